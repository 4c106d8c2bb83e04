"""Host-side logic of the multi-rank benchmark path: every rank derives its own seeded
batch (request-level data parallelism, no data-path collective) and the whole-job figure
is built from the max time over ranks.  Runs as two gloo ranks on CPU."""
import os
import subprocess
import sys
import textwrap

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = textwrap.dedent("""
    import os, sys, json
    sys.path.insert(0, %r)
    import numpy as np, torch, torch.distributed as dist
    import oracle
    from wuda_b200 import workloads
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    case = workloads.make_mqa_case(3, 2, 50, 400, seed=0xB201 + rank)
    logits = oracle.mqa_logits_fp8(case["q"], case["kv_pages"], case["weights"], case["context_lens"],
                                   case["block_table"], 2, 64, case["logits_stride"])
    pt = np.repeat(case["block_table"], 2, axis=0)
    pages, raw = oracle.topk(logits, case["context_lens"].reshape(-1), pt, 64, 64)
    # ranks hold different requests
    digest = torch.tensor([float(case["ctx"].sum()), float(raw.astype(np.int64).sum())], dtype=torch.float64)
    gathered = [torch.zeros_like(digest) for _ in range(world)]
    dist.all_gather(gathered, digest)
    t = torch.tensor([1.0 + rank], dtype=torch.float64)      # stand-in for a per-rank step time
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        print(json.dumps({"distinct": bool((gathered[0] != gathered[1]).any()), "max_time": float(t.item()),
                          "world": world}))
    dist.destroy_process_group()
""") % ROOT


def test_two_gloo_ranks_own_distinct_batches_and_take_max_time(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="2")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                          "--master-addr", "127.0.0.1", "--master-port", "29591", str(script)],
                         capture_output=True, text=True, env=env, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    line = [l for l in out.stdout.splitlines() if l.startswith("{")][-1]
    import json
    res = json.loads(line)
    assert res == {"distinct": True, "max_time": 2.0, "world": 2}


def test_reference_arm_prints_one_json_line():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1",
                          "--warmup", "1"], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    import json
    res = json.loads(out.stdout.strip().splitlines()[-1])
    assert res["impl"] == "reference" and res["cpu_baseline"]["kind"] == "port" and res["value"] > 0
    assert res["e2e"]["h2d_bytes_per_step"] == 0


def test_reference_arm_takes_all_cores_under_a_launcher_and_never_loads_the_product(tmp_path):
    """A multi-rank launcher exports OMP_NUM_THREADS=1 to its workers; the CPU arm must still use the cores
    the process may run on, and it must not map the CUDA library (it times the oracle, not the product)."""
    probe = tmp_path / "probe.py"
    probe.write_text(textwrap.dedent("""
        import json, runpy, sys
        sys.argv = [%r, "--impl", "reference", "--steps", "1", "--warmup", "1"]
        runpy.run_path(sys.argv[0], run_name="__main__")
        print(json.dumps({"mapped": sorted({l.split()[-1].rsplit("/", 1)[-1] for l in open("/proc/self/maps")
                                            if "libwuda" in l or "liboracle" in l})}))
    """) % os.path.join(ROOT, "bench.py"))
    env = dict(os.environ, OMP_NUM_THREADS="1", RANK="0", WORLD_SIZE="2", LOCAL_RANK="0")
    out = subprocess.run([sys.executable, str(probe)], capture_output=True, text=True, timeout=600, env=env)
    assert out.returncode == 0, out.stderr[-2000:]
    import json
    lines = [json.loads(l) for l in out.stdout.splitlines() if l.startswith("{")]
    cores = len(os.sched_getaffinity(0))
    assert lines[0]["impl"] == "reference" and lines[0]["cpu_baseline"]["cores"] == cores
    assert lines[1]["mapped"] == ["liboracle.so"]
    # every other rank leaves without work and without output
    env["RANK"] = "1"
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1"],
                         capture_output=True, text=True, timeout=600, env=env)
    assert out.returncode == 0 and out.stdout.strip() == ""


HANDLE_WORKER = textwrap.dedent("""
    import os, sys, json
    sys.path.insert(0, %r)
    import torch.distributed as dist
    dist.init_process_group("gloo")
    from wuda_b200.ops import exchange_handles
    rank = dist.get_rank()
    mine = bytes([rank + 1] * 64)
    peer = exchange_handles(mine)
    ok = peer == bytes([2 - rank] * 64)
    flags = [None, None]
    dist.all_gather_object(flags, ok)
    if rank == 0:
        print(json.dumps({"ok": all(flags)}))
    dist.destroy_process_group()
""") % ROOT


def test_tp2_handle_exchange_over_gloo(tmp_path):
    """Host-side bootstrap of the two-rank link: each rank ends up with the other's 64-byte handle."""
    script = tmp_path / "handles.py"
    script.write_text(HANDLE_WORKER)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                          "--master-addr", "127.0.0.1", "--master-port", "29593", str(script)],
                         capture_output=True, text=True, env=env, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    import json
    assert json.loads([l for l in out.stdout.splitlines() if l.startswith("{")][-1]) == {"ok": True}
