"""Benchmark of the indexer step (paged FP8 MQA logits + top-2048 selection) and of the decode layer.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (N = 1): batch 64 x next_n 2 = 128 query rows, 64 heads x 128 dims, FP8 e4m3
queries and keys, key pages of 64 tokens with per-token fp32 scales, context lengths
uniform in [16384, 65536], block table = a random permutation of the physical pages,
then the indices of the 2048 largest logits per row mapped through the block table.
Seeded synthetic data generated on the host.  With N > 1 every rank runs its own batch
of 64 requests (requests are independent: no collective on the data path, weak scaling).

A step is one MQA-logits launch plus one top-k launch.  `value` is the algorithmic bytes
of one step (keys and scales read once per request, fp32 logits written once and read
once, q/weights/indices) divided by the device time of the step, inputs resident in HBM.
`e2e` is the same number through the host-buffer C-ABI call, host<->device copies
included.  `--impl reference` times the CPU oracle (the reference ships no CPU
implementation of this path) on a bounded sample of the same workload, on every host core
the process may use (one rank only under a multi-rank launcher).

Beside the indexer step the line carries the decode layer (one random-init sparse-attention MoE
layer, batch 64, context 32768): `layer` = one GPU (N = 1), and for N >= 2 the ranks pair up
(0,1), (2,3), .. as independent tensor-parallel replicas: `tp2` = the wo_b projection with its
all-reduce fused into the GEMM epilogue over NVLink peer memory, checked against the CPU oracle;
`ep2` = the expert-parallel MoE block whose combine step exchanges rows over peer memory, checked
against the ranks' own partial sums; `layer_tp2` = the whole layer on a pair, decode
tokens/s/GPU = 64 / (t_layer x 2), checked against the same layer on one GPU.
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
# the pair legs exchange through plain peer loads and stores; NCCL (bootstrap and barriers only) stays
# off the NVLink multicast objects
os.environ.setdefault("NCCL_NVLS_ENABLE", "0")


def load_workloads():
    """The synthetic-input generators, loaded by path: importing the package would load the CUDA library,
    which the reference arm must not do."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("wuda_b200_workloads", os.path.join(ROOT, "wuda_b200", "workloads.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod

BATCH, NEXT_N, CTX_LO, CTX_HI, EPB, TOPK = 64, 2, 16384, 65536, 64, 2048
SEED = 0xB201
SAMPLE_REQUESTS = 8          # requests of the workload the CPU legs run
WORKLOAD = "paged MQA logits fp8 + top-2048: batch %d x next_n 2, 64 heads x 128, page 64, ctx U[16384,65536]"
METRIC = "MQA-logits + top-k HBM GB/s"


def step_bytes(case):
    workloads = load_workloads()
    rows = case["batch"] * case["next_n"]
    mqa = workloads.mqa_algorithmic_bytes(case)
    topk = int(case["context_lens"].sum()) * 4 + rows * TOPK * 4
    return mqa, topk


def measured_hbm_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def measured_traffic(algorithmic_bytes):
    """DRAM bytes of one MQA launch from the profiler capture recorded under profiles/ (DRAM bytes per
    algorithmic byte of a smaller batch), or None when no capture is recorded."""
    try:
        with open(os.path.join(ROOT, "profiles", "mqa_logits_fp8_traffic.json")) as f:
            return int(float(json.load(f)["dram_bytes_per_algorithmic_byte"]) * algorithmic_bytes)
    except Exception:
        return None


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.path = tempfile.mktemp(suffix=".csv")
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(gpu_index), "--query-gpu=" + self.FIELDS, "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        try:
            for line in open(self.path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 9:
                    continue
                try:
                    clk, clk_max, power = float(f[1]), float(f[2]), float(f[3])
                except ValueError:
                    continue
                if power < 250.0:      # idle sample taken before the load started
                    continue
                sm.append(clk)
                mx.append(clk_max)
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            out.update(sm_mhz=float(np.median(sm)), sm_max_mhz=float(max(mx)), reasons=sorted(reasons), samples=len(sm))
        return out


def cpu_sample(case):
    """The first SAMPLE_REQUESTS requests of the workload as a self-contained case."""
    n = min(SAMPLE_REQUESTS, case["batch"])
    rows = n * case["next_n"]
    sub = dict(case)
    sub.update(batch=n, q=case["q"][:rows], weights=case["weights"][:rows], context_lens=case["context_lens"][:n],
               block_table=case["block_table"][:n], ctx=case["ctx"][:n])
    return sub


def cpu_step(sub):
    import oracle
    logits = oracle.mqa_logits_fp8(sub["q"], sub["kv_pages"], sub["weights"], sub["context_lens"],
                                   sub["block_table"], sub["next_n"], sub["epb"], sub["logits_stride"])
    pt = np.repeat(sub["block_table"], sub["next_n"], axis=0)
    oracle.topk(logits, sub["context_lens"].reshape(-1), pt, TOPK, sub["epb"])


def time_cpu(sub, steps, warmup):
    import oracle
    oracle.set_num_threads()          # a launcher's OMP_NUM_THREADS=1 is for its GPU workers, not for this leg
    for _ in range(warmup):
        cpu_step(sub)
    t0 = time.perf_counter()
    for _ in range(steps):
        cpu_step(sub)
    dt = (time.perf_counter() - t0) / max(steps, 1)
    mqa_b, topk_b = step_bytes(sub)
    return (mqa_b + topk_b) / dt / 1e9, dt, oracle.num_threads()


def run_reference(args, rank):
    if rank != 0:
        return
    workloads = load_workloads()
    case = workloads.make_mqa_case(SAMPLE_REQUESTS, NEXT_N, CTX_LO, CTX_HI, epb=EPB, seed=SEED)
    gbs, dt, cores = time_cpu(case, args.steps, min(args.warmup, 1))
    sample = "first %d of 64 requests (same seed), every step" % SAMPLE_REQUESTS
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD % BATCH, "sample": sample},
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="wuda_b200", choices=["wuda_b200", "reference"])
    ap.add_argument("--e2e-steps", type=int, default=3)
    ap.add_argument("--batch", type=int, default=BATCH,
                    help="requests per rank (default 64 = the benchmark workload; smaller values are for profiler captures)")
    ap.add_argument("--capture", action="store_true",
                    help="profiler capture mode: no clock pre-warm, no end-to-end leg, no CPU baseline, no layer legs")
    ap.add_argument("--no-layer", action="store_true", help="skip the decode-layer legs (indexer step only)")
    ap.add_argument("--layer-reps", type=int, default=20, help="timed CUDA-graph replays of the layer legs")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        run_reference(args, rank)
        return

    import torch
    import torch.distributed as dist
    import wuda_b200 as wuda
    from wuda_b200 import workloads

    torch.cuda.set_device(local_rank)
    host_group = pair_group = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        # host-side groups (gloo) for the pair legs: IPC handles, barriers and result objects travel over them
        host_group = dist.new_group(backend="gloo")
        pairs = [dist.new_group([2 * i, 2 * i + 1], backend="gloo") for i in range(world // 2)]
        if rank // 2 < len(pairs):
            pair_group = pairs[rank // 2]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # every rank owns a batch of its own: request-level data parallelism, no exchange
    batch = args.batch
    case = workloads.make_mqa_case(batch, NEXT_N, CTX_LO, CTX_HI, epb=EPB, seed=SEED + rank)
    rows = batch * NEXT_N
    d = workloads.to_device(case)
    logits = torch.empty((rows, case["logits_stride"]), dtype=torch.float32, device="cuda")
    indices = torch.empty((rows, TOPK), dtype=torch.int32, device="cuda")
    seq_lens = d["context_lens"].reshape(-1).contiguous()
    status = wuda.device_status_word()

    def mqa():
        wuda.mqa_logits_fp8_decode_out(d["q"], d["kv_pages"], d["weights"], d["context_lens"], d["block_table"],
                                       None, logits, EPB, next_n=NEXT_N, status_word=status)

    def topk():
        wuda.topk_v2_transform(logits, seq_lens, d["block_table"], indices, EPB, rows_per_table_row=NEXT_N)

    def step():
        mqa()
        topk()

    # One step = one CUDA graph of the two launches, replayed: the host-side cost of a
    # launch (argument checks, tensor-map encoding, ~25 us) would otherwise leave the GPU
    # idle between the kernels.  A decode engine replays the layer as a graph too.
    step()
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        step_graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(step_graph, stream=side):
            step()
        topk_graph = torch.cuda.CUDAGraph()     # ten top-k launches, for the per-kernel split
        with torch.cuda.graph(topk_graph, stream=side):
            for _ in range(10):
                topk()
    torch.cuda.synchronize()

    # The sampler runs from here to the end of the timed region: the GPU is under the
    # same load throughout (the timed region alone is shorter than nvidia-smi's period).
    sampler = ClockSampler(local_rank)
    # bring the clocks up from idle before anything is measured
    t_end = time.perf_counter() + (0.0 if args.capture else 1.0)
    while time.perf_counter() < t_end:
        for _ in range(20):
            step_graph.replay()
        torch.cuda.synchronize()
    for _ in range(args.warmup):
        step_graph.replay()
    barrier()
    e0, e1, e2, e3 = (torch.cuda.Event(enable_timing=True) for _ in range(4))
    barrier()
    e0.record()
    for _ in range(args.steps):
        step_graph.replay()
    e1.record()
    barrier()
    total_ms = e0.elapsed_time(e1)
    # per-kernel durations, same stream, right after the timed region: the MQA kernel
    # launched back to back (the host is faster than the kernel), top-k as graphs of ten
    e1.record()
    for _ in range(args.steps):
        mqa()
    e2.record()
    reps = max(args.steps // 10, 1)
    for _ in range(reps):
        topk_graph.replay()
    e3.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    mqa_ms = e1.elapsed_time(e2) / args.steps
    topk_ms = e2.elapsed_time(e3) / (reps * 10)
    assert int(status.item()) == 0, "device status %d" % int(status.item())

    t = torch.tensor([total_ms], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms = float(t.item())
    ms_per_step = total_ms / args.steps
    mqa_b, topk_b = step_bytes(case)
    value = world * (mqa_b + topk_b) / (ms_per_step * 1e-3) / 1e9

    if args.capture:
        if rank == 0:
            print(json.dumps({"capture": True, "batch": batch, "ms_per_step": ms_per_step,
                              "kernels_us": {"mqa_logits_fp8": mqa_ms * 1e3, "topk": topk_ms * 1e3}}))
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- end to end through the host-buffer C-ABI call (pinned host inputs, results on the host)
    host = {k: torch.from_numpy(case[k]).pin_memory() for k in ("q", "kv_pages", "weights", "context_lens", "block_table")}
    out_host = torch.empty((rows, TOPK), dtype=torch.int32).pin_memory()
    plan = wuda.IndexerHostPlan(batch, NEXT_N, case["num_blocks"], EPB, case["page_stride"],
                                case["block_table"].shape[1], case["logits_stride"], TOPK)

    def e2e_step():
        plan.run(host["q"], host["kv_pages"], host["weights"], host["context_lens"], host["block_table"], out_host, batch)

    e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.e2e_steps):
        e2e_step()
    torch.cuda.synchronize()
    e2e_s = torch.tensor([(time.perf_counter() - t0) / args.e2e_steps], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(e2e_s, op=dist.ReduceOp.MAX)
    e2e_s = float(e2e_s.item())
    h2d = sum(int(v.numel() * v.element_size()) for v in host.values())
    d2h = int(out_host.numel() * 4) + 4
    same = np.array_equal(np.sort(out_host.numpy(), axis=1), np.sort(indices.cpu().numpy(), axis=1))

    # The same call with the key pool resident on the device, as a decode server keeps it: a step appends next_n
    # tokens per request, i.e. rewrites the page that holds each request's last tokens; only those pages travel.
    last_page = (case["context_lens"].reshape(batch, -1).max(axis=1) - 1) // EPB
    dirty = np.unique(case["block_table"][np.arange(batch), last_page]).astype(np.int32)
    dirty_host = torch.from_numpy(dirty).pin_memory()
    out_resident = torch.empty((rows, TOPK), dtype=torch.int32).pin_memory()

    def resident_step():
        plan.run(host["q"], host["kv_pages"], host["weights"], host["context_lens"], host["block_table"], out_resident, batch,
                 dirty_pages=dirty_host)

    resident_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(4 * args.e2e_steps):
        resident_step()
    torch.cuda.synchronize()
    res_s = torch.tensor([(time.perf_counter() - t0) / (4 * args.e2e_steps)], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(res_s, op=dist.ReduceOp.MAX)
    res_s = float(res_s.item())
    h2d_resident = h2d - int(host["kv_pages"].numel()) + int(dirty.size) * int(case["page_stride"])
    same_resident = np.array_equal(out_resident.numpy(), out_host.numpy())
    plan.close()

    if rank == 0:
        peak, peak_kind = measured_hbm_peak()
        achieved = mqa_b / (mqa_ms * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "fp8_e4m3 x fp8_e4m3 -> f32", "data": "synthetic",
            "config": {"workload": WORKLOAD % batch, "l2": "inputs (%.0f MB of key pages per rank) larger than the 126 MB L2; "
                       "no flush between iterations" % (case["kv_pages"].nbytes / 1e6),
                       "parallelism": "request-dp%d" % world, "rows_per_s": world * rows / (ms_per_step * 1e-3)},
            "kernels_us": {"mqa_logits_fp8": mqa_ms * 1e3, "topk": topk_ms * 1e3},
            "roofline": {"kernel": "mqa_logits_fp8_kernel<2>", "bound": "hbm", "achieved": achieved, "peak": peak,
                         "peak_kind": peak_kind, "unit": "GB/s", "frac": achieved / peak,
                         # DRAM read + write bytes per launch: the profiler's figure for a smaller batch of the
                         # same workload, scaled by algorithmic bytes (the traffic is the key stream)
                         "traffic": measured_traffic(mqa_b) if batch == BATCH else None, "algorithmic_bytes": mqa_b},
            "e2e": {"value": world * (mqa_b + topk_b) / e2e_s / 1e9, "unit": "GB/s", "ms_per_step": e2e_s * 1e3,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "matches_device_path": bool(same),
                    "note": "every input crosses PCIe every step, the whole key pool included"},
            "e2e_resident_pool": {"value": world * (mqa_b + topk_b) / res_s / 1e9, "unit": "GB/s", "ms_per_step": res_s * 1e3,
                                  "h2d_bytes_per_step": h2d_resident, "d2h_bytes_per_step": d2h,
                                  "matches_full_upload": bool(same_resident),
                                  "note": "the same host-buffer call with the key pool kept on the device between steps: "
                                          "q, weights, lengths, block table and the %d pages that hold the requests' "
                                          "newest tokens cross PCIe" % int(dirty.size)},
            "gpu_launches": 2 * args.steps, "launch": "one CUDA graph replay per step",
            "clocks": clocks,
        }
        if world == 1:
            gbs, dt, cores = time_cpu(cpu_sample(case), 3, 1)
            line["cpu_baseline"] = {"value": gbs, "unit": "GB/s", "cores": cores, "kind": "port",
                                    "sample": "first %d of %d requests, 3 timed passes of the C oracle "
                                              "(OpenMP), %.2f s each" % (min(SAMPLE_REQUESTS, batch), batch, dt)}
    else:
        line = None

    # ---- the decode layer: one GPU at N = 1, tensor-parallel pairs (and their exchange kernels) at N >= 2
    torch.cuda.empty_cache()
    if not args.no_layer:
        legs = layer_legs(args, rank, world, host_group, pair_group)
        if rank == 0:
            line.update(legs)
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def bf16_bits_to_f32(u16):
    return (u16.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_bits(x):
    """Round-to-nearest-even bf16 bits of finite fp32 values."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def layer_legs(args, rank, world, host_group, pair_group):
    """Runs the layer legs on every rank and returns, on rank 0, the blocks to add to the JSON line."""
    import torch
    import torch.distributed as dist
    from wuda_b200 import benchmarks

    if world == 1:
        res, _ = benchmarks.layer_leg(reps=args.layer_reps)
        res["parallelism"] = "1 GPU"
        return {"layer": res}
    if pair_group is None:          # an odd rank out: nothing to pair with
        mine = None
    else:
        import oracle
        pair_rank = rank % 2
        mine = {}
        # (1) wo_b with the fused all-reduce: both ranks of a pair must hold bf16(partial_0 + partial_1)
        res, gcase, got = benchmarks.tp2_gemm_leg(pair_group, pair_rank)
        both = [None, None]
        dist.all_gather_object(both, got.tobytes(), group=pair_group)
        res["ranks_identical"] = both[0] == both[1]
        if rank == 0:               # the oracle check runs once: every pair gets the same inputs
            oracle.set_num_threads()
            k = gcase["a"].shape[1]
            parts = [oracle.gemm_fp8_blockscaled(gcase["a"][:, sl], gcase["a_s"][:, sb], gcase["w"][:, sl], gcase["w_s"][:, sb],
                                                 out_bf16=False)
                     for sl, sb in ((slice(0, k // 2), slice(0, k // 256)), (slice(k // 2, k), slice(k // 256, k // 128)))]
            ref = parts[0] + parts[1]
            f = bf16_bits_to_f32(got)
            rms = float(np.sqrt(np.mean(ref.astype(np.float64) ** 2)))
            res["matches_oracle"] = bool(np.all(np.abs(f - ref) <= 1e-2 * np.abs(ref) + 1e-3 * rms))
            res["tolerance"] = "|got - (oracle partial 0 + partial 1)| <= 1e-2 |ref| + 1e-3 rms"
        res["output_digest"] = int(np.bitwise_xor.reduce(got.reshape(-1).astype(np.uint64) * np.arange(1, got.size + 1, dtype=np.uint64)))
        mine["tp2"] = res
        # (2) expert-parallel MoE block: y must be bf16(own partial + peer partial) bit for bit
        res, got, part = benchmarks.ep2_combine_leg(pair_group, pair_rank)
        both = [None, None]
        dist.all_gather_object(both, (got.tobytes(), part.tobytes()), group=pair_group)
        parts = [np.frombuffer(b[1], np.float32).reshape(part.shape) for b in both]
        res["ranks_identical"] = both[0][0] == both[1][0]
        res["equals_sum_of_partials"] = bool(np.array_equal(got, f32_to_bf16_bits(parts[0] + parts[1])))
        mine["ep2"] = res
        # (3) the whole layer on the pair
        res, out = benchmarks.layer_leg(reps=args.layer_reps, group=pair_group, pair_rank=pair_rank)
        both = [None, None]
        dist.all_gather_object(both, out.numpy().tobytes(), group=pair_group)
        res["ranks_identical"] = both[0] == both[1]
        res["finite"] = bool(torch.isfinite(out).all())
        if rank == 0:               # the same layer (same seed) on one GPU, one eager pass
            from wuda_b200.layer_setup import build_random_layer
            single, slots, x = build_random_layer(64, 32768)
            single.prepare(slots)
            ref = single.launch(x, 64).float().cpu()
            single.check_status()
            err = float((out - ref).norm() / ref.norm())
            res["rel_err_vs_one_gpu"] = err
            res["matches_one_gpu"] = bool(err < 2e-2)
            del single
        mine["layer_tp2"] = res
    gathered = [None] * world
    dist.all_gather_object(gathered, mine, group=host_group)
    if rank != 0:
        return None
    leaders = [g for i, g in enumerate(gathered) if g is not None and i % 2 == 0]
    followers = [g for i, g in enumerate(gathered) if g is not None and i % 2 == 1]
    out = {}
    for key in ("tp2", "ep2", "layer_tp2"):
        block = dict(leaders[0][key])
        block["pairs"] = len(leaders)
        block["status"] = max(g[key]["status"] for g in leaders + followers)
        block["ranks_identical"] = all(g[key]["ranks_identical"] for g in leaders)
        out[key] = block
    t = out["tp2"]
    t["gemm_allreduce_us"] = max(g["tp2"]["gemm_allreduce_us"] for g in leaders)
    t["local_gemm_us"] = max(g["tp2"]["local_gemm_us"] for g in leaders)
    t["roofline_frac"] = t["roofline_us"] / t["gemm_allreduce_us"]
    t["pairs_identical"] = all(g["tp2"]["output_digest"] == t["output_digest"] for g in leaders)
    t["parity_ok"] = bool(t["matches_oracle"] and t["ranks_identical"] and t["pairs_identical"] and t["status"] == 0)
    e = out["ep2"]
    e["block_us"] = max(g["ep2"]["block_us"] for g in leaders)
    e["equals_sum_of_partials"] = all(g["ep2"]["equals_sum_of_partials"] for g in leaders + followers)
    e["parity_ok"] = bool(e["equals_sum_of_partials"] and e["ranks_identical"] and e["status"] == 0)
    l = out["layer_tp2"]
    l["layer_us"] = max(g["layer_tp2"]["layer_us"] for g in leaders)
    l["tok_s_per_gpu"] = l["batch"] / (l["layer_us"] * 1e-6) / 2
    l["tok_s_all_gpus"] = l["tok_s_per_gpu"] * 2 * len(leaders)
    l["finite"] = all(g["layer_tp2"]["finite"] for g in leaders + followers)
    l["parallelism"] = "tp2 x %d replicas" % len(leaders)
    l["parity_ok"] = bool(l["matches_one_gpu"] and l["ranks_identical"] and l["finite"] and l["status"] == 0)
    return out


if __name__ == "__main__":
    main()
