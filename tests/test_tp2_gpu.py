"""The two-rank tensor-parallel GEMM with the all-reduce fused into its epilogue.

test_two_ranks needs two GPUs (one process per GPU, peer memory over NVLink) and is skipped
on a single-GPU box; the time-out path runs on one GPU with a peer that never answers."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import oracle
from wuda_b200 import workloads

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_peer_that_never_answers_times_out_cleanly(wuda):
    """A link whose peer is the rank itself: nothing ever raises the awaited flags, so every
    tile owner runs into the wait limit.  The kernel must end, report the code, and leave the
    context usable."""
    case = workloads.make_gemm_fp8_case(16, 1024, 1024, seed=3)
    a = torch.from_numpy(case["a"]).cuda().view(torch.float8_e4m3fn)
    w = torch.from_numpy(case["w"]).cuda().view(torch.float8_e4m3fn)
    a_s, w_s = torch.from_numpy(case["a_s"]).cuda(), torch.from_numpy(case["w_s"]).cuda()
    link = wuda.TP2Link(16, 1024, loopback=True)
    status = wuda.device_status_word()
    link.fp8_gemm(a, a_s, w, w_s, status_word=status, peer_wait_ms=20)
    torch.cuda.synchronize()
    assert int(status.item()) == 131
    link.close()
    # the context still works, and the ordinary GEMM (same scratch) is still right
    out = wuda.fp8_gemm(a, a_s, w, w_s)
    torch.cuda.synchronize()
    ref = oracle.gemm_fp8_blockscaled(case["a"], case["a_s"], case["w"], case["w_s"], out_bf16=False)
    f = oracle.bf16_to_f32(out.cpu().view(torch.int16).numpy().view(np.uint16))
    assert np.all(np.abs(f - ref) <= 1e-2 * np.abs(ref) + 1e-3 * np.sqrt(np.mean(ref.astype(np.float64) ** 2)))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_ranks_sum_over_nvlink_matches_oracle():
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", NCCL_NVLS_ENABLE="0")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                          "--master-addr", "127.0.0.1", "--master-port", "29611",
                          os.path.join(ROOT, "tests", "tp2_worker.py")],
                         capture_output=True, text=True, env=env, timeout=600)
    assert out.returncode == 0, out.stderr[-3000:]
    res = json.loads([l for l in out.stdout.splitlines() if l.startswith("{")][-1])
    assert len(res) == 3
    for shape, r in res.items():
        assert r == {"ok": True, "status": 0, "calls_identical": True, "ranks_identical": True}, (shape, r)
