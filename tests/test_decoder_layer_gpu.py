"""The whole decode layer (wuda_b200.layer.DecoderLayer: attention half, then mHC pre / ffn norm / router /
routed NVFP4 experts + shared expert / mHC post, the origin's Block.forward, origin/model.py:688-700) on one
GPU.  Every stage has its own parity test; here the wiring of the feed-forward half is checked by composing
the same tested entry points by hand from the layer's own intermediate tensors, the CUDA graph of the layer
must reproduce the eager pass bit for bit, and two runs from the same state must agree in every bit of every
pool and state ring (the reference's own race check, test/test_e2e_decode.py:1602-1628).

The two-GPU form (tensor-parallel pair) runs as child processes and is skipped on a single-GPU machine."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from wuda_b200 import moe, ops
from wuda_b200.layer_setup import build_random_layer

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SMALL = dict(topk=512, experts=32, inter=512, moe_topk=4)


def test_feed_forward_half_is_wired_like_block_forward():
    batch = 6
    layer, slots, x = build_random_layer(batch, 1500, seed=5, native=False, **SMALL)     # sequenced from Python
    layer.prepare(slots)
    out = layer.launch(x, batch).clone()
    torch.cuda.synchronize()
    layer.check_status()
    assert tuple(out.shape) == (batch, 4, 7168) and bool(torch.isfinite(out.float()).all())
    # by hand: the attention half's output is the residual of the feed-forward half
    f = layer.ffn
    x1 = layer.attn.out
    pre = ops.mhc_pre(x1, f.hc_weight, f.hc_base, f.hc_scale, f.ffn_norm, quant=False)
    rw, idx = ops.moe_gate(pre["normed"], f.gate_weight, f.gate_bias, f.score_func, f.route_scale, f.topk)
    assert torch.equal(idx, layer.route_indices)
    runner = moe.MoERunner(f.routed, batch, f.topk)
    y = runner.forward(pre["normed"], rw, idx, shared=f.shared.forward(pre["normed"]))
    want = ops.mhc_post_out(y, x1, pre["post"], pre["comb"], torch.empty_like(x1))
    torch.cuda.synchronize()
    assert torch.equal(out, want)
    # the MoE half changed the streams: the layer is not the attention half alone
    assert not torch.equal(out, x1)
    # graph replay == eager pass
    layer.capture(x, batch)
    again = layer.replay()
    torch.cuda.synchronize()
    layer.check_status()
    assert torch.equal(out, again)
    # the library's own C++ sequence (one call per step) gives the same bits from the same state
    native, slots_n, x_n = build_random_layer(batch, 1500, seed=5, native=True, **SMALL)
    native.prepare(slots_n)
    out_n = native.launch(x_n, batch)
    torch.cuda.synchronize()
    native.check_status()
    assert torch.equal(x, x_n) and torch.equal(out, out_n)
    assert torch.equal(native.view("mla_out", torch.bfloat16, batch, 128, 512), layer.attn.mla_out[:batch])
    assert torch.equal(native.route_indices, layer.route_indices)
    for pool in ("idx_pool", "cmp_pool", "swa_pool", "main_state", "idx_state"):
        assert torch.equal(getattr(native.attn.cache, pool), getattr(layer.attn.cache, pool))
    native.capture(x_n, batch)
    again = native.replay()
    torch.cuda.synchronize()
    native.check_status()
    assert torch.equal(out, again)


def _snapshot(layer):
    c, b = layer.attn.cache, layer.max_batch
    stride = layer.attn.stage.logits_stride
    return [t.clone() for t in (c.idx_pool, c.cmp_pool, c.swa_pool, c.main_state, c.idx_state,
                                layer.view("logits", torch.float32, b, stride), layer.view("topk_raw", torch.int32, b, layer.attn.topk).sort(-1).values,
                                layer.view("mla_out", torch.bfloat16, b, 128, 512), layer.out)]


def test_two_runs_from_the_same_state_agree_bit_for_bit():
    """Run-to-run determinism over outputs, pools and state rings: any race between the forked cache writers,
    the query tail and the main chain, or between stream-K partial sums, would show here."""
    batch = 5
    snaps = []
    for _ in range(2):
        layer, slots, x = build_random_layer(batch, 2052, seed=9, **SMALL)     # position 2051: a compress step
        layer.prepare(slots)
        layer.launch(x, batch)
        torch.cuda.synchronize()
        layer.check_status()
        snaps.append(_snapshot(layer))
        del layer
    for a, b in zip(*snaps):
        assert torch.equal(a.view(torch.uint8), b.view(torch.uint8))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_tensor_parallel_pair_matches_one_gpu():
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", NCCL_NVLS_ENABLE="0")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                          "--master-addr", "127.0.0.1", "--master-port", "29617",
                          os.path.join(ROOT, "tests", "layer_tp2_worker.py")],
                         capture_output=True, text=True, env=env, timeout=900)
    assert out.returncode == 0, out.stderr[-3000:]
    res = json.loads([l for l in out.stdout.splitlines() if l.startswith("{")][-1])
    assert res["status"] == [0, 0] and res["ranks_identical"] and res["replays_identical"] and res["finite"]
    # floating point: heads, K halves and experts are summed in another order on a pair, and the shared
    # expert's two halves are rounded to bf16 before they are added; tolerance 2e-2 of the output's norm
    assert res["rel_err_vs_one_gpu"] < 2e-2, res
