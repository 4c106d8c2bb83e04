"""Expert parallelism of the routed experts over two ranks: the expert-range dispatch, the combine step
that exchanges fp32 partial rows through peer memory, and its time-out path.

One-GPU tests use a rank that is its own peer (y = local + local) and a peer that never answers;
test_two_ranks needs two GPUs (one process per GPU) and is skipped on a single-GPU box."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import oracle
from wuda_b200 import moe

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def u16(t):
    return t.cpu().view(torch.int16).numpy().view(np.uint16)


def make(seed, tokens, experts, k, dim, inter):
    g = torch.Generator().manual_seed(seed)
    w1 = torch.randn(experts, inter, dim, generator=g) * 0.05
    w3 = torch.randn(experts, inter, dim, generator=g) * 0.05
    w2 = torch.randn(experts, dim, inter, generator=g) * 0.05
    x = torch.randn(tokens, dim, generator=g).bfloat16()
    idx = torch.stack([torch.randperm(experts, generator=g)[:k] for _ in range(tokens)]).int()
    rw = torch.rand(tokens, k, generator=g) + 0.1
    return w1, w3, w2, x, idx, rw


def local_sum(runner, tokens, k):
    """fp32 sum of the rank's own expert rows per token, in pair order (what the combine kernels add)."""
    of = oracle.bf16_to_f32(u16(runner.out))
    pr = runner.pair_row.cpu().numpy()[:tokens]
    acc = np.zeros((tokens, of.shape[1]), np.float32)
    for j in range(k):
        rows = np.where((pr[:, j] >= 0)[:, None], of[np.maximum(pr[:, j], 0)], 0.0).astype(np.float32)
        acc = (acc + rows).astype(np.float32)
    return acc


def test_expert_range_dispatch_takes_only_its_own_pairs(wuda):
    tokens, experts, k, dim, inter = 24, 8, 3, 512, 256
    w1, w3, w2, x, idx, rw = make(3, tokens, experts, k, dim, inter)
    half = experts // 2
    for first in (0, half):
        sl = slice(first, first + half)
        weights = moe.RoutedExperts(w1[sl], w3[sl], w2[sl], 4.0 / 2688, 3.0 / 2688)
        runner = moe.MoERunner(weights, tokens, k, expert_first=first, experts_total=experts)
        y = runner.forward(x.cuda(), rw.cuda(), idx.cuda())
        torch.cuda.synchronize()
        assert int(runner.status.item()) == 0
        mine = (idx.numpy() >= first) & (idx.numpy() < first + half)
        local = np.where(mine, idx.numpy() - first, -1)
        ge, rt, pr = oracle.moe_dispatch(local, half)
        groups = len(ge)
        assert int(runner.num_groups.item()) == groups
        assert np.array_equal(runner.group_expert.cpu().numpy()[:groups], ge)
        assert np.array_equal(runner.row_token.cpu().numpy()[:groups * 16], rt)
        assert np.array_equal(runner.pair_row.cpu().numpy()[:tokens], pr)
        assert np.array_equal(u16(y), oracle.f32_to_bf16(local_sum(runner, tokens, k)))
    # an index outside [0, experts_total) is still reported
    bad = idx.clone()
    bad[0, 0] = experts
    runner.forward(x.cuda(), rw.cuda(), bad.cuda())
    torch.cuda.synchronize()
    assert int(runner.status.item()) == 143


def test_rank_that_is_its_own_peer_adds_its_row_twice(wuda):
    tokens, experts, k, dim, inter = 40, 6, 2, 768, 256
    w1, w3, w2, x, idx, rw = make(4, tokens, experts, k, dim, inter)
    weights = moe.RoutedExperts(w1, w3, w2, 4.0 / 2688, 3.0 / 2688)
    link = moe.EP2Link(64, dim, loopback=True)
    runner = moe.MoERunner(weights, 64, k, link=link)
    shared = torch.randn(tokens, dim, generator=torch.Generator().manual_seed(1)).bfloat16()
    for _ in range(3):                       # both inbox sets and their reuse
        y = runner.forward(x.cuda(), rw.cuda(), idx.cuda(), shared=shared.cuda())
    torch.cuda.synchronize()
    assert int(runner.status.item()) == 0
    part = (local_sum(runner, tokens, k) + oracle.bf16_to_f32(u16(shared))).astype(np.float32)
    assert np.array_equal(u16(y), oracle.f32_to_bf16((part + part).astype(np.float32)))
    link.close()


def test_peer_that_never_answers_times_out_cleanly(wuda):
    tokens, experts, k, dim, inter = 8, 4, 2, 512, 256
    w1, w3, w2, x, idx, rw = make(5, tokens, experts, k, dim, inter)
    weights = moe.RoutedExperts(w1, w3, w2, 4.0 / 2688, 3.0 / 2688)
    link = moe.EP2Link(16, dim, mute=True)
    runner = moe.MoERunner(weights, 16, k, link=link, peer_wait_ms=20)
    y = runner.forward(x.cuda(), rw.cuda(), idx.cuda())
    torch.cuda.synchronize()
    assert int(runner.status.item()) == 131                 # WUDA_DEV_TIMEOUT_PEER_FLAG
    assert np.array_equal(u16(y), oracle.f32_to_bf16(local_sum(runner, tokens, k)))   # the local sum stays
    link.close()
    runner.status.zero_()
    plain = moe.MoERunner(weights, 16, k)                   # the context still works
    y2 = plain.forward(x.cuda(), rw.cuda(), idx.cuda())
    torch.cuda.synchronize()
    assert torch.equal(y, y2)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_ranks_match_the_sum_of_their_parts():
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", NCCL_NVLS_ENABLE="0")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                          "--master-addr", "127.0.0.1", "--master-port", "29621",
                          os.path.join(ROOT, "tests", "ep2_worker.py")],
                         capture_output=True, text=True, env=env, timeout=600)
    assert out.returncode == 0, out.stderr[-3000:]
    res = json.loads([l for l in out.stdout.splitlines() if l.startswith("{")][-1])
    assert res == {"status": [0, 0], "ranks_identical": True, "calls_identical": True, "equals_sum_of_parts": True,
                   "close_to_one_rank": True}, res
