"""GPU parity of the routed-expert block (dispatch, NVFP4 gather-quantisation, grouped NVFP4 GEMMs,
SwiGLU + quantisation, combine; all through the C ABI) against the CPU oracle, stage by stage: every
stage's GPU output is compared with the oracle applied to that stage's GPU inputs."""
import numpy as np
import pytest
import torch

import oracle
from wuda_b200 import moe

pytestmark = pytest.mark.gpu


def u16(t):
    return t.cpu().view(torch.int16).numpy().view(np.uint16)


def unpack_sf(packed, groups, kb):
    """[groups, kb, 2048] image -> scale bytes [groups*16, kb*16] (rows 0..15 of every 128-row image)."""
    v = packed.reshape(groups, kb, 4, 32, 4, 4)            # [g][kb][step][row%32][row/32][byte]
    rows = v[:, :, :, :16, 0, :]                           # [g][kb][step][r][byte]
    return np.ascontiguousarray(rows.transpose(0, 3, 1, 2, 4)).reshape(groups * 16, kb * 16)


def close_bf16(got, ref, rel=1e-2):
    g, r = oracle.bf16_to_f32(got), oracle.bf16_to_f32(ref)
    assert np.all(np.abs(g - r) <= rel * np.abs(r) + 2e-3 * np.abs(r).max())


@pytest.mark.parametrize("tokens,experts,k,dim,inter,limit", [(20, 6, 3, 512, 256, 0.0), (64, 16, 4, 768, 512, 7.0),
                                                              (1, 4, 2, 256, 256, 0.0)])
def test_routed_experts_stagewise(wuda, tokens, experts, k, dim, inter, limit):
    g = torch.Generator().manual_seed(tokens * 13 + experts)
    w1 = torch.randn(experts, inter, dim, generator=g) * 0.05
    w3 = torch.randn(experts, inter, dim, generator=g) * 0.05
    w2 = torch.randn(experts, dim, inter, generator=g) * 0.05
    weights = moe.RoutedExperts(w1, w3, w2, act_scale_in=4.0 / (448 * 6), act_scale_mid=3.0 / (448 * 6), swiglu_limit=limit)
    runner = moe.MoERunner(weights, tokens, k)
    x = torch.randn(tokens, dim, generator=g).bfloat16()
    # a skewed routing: expert 0 takes more than one group of 16 when there are enough tokens
    idx = torch.stack([torch.randperm(experts, generator=g)[:k] for _ in range(tokens)]).int()
    if tokens >= 20:
        idx[:18, 0] = 0
        for t in range(18):                                # keep the k experts of a token distinct
            for j in range(1, k):
                if idx[t, j] == 0:
                    idx[t, j] = experts - 1 if (experts - 1) not in idx[t].tolist() else experts - 2
    rw = torch.rand(tokens, k, generator=g) + 0.1
    shared = torch.randn(tokens, dim, generator=g).bfloat16()
    y = runner.forward(x.cuda(), rw.cuda(), idx.cuda(), shared=shared.cuda())
    torch.cuda.synchronize()
    assert int(runner.status.item()) == 0

    # 1 dispatch: identical
    ge, rt, pr = oracle.moe_dispatch(idx.numpy(), experts)
    groups = len(ge)
    assert int(runner.num_groups.item()) == groups
    assert np.array_equal(runner.group_expert.cpu().numpy()[:groups], ge)
    assert np.array_equal(runner.row_token.cpu().numpy()[:groups * 16], rt)
    assert np.array_equal(runner.pair_row.cpu().numpy()[:tokens], pr)
    rows = groups * 16
    live = rt >= 0
    row_w = np.zeros(rows, np.float32)
    row_w[pr.reshape(-1)] = rw.numpy().reshape(-1)
    assert np.array_equal(runner.row_weight.cpu().numpy()[:rows], row_w)
    # 2 gather + quantise: bit-exact on the rows that hold a token.  Padding rows are never written (neither values
    # nor scales): the grouped GEMM does not store their outputs and nothing reads them.
    xr = np.zeros((rows, dim), np.float32)
    xr[live] = oracle.bf16_to_f32(u16(x))[rt[live]]
    q, sf = oracle.quantize_nvfp4_rows(xr, weights.act_scale_in)
    assert np.array_equal(runner.a1.cpu().numpy()[:rows][live], q[live])
    a1_sf = unpack_sf(runner.a1_sf.cpu().numpy()[:groups], groups, dim // 256)
    assert np.array_equal(a1_sf[live], sf[live])
    # 3 grouped w1|w3 GEMM on the GPU's own quantised rows
    h = u16(runner.h)[:rows]
    for gi, e in enumerate(ge):
        sl = slice(gi * 16, gi * 16 + 16)
        ref = oracle.gemm_nvfp4(q[sl], sf[sl], weights.act_scale_in, weights.host["w13"][e], weights.raw_scales["w13"][e],
                                weights.host["w13_gs"][e])
        close_bf16(h[sl][live[sl]], ref[live[sl]])
    # 4 SwiGLU + routing weight + quantise, from the GPU's h
    act = oracle.moe_swiglu(h, row_w, limit)
    act[~live] = 0
    q2, sf2 = oracle.quantize_nvfp4_rows(oracle.bf16_to_f32(act), weights.act_scale_mid)
    a2 = runner.a2.cpu().numpy()[:rows]
    a2_sf = unpack_sf(runner.a2_sf.cpu().numpy()[:groups], groups, inter // 256)
    assert np.mean(a2[live] == q2[live]) >= 0.995 and np.mean(a2_sf[live] == sf2[live]) >= 0.995     # expf differs in the last bit
    # 5 grouped w2 GEMM on the GPU's own a2
    out = u16(runner.out)[:rows]
    for gi, e in enumerate(ge):
        sl = slice(gi * 16, gi * 16 + 16)
        ref = oracle.gemm_nvfp4(a2[sl], a2_sf[sl], weights.act_scale_mid, weights.host["w2"][e],
                                weights.raw_scales["w2"][e], weights.host["w2_gs"][e])
        close_bf16(out[sl][live[sl]], ref[live[sl]])
    # 6 combine: exact, pairs in slot order, then the shared expert's row
    of = oracle.bf16_to_f32(out)
    acc = np.zeros((tokens, dim), np.float32)
    for j in range(k):
        acc = (acc + of[pr[:, j]]).astype(np.float32)
    acc = (acc + oracle.bf16_to_f32(u16(shared))).astype(np.float32)
    assert np.array_equal(u16(y), oracle.f32_to_bf16(acc))


def test_end_to_end_against_a_float_reference(wuda):
    """The whole block against an fp32 evaluation of the origin's formula on the unquantised weights.  e2m1
    has about 10 % of rounding noise per element; with both operands of both projections quantised and
    uncorrelated random data the block's relative error is 20-25 % (a gross error - a wrong scale, a
    misplaced row - gives 100 % or more)."""
    g = torch.Generator().manual_seed(5)
    tokens, experts, k, dim, inter = 32, 8, 2, 512, 256
    w1 = torch.randn(experts, inter, dim, generator=g) * 0.05
    w3 = torch.randn(experts, inter, dim, generator=g) * 0.05
    w2 = torch.randn(experts, dim, inter, generator=g) * 0.05
    weights = moe.RoutedExperts(w1, w3, w2, act_scale_in=5.0 / (448 * 6), act_scale_mid=24.0 / (448 * 6))
    runner = moe.MoERunner(weights, tokens, k)
    x = torch.randn(tokens, dim, generator=g).bfloat16()
    idx = torch.stack([torch.randperm(experts, generator=g)[:k] for _ in range(tokens)]).int()
    rw = torch.rand(tokens, k, generator=g) + 0.1
    y = runner.forward(x.cuda(), rw.cuda(), idx.cuda()).float().cpu()
    ref = torch.zeros(tokens, dim)
    for t in range(tokens):
        for j in range(k):
            e = int(idx[t, j])
            hgate, hup = w1[e] @ x[t].float(), w3[e] @ x[t].float()
            ref[t] += w2[e] @ (rw[t, j] * torch.nn.functional.silu(hgate) * hup)
    err = (y - ref).norm() / ref.norm()
    assert err < 0.30, float(err)


@pytest.mark.parametrize("name", ["plain", "limit"])
def test_block_against_the_origin_module(wuda, name):
    """The whole block (router, routed NVFP4 experts, FP8 shared expert, sum) on the weights and inputs of the
    fixture made with the origin's MoE module (Gate / Expert / MoE, origin/model.py:546-644, bf16 weights, CPU):
    the same experts must be selected with the same routing weights, and the output must stay within the
    quantisation noise of the origin's - e2m1 on both operands of both routed projections gives 10-15 % of
    relative error on uncorrelated data (a misplaced row, a missing routing weight or a dropped shared expert
    gives 50 % or more); tolerance 25 % of the output's norm, floating point."""
    from conftest import load_golden
    from wuda_b200 import workloads
    g = load_golden("moe_block_origin.npz")
    f32 = lambda key: torch.from_numpy(oracle.bf16_to_f32(g[key + "_" + name]))
    w1, w3, w2, x = f32("w1"), f32("w3"), f32("w2"), f32("x")
    experts, topk, limit = w1.size(0) - 1, int(g["topk"]), float(g["limit_" + name])
    tokens, dim = x.shape
    routed_w = moe.RoutedExperts(w1[:experts], w3[:experts], w2[:experts], act_scale_in=8.0 / 2688, act_scale_mid=32.0 / 2688,
                                 swiglu_limit=limit)
    runner = moe.MoERunner(routed_w, tokens, topk)
    t8 = lambda a: torch.from_numpy(a).cuda().view(torch.float8_e4m3fn)
    w13, w13s = workloads.quantize_fp8_128x128(torch.cat([w1[experts], w3[experts]]))
    w2q, w2s = workloads.quantize_fp8_128x128(w2[experts])
    shared = moe.SharedExpert(t8(w13), torch.from_numpy(w13s).cuda(), t8(w2q), torch.from_numpy(w2s).cuda(), swiglu_limit=limit)
    gate_w = torch.from_numpy(g["gate_w_" + name].view(np.int16)).view(torch.bfloat16).cuda()
    bias = torch.from_numpy(g["gate_bias_" + name]).cuda()
    xb = x.bfloat16().cuda()
    rw, idx = wuda.moe_gate(xb, gate_w, bias, "sqrtsoftplus", float(g["route_scale"]), topk)
    y = moe.moe_block(xb, gate_w, bias, runner, shared, "sqrtsoftplus", float(g["route_scale"]))
    torch.cuda.synchronize()
    assert int(runner.status.item()) == 0
    got_idx, want_idx = idx.cpu().numpy(), g["indices_" + name]
    assert np.array_equal(np.sort(got_idx, 1), np.sort(want_idx, 1))
    a, b = np.argsort(got_idx, 1), np.argsort(want_idx, 1)
    assert np.allclose(np.take_along_axis(rw.cpu().numpy(), a, 1), np.take_along_axis(g["weights_" + name], b, 1),
                       rtol=1e-4, atol=1e-6)
    want = oracle.bf16_to_f32(g["y_" + name])
    got = y.float().cpu().numpy()
    err = np.linalg.norm(got - want) / np.linalg.norm(want)
    assert err < 0.25, float(err)
    # and the oracle's restatement of the module (pinned by the same fixture) stands between the two
    oy, _, _ = oracle.moe_block(g["x_" + name], g["gate_w_" + name], g["gate_bias_" + name], g["w1_" + name], g["w3_" + name],
                                g["w2_" + name], topk, 2, float(g["route_scale"]), limit)
    assert np.linalg.norm(got - oracle.bf16_to_f32(oy)) / np.linalg.norm(want) < 0.25


def test_rejects_bad_arguments(wuda):
    from wuda_b200._lib import check
    with pytest.raises(wuda.WudaError, match="max_groups"):
        z = torch.zeros(64, dtype=torch.int32, device="cuda")
        check(wuda.lib.wuda_moe_dispatch(z.data_ptr(), z.data_ptr(), z.data_ptr(), z.data_ptr(), z.data_ptr(), z.data_ptr(),
                                         z.data_ptr(), 8, 2, 4, 1, None, None))
    assert wuda.lib.wuda_moe_max_groups(64, 8, 256) == 288 and wuda.lib.wuda_moe_max_groups(1, 2, 256) == 2


def test_shared_expert_and_block(wuda):
    """Dense shared expert: SwiGLU + FP8 quantisation against numpy on the GPU's own projection, and the
    whole block (router + routed + shared) against its parts."""
    from wuda_b200 import workloads
    from wuda_b200._lib import check
    g = torch.Generator().manual_seed(21)
    tokens, experts, k, dim, inter = 12, 8, 2, 512, 256
    h = (torch.randn(tokens, 2 * inter, generator=g) * 3).bfloat16()
    a8 = torch.empty(tokens, inter, dtype=torch.float8_e4m3fn, device="cuda")
    a_s = torch.empty(tokens, inter // 128, device="cuda")
    y16 = torch.empty(tokens, inter, dtype=torch.bfloat16, device="cuda")
    hc = h.cuda()
    check(wuda.lib.wuda_swiglu_quant_fp8(hc.data_ptr(), y16.data_ptr(), a8.data_ptr(), a_s.data_ptr(), tokens, inter, 5.0, 1, None))
    torch.cuda.synchronize()
    ref = oracle.moe_swiglu(u16(h), np.ones(tokens, np.float32), 5.0)
    got = u16(y16)
    assert np.mean(got == ref) >= 0.995 and np.abs(got.astype(np.int32) - ref.astype(np.int32)).max() <= 1
    q, s = oracle.act_quant_fp8(got, 128, round_scale=True)          # exact on the GPU's own bf16 values
    assert np.array_equal(a8.view(torch.uint8).cpu().numpy(), q) and np.array_equal(a_s.cpu().numpy(), s)

    mk = lambda n, kk: workloads.quantize_fp8_128x128(torch.randn(n, kk, generator=g) * 0.05)
    t8 = lambda a: torch.from_numpy(a).cuda().view(torch.float8_e4m3fn)
    w13, w13s = mk(2 * inter, dim)
    w2, w2s = mk(dim, inter)
    shared = moe.SharedExpert(t8(w13), torch.from_numpy(w13s).cuda(), t8(w2), torch.from_numpy(w2s).cuda())
    routed_w = moe.RoutedExperts(torch.randn(experts, inter, dim, generator=g) * 0.05, torch.randn(experts, inter, dim, generator=g) * 0.05,
                                 torch.randn(experts, dim, inter, generator=g) * 0.05, 5.0 / 2688, 24.0 / 2688)
    runner = moe.MoERunner(routed_w, tokens, k)
    x = torch.randn(tokens, dim, generator=g).bfloat16().cuda()
    gate_w = (torch.randn(experts, dim, generator=g) * 0.05).bfloat16().cuda()
    y = moe.moe_block(x, gate_w, None, runner, shared, "sigmoid", 1.5)
    rw, idx = wuda.moe_gate(x, gate_w, None, "sigmoid", 1.5, k)
    sh = shared.forward(x)
    y_parts = runner.forward(x, rw, idx, shared=sh)
    y_routed = runner.forward(x, rw, idx)
    torch.cuda.synchronize()
    assert torch.equal(y, y_parts)                                    # deterministic
    assert torch.allclose(y.float(), y_routed.float() + sh.float(), rtol=2 ** -7, atol=1e-2)
    # the shared expert against the FP8 oracle chain on its own activations
    x8, xs = oracle.act_quant_fp8(u16(x), 128, round_scale=True)
    hh = oracle.gemm_fp8_blockscaled(x8, xs, w13, w13s)
    act = oracle.moe_swiglu(hh, np.ones(tokens, np.float32), 0.0)
    q2, s2 = oracle.act_quant_fp8(act, 128, round_scale=True)
    ref_sh = oracle.bf16_to_f32(oracle.gemm_fp8_blockscaled(q2, s2, w2, w2s))
    got_sh = sh.float().cpu().numpy()
    assert np.all(np.abs(got_sh - ref_sh) <= 3e-2 * np.abs(ref_sh) + 1e-2 * np.abs(ref_sh).max())
