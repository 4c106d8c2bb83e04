"""The reference's fused entry points by their own names (wuda_b200.shims), called with the argument order and the
tensor layouts of the reference's decode_step (test/test_e2e_decode.py:441-575) and held against this library's own
entry points, which have their parity tests elsewhere: the shims add layout translation, not arithmetic."""
import numpy as np
import pytest
import torch

import oracle
from wuda_b200 import ops, shims

pytestmark = pytest.mark.gpu
HIDDEN = 7168


def tables(max_pos=4096):
    ang = torch.outer(torch.arange(max_pos, dtype=torch.float32), 1.0 / (10000.0 ** (torch.arange(32) / 32.0)))
    return torch.cos(ang).cuda().contiguous(), torch.sin(ang).cuda().contiguous()


def fp8_weight(g, n, k):
    b = torch.randint(0, 0x48, (n, k), generator=g, dtype=torch.uint8) | (torch.randint(0, 2, (n, k), generator=g, dtype=torch.uint8) << 7)
    sf = torch.randint(118, 123, ((n + 127) // 128, k // 128), generator=g, dtype=torch.uint8)       # UE8M0: 2^-9 .. 2^-5
    return b.cuda().view(torch.float8_e4m3fn), sf.cuda()


@pytest.mark.parametrize("m,heads", [(5, 128), (64, 64)])
def test_inv_rope_quant_layouts(wuda, m, heads):
    g = torch.Generator().manual_seed(m)
    x = torch.randn(m, heads, 512, generator=g).bfloat16().cuda()
    pos = torch.randint(0, 4096, (m,), generator=g).cuda()
    cos, sin = tables()
    groups, m4 = heads // 8, (m + 3) // 4 * 4
    out8 = torch.empty(groups, m, 4096, dtype=torch.float8_e4m3fn, device="cuda").permute(1, 0, 2)      # [M, groups, 4096]
    out_s = torch.empty(groups, 8, m4, dtype=torch.int32, device="cuda").permute(2, 0, 1)[:m]            # strides (1, 8*M4, M4)
    assert out_s.stride() == (1, 8 * m4, m4)
    shims.inv_rope_quant(x, pos, torch.cat([cos, sin], dim=1).contiguous(), out8, out_s)
    _, y8, sc = ops.rope_quant(x, pos, cos, sin, 64, inverse=True, quant=True, scale_fmt="ue8m0")
    torch.cuda.synchronize()
    assert torch.equal(out8.contiguous().view(torch.uint8).view(m, heads * 512), y8.view(torch.uint8))
    words = out_s.contiguous().view(m, heads)
    for j in range(4):
        assert torch.equal(shims.ue8m0_to_f32(((words >> (8 * j)) & 0xFF).to(torch.uint8)), sc.view(m, heads, 4)[..., j])
    # and the arithmetic itself: inverse rotation + power-of-two quantisation of the oracle
    rot = oracle.rope_bf16(x.cpu().view(torch.int16).numpy().view(np.uint16), pos.cpu().numpy(), cos.cpu().numpy(), sin.cpu().numpy(),
                           64, inverse=True)
    q, s = oracle.act_quant_fp8(rot.reshape(m, heads * 512), 128, round_scale=True)
    assert np.array_equal(s, sc.cpu().numpy()) and np.mean(q == y8.view(torch.uint8).cpu().numpy()) >= 0.999


def test_mhc_pair_and_front_projection_with_tail(wuda):
    g = torch.Generator().manual_seed(3)
    m, splits = 9, 16
    hidden_states = torch.randn(m, 4, HIDDEN, generator=g).bfloat16().cuda()
    w = (torch.randn(24, 4 * HIDDEN, generator=g) * 0.01).cuda()
    base, scale = (torch.randn(24, generator=g) * 0.1).cuda(), (torch.rand(3, generator=g) + 0.5).cuda()
    gamma = (torch.randn(HIDDEN, generator=g) * 0.1 + 1).bfloat16().cuda()
    want = ops.mhc_pre(hidden_states, w, base, scale, gamma)
    # the reference's pair: split-K mix projection, then the reduce-and-fuse epilogue exporting mix for the tail
    mul = torch.empty(splits, m, 24, device="cuda")
    sqr = torch.empty(splits, m, device="cuda")
    shims.tf32_hc_prenorm_gemm(hidden_states.view(m, -1), w, mul, sqr, splits)
    collapsed = torch.empty(m, HIDDEN, dtype=torch.bfloat16, device="cuda")
    pre, po, cb = torch.empty(m, 4, device="cuda"), torch.empty(m, 4, device="cuda"), torch.empty(m, 4, 4, device="cuda")
    mix = torch.empty(m, 24, device="cuda")
    x_fp8 = torch.empty(m, HIDDEN, dtype=torch.float8_e4m3fn, device="cuda")
    x_sf = torch.empty(m, HIDDEN // 128, dtype=torch.uint8, device="cuda")
    shims.hc_reduce_fuse_out(hidden_states, mul, sqr, base, scale, 1e-6, 1e-6, collapsed, pre, po, cb, with_post_comb=False,
                             attn_norm_w=gamma, attn_norm_eps=1e-6, mix_out=mix, xq_out=x_fp8.view(torch.uint8), xsf_out=x_sf)
    torch.cuda.synchronize()
    # the splits are added in another order than the 56 slices: the gates move in their last fp32 bits, a sum of four
    # products near zero then moves by a bf16 step of its largest term
    assert torch.allclose(pre, want["pre"], rtol=1e-5, atol=1e-6)
    assert torch.allclose(collapsed.float(), want["normed"].float(), rtol=2.0 ** -7, atol=2.0 ** -7)
    assert float((collapsed.view(torch.int16) == want["normed"].view(torch.int16)).float().mean()) >= 0.99
    assert float((x_fp8.view(torch.uint8) == want["xq"].view(torch.uint8)).float().mean()) >= 0.99
    assert float((shims.ue8m0_to_f32(x_sf) == want["xsf"]).float().mean()) >= 0.99
    # front projection with FRONT-EMIT and the tail, reference argument order
    w16 = (torch.randn(2624, HIDDEN, generator=g) * 0.02).bfloat16().cuda()
    w8, w8_sf = fp8_weight(g, 2048, HIDDEN)
    rows_total, pos = 40, torch.tensor([3, 4, 5, 6, 7, 8, 9, 10, 11]).cuda()
    state_row = torch.arange(m).cuda() * 3
    ape, idx_ape = torch.randn(4, 1024, generator=g).cuda(), torch.randn(4, 256, generator=g).cuda()

    def run(fn):
        main_state, idx_state = torch.zeros(rows_total, 2048, device="cuda"), torch.zeros(rows_total, 512, device="cuda")
        win_y2, w64 = torch.empty(m, 512, device="cuda"), torch.empty(m, 64, device="cuda")
        return fn(main_state, idx_state, win_y2, w64), main_state, idx_state, win_y2, w64

    hc_post, hc_comb = torch.empty(m, 4, device="cuda"), torch.empty(m, 16, device="cuda")
    got = run(lambda ms, st, wy, w6: shims.front_mixed_gemm_csa_swapab(
        collapsed, x_fp8, x_sf, w16, w8, w8_sf, hc_mix=mix, hc_base=base, hc_scale=scale, hc_post=hc_post, hc_comb=hc_comb,
        enable_tail=True, main_state=ms, main_ape=ape, main_state_row=state_row, ape_phase=(pos % 4).int(), idx_state=st,
        idx_state_row=state_row, idx_ape=idx_ape, win_y2=wy, w64=w6, pdl=True))
    y8 = torch.empty(m, 2048, dtype=torch.bfloat16, device="cuda")
    ref = run(lambda ms, st, wy, w6: ops.front_mixed_gemm(
        collapsed, x_fp8, shims.ue8m0_to_f32(x_sf).contiguous(), w16, w8, shims.ue8m0_to_f32(w8_sf).contiguous(), y8, pos=pos,
        main_state=ms, ape=ape, main_state_row=state_row, idx_state=st, idx_state_row=state_row, idx_ape=idx_ape, win_y2=wy,
        w64=w6))
    torch.cuda.synchronize()
    assert tuple(got[0].shape) == (m, 4672) and torch.equal(got[0][:, :2048], y8)
    for a, b in zip(got[1:], ref[1:]):
        assert torch.equal(a, b)
    # post / comb of the tail against the one-call form (same mixes, another summation order upstream)
    assert torch.allclose(hc_post, want["post"], rtol=1e-5, atol=1e-6)
    assert torch.allclose(hc_comb.view(m, 4, 4), want["comb"], rtol=1e-4, atol=1e-6)


def test_merged_q_projection_call_of_decode_step(wuda):
    g = torch.Generator().manual_seed(4)
    m, n_total = 7, 8192 + 128 * 512
    w8, w_sf = fp8_weight(g, n_total, 1536)
    q_norm = (torch.rand(1536, generator=g) + 0.5).cuda()
    y_front = torch.randn(m, 4672, generator=g).bfloat16().cuda()
    q_pos = torch.tensor([0, 5, 17, 100, 1000, 2047, 4095], dtype=torch.int32).cuda()
    pos = q_pos.long()
    cos, sin = tables()
    w64 = (torch.randn(m, 64, generator=g) / 8).cuda()
    win_y2 = torch.randn(m, 512, generator=g).cuda()
    idx_norm, win_norm = (torch.rand(128, generator=g) + 0.5).cuda(), (torch.rand(512, generator=g) + 0.5).cuda()
    idx_state = torch.randn(m, 8, 512, generator=g).cuda()
    state_row = (torch.arange(m) * 8 + pos.cpu() % 8).cuda()
    xq = torch.empty(m, 1536, dtype=torch.float8_e4m3fn, device="cuda")
    xq_sf = torch.empty(m, 12, dtype=torch.uint8, device="cuda")
    rets = shims.wq_b_proj_gemm_merged(
        xq, xq_sf, w8, w_sf, q_pos, cos, sin, head_ssq=None, enable_ssq=False, mock_post=False, cmp_pos=pos, idx_norm=idx_norm,
        cos_tab=cos, sin_tab=sin, idx_state=idx_state, idx_state_row=state_row, state_ring_entries=8, win_y2=win_y2,
        win_norm=win_norm, q_y=y_front[:, :1536], q_norm_w=q_norm, indexer_fp8=True, iq_weights=w64, pdl=True)
    yq, iq, iq_sf = rets[0], rets[1], rets[2]
    # by hand with the library's own entry points
    _, x8, xs = ops.rmsnorm_quant(y_front[:, :1536], q_norm, 1e-6, quant=True, scale_fmt="ue8m0", return_bf16=False)
    y_all = ops.fp8_gemm(x8, xs, w8, shims.ue8m0_to_f32(w_sf).contiguous())
    q8, wf = ops.idx_postprocess_fp8(y_all[:, :8192].unflatten(-1, (64, 128)), w64, q_pos, cos, sin)
    torch.cuda.synchronize()
    assert torch.equal(xq.view(torch.uint8), x8.view(torch.uint8)) and torch.equal(shims.ue8m0_to_f32(xq_sf), xs)
    assert tuple(yq.shape) == (m, 128 * 512) and torch.equal(yq, y_all[:, 8192:])
    assert yq.view(m, 1, 128, 512).shape == (m, 1, 128, 512)                      # the caller's in-place query view
    assert torch.equal(iq.view(torch.uint8), q8.view(torch.uint8)) and torch.equal(iq_sf, wf)
    win_q8, win_s8, win_rope = rets[3], rets[4], rets[5]
    oq, os_, orope = oracle.window_kv_fp8(win_y2.cpu().numpy(), pos.cpu().numpy(), win_norm.cpu().numpy(), cos.cpu().numpy(),
                                          sin.cpu().numpy())
    assert np.array_equal(win_q8.cpu().numpy(), oq) and np.array_equal(win_s8.cpu().numpy(), os_)
    assert np.array_equal(win_rope.cpu().view(torch.int16).numpy().view(np.uint16), orope)
    # the same call in the indexer's FP4 form: Hadamard + MXFP4 query, FP4 compressor records into a pool
    epb = 64
    pool = torch.full((2, epb * 68), 0xA5, dtype=torch.uint8, device="cuda")
    dst = torch.where((pos + 1) % 4 == 0, torch.arange(m, device="cuda") * 3, torch.full_like(pos, -1))
    rets4 = shims.wq_b_proj_gemm_merged(
        xq, xq_sf, w8, w_sf, q_pos, cos, sin, head_ssq=None, enable_ssq=False, mock_post=False, cmp_pos=pos, idx_norm=idx_norm,
        cos_tab=cos, sin_tab=sin, idx_state=idx_state, idx_state_row=state_row, state_ring_entries=8, idx_cache=pool,
        idx_dst=dst, idx_entries_per_block=epb, indexer_fp8=False, pdl=True)
    torch.cuda.synchronize()
    iq4, iq4_sf = rets4[1], rets4[2]
    assert iq4.dtype == torch.int8 and tuple(iq4.shape) == (m, 64, 64) and iq4_sf.dtype == torch.int32
    y_idx = y_all[:, :8192].cpu().view(torch.int16).numpy().view(np.uint16).reshape(m, 64, 128)
    oq4, osf = oracle.index_q_post_fp4(y_idx, q_pos.cpu().numpy(), cos.cpu().numpy(), sin.cpu().numpy())
    assert np.array_equal(iq4.view(torch.uint8).cpu().numpy(), oq4)
    assert np.array_equal(iq4_sf.cpu().numpy().view(np.uint32), osf)
    want = np.full((2, epb * 68), 0xA5, np.uint8)
    oracle.indexer_compressor_fp4(idx_state.cpu().numpy(), state_row.cpu().numpy(), pos.cpu().numpy(), idx_norm.cpu().numpy(),
                                  cos.cpu().numpy(), sin.cpu().numpy(), pool=want, dst=dst.cpu().numpy(), epb=epb)
    got_pool = pool.cpu().numpy()
    assert (want != 0xA5).any() and np.mean(got_pool == want) >= 0.999
