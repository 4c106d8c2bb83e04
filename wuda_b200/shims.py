"""The reference's fused entry points by their own names and argument lists, over this library's entry points,
so that a caller written against the reference's decode_step (dsv4_megakernel/megakernel/test/
test_e2e_decode.py:441-800) can be pointed at this package without rewriting its call sites:

    inv_rope_quant               kernels/mla_o_inv_rope_quant.cu:287-290
    tf32_hc_prenorm_gemm         the third-party split-K mix GEMM as called at test/test_e2e_decode.py:466
    hc_reduce_fuse_out           kernels/hc_fused_kernel_tc.cu:524-540
    front_mixed_gemm_csa_swapab  kernels/front_mixed_gemm_csa_swapab.cu:262-279
    wq_b_proj_gemm_merged        kernels/wq_b_fp8_gemm.cu:1375-1460

The reference fuses each of these into one kernel; here a call is the sequence of this library's launches that
produces the same outputs in the same layouts (the fusion state of each is described with its entry point).
Scale tensors arrive in the reference's packed forms - UE8M0 bytes, or int32 words of four such bytes in the
"MN-major" order its GEMM library wants - and are translated to and from the fp32 power-of-two scales this
library's GEMMs take by a few torch element-wise kernels; that translation is the price of the drop-in form and
is not on the path of wuda_layer_decode.
"""
import torch

from . import ops
from ._lib import check, lib

__all__ = ["inv_rope_quant", "tf32_hc_prenorm_gemm", "hc_reduce_fuse_out", "front_mixed_gemm_csa_swapab",
           "wq_b_proj_gemm_merged", "ue8m0_to_f32", "f32_to_ue8m0"]

N_INDEX, Q_LORA = 8192, 1536


def ue8m0_to_f32(sf):
    """UE8M0 exponent bytes (uint8 or float8_e8m0fnu) -> the fp32 powers of two they stand for."""
    b = sf.view(torch.uint8) if sf.dtype != torch.uint8 else sf
    return (b.to(torch.int32) << 23).view(torch.float32)


def f32_to_ue8m0(scale):
    """fp32 powers of two -> UE8M0 exponent bytes."""
    return ((scale.contiguous().view(torch.int32) >> 23) & 0xFF).to(torch.uint8)


_weight_scales = {}


def _cached_weight_scales(w_sf):
    """fp32 copy of a weight's UE8M0 scale bytes, converted once per tensor (weights do not change)."""
    key = (w_sf.data_ptr(), tuple(w_sf.shape))
    hit = _weight_scales.get(key)
    if hit is None:
        hit = _weight_scales[key] = ue8m0_to_f32(w_sf).contiguous()
    return hit


def inv_rope_quant(input, positions, cos_sin, output_fp8, output_scale):
    """Inverse RoPE on the last 64 dims of every 512-wide head of the attention output + per-128 power-of-two
    FP8 quantisation, written in the reference's grouped layouts: output_fp8 e4m3 [M, groups, 8 * 512] (a view of
    a [groups, M, 4096] buffer), output_scale int32 [M, groups, 8] with strides (1, 8 * M4, M4), M4 = M rounded up
    to 4: one word of four UE8M0 bytes per head.  cos_sin fp32 [max_pos, 64] = 32 cosines then 32 sines."""
    ops._require(input.is_cuda and input.is_contiguous() and input.dtype == torch.bfloat16 and input.dim() == 3
                 and input.size(2) == 512 and input.size(1) in (64, 128) and 1 <= input.size(0) <= 128,
                 "input must be contiguous CUDA BF16 [M,H,512] with M in [1,128] and H in {64,128}")
    m, heads, _ = input.shape
    groups = heads // 8
    ops._require(cos_sin.is_cuda and cos_sin.is_contiguous() and cos_sin.dtype == torch.float32 and cos_sin.dim() == 2
                 and cos_sin.size(1) == 64, "cos_sin must be contiguous CUDA FP32 [max_pos,64]")
    ops._require(tuple(output_fp8.shape) == (m, groups, 4096) and output_fp8.element_size() == 1 and output_fp8.stride(2) == 1,
                 "output_fp8 has the wrong grouped layout")
    ops._require(tuple(output_scale.shape) == (m, groups, 8) and output_scale.dtype == torch.int32,
                 "output_scale has the wrong MN-major layout")
    cos, sin = cos_sin[:, :32].contiguous(), cos_sin[:, 32:].contiguous()
    _, y8, sc = ops.rope_quant(input, positions, cos, sin, 64, inverse=True, quant=True, scale_fmt="ue8m0")
    output_fp8.view(torch.uint8).copy_(y8.view(torch.uint8).view(m, groups, 4096))
    words = f32_to_ue8m0(sc).view(m, heads, 4).contiguous().view(torch.int32).view(m, groups, 8)
    output_scale.copy_(words)
    return output_fp8, output_scale


def tf32_hc_prenorm_gemm(x, w, out_mul, out_sqrsum, num_splits=None):
    """The split-K mix projection in front of hc_reduce_fuse_out: x bf16 [M, 4*hidden] (or [M, 4, hidden]), w fp32
    [24, 4*hidden] -> out_mul fp32 [S, M, 24] partial dot products and out_sqrsum fp32 [S, M] partial sums of
    squares.  fp32 products on CUDA cores (the third-party kernel rounds its operands to TF32); this library's 56
    K-slices are folded into the S splits the caller's tensors have (slice s goes to split s % S)."""
    m = out_mul.size(1)
    hidden = x.numel() // (4 * m)
    splits = out_mul.size(0)
    need = lib.wuda_mhc_pre_workspace_bytes(m, hidden)
    ws = torch.empty(need // 4, dtype=torch.float32, device=x.device)
    check(lib.wuda_mhc_pre_mix(x.data_ptr(), w.data_ptr(), ws.data_ptr(), need, m, hidden, ops._stream()))
    part = ws.view(-1, m, 25)
    slices = part.size(0)
    if splits == slices:
        folded = part
    else:
        pad = (-slices) % splits
        if pad:
            part = torch.cat([part, part.new_zeros(pad, m, 25)])
        folded = part.view(-1, splits, m, 25).sum(0)
    out_mul.copy_(folded[..., :24])
    out_sqrsum.copy_(folded[..., 24])
    return out_mul, out_sqrsum


def hc_reduce_fuse_out(hidden_states, workspace, sqr_sum, attn_hc_base, attn_hc_scale, hc_eps, rms_norm_eps, collapsed, pre,
                       post, comb, with_post_comb=False, attn_norm_w=None, attn_norm_eps=1e-6, pdl=True, mix_out=None,
                       xq_out=None, xsf_out=None):
    """Everything of mHC pre behind the mix projection, on an EXTERNAL split-K workspace (workspace fp32 [S, M, 24],
    sqr_sum fp32 [S, M]): pre (and, with with_post_comb, post and comb), the collapsed stream - which becomes the
    attention RMSNorm's output when attn_norm_w is given, as in the reference - its FP8 form xq_out uint8 [M, hidden]
    with UE8M0 bytes xsf_out uint8 [M, hidden / 128], and mix_out fp32 [M, 24] for the front projection's tail."""
    m = workspace.size(1)
    hidden = hidden_states.numel() // (4 * m)
    partials = torch.cat([workspace, sqr_sum.view(-1, m, 1)], dim=2).contiguous()
    normed = collapsed if attn_norm_w is not None else None
    scales = torch.empty(m, hidden // 128, dtype=torch.float32, device=workspace.device) if xq_out is not None else None
    check(lib.wuda_mhc_pre_finish(hidden_states.data_ptr(), partials.data_ptr(), partials.size(0), attn_hc_base.data_ptr(),
                                  attn_hc_scale.data_ptr(), ops._ptr(attn_norm_w), float(hc_eps), float(rms_norm_eps),
                                  float(attn_norm_eps), pre.data_ptr(), post.data_ptr() if with_post_comb else None,
                                  comb.data_ptr() if with_post_comb else None, ops._ptr(mix_out),
                                  None if normed is not None else collapsed.data_ptr(), ops._ptr(normed), ops._ptr(xq_out),
                                  ops._ptr(scales), m, hidden, ops._stream()))
    if xsf_out is not None and scales is not None:
        xsf_out.view(torch.uint8).copy_(f32_to_ue8m0(scales))
    return collapsed


def front_mixed_gemm_csa_swapab(x, x_fp8, x_sf, w_bf16, w_fp8, w_sf, out=None, batch_n_override=0, task_times=None, hc_mix=None,
                                hc_base=None, hc_scale=None, hc_post=None, hc_comb=None, enable_tail=False, hc_eps=1e-6,
                                main_state=None, main_ape=None, main_state_row=None, ape_phase=None, idx_state=None,
                                idx_state_row=None, idx_ape=None, win_y2=None, w64=None, pdl=False):
    """The front projection y[M, 4672] = x . [W8 (2048 rows, FP8 with UE8M0 1x128 / 128x128 scales) | W16 (2624 rows,
    BF16)]^T with the FRONT-EMIT scatter of the BF16 segment into the state rings, win_y2 and w64, and - with
    enable_tail - post and comb computed from hc_mix behind it.  Returns the bf16 [M, 4672] output; with the scatter
    only its first 2048 columns are written (the reference leaves the others unwritten too).  ape_phase int [M] is
    position % 4.  Four launches (FP8 GEMM, BF16 GEMM, scatter, tail) where the reference has one."""
    m = x.size(0)
    if out is None:
        out = torch.empty(m, 4672, dtype=torch.bfloat16, device=x.device)
    xs = ue8m0_to_f32(x_sf).contiguous()
    ws = _cached_weight_scales(w_sf)
    y8 = torch.empty(m, 2048, dtype=torch.bfloat16, device=x.device)
    emit = main_state is not None or idx_state is not None
    pos = ape_phase.to(torch.int64) if ape_phase is not None else None
    _, y16 = ops.front_mixed_gemm(x, x_fp8.view(torch.float8_e4m3fn), xs, w_bf16, w_fp8.view(torch.float8_e4m3fn), ws, y8,
                                  pos=pos if emit else None, main_state=main_state, ape=main_ape, main_state_row=main_state_row,
                                  idx_state=idx_state, idx_state_row=idx_state_row, idx_ape=idx_ape, win_y2=win_y2, w64=w64)
    out[:, :2048].copy_(y8)
    if not emit:
        out[:, 2048:].copy_(y16)
    if enable_tail:
        check(lib.wuda_mhc_tail(hc_mix.data_ptr(), hc_base.data_ptr(), hc_scale.data_ptr(), float(hc_eps), hc_post.data_ptr(),
                                hc_comb.data_ptr(), m, ops._stream()))
    return out


def wq_b_proj_gemm_merged(x_fp8, x_sf, w_fp8, w_sf, q_pos, rope_cos, rope_sin, head_ssq=None, mock_post=True, enable_ssq=True,
                          cmp_pos=None, idx_norm=None, cos_tab=None, sin_tab=None, idx_state=None, idx_state_row=None,
                          state_ring_entries=0, win_y2=None, win_norm=None, q_y=None, q_norm_w=None, q_eps=1e-6, idx_cache=None,
                          idx_dst=None, idx_entries_per_block=64, idx_block_stride_bytes=0, swa_cache=None, swa_dst=None,
                          swa_entries_per_block=256, swa_block_stride_bytes=0, iq_dst=None, iq_dst_sf=None, indexer_fp8=True,
                          iq_weights=None, iq_head_base=0, iq_prof=None, pdl=True):
    """The merged q projection (weight [8192 + n_main, 1536]: indexer rows first) with what the reference fuses onto it:
    the q RMSNorm + quantisation producer (q_y bf16 [M, 1536] strided, q_norm_w fp32 -> fills x_fp8 / x_sf), the FP8
    indexer-q post (indexer_fp8=True: e4m3 [M, 64, 128] and iq_weights times the row scale), the indexer compressor
    and the window-KV writer into their pools.  Returns [y bf16 [M, n_main] (a column view of the projection output),
    iq, iq_weights_folded] (+ [win_q8, win_s8, win_rope] when the window writer ran without a pool).  With
    indexer_fp8=False the indexer takes its FP4 form: the indexer-q post runs the Hadamard transform and emits packed
    e2m1 codes int8 [M, 64, 64] with their scale words int32 [M, 64] (returned in the place of iq and the folded
    weights; iq_weights is not used), and the compressor writes 68-byte MXFP4 records.  head_ssq / enable_ssq /
    mock_post are accepted and ignored.  Up to five launches where the reference has one."""
    m = x_fp8.size(0)
    dev = x_fp8.device
    if q_y is not None:      # producer: RMSNorm(q_norm_w) + power-of-two quantisation into the caller's x_fp8 / x_sf
        xs = torch.empty(m, Q_LORA // 128, dtype=torch.float32, device=dev)
        check(lib.wuda_rmsnorm_quant_fp8(q_y.data_ptr(), q_y.stride(0), q_norm_w.data_ptr(), 0, float(q_eps), None,
                                         x_fp8.data_ptr(), xs.data_ptr(), m, Q_LORA, 1, ops._stream()))
        x_sf.view(torch.uint8).copy_(f32_to_ue8m0(xs))
    else:
        xs = ue8m0_to_f32(x_sf).contiguous()
    ws = _cached_weight_scales(w_sf)
    y_all = ops.fp8_gemm(x_fp8.view(torch.float8_e4m3fn), xs, w_fp8.view(torch.float8_e4m3fn), ws)
    n_total = y_all.size(1)
    if indexer_fp8:
        iq, wf = ops.idx_postprocess_fp8(y_all[:, :N_INDEX].unflatten(-1, (64, 128)), iq_weights, q_pos, rope_cos, rope_sin,
                                         q_fp8=iq_dst, weights_out=iq_dst_sf)
    else:
        iq, wf = ops.idx_postprocess(y_all[:, :N_INDEX].unflatten(-1, (64, 128)), q_pos, rope_cos, rope_sin, iq_fp4=iq_dst,
                                     iq_sf=iq_dst_sf)
    rets = [y_all[:, N_INDEX:], iq, wf]
    indexer = window = None
    if idx_state is not None:
        indexer = dict(state=idx_state, state_row=idx_state_row, norm_w=idx_norm, ring_entries=state_ring_entries)
        if idx_cache is not None:
            indexer.update(pool=idx_cache, dst=idx_dst, entries_per_block=idx_entries_per_block)
    if win_y2 is not None:
        window = dict(y=win_y2, norm_w=win_norm)
        if swa_cache is not None:
            window.update(pool=swa_cache, dst=swa_dst, entries_per_block=swa_entries_per_block)
        else:
            window.update(q8=torch.empty(m, 448, dtype=torch.uint8, device=dev), s8=torch.empty(m, 7, device=dev),
                          rope=torch.empty(m, 64, dtype=torch.bfloat16, device=dev))
            rets += [window["q8"], window["s8"], window["rope"]]
    if indexer is not None or window is not None:
        ops.cache_writers_fp8(cmp_pos, cos_tab, sin_tab, indexer=indexer, window=window, indexer_fp4=not indexer_fp8)
    del n_total
    return rets
