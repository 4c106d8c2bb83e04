"""The output projection of an attention half-layer and the mHC post mix behind it.

Mirrors run_o_proj_mhc_post, OProjWeights and quantize_o_proj_weights of the reference
(dsv4_megakernel/megakernel/test/o_proj_csa.py:319-494, :90-109, :498-555): inverse RoPE on the
last 64 dims of every 512-wide head of the attention output + 1x128 power-of-two FP8 quantisation,
the grouped low-rank projection wo_a ([groups, 1024, heads_per_group * 512]), a second
quantisation, the projection wo_b ([hidden, groups * 1024]) and mhc_post.  The reference runs the
two projections through a third-party GEMM library with packed UE8M0 scales; here they are this
library's block-scaled FP8 GEMMs (plain and grouped) with the same power-of-two scales held as fp32.
With a TP2Link the wo_b projection is the K-split form whose all-reduce is fused into the GEMM.
"""
from dataclasses import dataclass

import torch

from . import ops
from ._lib import check, lib

HEAD_DIM, ROPE_DIM, O_LORA_RANK = 512, 64, 1024


@dataclass
class OProjWeights:
    wo_a: torch.Tensor         # e4m3 [groups, n_per_group, heads_per_group * 512]
    wo_a_scale: torch.Tensor   # fp32 [groups * n_per_group / 128, heads_per_group * 4]
    wo_b: torch.Tensor         # e4m3 [hidden, groups * n_per_group]  (or this rank's K slice)
    wo_b_scale: torch.Tensor   # fp32 [ceil(hidden / 128), K / 128]
    scales_pow2: bool = False  # every scale is a power of two: wo_a runs on the GEMM that applies them in the tensor core


def _pow2_block_quant(w):
    """fp32 [N, K] -> (e4m3 [N, K], fp32 power-of-two scales [N/128, K/128]).  Setup only."""
    n, k = w.shape
    v = w.float().view(n // 128, 128, k // 128, 128)
    amax = v.abs().amax(dim=(1, 3)).clamp_min(1e-4)
    s = torch.exp2(torch.ceil(torch.log2(amax / 448.0)))
    q = (v / s[:, None, :, None]).clamp(-448, 448).reshape(n, k).to(torch.float8_e4m3fn)
    return q, s.contiguous()


def quantize_o_proj_weights(wo_a, wo_b):
    """bf16 wo_a [groups, n_per_group, K_a] and wo_b [hidden, groups * n_per_group] -> OProjWeights.
    Never call this in the decode hot region."""
    groups, npg, ka = wo_a.shape
    if npg % 128 or ka % 128 or wo_b.size(0) % 128 or wo_b.size(1) != groups * npg:
        raise ValueError("wo_a must be [groups, 128*i, 128*j] and wo_b [128*h, groups * n_per_group]")
    qa, sa = _pow2_block_quant(wo_a.reshape(groups * npg, ka))
    qb, sb = _pow2_block_quant(wo_b)
    return OProjWeights(qa.view(groups, npg, ka), sa, qb, sb, scales_pow2=True)


def fp8_gemm_grouped(a, a_s, w, w_s, *, out=None, status_word=None, pow2_scales=False):
    """c[m, g, :] = a[m, g, :] @ w[g]^T for every group g in one launch (wuda_gemm_fp8_grouped, or with
    pow2_scales=True - every scale a power of two - wuda_gemm_fp8_grouped_pow2).
    a e4m3 [M, groups * K] with fp32 scales [M, groups * K / 128]; w e4m3 [groups, N, K] with fp32
    scales [groups * N / 128, K / 128]; returns bf16 [M, groups * N]."""
    groups, n, k = w.shape
    m = a.size(0)
    if not (a.is_cuda and a.is_contiguous() and a.element_size() == 1 and a.numel() == m * groups * k):
        raise ValueError("a must be contiguous CUDA e4m3 [M, groups * K]")
    if not (w.is_cuda and w.is_contiguous() and w.element_size() == 1):
        raise ValueError("w must be contiguous CUDA e4m3 [groups, N, K]")
    if a_s.numel() != m * groups * (k // 128) or w_s.numel() != groups * (n // 128) * (k // 128):
        raise ValueError("scale shapes do not match the operands")
    if out is None:
        out = torch.empty(m, groups * n, dtype=torch.bfloat16, device=a.device)
    need = lib.wuda_gemm_fp8_scratch_bytes(m, groups * n)
    scratch = ops._scratch_for(a.device, need)
    entry = lib.wuda_gemm_fp8_grouped_pow2 if pow2_scales else lib.wuda_gemm_fp8_grouped
    check(entry(a.data_ptr(), a_s.data_ptr(), w.data_ptr(), w_s.data_ptr(), out.data_ptr(), m, n, k, groups, scratch.data_ptr(),
                scratch.numel(), status_word.data_ptr() if status_word is not None else None,
                torch.cuda.current_stream().cuda_stream))
    return out


def run_o_proj_mhc_post(mla_out, positions, cos_table, sin_table, residual, post, comb, weights, *, run_mhc_post=True,
                        tp_link=None, status_word=None):
    """mla_out bf16 [M, heads, 512] -> mhc output bf16 [M, 4, hidden] (or, with run_mhc_post=False,
    the projected bf16 [M, hidden]).  `tp_link` (ops.TP2Link) makes wo_b the K-split GEMM with the
    fused two-rank all-reduce; weights.wo_b is then this rank's [hidden, K/2] slice and mla_out this
    rank's heads."""
    if mla_out.dim() == 4:
        mla_out = mla_out[:, 0]
    m, heads, head_dim = mla_out.shape
    if head_dim != HEAD_DIM or not 1 <= m <= 128:
        raise ValueError("mla_out must be [M, heads, 512] with M in [1, 128]")
    groups = weights.wo_a.size(0)
    if heads % groups or weights.wo_a.size(2) != heads // groups * HEAD_DIM:
        raise ValueError("heads do not match wo_a's groups")
    _, o_fp8, o_scale = ops.rope_quant(mla_out, positions, cos_table, sin_table, ROPE_DIM, inverse=True, quant=True,
                                       scale_fmt="ue8m0")
    z = fp8_gemm_grouped(o_fp8, o_scale, weights.wo_a, weights.wo_a_scale, status_word=status_word,
                         pow2_scales=weights.scales_pow2)
    z_fp8, z_scale = ops.act_quant(z, 128, "ue8m0")
    if tp_link is None:
        projected = ops.fp8_gemm(z_fp8, z_scale, weights.wo_b, weights.wo_b_scale, status_word=status_word)
    else:
        projected = tp_link.fp8_gemm(z_fp8, z_scale, weights.wo_b, weights.wo_b_scale, status_word=status_word)
    if not run_mhc_post:
        return projected
    out = torch.empty_like(residual)
    return ops.mhc_post_out(projected, residual, post, comb, out)
