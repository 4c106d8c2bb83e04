"""GPU parity of the grouped FP8 GEMM and of the output-projection chain (inverse RoPE + quant ->
grouped wo_a -> quant -> wo_b -> mhc_post) against the CPU oracle applied stage by stage to the
GPU's own intermediate results."""
import numpy as np
import pytest
import torch

import oracle
from wuda_b200 import o_proj, workloads

pytestmark = pytest.mark.gpu


def u16(t):
    return t.cpu().view(torch.int16).numpy().view(np.uint16)


def close(got_bf16, ref_bf16):
    g, r = oracle.bf16_to_f32(got_bf16), oracle.bf16_to_f32(ref_bf16)
    assert np.all(np.abs(g - r) <= 1e-2 * np.abs(r) + 1e-3 * np.abs(r).max())


@pytest.mark.parametrize("m,groups,n,k", [(1, 2, 128, 128), (5, 3, 256, 512), (64, 8, 1024, 4096), (128, 2, 384, 1024)])
def test_grouped_gemm_equals_per_group_oracle(wuda, m, groups, n, k):
    g = torch.Generator().manual_seed(m + groups * 7 + n)
    a = torch.randn(m, groups * k, generator=g)
    a8, a_s = workloads.quantize_fp8_1x128(a)
    w = torch.randn(groups * n, k, generator=g) * 0.03
    w8, w_s = workloads.quantize_fp8_128x128(w)
    status = wuda.device_status_word()
    out = o_proj.fp8_gemm_grouped(torch.from_numpy(a8).cuda().view(torch.float8_e4m3fn), torch.from_numpy(a_s).cuda(),
                                  torch.from_numpy(w8).cuda().view(torch.float8_e4m3fn).view(groups, n, k),
                                  torch.from_numpy(w_s).cuda(), status_word=status)
    torch.cuda.synchronize()
    assert status.item() == 0
    got = u16(out)
    kb, nb = k // 128, n // 128
    for j in range(groups):
        ref = oracle.gemm_fp8_blockscaled(a8[:, j * k:(j + 1) * k], a_s[:, j * kb:(j + 1) * kb],
                                          w8[j * n:(j + 1) * n], w_s[j * nb:(j + 1) * nb])
        close(got[:, j * n:(j + 1) * n], ref)


def test_o_proj_chain_stagewise(wuda):
    g = torch.Generator().manual_seed(99)
    m, heads, groups, npg, hidden = 6, 8, 2, 256, 512
    mla = torch.randn(m, heads, 512, generator=g).bfloat16()
    pos = torch.tensor([0, 5, 77, 1000, 4095, 31])
    ang = torch.outer(torch.arange(4096, dtype=torch.float32), 1.0 / (10000.0 ** (torch.arange(32) / 32.0)))
    cos, sin = torch.cos(ang).contiguous(), torch.sin(ang).contiguous()
    wo_a = (torch.randn(groups, npg, heads // groups * 512, generator=g) * 0.03).bfloat16()
    wo_b = (torch.randn(hidden, groups * npg, generator=g) * 0.05).bfloat16()
    weights = o_proj.quantize_o_proj_weights(wo_a.cuda(), wo_b.cuda())
    assert torch.all(torch.log2(weights.wo_a_scale) == torch.round(torch.log2(weights.wo_a_scale)))
    residual = torch.randn(m, 4, hidden, generator=g).bfloat16().cuda()
    post = torch.rand(m, 4, generator=g).cuda()
    comb = torch.softmax(torch.randn(m, 4, 4, generator=g), -1).cuda()
    status = wuda.device_status_word()
    out = o_proj.run_o_proj_mhc_post(mla.cuda(), pos.cuda(), cos.cuda(), sin.cuda(), residual, post, comb, weights,
                                     status_word=status)
    projected = o_proj.run_o_proj_mhc_post(mla.cuda(), pos.cuda(), cos.cuda(), sin.cuda(), residual, post, comb, weights,
                                           run_mhc_post=False, status_word=status)
    torch.cuda.synchronize()
    assert status.item() == 0
    # the oracle's chain end to end (every stage's tolerance is already checked elsewhere): within the
    # FP8 GEMM tolerance of the final projection
    rot = oracle.rope_bf16(u16(mla), pos.numpy(), cos.numpy(), sin.numpy(), 64, inverse=True)
    o8, o_s = oracle.act_quant_fp8(rot.reshape(m, -1), 128, round_scale=True)
    wa8 = weights.wo_a.view(torch.uint8).cpu().numpy().reshape(groups * npg, -1)
    wa_s = weights.wo_a_scale.cpu().numpy()
    ka, kb = wa8.shape[1], wa8.shape[1] // 128
    z = np.concatenate([oracle.gemm_fp8_blockscaled(o8[:, j * ka:(j + 1) * ka], o_s[:, j * kb:(j + 1) * kb],
                                                    wa8[j * npg:(j + 1) * npg], wa_s[j * (npg // 128):(j + 1) * (npg // 128)])
                        for j in range(groups)], axis=1)
    z8, z_s = oracle.act_quant_fp8(z, 128, round_scale=True)
    ref_proj = oracle.gemm_fp8_blockscaled(z8, z_s, weights.wo_b.view(torch.uint8).cpu().numpy(),
                                           weights.wo_b_scale.cpu().numpy())
    g_p, r_p = oracle.bf16_to_f32(u16(projected)), oracle.bf16_to_f32(ref_proj)
    assert np.all(np.abs(g_p - r_p) <= 2e-2 * np.abs(r_p) + 5e-3 * np.abs(r_p).max())
    # mhc_post on the GPU's own projection: exact
    ref_out = oracle.mhc_post(u16(projected), u16(residual), post.cpu().numpy(), comb.cpu().numpy())
    assert np.array_equal(u16(out), ref_out)
