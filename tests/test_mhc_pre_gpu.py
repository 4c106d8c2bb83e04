"""GPU parity of mHC pre (through the C ABI) against the CPU oracle and the fixture made with the
reference's torch twin.  The 24 mixes are fp32 sums of 28672 products in different orders on the two
sides, so the gates agree to ~1e-6 and the bf16 / FP8 outputs are compared by match rate and step."""
import os
import sys

import numpy as np
import pytest
import torch

import oracle
from conftest import load_golden

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))
from make_golden import mhc_pre_inputs  # noqa: E402

pytestmark = pytest.mark.gpu


def u16(t):
    return t.cpu().view(torch.int16).numpy().view(np.uint16)


def bf16_near(got, ref, frac=0.999, steps=1):
    g, r = oracle.bf16_to_f32(got), oracle.bf16_to_f32(ref)
    assert np.mean(got == ref) >= frac, np.mean(got == ref)
    # `steps` bf16 steps, or the fp32 noise of a sum whose terms cancel (terms are O(1))
    bad = np.abs(g - r) > np.abs(r) * steps * 2.0 ** -7 + 2e-4
    assert not bad.any(), (g[bad][:4], r[bad][:4])


def test_golden(wuda):
    g = load_golden("mhc_pre_7168.npz")
    x, weight, base, scale = mhc_pre_inputs()
    out = wuda.mhc_pre(x.cuda(), torch.from_numpy(weight).cuda(), torch.from_numpy(base).cuda(),
                       torch.from_numpy(scale).cuda())
    torch.cuda.synchronize()
    for key in ("pre", "post", "comb"):
        assert np.abs(out[key].cpu().numpy() - g[key]).max() <= 5e-6, key
    bf16_near(u16(out["collapsed"]), g["collapsed"])


@pytest.mark.parametrize("m,hidden", [(1, 7168), (9, 7168), (64, 7168), (128, 7168), (5, 128), (3, 2048)])
def test_against_oracle(wuda, m, hidden):
    rng = np.random.default_rng(m * 7 + hidden)
    x = torch.from_numpy(rng.standard_normal((m, 4, hidden), dtype=np.float32)).bfloat16()
    weight = rng.standard_normal((24, 4 * hidden), dtype=np.float32) * np.float32(0.02)
    base = rng.standard_normal(24, dtype=np.float32) * np.float32(0.3)
    scale = np.array([0.9, 1.1, 2.0], np.float32)
    gamma = torch.from_numpy(1 + 0.1 * rng.standard_normal(hidden, dtype=np.float32)).bfloat16()
    out = wuda.mhc_pre(x.cuda(), torch.from_numpy(weight).cuda(), torch.from_numpy(base).cuda(),
                       torch.from_numpy(scale).cuda(), gamma.cuda())
    torch.cuda.synchronize()
    ref = oracle.mhc_pre(u16(x), weight, base, scale, u16(gamma))
    for key in ("pre", "post", "comb"):
        assert np.abs(out[key].cpu().numpy() - ref[key]).max() <= 5e-6, key
    bf16_near(u16(out["collapsed"]), ref["collapsed"])
    # a one-step difference of the collapsed value moves the normalised one by up to two steps
    bf16_near(u16(out["normed"]), ref["normed"], 0.995, steps=2)
    xq, xsf = out["xq"].view(torch.uint8).cpu().numpy(), out["xsf"].cpu().numpy()
    assert np.mean(xsf == ref["xsf"]) >= 0.99 and np.mean(xq == ref["xq"]) >= 0.99
    # self-consistency, exact: the FP8 copy is the power-of-two quantisation of the GPU's own normed row
    q2, s2 = oracle.act_quant_fp8(u16(out["normed"]), 128, round_scale=True)
    assert np.array_equal(xsf, s2) and np.array_equal(xq, q2)


def test_feeds_mhc_post(wuda):
    """pre/post/comb of the pre stage are what mhc_post consumes: with attention_out = 0 the post
    mix is comb^T applied to the residual streams."""
    rng = np.random.default_rng(3)
    m, hidden = 4, 7168
    x = torch.from_numpy(rng.standard_normal((m, 4, hidden), dtype=np.float32)).bfloat16().cuda()
    w = torch.from_numpy(rng.standard_normal((24, 4 * hidden), dtype=np.float32) * np.float32(0.01)).cuda()
    out = wuda.mhc_pre(x, w, torch.zeros(24, device="cuda"), torch.ones(3, device="cuda"))
    y = torch.empty_like(x)
    wuda.mhc_post_out(torch.zeros(m, hidden, dtype=torch.bfloat16, device="cuda"), x, out["post"], out["comb"], y)
    torch.cuda.synchronize()
    ref = torch.einsum("mij,mih->mjh", out["comb"], x.float())
    assert torch.allclose(y.float(), ref, rtol=2 ** -7, atol=1e-2)


def test_rejects_bad_arguments(wuda):
    x = torch.zeros(2, 4, 200, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(wuda.WudaError, match="hidden"):
        wuda.mhc_pre(x, torch.zeros(24, 800, device="cuda"), torch.zeros(24, device="cuda"), torch.ones(3, device="cuda"))
    x = torch.zeros(2, 4, 256, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(wuda.WudaError, match="weight"):
        wuda.mhc_pre(x, torch.zeros(24, 512, device="cuda"), torch.zeros(24, device="cuda"), torch.ones(3, device="cuda"))
