"""GPU parity of the mHC post mix (through the C ABI): bit-exact against the CPU oracle, which
follows the reference kernel's operation order, and within one bf16 step of the fixture made
with the reference's torch twin."""
import numpy as np
import pytest
import torch

import oracle
from conftest import load_golden

pytestmark = pytest.mark.gpu


def u16(t):
    return t.cpu().view(torch.int16).numpy().view(np.uint16)


def from_u16(a):
    return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16).cuda()


def run(wuda, x, res, post, comb):
    out = torch.empty_like(res)
    assert wuda.mhc_post_out(x, res, post, comb, out) is out
    torch.cuda.synchronize()
    return out


def test_golden(wuda):
    g = load_golden("mhc_post_7168.npz")
    out = run(wuda, from_u16(g["x"]), from_u16(g["residual"]), torch.from_numpy(g["post"]).cuda(),
              torch.from_numpy(g["comb"]).cuda())
    d = np.abs(u16(out).astype(np.int32) - g["out"].astype(np.int32))
    assert d.max() <= 1 and (d == 0).mean() >= 0.99
    assert np.array_equal(u16(out), oracle.mhc_post(g["x"], g["residual"], g["post"], g["comb"]))


@pytest.mark.parametrize("m,hidden", [(1, 7168), (7, 7168), (64, 7168), (128, 7168), (5, 8), (3, 1000)])
def test_bit_exact_against_oracle(wuda, m, hidden):
    g = torch.Generator().manual_seed(m * 100003 + hidden)
    x = (torch.randn(m, hidden, generator=g) * 3).bfloat16()
    res = torch.randn(m, 4, hidden, generator=g).bfloat16()
    post = torch.randn(m, 4, generator=g)
    comb = torch.randn(m, 4, 4, generator=g)
    comb[0, 1, 2] = 0.0
    post[0, 3] = 0.0
    x[0, :8] = torch.tensor([0.0, -0.0, 3.3895e38, -3.3895e38, 1e-38, 1.0, -1.0, 65504.0]).bfloat16()
    from wuda_b200._lib import check
    lib = wuda.lib
    out = torch.empty_like(res).cuda()
    xc, rc, pc, cc = x.cuda(), res.cuda(), post.cuda(), comb.cuda()
    check(lib.wuda_mhc_post(xc.data_ptr(), rc.data_ptr(), pc.data_ptr(), cc.data_ptr(), out.data_ptr(), m, hidden,
                                 None))
    torch.cuda.synchronize()
    ref = oracle.mhc_post(u16(x), u16(res), post.numpy(), comb.numpy())
    got = u16(out)
    same = (got == ref) | (np.isnan(oracle.bf16_to_f32(got)) & np.isnan(oracle.bf16_to_f32(ref)))
    assert same.all()


def test_identity_mix_returns_the_residual(wuda):
    m = 4
    res = torch.randn(m, 4, 7168).bfloat16().cuda()
    x = torch.randn(m, 7168).bfloat16().cuda()
    out = run(wuda, x, res, torch.zeros(m, 4, device="cuda"), torch.eye(4, device="cuda").expand(m, 4, 4).contiguous())
    assert torch.equal(out, res)
    out = run(wuda, x, res, torch.ones(m, 4, device="cuda"), torch.zeros(m, 4, 4, device="cuda"))
    assert torch.equal(out, x[:, None, :].expand(m, 4, 7168))


def test_rejects_bad_arguments(wuda):
    from wuda_b200._lib import check
    x = torch.zeros(2, 7168, dtype=torch.bfloat16, device="cuda")
    res = torch.zeros(2, 4, 7168, dtype=torch.bfloat16, device="cuda")
    post, comb = torch.zeros(2, 4, device="cuda"), torch.zeros(2, 4, 4, device="cuda")
    with pytest.raises(wuda.WudaError, match="overlap"):
        wuda.mhc_post_out(x, res, post, comb, res)                      # in place
    with pytest.raises(wuda.WudaError, match="hidden"):
        check(wuda.lib.wuda_mhc_post(x.data_ptr(), res.data_ptr(), post.data_ptr(), comb.data_ptr(),
                                          torch.empty_like(res).data_ptr(), 2, 7164, None))
    with pytest.raises(wuda.WudaError, match="m must be"):
        check(wuda.lib.wuda_mhc_post(x.data_ptr(), res.data_ptr(), post.data_ptr(), comb.data_ptr(),
                                          torch.empty_like(res).data_ptr(), 0, 7168, None))
    with pytest.raises(wuda.WudaError, match="comb"):
        wuda.mhc_post_out(x, res, post, comb.double(), torch.empty_like(res))
    big = torch.zeros(129, 7168, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(wuda.WudaError, match="128"):
        wuda.mhc_post_out(big, big[:, None].expand(129, 4, 7168).contiguous(), torch.zeros(129, 4, device="cuda"),
                          torch.zeros(129, 4, 4, device="cuda"), torch.empty(129, 4, 7168, dtype=torch.bfloat16,
                                                                             device="cuda"))
