"""GPU parity of the fused RMSNorm / RoPE / FP8-quantisation kernels (through the C ABI)
against the CPU oracle and the golden fixtures made with the origin model's functions."""
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


def bf16_close(got, ref, min_equal=0.999):
    """bf16 outputs: >= 99.9 % identical bytes and never more than one bf16 step apart
    (the only difference allowed is the summation order of the row's mean square)."""
    assert got.shape == ref.shape
    d = np.abs(got.astype(np.int32) - ref.astype(np.int32))
    assert d.max() <= 1, "bf16 values differ by %d steps" % d.max()
    assert (d == 0).mean() >= min_equal, "only %.4f of the values are identical" % (d == 0).mean()


def quant_close(q, s, ref_q, ref_s, x_ref_bf16):
    """FP8 outputs given bf16 inputs that may differ from the oracle's by one step in rare
    places: scales identical except for groups holding such an element, payload >= 99.9 %."""
    assert np.mean(s == ref_s) >= 0.999
    assert np.allclose(s, ref_s, rtol=2 ** -7)
    assert np.mean(q == ref_q) >= 0.999
    deq = oracle.e4m3_decode(q).reshape(s.shape + (128,)) * s[..., None]
    x = oracle.bf16_to_f32(x_ref_bf16).reshape(s.shape + (128,))
    assert np.all(np.abs(deq - x) <= s[..., None] * 16 * 1.01 + np.abs(x) * 2 ** -7)


def test_rmsnorm_golden(wuda):
    g = load_golden("rmsnorm_7168.npz")
    y16, _, _ = wuda.rmsnorm_quant(from_u16(g["x"]), from_u16(g["gamma"]), float(g["eps"]), quant=False)
    torch.cuda.synchronize()
    bf16_close(u16(y16), g["y"])


def test_rope_golden_forward_and_inverse(wuda):
    g = load_golden("rope_192.npz")
    rows = {int(p): i for i, p in enumerate(g["table_rows"])}
    pos = torch.tensor([rows[int(p)] for p in g["positions"]], dtype=torch.int64, device="cuda")
    cos, sin = torch.from_numpy(g["cos"]).cuda(), torch.from_numpy(g["sin"]).cuda()
    for inverse, key in ((False, "y"), (True, "y_inverse")):
        y16, _, _ = wuda.rope_quant(from_u16(g["x"]), pos, cos, sin, int(g["rope_dim"]), inverse=inverse,
                                    quant=False, return_bf16=True)
        torch.cuda.synchronize()
        assert np.array_equal(u16(y16), g[key])     # same fp32 operations: bit-exact


@pytest.mark.parametrize("scale_fmt", [None, "ue8m0"])
def test_act_quant_golden_and_oracle(wuda, scale_fmt):
    g = load_golden("act_quant_pow2_7168.npz")
    y8, sc = wuda.act_quant(from_u16(g["x"]), 128, scale_fmt)
    torch.cuda.synchronize()
    q, s = y8.cpu().view(torch.uint8).numpy(), sc.cpu().numpy()
    ref_q, ref_s = oracle.act_quant_fp8(g["x"], 128, round_scale=scale_fmt is not None)
    assert np.array_equal(s, ref_s) and np.array_equal(q, ref_q)      # same input bytes: bit-exact
    if scale_fmt is not None:
        assert np.array_equal(s, g["scale"]) and np.array_equal(q, g["q"])


def make_config3(tokens, seed):
    gen = torch.Generator().manual_seed(seed)
    x = torch.randn(tokens, 7168, generator=gen).bfloat16()
    gamma = (1 + 0.1 * torch.randn(7168, generator=gen)).bfloat16()
    proj = torch.randn(tokens, 128, 192, generator=gen).bfloat16()      # stands for the projection's output
    pos = torch.randint(0, 65536, (tokens,), generator=gen)
    freqs = 1.0 / (10000 ** (torch.arange(0, 64, 2, dtype=torch.float32) / 64))
    ang = torch.outer(torch.arange(65536).float(), freqs)
    return x, gamma, proj, pos, ang.cos().contiguous(), ang.sin().contiguous()


@pytest.mark.parametrize("tokens", [1, 64, 256])
@pytest.mark.parametrize("scale_fmt", [None, "ue8m0"])
def test_config3_rmsnorm_quant_stage(wuda, tokens, scale_fmt):
    """tokens x 7168 bf16 ~ N(0,1), bf16 gamma ~ N(1, 0.1), eps 1e-6 -> bf16 + e4m3 with 1x128 scales."""
    x, gamma, *_ = make_config3(tokens, 100 + tokens)
    y16, y8, sc = wuda.rmsnorm_quant(x.cuda(), gamma.cuda(), 1e-6, quant=True, scale_fmt=scale_fmt)
    torch.cuda.synchronize()
    ref16 = oracle.rmsnorm_bf16(u16(x), u16(gamma), 1e-6)
    bf16_close(u16(y16), ref16)
    # the FP8 output must be the quantisation of the kernel's OWN bf16 output, bit for bit
    own_q, own_s = oracle.act_quant_fp8(u16(y16), 128, round_scale=scale_fmt is not None)
    assert np.array_equal(sc.cpu().numpy(), own_s)
    assert np.array_equal(y8.cpu().view(torch.uint8).numpy(), own_q)
    ref_q, ref_s = oracle.act_quant_fp8(ref16, 128, round_scale=scale_fmt is not None)
    quant_close(y8.cpu().view(torch.uint8).numpy(), sc.cpu().numpy(), ref_q, ref_s, ref16)


@pytest.mark.parametrize("tokens", [1, 64, 256])
def test_config3_rope_quant_stage(wuda, tokens):
    """tokens x 128 heads x 192 (128 nope + 64 rope), RoPE base 10000 at random positions < 65536,
    e4m3 with one fp32 scale per 128 consecutive elements of the flat row."""
    _, _, proj, pos, cos, sin = make_config3(tokens, 200 + tokens)
    y16, y8, sc = wuda.rope_quant(proj.cuda(), pos.cuda(), cos.cuda(), sin.cuda(), 64, quant=True, return_bf16=True)
    torch.cuda.synchronize()
    ref16 = oracle.rope_bf16(u16(proj), pos.numpy(), cos.numpy(), sin.numpy(), 64)
    assert np.array_equal(u16(y16), ref16)
    ref_q, ref_s = oracle.act_quant_fp8(ref16.reshape(tokens, -1), 128, round_scale=False)
    assert np.array_equal(sc.cpu().numpy(), ref_s)
    assert np.array_equal(y8.cpu().view(torch.uint8).numpy(), ref_q)


def test_strided_rows_fp32_gamma_and_other_widths(wuda):
    gen = torch.Generator().manual_seed(5)
    wide = torch.randn(9, 4672, generator=gen).bfloat16().cuda()          # rows are a slice of a wider tensor
    x = wide[:, :1536]
    gamma = (torch.rand(1536, generator=gen) + 0.5).cuda()                 # fp32 gamma, as qnorm_quant takes it
    y16, y8, sc = wuda.rmsnorm_quant(x, gamma, 1e-6, scale_fmt="ue8m0")
    torch.cuda.synchronize()
    ref16 = oracle.rmsnorm_bf16(u16(x.contiguous()), gamma.cpu().numpy(), 1e-6)
    bf16_close(u16(y16), ref16)
    own_q, own_s = oracle.act_quant_fp8(u16(y16), 128, round_scale=True)
    assert np.array_equal(sc.cpu().numpy(), own_s) and np.array_equal(y8.cpu().view(torch.uint8).numpy(), own_q)
    for dim in (128, 512, 24576):
        xx = torch.randn(3, dim, generator=gen).bfloat16()
        y, _, _ = wuda.rmsnorm_quant(xx.cuda(), torch.ones(dim).cuda(), 1e-6, quant=False)
        bf16_close(u16(y), oracle.rmsnorm_bf16(u16(xx), np.ones(dim, np.float32), 1e-6))


def test_query_rmsnorm_rope_reference_signature(wuda):
    """rmsnorm_rope_out(x, positions, cos, sin, out, ...): per-head RMSNorm(512, no gamma) + RoPE(last 64)."""
    gen = torch.Generator().manual_seed(6)
    x = torch.randn(3, 64, 512, generator=gen).bfloat16()
    pos = torch.tensor([5, 70000 % 4096, 17])
    freqs = 1.0 / (10000 ** (torch.arange(0, 64, 2, dtype=torch.float32) / 64))
    ang = torch.outer(torch.arange(4096).float(), freqs)
    out = torch.empty(3, 64, 512, dtype=torch.bfloat16, device="cuda")
    wuda.rmsnorm_rope_out(x.cuda(), pos.cuda(), ang.cos().cuda().contiguous(), ang.sin().cuda().contiguous(), out, 64, 1e-6)
    torch.cuda.synchronize()
    ref = oracle.query_rms_rope(u16(x), pos.numpy(), ang.cos().numpy(), ang.sin().numpy())
    assert np.array_equal(u16(out), ref)              # same operations in the same order: bit-exact
    # against the two-pass form (norm -> bf16 -> rotate -> bf16) only the 64 rotated dims may move a step
    normed = oracle.rmsnorm_bf16(u16(x).reshape(-1, 512), np.ones(512, np.float32), 1e-6).reshape(3, 64, 512)
    two_pass = oracle.rope_bf16(normed, pos.numpy(), ang.cos().numpy(), ang.sin().numpy(), 64)
    bf16_close(u16(out)[..., :448], two_pass[..., :448], min_equal=0.995)
    # the rotated dims are differences of products: compare them by value (normalised inputs are O(1))
    assert np.allclose(oracle.bf16_to_f32(u16(out)), oracle.bf16_to_f32(two_pass), rtol=2 ** -6, atol=3e-2)


@pytest.mark.parametrize("name,input_heads", [("full", 8), ("half", 4)])
def test_query_rmsnorm_rope_golden(wuda, name, input_heads):
    """Fixture from the reference's inline twin of the fused query tail (test/test_mqa_logits_fp4.py:404-413):
    the twin's own gate is max_abs == 0 against its kernel; torch's rsqrt and this kernel's 1 / sqrt may
    differ in the last bit of a few values, so: within one bf16 step, >= 99.9 % identical."""
    g = load_golden("query_rms_rope.npz")
    x = torch.from_numpy(g["x_" + name].view(np.int16)).view(torch.bfloat16).cuda()
    out = torch.empty(x.size(0), 8, 512, dtype=torch.bfloat16, device="cuda")
    wuda.rmsnorm_rope_out(x, torch.from_numpy(g["positions"]).cuda(), torch.from_numpy(g["cos"]).cuda(),
                          torch.from_numpy(g["sin"]).cuda(), out, input_heads, float(g["eps"]))
    torch.cuda.synchronize()
    bf16_close(u16(out), g["out_" + name], min_equal=0.999)


def test_query_rmsnorm_rope_strided_input_and_head_duplication(wuda):
    """x is read in place from a wider projection output; out head h reads head h % heads."""
    gen = torch.Generator().manual_seed(8)
    wide = torch.randn(5, 8192 + 4 * 512, generator=gen).bfloat16().cuda()
    x = wide[:, 8192:].unflatten(-1, (4, 512))
    pos = torch.tensor([0, 1, 100, 4095, 9999], device="cuda")     # the last one is clamped to the table
    freqs = 1.0 / (10000 ** (torch.arange(0, 64, 2, dtype=torch.float32) / 64))
    ang = torch.outer(torch.arange(4096).float(), freqs)
    out = torch.empty(5, 8, 512, dtype=torch.bfloat16, device="cuda")
    wuda.rmsnorm_rope_out(x, pos, ang.cos().cuda().contiguous(), ang.sin().cuda().contiguous(), out, 4, 1e-6)
    torch.cuda.synchronize()
    ref = oracle.query_rms_rope(u16(x.contiguous()), pos.cpu().numpy(), ang.cos().numpy(), ang.sin().numpy(), out_heads=8)
    assert np.array_equal(u16(out), ref)
    assert torch.equal(out[:, :4], out[:, 4:])


def test_index_q_post_golden_and_oracle(wuda):
    g = load_golden("index_q_post_fp8.npz")
    iq = from_u16(g["iq"])
    q, w = wuda.idx_postprocess_fp8(iq, torch.from_numpy(g["weights"]).cuda(), torch.from_numpy(g["q_pos"]).cuda(),
                                    torch.from_numpy(g["cos"]).cuda(), torch.from_numpy(g["sin"]).cuda())
    torch.cuda.synchronize()
    oq, ow = oracle.index_q_post_fp8(g["iq"], g["q_pos"], g["cos"], g["sin"], g["weights"])
    assert np.array_equal(q.view(torch.uint8).cpu().numpy(), oq)    # correctly rounded operations only: exact
    assert np.array_equal(w.cpu().numpy(), ow)
    assert np.mean(oq == g["q8"]) >= 0.999 and np.allclose(ow, g["w_folded"], rtol=1e-6)
    # strided input (a slice of the projection output), no weights -> bare scales
    wide = torch.zeros(iq.size(0), 4096 + iq.size(1) * 128, dtype=torch.bfloat16, device="cuda")
    wide[:, :iq.size(1) * 128] = iq.flatten(1)
    q2, s2 = wuda.idx_postprocess_fp8(wide[:, :iq.size(1) * 128].unflatten(-1, (iq.size(1), 128)), None,
                                      torch.from_numpy(g["q_pos"]).cuda(), torch.from_numpy(g["cos"]).cuda(),
                                      torch.from_numpy(g["sin"]).cuda())
    torch.cuda.synchronize()
    assert torch.equal(q2.view(torch.uint8), q.view(torch.uint8))
    assert np.array_equal(s2.cpu().numpy() * g["weights"], ow)


def test_bad_arguments(wuda):
    x = torch.zeros(2, 200, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError):
        wuda.rmsnorm_quant(x, None)                 # dim not a multiple of 128
    with pytest.raises(RuntimeError):
        wuda.rmsnorm_quant(x.float(), None)
    x3 = torch.zeros(2, 4, 192, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError):
        wuda.rope_quant(x3, torch.zeros(2, dtype=torch.int32, device="cuda"), torch.zeros(8, 32, device="cuda"),
                        torch.zeros(8, 32, device="cuda"), 64)
