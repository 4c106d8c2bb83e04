"""GPU parity (through the C ABI) of the operators that carry the origin's and the reference modules' remaining export
names: fp4_gemm (FP8 activations x FP4 weights, origin/kernel.py:441-536), fp4_act_quant (:126-200), hc_split_sinkhorn
(:355-436), head_ssq_standalone, idx_postprocess[_fp8]_standalone (kernels/wq_b_fp8_gemm.cu:1474-1566),
mqa_compressor_standalone / mqa_compressor_paged (kernels/mqa_logits_fp4.cu:653-750) and topk_v2_plan
(kernels/topk_v2.cu:329-345), each against the CPU oracle.
Tolerances: the FP4 GEMM adds exact products in fp32 inside the tensor core where the origin adds them 32-block by
32-block: |got - ref| <= 2^-7 |ref| + 2e-3 rms (one bf16 ulp plus the summation order).  The quantiser and the head
sums are correctly rounded operations in a fixed order: identical bytes.  The Sinkhorn split contains expf: 2e-6."""
import numpy as np
import pytest
import torch

import oracle
from conftest import load_golden

pytestmark = pytest.mark.gpu


def cu(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def bf16_bits(t):
    return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def make_fp4_operands(m, n, k, seed):
    """Seeded operands of the origin's fp4_gemm: activations quantised to e4m3 with power-of-two 1x128 scales,
    weights to e2m1 with exponent bytes per 32 (both by the oracle's quantisers)."""
    rng = np.random.default_rng(seed)
    x = (rng.standard_normal((m, k)) * np.exp(rng.standard_normal((m, 1)))).astype(np.float32)
    a8, a_s = oracle.act_quant_fp8(oracle.f32_to_bf16(x), 128, round_scale=True)
    w = (rng.standard_normal((n, k)) * 0.02 * np.exp(rng.standard_normal((n, 1)) * 0.5)).astype(np.float32)
    codes, sf, _ = oracle.fp4_act_quant(oracle.f32_to_bf16(w))
    return a8, a_s, codes, sf


def check_fp4_gemm(wuda, m, n, k, seed):
    a8, a_s, codes, sf = make_fp4_operands(m, n, k, seed)
    status = wuda.device_status_word()
    out = wuda.fp4_gemm(cu(a8).view(torch.float8_e4m3fn), cu(a_s), cu(codes), cu(sf), status_word=status)
    torch.cuda.synchronize()
    assert status.item() == 0
    got = out.float().cpu().numpy()
    ref = oracle.gemm_fp8_fp4(a8, a_s, codes, sf, out_bf16=False)
    rms = np.sqrt(np.mean(ref.astype(np.float64) ** 2))
    err = np.abs(got - ref)
    assert np.all(err <= 2.0 ** -7 * np.abs(ref) + 2e-3 * rms), (m, n, k, float(err.max()), float(rms))
    return out


def test_fp4_gemm_golden(wuda):
    """The fixture made with the reference's FP4 quantiser / dequantiser and the origin's lossless cast to e4m3
    (origin/convert.py:20-52): the FP4 GEMM, and the FP8 GEMM over the cast weights, against the product of the
    dequantised operands; the GPU quantiser against the reference's scale bytes."""
    g = load_golden("fp4_gemm.npz")
    a = cu(g["a"]).view(torch.float8_e4m3fn)
    status = wuda.device_status_word()
    c4 = wuda.fp4_gemm(a, cu(g["a_s"]), cu(g["w4"]), cu(g["w_sf"]), status_word=status)
    c8 = wuda.fp8_gemm(a, cu(g["a_s"]), cu(g["w8"]).view(torch.float8_e4m3fn), cu(g["w8_scale"]), pow2_scales=True,
                       status_word=status)
    torch.cuda.synchronize()
    assert status.item() == 0
    ref = g["c"]
    rms = np.sqrt(np.mean(ref.astype(np.float64) ** 2))
    for got in (c4, c8):
        assert np.all(np.abs(got.float().cpu().numpy() - ref) <= 2.0 ** -8 * np.abs(ref) + 1e-5 * rms)   # one bf16 rounding
    assert (c4 == c8).float().mean().item() >= 0.99      # same products; the tensor core aligns them per instruction
    codes, sf = wuda.fp4_act_quant(torch.from_numpy(g["w"]).bfloat16().cuda())
    assert np.array_equal(sf.view(torch.uint8).cpu().numpy(), g["w_sf"])
    unpack = lambda b: np.stack([b & 15, b >> 4], -1).reshape(b.shape[0], -1)
    mine, want = unpack(codes.view(torch.uint8).cpu().numpy()), unpack(g["w4"])
    mine = np.where((mine & 7) == 0, 0, mine)            # the hardware conversion keeps the sign of a zero
    assert np.mean(mine == want) > 0.98                  # what is left are exact ties (down there, to even here)


@pytest.mark.parametrize("m", [1, 8, 32, 64, 128, 256])
def test_fp4_gemm_small_every_row_count(wuda, m):
    check_fp4_gemm(wuda, m, 512, 1024, 100 + m)


@pytest.mark.parametrize("m,n,k", [(64, 4096, 7168), (64, 7168, 2048), (33, 2112, 7168), (5, 200, 256), (128, 1000, 1536),
                                   (64, 384, 128), (8, 512, 640), (64, 256, 1920), (256, 2048, 2048)])
def test_fp4_gemm_shapes(wuda, m, n, k):
    """The origin's expert shapes (w1/w3: 2048 x 7168 pairs, w2: 7168 x 2048), ragged N, short K (activations resident
    in shared memory), one K block, an odd number of K blocks, two passes of 128 rows."""
    check_fp4_gemm(wuda, m, n, k, m * 7 + n)


def test_fp4_gemm_scale_dtypes_and_reruns(wuda):
    """float8_e8m0fnu activation scales and torch's FP4 dtype are what the origin passes; a rerun writes the same bytes."""
    a8, a_s, codes, sf = make_fp4_operands(64, 1024, 2048, 5)
    a = cu(a8).view(torch.float8_e4m3fn)
    first = wuda.fp4_gemm(a, cu(a_s), cu(codes), cu(sf))
    exps = cu(((a_s.view(np.uint32) >> 23) & 0xFF).astype(np.uint8))
    e8 = getattr(torch, "float8_e8m0fnu", None)
    fp4 = getattr(torch, "float4_e2m1fn_x2", None)
    b, b_s = cu(codes), cu(sf)
    second = wuda.fp4_gemm(a, exps.view(e8) if e8 is not None else exps, b.view(fp4) if fp4 is not None else b,
                           b_s.view(e8) if e8 is not None else b_s, e8 if e8 is not None else torch.float32)
    torch.cuda.synchronize()
    assert torch.equal(first, second)
    for _ in range(3):
        assert torch.equal(wuda.fp4_gemm(a, cu(a_s), b, b_s), first)


def test_fp4_gemm_reports_a_scale_that_is_no_power_of_two(wuda):
    a8, a_s, codes, sf = make_fp4_operands(8, 256, 256, 9)
    a_s = a_s.copy()
    a_s[3, 1] *= 1.5
    status = wuda.device_status_word()
    wuda.fp4_gemm(cu(a8).view(torch.float8_e4m3fn), cu(a_s), cu(codes), cu(sf), status_word=status)
    torch.cuda.synchronize()
    assert status.item() != 0
    with pytest.raises(wuda.WudaError, match="K"):
        wuda.fp4_gemm(cu(a8).view(torch.float8_e4m3fn), cu(a_s), cu(codes[:, :64]), cu(sf))


@pytest.mark.parametrize("rows,cols,seed", [(1, 32, 1), (7, 128, 2), (64, 7168, 3), (300, 512, 4), (2049, 7168, 5)])
def test_fp4_act_quant_against_oracle(wuda, rows, cols, seed):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((rows, cols)) * np.exp(rng.standard_normal((rows, 1)) * 4)
    x[0, :32] = 0.0                                                   # a block of zeros: the amax floor
    if rows > 2:
        x[2, 5] = 3.0e38                                              # the largest scales
        x[1] *= 1e-36                                                 # the smallest
    xb = torch.from_numpy(x).bfloat16().cuda()
    y, s = wuda.fp4_act_quant(xb)
    torch.cuda.synchronize()
    oc, osf, odeq = oracle.fp4_act_quant(bf16_bits(xb))
    assert np.array_equal(s.view(torch.uint8).cpu().numpy(), osf)
    assert np.array_equal(y.view(torch.uint8).cpu().numpy(), oc)
    z = xb.clone()
    back = wuda.fp4_act_quant(z, 32, True)
    torch.cuda.synchronize()
    assert back.data_ptr() == z.data_ptr()
    assert np.array_equal(bf16_bits(z), odeq)
    # a column slice of a wider matrix is read, and in place written, where it lies
    wide = torch.full((rows, cols + 64), 7.0, dtype=torch.bfloat16, device="cuda")
    wide[:, 32:32 + cols] = xb
    ys, ss = wuda.fp4_act_quant(wide[:, 32:32 + cols])
    assert torch.equal(ys.view(torch.uint8), y.view(torch.uint8)) and torch.equal(ss.view(torch.uint8), s.view(torch.uint8))
    wuda.fp4_act_quant(wide[:, 32:32 + cols], 32, True)
    torch.cuda.synchronize()
    assert np.array_equal(bf16_bits(wide[:, 32:32 + cols]), odeq)
    assert (wide[:, :32] == 7.0).all() and (wide[:, 32 + cols:] == 7.0).all()
    # a view of a wider tensor (3-D, last dimension dense) quantises row by row like the origin's .view(-1, N)
    y3, s3 = wuda.fp4_act_quant(xb.view(rows, 1, cols))
    torch.cuda.synchronize()
    assert y3.shape == (rows, 1, cols // 2) and s3.shape == (rows, 1, cols // 32)
    assert torch.equal(y3.view(torch.uint8).flatten(), y.view(torch.uint8).flatten())


def test_fp4_quantised_weights_feed_the_gemm(wuda):
    """fp4_act_quant's outputs are what fp4_gemm reads as weights: quantise on the GPU, multiply, compare with the
    oracle run on the same bytes."""
    rng = np.random.default_rng(11)
    w = torch.from_numpy(rng.standard_normal((768, 1024)) * 0.05).bfloat16().cuda()
    codes, sf = wuda.fp4_act_quant(w)
    x = torch.from_numpy(rng.standard_normal((16, 1024))).bfloat16().cuda()
    a8, a_s = wuda.act_quant(x, 128, "ue8m0")
    out = wuda.fp4_gemm(a8, a_s, codes, sf)
    torch.cuda.synchronize()
    ref = oracle.gemm_fp8_fp4(a8.view(torch.uint8).cpu().numpy(), a_s.cpu().numpy(), codes.view(torch.uint8).cpu().numpy(),
                              sf.view(torch.uint8).cpu().numpy(), out_bf16=False)
    rms = np.sqrt(np.mean(ref.astype(np.float64) ** 2))
    assert np.all(np.abs(out.float().cpu().numpy() - ref) <= 2.0 ** -7 * np.abs(ref) + 2e-3 * rms)


@pytest.mark.parametrize("b,s", [(1, 1), (64, 1), (3, 17)])
def test_hc_split_sinkhorn_against_oracle(wuda, b, s):
    rng = np.random.default_rng(b * 31 + s)
    mixes = (rng.standard_normal((b, s, 24)) * 2).astype(np.float32)
    scale = np.array([0.7, 1.3, 0.9], np.float32)
    base = (rng.standard_normal(24) * 0.3).astype(np.float32)
    pre, post, comb = wuda.hc_split_sinkhorn(cu(mixes), cu(scale), cu(base))
    torch.cuda.synchronize()
    assert pre.shape == (b, s, 4) and post.shape == (b, s, 4) and comb.shape == (b, s, 4, 4)
    opre, opost, ocomb = oracle.hc_split_sinkhorn(mixes, scale, base)
    assert np.allclose(pre.cpu().numpy().reshape(-1, 4), opre, rtol=2e-6, atol=2e-6)
    assert np.allclose(post.cpu().numpy().reshape(-1, 4), opost, rtol=2e-6, atol=2e-6)
    assert np.allclose(comb.cpu().numpy().reshape(-1, 4, 4), ocomb, rtol=2e-6, atol=2e-6)
    c = comb.cpu().numpy()
    assert np.allclose(c.sum(-2), 1.0, atol=1e-4)            # the last step normalises the columns
    with pytest.raises(wuda.WudaError, match="hc_mult"):
        wuda.hc_split_sinkhorn(cu(mixes), cu(scale), cu(base), 2)


@pytest.mark.parametrize("rows,heads", [(1, 1), (64, 128), (5, 3)])
def test_head_ssq_is_the_reference_sum_bit_for_bit(wuda, rows, heads):
    rng = np.random.default_rng(rows + heads)
    y = torch.from_numpy(rng.standard_normal((rows, heads * 512)) * 3).bfloat16().cuda()
    ssq = wuda.head_ssq_standalone(y)
    torch.cuda.synchronize()
    ref = oracle.head_ssq(bf16_bits(y).reshape(rows, heads, 512))
    assert np.array_equal(ssq.cpu().numpy().view(np.uint32), ref.view(np.uint32))
    wide = torch.zeros(rows, heads * 512 + 1024, dtype=torch.bfloat16, device="cuda")
    wide[:, :heads * 512] = y
    assert torch.equal(wuda.head_ssq_standalone(wide[:, :heads * 512]), ssq)


def rope_tables(max_pos):
    ang = np.outer(np.arange(max_pos, dtype=np.float32), (1.0 / (10000.0 ** (np.arange(32) / 32.0))).astype(np.float32))
    return np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)


def test_standalone_names_of_the_indexer_q_post(wuda):
    rng = np.random.default_rng(3)
    iq = torch.from_numpy(rng.standard_normal((9, 64, 128))).bfloat16().cuda()
    cos, sin = rope_tables(256)
    pos = cu(rng.integers(0, 256, size=9).astype(np.int32))
    w = cu(rng.standard_normal((9, 64)).astype(np.float32))
    q4, sf = wuda.idx_postprocess_standalone(iq, pos, cu(cos), cu(sin))
    r4, rsf = wuda.idx_postprocess(iq, pos, cu(cos), cu(sin))
    assert torch.equal(q4, r4) and torch.equal(sf, rsf) and q4.dtype == torch.int8 and sf.dtype == torch.int32
    f4, fsf = wuda.idx_postprocess_standalone(iq.float(), pos, cu(cos), cu(sin))       # fp32 input holding bf16 values
    assert torch.equal(f4, r4) and torch.equal(fsf, rsf)
    q8, wf = wuda.idx_postprocess_fp8_standalone(iq, w, pos, cu(cos), cu(sin))
    r8, rwf = wuda.idx_postprocess_fp8(iq, w, pos, cu(cos), cu(sin))
    torch.cuda.synchronize()
    assert torch.equal(q8.view(torch.uint8), r8.view(torch.uint8)) and torch.equal(wf, rwf)


def test_main_compressor_under_the_fp4_module_names(wuda):
    """mqa_compressor_standalone and mqa_compressor_paged with the reference's int32 row arguments."""
    rng = np.random.default_rng(21)
    rows, ring, epb, stride = 16, 8, 64, 64 * 584 + 128
    pos = (rng.integers(1, 500, size=rows) * 4 + 3).astype(np.int64)
    pos[::3] -= 1                                                      # rows that do not compress
    cos, sin = rope_tables(2048)
    state = rng.normal(size=(rows, ring, 2048)).astype(np.float32)
    state_row = (np.arange(rows) * ring + pos % ring).astype(np.int32)
    norm = (rng.random(512) + 0.5).astype(np.float32)
    q8 = torch.full((rows, 448), 0xAB, dtype=torch.uint8, device="cuda")
    s8 = torch.full((rows, 7), -1.0, device="cuda")
    rope = torch.zeros((rows, 64), dtype=torch.bfloat16, device="cuda")
    wuda.mqa_compressor_standalone(cu(pos), cu(norm), cu(cos), cu(sin), cu(state), cu(state_row), ring, q8, s8, rope)
    oq, os_, orope = oracle.main_compressor_fp8(state, state_row.astype(np.int64), pos, norm, cos, sin)
    assert np.mean(q8.cpu().numpy() == oq) >= 0.999
    pages = 3
    pool = np.full((pages, stride), 0xA5, np.uint8)
    dst = rng.permutation(pages * epb)[:rows].astype(np.int32)
    dst[(pos + 1) % 4 != 0] = -1
    ref_pool = pool.copy()
    oracle.main_compressor_fp8(state, state_row.astype(np.int64), pos, norm, cos, sin, pool=ref_pool,
                               dst=dst.astype(np.int64), epb=epb)
    d_pool = cu(pool)
    wuda.mqa_compressor_paged(cu(pos), cu(norm), cu(cos), cu(sin), cu(state), cu(state_row), ring, d_pool.flatten(), cu(dst),
                              epb, stride)
    torch.cuda.synchronize()
    got = d_pool.cpu().numpy()
    changed = ref_pool != pool
    assert changed.any() and not np.any((got != pool) & ~changed)
    assert np.mean(got == ref_pool) >= 1 - 1e-3
    with pytest.raises(wuda.WudaError, match="geometry"):
        wuda.mqa_compressor_paged(cu(pos), cu(norm), cu(cos), cu(sin), cu(state), cu(state_row), ring, d_pool.flatten(),
                                  cu(dst), epb, 1000)


def test_topk_v2_plan_checks_like_the_reference_and_changes_nothing(wuda):
    lens = torch.tensor([5, 70000, 123], dtype=torch.int32, device="cuda")
    meta = torch.full((4, 2), 7, dtype=torch.int32, device="cuda")
    wuda.topk_v2_plan(lens, meta)
    assert (meta == 7).all()
    with pytest.raises(wuda.WudaError, match="metadata"):
        wuda.topk_v2_plan(lens, meta[:3].contiguous())
    scores = torch.randn(3, 70016, device="cuda")
    table = torch.arange(3 * 1100, dtype=torch.int32, device="cuda").view(3, 1100)
    out = torch.empty((3, 64), dtype=torch.int32, device="cuda")
    wuda.topk_v2_transform(scores, lens, table, out, 64, meta)      # the planned call of the reference's test
    torch.cuda.synchronize()
    assert (out[0, :5] >= 0).all() and (out[0, 5:] == -1).all()
