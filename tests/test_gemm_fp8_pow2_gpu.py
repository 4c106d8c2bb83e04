"""GPU parity of the FP8 GEMM that applies power-of-two block scales inside the tensor core (through the C ABI)
against the CPU oracle of the block-scaled product (origin/kernel.py:203-273) on the same inputs."""
import numpy as np
import pytest
import torch

import oracle
from wuda_b200 import o_proj, workloads

pytestmark = pytest.mark.gpu


def pow2(x):
    """Nearest power of two of every (positive) scale."""
    return np.exp2(np.round(np.log2(x))).astype(np.float32)


def make(m, n, k, seed):
    case = workloads.make_gemm_fp8_case(m, n, k, seed)
    case["a_s"], case["w_s"] = pow2(case["a_s"]), pow2(case["w_s"])
    return case


def run(wuda, case, expect_status=0):
    a = torch.from_numpy(case["a"]).cuda().view(torch.float8_e4m3fn)
    w = torch.from_numpy(case["w"]).cuda().view(torch.float8_e4m3fn)
    a_s, w_s = torch.from_numpy(case["a_s"]).cuda(), torch.from_numpy(case["w_s"]).cuda()
    status = wuda.device_status_word()
    out = wuda.fp8_gemm(a, a_s, w, w_s, status_word=status, pow2_scales=True)
    torch.cuda.synchronize()
    assert int(status.item()) == expect_status
    return out.cpu().view(torch.int16).numpy().view(np.uint16)


def close(got_bits, ref):
    got = oracle.bf16_to_f32(got_bits).astype(np.float64)
    ref = ref.astype(np.float64)
    rms = np.sqrt(np.mean(ref ** 2))
    err = np.abs(got - ref)
    # bf16 output rounding (2^-9 relative) plus the order of the fp32 additions; the stated bar is 1e-2 relative
    assert np.all(err <= 1e-2 * np.abs(ref) + 1e-3 * rms), "max err %g at rms %g" % (err.max(), rms)


def check(wuda, m, n, k, seed=1):
    case = make(m, n, k, seed)
    ref = oracle.gemm_fp8_blockscaled(case["a"], case["a_s"], case["w"], case["w_s"], out_bf16=False)
    got = run(wuda, case)
    assert got.shape == (m, n)
    close(got, ref)


@pytest.mark.parametrize("m", [1, 8, 16, 17, 32, 64, 65, 128, 129, 256])
def test_small_shapes_every_m(wuda, m):
    check(wuda, m, 512, 1024, seed=m)


@pytest.mark.parametrize("m,n,k", [(1, 128, 128), (3, 128, 256), (17, 384, 128), (64, 2112, 7168), (5, 1000, 512),
                                   (100, 130, 384), (200, 7168, 2048), (64, 8192, 1536), (33, 256, 16384)])
def test_ragged_shapes_partial_tiles_short_and_long_k(wuda, m, n, k):
    check(wuda, m, n, k, seed=m + n + k)


@pytest.mark.parametrize("m", [8, 64, 128, 256])
@pytest.mark.parametrize("n,k", [(24576, 7168), (7168, 16384), (2112, 7168)])
def test_decode_shapes_on_sampled_column_blocks(wuda, n, k, m):
    """The large decode shapes: the GPU computes the full product, the oracle checks every row on the first, the
    last and four seeded 128-column blocks."""
    case = make(m, n, k, seed=n % 101)
    got = oracle.bf16_to_f32(run(wuda, case)).astype(np.float64)
    tiles = (n + 127) // 128
    rng = np.random.default_rng(n + m)
    for t in sorted({0, tiles - 1} | set(rng.integers(0, tiles, size=4).tolist())):
        lo, hi = t * 128, min(n, t * 128 + 128)
        ref = oracle.gemm_fp8_blockscaled(case["a"], case["a_s"], case["w"][lo:hi], case["w_s"][t:t + 1],
                                          out_bf16=False).astype(np.float64)
        rms = np.sqrt(np.mean(ref ** 2))
        err = np.abs(got[:, lo:hi] - ref)
        assert np.all(err <= 1e-2 * np.abs(ref) + 1e-3 * rms), "block %d: max err %g at rms %g" % (t, err.max(), rms)


@pytest.mark.parametrize("m,groups,n,k", [(5, 3, 128, 256), (64, 4, 256, 512), (64, 16, 1024, 4096), (130, 2, 384, 128)])
def test_grouped(wuda, m, groups, n, k):
    """Every group multiplies its own K columns of the activation row by its own weight rows."""
    rng = np.random.default_rng(m + groups)
    a = rng.integers(0, 256, size=(m, groups * k), dtype=np.uint8)
    w = rng.integers(0, 256, size=(groups * n, k), dtype=np.uint8)
    a[(a & 0x7f) == 0x7f] = 0
    w[(w & 0x7f) == 0x7f] = 0
    a &= 0xbf                                     # |a| < 2: keeps the sums moderate
    a_s = pow2(rng.uniform(0.01, 1.0, size=(m, groups * k // 128)))
    w_s = pow2(rng.uniform(0.001, 0.1, size=(groups * n // 128, k // 128)))
    status = wuda.device_status_word()
    out = o_proj.fp8_gemm_grouped(torch.from_numpy(a).cuda().view(torch.float8_e4m3fn), torch.from_numpy(a_s).cuda(),
                                  torch.from_numpy(w).cuda().view(torch.float8_e4m3fn).view(groups, n, k),
                                  torch.from_numpy(w_s).cuda(), status_word=status, pow2_scales=True)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    got = out.cpu().view(torch.int16).numpy().view(np.uint16)
    for g in range(groups):
        ref = oracle.gemm_fp8_blockscaled(np.ascontiguousarray(a[:, g * k:(g + 1) * k]),
                                          np.ascontiguousarray(a_s[:, g * k // 128:(g + 1) * k // 128]),
                                          w[g * n:(g + 1) * n], w_s[g * n // 128:(g + 1) * n // 128], out_bf16=False)
        close(got[:, g * n:(g + 1) * n], ref)


def test_agrees_with_the_general_kernel(wuda):
    case = make(64, 1024, 2048, seed=9)
    a = torch.from_numpy(case["a"]).cuda().view(torch.float8_e4m3fn)
    w = torch.from_numpy(case["w"]).cuda().view(torch.float8_e4m3fn)
    a_s, w_s = torch.from_numpy(case["a_s"]).cuda(), torch.from_numpy(case["w_s"]).cuda()
    general = wuda.fp8_gemm(a, a_s, w, w_s).float()
    fused = wuda.fp8_gemm(a, a_s, w, w_s, pow2_scales=True).float()
    torch.cuda.synchronize()
    rms = general.pow(2).mean().sqrt()
    assert (general - fused).abs().max() <= 2e-2 * rms


def test_a_scale_that_is_no_power_of_two_is_reported(wuda):
    case = make(8, 256, 256, seed=3)
    case["w_s"][1, 0] *= 1.5
    run(wuda, case, expect_status=125)
    case = make(8, 256, 256, seed=3)
    case["a_s"][2, 1] *= 1.25
    run(wuda, case, expect_status=125)


def test_repeated_calls_share_a_scratch_with_the_general_kernel(wuda):
    """Stream-K flags are left zero: calls of both kernels and of different row counts alternate on one scratch."""
    ref = {}
    for m in (64, 5, 128, 64, 20):
        case = make(m, 2112, 7168, seed=m)
        if m not in ref:
            ref[m] = oracle.gemm_fp8_blockscaled(case["a"], case["a_s"], case["w"], case["w_s"], out_bf16=False)
        close(run(wuda, case), ref[m])
        a = torch.from_numpy(case["a"]).cuda().view(torch.float8_e4m3fn)
        w = torch.from_numpy(case["w"]).cuda().view(torch.float8_e4m3fn)
        out = wuda.fp8_gemm(a, torch.from_numpy(case["a_s"]).cuda(), w, torch.from_numpy(case["w_s"]).cuda())
        torch.cuda.synchronize()
        close(out.cpu().view(torch.int16).numpy().view(np.uint16), ref[m])


def test_exponent_byte_scales_take_the_same_path(wuda):
    """The origin passes float8_e8m0fnu scales (origin/kernel.py:257-273, scale_dtype): fp8_gemm converts the bytes to
    the fp32 powers of two they stand for and applies them in the tensor core; same bytes out as with fp32 scales."""
    case = make(33, 640, 1024, 17)
    a = torch.from_numpy(case["a"]).cuda().view(torch.float8_e4m3fn)
    w = torch.from_numpy(case["w"]).cuda().view(torch.float8_e4m3fn)
    a_s, w_s = torch.from_numpy(case["a_s"]).cuda(), torch.from_numpy(case["w_s"]).cuda()
    want = wuda.fp8_gemm(a, a_s, w, w_s, pow2_scales=True)
    exps = lambda t: ((t.view(torch.int32) >> 23) & 0xFF).to(torch.uint8)
    e8 = getattr(torch, "float8_e8m0fnu", None)
    a_e, w_e = exps(a_s), exps(w_s)
    if e8 is not None:
        a_e, w_e = a_e.view(e8), w_e.view(e8)
    got = wuda.fp8_gemm(a, a_e, w, w_e, e8 if e8 is not None else torch.float32)
    torch.cuda.synchronize()
    assert torch.equal(got, want)
