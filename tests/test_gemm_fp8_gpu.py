"""GPU parity of the block-scaled FP8 GEMM (through the C ABI) against the CPU oracle
(fp32 accumulation per 128-wide K block, promoted with the block scales)."""
import numpy as np
import pytest
import torch

import oracle
from wuda_b200 import workloads

pytestmark = pytest.mark.gpu


def run(wuda, case):
    a = torch.from_numpy(case["a"]).cuda().view(torch.float8_e4m3fn)
    w = torch.from_numpy(case["w"]).cuda().view(torch.float8_e4m3fn)
    a_s, w_s = torch.from_numpy(case["a_s"]).cuda(), torch.from_numpy(case["w_s"]).cuda()
    status = wuda.device_status_word()
    out = wuda.fp8_gemm(a, a_s, w, w_s, status_word=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    return out.cpu().view(torch.int16).numpy().view(np.uint16)


def check(wuda, m, n, k, seed=1):
    case = workloads.make_gemm_fp8_case(m, n, k, seed)
    got = oracle.bf16_to_f32(run(wuda, case)).astype(np.float64)
    ref = oracle.gemm_fp8_blockscaled(case["a"], case["a_s"], case["w"], case["w_s"], out_bf16=False).astype(np.float64)
    assert got.shape == ref.shape == (m, n)
    rms = np.sqrt(np.mean(ref ** 2))
    err = np.abs(got - ref)
    # bf16 output rounding (2^-9 relative) plus fp32 summation order; the stated bar is 1e-2 relative
    assert np.all(err <= 1e-2 * np.abs(ref) + 1e-3 * rms), "max err %g at rms %g" % (err.max(), rms)
    return err.max() / rms


@pytest.mark.parametrize("m", [1, 8, 32, 64, 128, 256])
def test_small_shapes_every_m(wuda, m):
    check(wuda, m, 512, 1024, seed=m)


@pytest.mark.parametrize("m,n,k", [(1, 128, 128), (3, 128, 256), (17, 384, 128), (64, 2112, 7168), (5, 1000, 512),
                                   (100, 130, 384), (200, 7168, 2048)])
def test_ragged_shapes_and_partial_tiles(wuda, m, n, k):
    check(wuda, m, n, k, seed=m + n + k)


CONFIG2_SHAPES = [(24576, 7168), (7168, 16384), (2112, 7168), (4096, 7168)]
_config2_cases = {}


def _config2_case(n, k):
    """One seeded case per shape, 256 activation rows; smaller M take the first rows."""
    if (n, k) not in _config2_cases:
        _config2_cases.clear()                       # one shape at a time: the largest case holds 180 MB
        _config2_cases[(n, k)] = workloads.make_gemm_fp8_case(256, n, k, seed=n % 101)
    return _config2_cases[(n, k)]


@pytest.mark.parametrize("m", [1, 8, 32, 64, 128, 256])
@pytest.mark.parametrize("n,k", CONFIG2_SHAPES)
def test_config2_sweep_every_m_on_every_shape(wuda, n, k, m):
    """The whole (N, K) x M sweep of the block-scaled decode GEMM: the GPU computes
    the full product; the oracle checks every row on a sample of 128-column blocks - the first, the last (ragged
    for N = 2112), and four seeded ones - which is where the stream-K splits, the resident-activation switch and
    the two-pass path above 128 rows differ between M."""
    full = _config2_case(n, k)
    case = dict(a=full["a"][:m], a_s=full["a_s"][:m], w=full["w"], w_s=full["w_s"])
    got = oracle.bf16_to_f32(run(wuda, case)).astype(np.float64)
    tiles = (n + 127) // 128
    rng = np.random.default_rng(n + m)
    blocks = sorted({0, tiles - 1} | set(rng.integers(0, tiles, size=4).tolist()))
    for t in blocks:
        lo, hi = t * 128, min(n, t * 128 + 128)
        ref = oracle.gemm_fp8_blockscaled(case["a"], case["a_s"], full["w"][lo:hi], full["w_s"][t:t + 1],
                                          out_bf16=False).astype(np.float64)
        rms = np.sqrt(np.mean(ref ** 2))
        err = np.abs(got[:, lo:hi] - ref)
        assert np.all(err <= 1e-2 * np.abs(ref) + 1e-3 * rms), "block %d: max err %g at rms %g" % (t, err.max(), rms)


def test_scratch_is_left_clean_and_results_repeat(wuda):
    case = workloads.make_gemm_fp8_case(48, 7168, 4096, 9)
    first = run(wuda, case)
    second = run(wuda, case)
    third = run(wuda, workloads.make_gemm_fp8_case(48, 7168, 4096, 9))
    ref = oracle.gemm_fp8_blockscaled(case["a"], case["a_s"], case["w"], case["w_s"], out_bf16=False)
    f = oracle.bf16_to_f32(first)
    assert np.all(np.abs(f - ref) <= 1e-2 * np.abs(ref) + 1e-3 * np.sqrt(np.mean(ref ** 2)))
    # same scratch reused: a dirty scratch would show up as a changed result
    assert np.mean(first == second) > 0.999 and np.mean(first == third) > 0.999
    assert np.max(np.abs(oracle.bf16_to_f32(second) - f)) <= np.max(np.abs(f)) * 2 ** -7


def test_gemm_launched_while_another_kernel_holds_the_sms(wuda):
    """The stream-K fix-up makes a tile's first CTA wait for the CTAs that hold the rest of its K range, which
    is only sound while those can become resident.  Here every SM is held by another stream's persistent
    kernel (the paged MQA logits, one 170 KB CTA per SM, launched back to back) while the GEMMs are launched:
    their CTAs trickle onto SMs as that kernel's CTAs leave.  Every GEMM must finish with status 0 and the
    bits of an undisturbed run (the partial sums are added in CTA order whatever the arrival order)."""
    case = workloads.make_gemm_fp8_case(64, 7168, 4096, seed=77)      # 56 tiles over 148 SMs: most tiles are split
    a = torch.from_numpy(case["a"]).cuda().view(torch.float8_e4m3fn)
    w = torch.from_numpy(case["w"]).cuda().view(torch.float8_e4m3fn)
    a_s, w_s = torch.from_numpy(case["a_s"]).cuda(), torch.from_numpy(case["w_s"]).cuda()
    status = wuda.device_status_word()
    quiet = wuda.fp8_gemm(a, a_s, w, w_s, status_word=status).clone()
    torch.cuda.synchronize()
    mqa = workloads.make_mqa_case(24, 2, 30000, 60000, seed=5)
    d = workloads.to_device(mqa)
    logits = torch.empty((48, mqa["logits_stride"]), dtype=torch.float32, device="cuda")
    mqa_status = wuda.device_status_word()
    busy, side = torch.cuda.Stream(), torch.cuda.Stream()
    outs = [torch.empty_like(quiet) for _ in range(12)]
    torch.cuda.synchronize()
    with torch.cuda.stream(busy):
        for _ in range(40):
            wuda.mqa_logits_fp8_decode_out(d["q"], d["kv_pages"], d["weights"], d["context_lens"], d["block_table"], None,
                                           logits, 64, next_n=2, status_word=mqa_status)
    with torch.cuda.stream(side):
        for out in outs:
            wuda.fp8_gemm(a, a_s, w, w_s, out=out, status_word=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0 and int(mqa_status.item()) == 0
    for out in outs:
        assert torch.equal(out, quiet)


def test_exactly_representable_products_are_bit_exact(wuda):
    """Small integer operands and power-of-two scales: every partial sum is exact in fp32, so any
    mis-indexed tile, K block or scale shows as a bit difference."""
    rng = np.random.default_rng(4)
    m, n, k = 37, 1152, 1536
    a = oracle.e4m3_encode(rng.integers(-3, 4, size=(m, k)).astype(np.float32))
    w = oracle.e4m3_encode(rng.integers(-3, 4, size=(n, k)).astype(np.float32))
    a_s = (2.0 ** rng.integers(-2, 3, size=(m, k // 128))).astype(np.float32)
    w_s = (2.0 ** rng.integers(-2, 3, size=(n // 128, k // 128))).astype(np.float32)
    case = dict(a=a, a_s=a_s, w=w, w_s=w_s)
    got = run(wuda, case)
    ref = oracle.gemm_fp8_blockscaled(a, a_s, w, w_s, out_bf16=True)
    assert np.array_equal(got, ref)


def test_bad_arguments(wuda):
    a = torch.zeros(4, 256, device="cuda").to(torch.float8_e4m3fn)
    w = torch.zeros(128, 256, device="cuda").to(torch.float8_e4m3fn)
    a_s = torch.ones(4, 2, device="cuda")
    w_s = torch.ones(1, 2, device="cuda")
    with pytest.raises(RuntimeError):
        wuda.fp8_gemm(a, a_s[:, :1].contiguous(), w, w_s)
    with pytest.raises(RuntimeError):
        wuda.fp8_gemm(a[:, :200].contiguous(), a_s, w[:, :200].contiguous(), w_s)
    with pytest.raises(RuntimeError):
        wuda.fp8_gemm(torch.zeros(300, 256, device="cuda").to(torch.float8_e4m3fn), torch.ones(300, 2, device="cuda"), w, w_s)
