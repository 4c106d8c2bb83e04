"""The allocation-free FP8 GEMM entry point (scratch inside the library's device image, for
callers that cannot hand scratch memory to a library or tolerate a device allocation)
must give exactly what the regular entry point gives, call after call: the second call
finds whatever the first one left in the shared scratch array.

Collected last on purpose (file name), so that a run that stops at the first failure has
already run every other test; it also passes alone in a fresh process."""
import ctypes

import numpy as np
import pytest
import torch

import oracle
from wuda_b200 import workloads

pytestmark = pytest.mark.gpu


def _dev(case):
    a = torch.from_numpy(case["a"]).cuda().view(torch.float8_e4m3fn)
    w = torch.from_numpy(case["w"]).cuda().view(torch.float8_e4m3fn)
    return a, torch.from_numpy(case["a_s"]).cuda(), w, torch.from_numpy(case["w_s"]).cuda()


def _regular(wuda, case):
    a, a_s, w, w_s = _dev(case)
    out = wuda.fp8_gemm(a, a_s, w, w_s)
    torch.cuda.synchronize()
    return out.cpu().view(torch.int16).numpy().view(np.uint16)


def _noalloc(wuda, case):
    a, a_s, w, w_s = _dev(case)
    m, k = case["a"].shape
    n = case["w"].shape[0]
    out = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    status = wuda.device_status_word()
    st = wuda.lib.wuda_gemm_fp8_blockscaled_noalloc(a.data_ptr(), a_s.data_ptr(), w.data_ptr(), w_s.data_ptr(),
                                                    out.data_ptr(), m, n, k, status.data_ptr(),
                                                    torch.cuda.current_stream().cuda_stream)
    assert st == 0, wuda.lib.wuda_last_error()
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    return out.cpu().view(torch.int16).numpy().view(np.uint16)


def test_noalloc_entry_matches_regular_entry_on_two_calls_in_a_row(wuda):
    # (7168, 4096): 56 weight tiles over 148 SMs, so most tiles are split across SMs and go through the scratch
    first = workloads.make_gemm_fp8_case(64, 7168, 4096, seed=41)
    second = workloads.make_gemm_fp8_case(33, 2112, 7168, seed=42)
    for case in (first, second, first):
        got = _noalloc(wuda, case)
        ref = _regular(wuda, case)
        assert np.array_equal(got, ref)
        # and both are right: same bar as the GEMM parity tests
        exact = oracle.gemm_fp8_blockscaled(case["a"], case["a_s"], case["w"], case["w_s"], out_bf16=False)
        f = oracle.bf16_to_f32(got)
        assert np.all(np.abs(f - exact) <= 1e-2 * np.abs(exact) + 1e-3 * np.sqrt(np.mean(exact.astype(np.float64) ** 2)))


def test_noalloc_calls_of_different_row_counts_share_the_array(wuda):
    """5, 20 and 64 rows use partial-tile slots of 16, 32 and 64 columns: consecutive calls lay their slots
    out differently over the one shared array (the flags stay where they are), and each must still give
    the regular entry point's bits."""
    wide = workloads.make_gemm_fp8_case(64, 7168, 2048, seed=43)
    narrow = workloads.make_gemm_fp8_case(5, 7168, 2048, seed=44)
    middle = workloads.make_gemm_fp8_case(20, 2112, 4096, seed=45)
    refs = {id(c): _regular(wuda, c) for c in (wide, narrow, middle)}
    for case in (wide, narrow, wide, middle, narrow, middle, wide):
        assert np.array_equal(_noalloc(wuda, case), refs[id(case)])


def test_noalloc_entry_refuses_sizes_beyond_its_scratch(wuda):
    fake = ctypes.c_void_p(0x1000)
    st = wuda.lib.wuda_gemm_fp8_blockscaled_noalloc(fake, fake, fake, fake, fake, 65, 4096, 4096, None, None)
    assert st == 2
    msg = wuda.lib.wuda_last_error().decode()
    assert "m <= 64" in msg and "6292480" in msg
