"""GPU parity of the NVFP4 block-scaled GEMM (through the C ABI) against the CPU oracle (fp32
accumulation of the dequantised operands)."""
import numpy as np
import pytest
import torch

import oracle
from wuda_b200 import workloads

pytestmark = pytest.mark.gpu


def run(wuda, case):
    t = lambda x: torch.from_numpy(np.ascontiguousarray(x)).cuda()
    status = wuda.device_status_word()
    out = wuda.nvfp4_gemm(t(case["a"]), t(case["a_sf_packed"]), case["a_gs"], t(case["w"]), t(case["w_sf_packed"]),
                          case["w_gs"], status_word=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    return out.cpu().view(torch.int16).numpy().view(np.uint16)


def reference(case, out_bf16=False):
    return oracle.gemm_nvfp4(case["a"], case["a_sf"], case["a_gs"], case["w"], case["w_sf"], case["w_gs"], out_bf16)


def check(wuda, m, n, k, seed=1):
    case = workloads.make_gemm_nvfp4_case(m, n, k, seed)
    got = oracle.bf16_to_f32(run(wuda, case)).astype(np.float64)
    ref = reference(case).astype(np.float64)
    rms = np.sqrt(np.mean(ref ** 2))
    err = np.abs(got - ref)
    assert np.all(err <= 1e-2 * np.abs(ref) + 1e-3 * rms), "max err %g at rms %g" % (err.max(), rms)


def pack_codes(vals):
    """integers in {-6..6} representable in e2m1 -> packed bytes"""
    table = {0.0: 0, 0.5: 1, 1.0: 2, 1.5: 3, 2.0: 4, 3.0: 5, 4.0: 6, 6.0: 7}
    mag = np.vectorize(lambda v: table[abs(float(v))])(vals).astype(np.uint8)
    code = mag | ((vals < 0) & (mag != 0)).astype(np.uint8) << 3
    code = code.reshape(vals.shape[0], -1, 2)
    return (code[:, :, 0] | (code[:, :, 1] << 4)).astype(np.uint8)


def test_unit_scales_small_integers_exact(wuda):
    """All block scales 1.0: the result is a plain integer GEMM, exact in fp32 and in bf16."""
    rng = np.random.default_rng(1)
    m, n, k = 16, 256, 512
    a = rng.choice([-2.0, -1.0, 0.0, 1.0, 2.0], size=(m, k))
    w = rng.choice([-1.0, 0.0, 1.0], size=(n, k))
    one = np.full((1,), 0x38, np.uint8)      # 1.0 in ue4m3
    case = dict(a=pack_codes(a), w=pack_codes(w), a_sf=np.full((m, k // 16), 0x38, np.uint8),
                w_sf=np.full((n, k // 16), 0x38, np.uint8), a_gs=np.float32(1), w_gs=np.float32(1))
    case["a_sf_packed"] = workloads.pack_nvfp4_scales(case["a_sf"])
    case["w_sf_packed"] = workloads.pack_nvfp4_scales(case["w_sf"])
    got = oracle.bf16_to_f32(run(wuda, case))
    ref = (a @ w.T).astype(np.float32)
    assert np.array_equal(got, ref), np.abs(got - ref).max()
    del one


def test_scale_layout_is_pinned_by_power_of_two_scales(wuda):
    """Power-of-two block scales that differ per row, per 16-element group and per operand: every
    product is exact, so a scale applied to the wrong row or K group changes bits."""
    rng = np.random.default_rng(2)
    m, n, k = 48, 384, 1024
    a = rng.choice([-1.0, 0.0, 1.0, 2.0], size=(m, k))
    w = rng.choice([-1.0, 0.0, 1.0], size=(n, k))
    a_sf = (0x38 + 8 * rng.integers(-2, 3, size=(m, k // 16))).astype(np.uint8)     # 2^-2 .. 2^2
    w_sf = (0x38 + 8 * rng.integers(-2, 3, size=(n, k // 16))).astype(np.uint8)
    case = dict(a=pack_codes(a), w=pack_codes(w), a_sf=a_sf, w_sf=w_sf, a_gs=np.float32(0.5), w_gs=np.float32(4))
    case["a_sf_packed"] = workloads.pack_nvfp4_scales(a_sf)
    case["w_sf_packed"] = workloads.pack_nvfp4_scales(w_sf)
    got = run(wuda, case)
    ref = reference(case, out_bf16=True)
    assert np.array_equal(got, ref)


@pytest.mark.parametrize("m", [1, 8, 32, 64, 128, 200, 256])
def test_random_every_m(wuda, m):
    check(wuda, m, 512, 1024, seed=m)


@pytest.mark.parametrize("m,n,k", [(3, 128, 256), (17, 1000, 512), (64, 2112, 7168), (100, 130, 768)])
def test_ragged_shapes(wuda, m, n, k):
    check(wuda, m, n, k, seed=m + n)


CONFIG2_SHAPES = [(24576, 7168), (7168, 16384), (2112, 7168), (4096, 7168)]
_config2_cases = {}


def _config2_case(n, k):
    if (n, k) not in _config2_cases:
        _config2_cases.clear()
        _config2_cases[(n, k)] = workloads.make_gemm_nvfp4_case(256, n, k, seed=n % 103)
    return _config2_cases[(n, k)]


@pytest.mark.parametrize("m", [1, 8, 32, 64, 128, 256])
@pytest.mark.parametrize("n,k", CONFIG2_SHAPES)
def test_config2_sweep_every_m_on_every_shape(wuda, n, k, m):
    """Every M of the decode sweep on every (N, K) pair, (2112, 7168) and the two-pass M = 256 included.  The GPU
    computes the full product; the oracle checks every row on the first, the last and four seeded 128-column
    blocks."""
    full = _config2_case(n, k)
    case = dict(full, a=np.ascontiguousarray(full["a"][:m]), a_sf=full["a_sf"][:m],
                a_sf_packed=workloads.pack_nvfp4_scales(full["a_sf"][:m]))
    got = oracle.bf16_to_f32(run(wuda, case)).astype(np.float64)
    assert got.shape == (m, n)
    tiles = (n + 127) // 128
    rng = np.random.default_rng(n + m)
    for t in sorted({0, tiles - 1} | set(rng.integers(0, tiles, size=4).tolist())):
        lo, hi = t * 128, min(n, t * 128 + 128)
        ref = oracle.gemm_nvfp4(case["a"], case["a_sf"], case["a_gs"], np.ascontiguousarray(full["w"][lo:hi]),
                                np.ascontiguousarray(full["w_sf"][lo:hi]), full["w_gs"], False).astype(np.float64)
        rms = np.sqrt(np.mean(ref ** 2))
        err = np.abs(got[:, lo:hi] - ref)
        assert np.all(err <= 1e-2 * np.abs(ref) + 1e-3 * rms), "block %d: max err %g at rms %g" % (t, err.max(), rms)


def test_bad_arguments(wuda):
    a = torch.zeros(4, 128, dtype=torch.uint8, device="cuda")
    w = torch.zeros(128, 128, dtype=torch.uint8, device="cuda")
    sf = torch.zeros(128 * 16, dtype=torch.uint8, device="cuda")
    with pytest.raises(RuntimeError):
        wuda.nvfp4_gemm(a, sf[:100], 1.0, w, sf, 1.0)
    with pytest.raises(RuntimeError):
        wuda.nvfp4_gemm(a[:, :100].contiguous(), sf, 1.0, w[:, :100].contiguous(), sf, 1.0)
