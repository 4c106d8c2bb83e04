"""GPU parity of the BF16 GEMM and of the front mixed GEMM with its FRONT-EMIT scatter (through
the C ABI) against the CPU oracle.  Products of bf16 values are exact in fp32, so only the order of
the fp32 sum differs: fp32 outputs are held to 2e-5 of the row scale against a double-precision
sum, bf16 outputs to one step."""
import numpy as np
import pytest
import torch

import oracle
from wuda_b200 import workloads

pytestmark = pytest.mark.gpu


def u16(t):
    return t.cpu().view(torch.int16).numpy().view(np.uint16)


def check_fp32(got, ref):
    scale = np.sqrt((ref ** 2).mean(axis=1, keepdims=True)) + 1e-30
    assert np.all(np.abs(got - ref) <= 2e-5 * scale + 1e-5 * np.abs(ref))


@pytest.mark.parametrize("m,n,k", [(1, 128, 64), (7, 200, 448), (16, 2624, 7168), (33, 1000, 1024), (64, 2624, 7168),
                                   (128, 384, 2048), (5, 24576, 512)])
def test_fp32_and_bf16_outputs(wuda, m, n, k):
    g = torch.Generator().manual_seed(m * 1009 + n + k)
    a = torch.randn(m, k, generator=g).bfloat16()
    w = (torch.randn(n, k, generator=g) * 0.05).bfloat16()
    ref = oracle.gemm_bf16(u16(a), u16(w))
    status = wuda.device_status_word()
    out32 = wuda.bf16_gemm(a.cuda(), w.cuda(), out_dtype=torch.float32, status_word=status)
    out16 = wuda.bf16_gemm(a.cuda(), w.cuda(), status_word=status)
    out32_again = wuda.bf16_gemm(a.cuda(), w.cuda(), out_dtype=torch.float32, status_word=status)
    torch.cuda.synchronize()
    assert status.item() == 0
    check_fp32(out32.cpu().numpy().astype(np.float64), ref)
    assert torch.equal(out32, out32_again)                       # partial tiles are added in a fixed order
    assert np.array_equal(u16(out16), oracle.f32_to_bf16(out32.cpu().numpy()))   # same sums, rounded once


def test_rejects_bad_arguments(wuda):
    a = torch.zeros(4, 100, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(wuda.WudaError, match="multiple of 64"):
        wuda.bf16_gemm(a, torch.zeros(8, 100, dtype=torch.bfloat16, device="cuda"))
    a = torch.zeros(129, 128, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(wuda.WudaError):
        wuda.bf16_gemm(a, torch.zeros(8, 128, dtype=torch.bfloat16, device="cuda"))


@pytest.mark.parametrize("m", [1, 9, 64])
def test_front_mixed_gemm_with_emit(wuda, m):
    g = torch.Generator().manual_seed(50 + m)
    k, ring, blocks = 7168, 8, m + 2
    x = torch.randn(m, k, generator=g).bfloat16()
    x8, xs = workloads.quantize_fp8_1x128(x.float())
    w8, w8s = workloads.quantize_fp8_128x128(torch.randn(2048, k, generator=g) * 0.02)
    w16 = (torch.randn(2624, k, generator=g) * 0.02).bfloat16()
    pos = torch.randint(0, 5000, (m,), generator=g)
    main_row = torch.arange(m) * ring + pos % ring
    idx_row = main_row.clone()
    if m > 1:
        main_row[1] = -1                                          # this token publishes no MAIN entry
    ape, idx_ape = torch.randn(4, 1024, generator=g), torch.randn(4, 256, generator=g)
    main_state = torch.full((blocks, ring, 2048), 7.0)
    idx_state = torch.full((blocks, ring, 512), 7.0)
    d = dict(main_state=main_state.cuda(), idx_state=idx_state.cuda(), win_y2=torch.empty(m, 512, device="cuda"),
             w64=torch.empty(m, 64, device="cuda"))
    out = torch.empty(m, 2048, dtype=torch.bfloat16, device="cuda")
    status = wuda.device_status_word()
    to_t = lambda a, dt=None: torch.from_numpy(a).cuda() if dt is None else torch.from_numpy(a).cuda().view(dt)
    _, y16 = wuda.front_mixed_gemm(x.cuda(), to_t(x8, torch.float8_e4m3fn), to_t(xs), w16.cuda(),
                                   to_t(w8, torch.float8_e4m3fn), to_t(w8s), out, pos=pos.cuda(), ape=ape.cuda(),
                                   main_state_row=main_row.cuda(), idx_state_row=idx_row.cuda(), idx_ape=idx_ape.cuda(),
                                   status_word=status, **d)
    torch.cuda.synchronize()
    assert status.item() == 0
    # FP8 segment against the block-scaled oracle, BF16 segment against the double-precision sum
    ref8 = oracle.bf16_to_f32(oracle.gemm_fp8_blockscaled(x8, xs, w8, w8s))
    got8 = out.float().cpu().numpy()
    assert np.all(np.abs(got8 - ref8) <= 1e-2 * np.abs(ref8) + 1e-3 * np.abs(ref8).max())
    check_fp32(y16.cpu().numpy().astype(np.float64), oracle.gemm_bf16(u16(x), u16(w16)))
    # the scatter, exactly, from the GPU's own GEMM outputs
    ms, isr = main_state.numpy().copy(), idx_state.numpy().copy()
    win, w64 = oracle.front_emit(u16(out), y16.cpu().numpy(), pos.numpy(), ms, ape.numpy(), main_row.numpy(), isr,
                                 idx_ape.numpy(), idx_row.numpy())
    assert np.array_equal(d["win_y2"].cpu().numpy(), win) and np.array_equal(d["w64"].cpu().numpy(), w64)
    assert np.array_equal(d["main_state"].cpu().numpy(), ms) and np.array_equal(d["idx_state"].cpu().numpy(), isr)
    assert (ms == 7.0).sum() > 0                                   # untouched entries keep their fill
