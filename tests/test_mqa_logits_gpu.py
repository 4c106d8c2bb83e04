"""GPU parity of the paged FP8 MQA-logits kernel (through the C ABI) against the CPU
oracle and the golden fixtures."""
import numpy as np
import pytest
import torch

import oracle
from conftest import assert_close_logits, load_golden
from wuda_b200 import workloads

pytestmark = pytest.mark.gpu

SENTINEL = -12345.0


def run_kernel(wuda, case, rows_extra=0):
    d = workloads.to_device(case)
    rows = case["batch"] * case["next_n"]
    logits = torch.full((rows + rows_extra, case["logits_stride"]), SENTINEL, dtype=torch.float32, device="cuda")
    status = wuda.device_status_word()
    wuda.mqa_logits_fp8_decode_out(d["q"], d["kv_pages"], d["weights"], d["context_lens"], d["block_table"],
                                   None, logits, case["epb"], next_n=case["next_n"], status_word=status)
    torch.cuda.synchronize()
    return logits.cpu().numpy(), int(status.item())


def check_case(wuda, case, ref=None):
    got, status = run_kernel(wuda, case, rows_extra=1)
    assert status == 0, "device status %d" % status
    rows = case["batch"] * case["next_n"]
    if ref is None:
        ref = oracle.mqa_logits_fp8(case["q"], case["kv_pages"], case["weights"], case["context_lens"],
                                    case["block_table"], case["next_n"], case["epb"], case["logits_stride"])
    cols = np.arange(case["logits_stride"])[None, :]
    valid = cols < case["context_lens"].reshape(-1)[:, None]
    # nothing outside t < context is written, including the spare row
    assert np.all(got[:rows][~valid] == SENTINEL)
    assert np.all(got[rows:] == SENTINEL)
    return assert_close_logits(got[:rows], ref, valid, rtol=1e-2, atol_frac=1e-4)


@pytest.mark.parametrize("name", ["mqa_logits_fp8_n1.npz", "mqa_logits_fp8_n2_epb32.npz"])
def test_golden_fixture(wuda, name):
    g = load_golden(name)
    case = dict(g, batch=g["context_lens"].shape[0], next_n=int(g["next_n"]), epb=int(g["epb"]),
                logits_stride=int(g["logits_stride"]))
    check_case(wuda, case, ref=g["expected"])


def test_config0_batch4_ctx_up_to_4096(wuda):
    check_case(wuda, workloads.make_mqa_case(4, 1, 1, 4096, epb=64, seed=0xB200))


@pytest.mark.parametrize("ctx", [1, 63, 64, 65, 127, 128, 129, 255, 256, 257, 1000])
def test_single_request_edge_lengths(wuda, ctx):
    check_case(wuda, workloads.make_mqa_case(1, 1, 0, 0, ctx=[ctx], seed=ctx))


@pytest.mark.parametrize("epb,pad", [(32, 128), (64, 0), (64, 64), (128, 256)])
@pytest.mark.parametrize("next_n", [1, 2])
def test_page_geometries_and_next_n(wuda, epb, pad, next_n):
    check_case(wuda, workloads.make_mqa_case(5, next_n, 2, 1500, epb=epb, page_pad=pad, seed=epb + pad + next_n))


def test_ragged_batch_with_empty_requests(wuda):
    ctx = [0, 300, 0, 0, 1, 129, 0, 2047, 64, 0]
    check_case(wuda, workloads.make_mqa_case(len(ctx), 1, 0, 0, ctx=ctx, seed=7))
    # next_n = 2 with a request whose first row is empty (ctx 1 -> rows see 0 and 1 tokens)
    check_case(wuda, workloads.make_mqa_case(4, 2, 0, 0, ctx=[1, 2, 500, 0], seed=8))


def test_many_short_requests_more_than_sms(wuda):
    rng = np.random.default_rng(3)
    check_case(wuda, workloads.make_mqa_case(400, 1, 0, 0, ctx=rng.integers(1, 300, 400), seed=9))


def test_long_request_spanning_many_ctas(wuda):
    check_case(wuda, workloads.make_mqa_case(2, 2, 0, 0, ctx=[70000, 33333], seed=10))


def test_paging_is_bit_exact(wuda):
    """Keys and scales are chosen so that every logit is an exactly representable
    function of (physical page, slot): any wrong page, slot or row shows as a bit
    difference."""
    case = workloads.make_mqa_case(6, 2, 1, 3000, epb=64, seed=21)
    nb, epb = case["num_blocks"], 64
    vals = oracle.e4m3_decode(np.arange(0x30, 0x70, dtype=np.uint8))          # 64 distinct positive values
    kv = case["kv_pages"]
    kv[:, :epb * 128] = 0
    codes = (0x30 + (np.arange(nb) % 64)).astype(np.uint8)
    kv[:, 0:epb * 128:128] = codes[:, None]                                   # dim 0 of every token
    scales = (np.arange(nb)[:, None] * 128 + np.arange(epb)[None, :] + 1).astype(np.float32)
    kv[:, epb * 128:epb * 132] = scales.view(np.uint8).reshape(nb, epb * 4)
    q = np.zeros_like(case["q"])
    q[:, 0, 0] = 0x38                                                          # 1.0 in e4m3, head 0, dim 0
    case["q"] = q
    w = np.zeros_like(case["weights"])
    w[:, 0] = 1.0
    w[1::2, 0] = 2.0
    case["weights"] = w
    got, status = run_kernel(wuda, case)
    assert status == 0
    ref = oracle.mqa_logits_fp8(case["q"], kv, w, case["context_lens"], case["block_table"], 2, epb,
                                case["logits_stride"], fill=SENTINEL)
    assert np.array_equal(got.view(np.uint32), ref.view(np.uint32))
    del vals


def test_out_of_pool_page_is_reported_not_faulted(wuda):
    case = workloads.make_mqa_case(2, 1, 0, 0, ctx=[200, 300], seed=5)
    case["block_table"][1, 2] = case["num_blocks"] + 7
    got, status = run_kernel(wuda, case)
    assert status == 110
    # request 0 is unaffected
    ref = oracle.mqa_logits_fp8(case["q"][:1], case["kv_pages"], case["weights"][:1], case["context_lens"][:1],
                                case["block_table"][:1], 1, 64, case["logits_stride"])
    assert_close_logits(got[:1], ref, np.isfinite(ref))


def test_context_beyond_the_logits_row_is_cut_and_reported(wuda):
    """A context length larger than logits_stride (or negative) must neither write past the row nor
    corrupt the tile count: the row is cut at the stride, the cut is reported as code 111, the guard
    rows behind the logits stay untouched and the other requests are unaffected."""
    case = workloads.make_mqa_case(3, 1, 0, 0, ctx=[700, 300, 500], seed=41)
    stride = case["logits_stride"]
    assert stride == 768
    d = workloads.to_device(case)
    lens = d["context_lens"].clone()
    lens[0] = stride + 1000           # claims more tokens than its row of the logits holds
    lens[1] = -5000                   # negative: counts as empty
    logits = torch.full((3 + 2, stride), SENTINEL, dtype=torch.float32, device="cuda")
    status = wuda.device_status_word()
    wuda.mqa_logits_fp8_decode_out(d["q"], d["kv_pages"], d["weights"], lens, d["block_table"], None, logits,
                                   case["epb"], status_word=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 111
    got = logits.cpu().numpy()
    ref = oracle.mqa_logits_fp8(case["q"], case["kv_pages"], case["weights"], case["context_lens"],
                                case["block_table"], 1, 64, stride)
    assert np.all(got[3:] == SENTINEL) and np.all(got[1] == SENTINEL)       # guard rows, the "negative" request
    valid = np.isfinite(ref)
    valid[1] = False
    assert_close_logits(got[:3], ref, valid)                               # rows 0 (its real 700 tokens) and 2
    assert np.all(got[2][500:] == SENTINEL)


def test_reference_call_shape_allocating_form(wuda):
    case = workloads.make_mqa_case(3, 2, 100, 900, seed=31)
    d = workloads.to_device(case)
    max_ctx = int(case["ctx"].max())
    out = wuda.fp8_paged_mqa_logits(d["q"].view(3, 2, 64, 128), d["kv_pages"], d["weights"], d["context_lens"],
                                    d["block_table"], None, max_ctx)
    torch.cuda.synchronize()
    ref = oracle.mqa_logits_fp8(case["q"], case["kv_pages"], case["weights"], case["context_lens"],
                                case["block_table"], 2, 64, case["logits_stride"])[:, :max_ctx]
    got = out.cpu().numpy()
    assert np.array_equal(np.isfinite(got), np.isfinite(ref))
    assert_close_logits(got, ref, np.isfinite(ref))


def test_shim_rejects_bad_arguments_like_the_reference(wuda):
    case = workloads.make_mqa_case(2, 1, 10, 100, seed=1)
    d = workloads.to_device(case)
    logits = torch.zeros(2, 256, device="cuda")
    with pytest.raises(RuntimeError):
        wuda.mqa_logits_fp8_decode_out(d["q"].view(torch.uint8), d["kv_pages"], d["weights"], d["context_lens"],
                                       d["block_table"], None, logits)
    with pytest.raises(RuntimeError):
        wuda.mqa_logits_fp8_decode_out(d["q"], d["kv_pages"], d["weights"][:, :32].contiguous(),
                                       d["context_lens"], d["block_table"], None, logits)
    with pytest.raises(RuntimeError):
        wuda.mqa_logits_fp8_decode_out(d["q"], d["kv_pages"], d["weights"], d["context_lens"],
                                       d["block_table"], None, logits, 48)


def test_config1_full_size_against_oracle(wuda):
    """batch 64 x next_n 2, contexts 16384..65536 (the benchmark workload), every
    valid logit checked against the CPU oracle."""
    case = workloads.make_mqa_case(64, 2, 16384, 65536, epb=64, seed=0xB201)
    check_case(wuda, case)
