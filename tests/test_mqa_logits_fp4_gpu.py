"""GPU parity of the MXFP4 paged MQA logits (through the C ABI) against the CPU oracle (the reference's torch
twin over dequantised operands, sums in double) and the fixture made with the reference's own quantiser,
page builder and twin.  Floating point: products of e2m1 values and power-of-two scales are exact and the
tensor core sums them in fp32, so the tolerance only covers the order of the fp32 additions:
|got - ref| <= 1e-4 |ref| + 1e-5 rms(ref)."""
import numpy as np
import pytest
import torch

import oracle
from conftest import load_golden

pytestmark = pytest.mark.gpu

E2M1_BOUNDS = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0])


def quantize_mxfp4(x):
    """x float [rows, 128] -> (packed uint8 [rows, 64], scale words uint32 [rows]): one power-of-two scale per 32
    values (amax / 6 rounded up, at least 1e-4 before rounding), nearest e2m1 code, ties to the smaller magnitude."""
    rows = x.shape[0]
    v = x.reshape(rows, 4, 32).astype(np.float32)
    amax = np.maximum(np.abs(v).max(-1), 1e-4) / 6.0
    m, e = np.frexp(amax)                        # amax = m * 2^e, m in [0.5, 1)
    exp = np.where(m == 0.5, e - 1, e)           # ceil(log2(amax))
    scaled = v / np.ldexp(1.0, exp)[..., None]
    code = np.searchsorted(E2M1_BOUNDS, np.minimum(np.abs(scaled), 6.0), side="left").astype(np.uint8)
    code |= ((scaled < 0) & (code != 0)).astype(np.uint8) << 3
    code = code.reshape(rows, 64, 2)
    packed = (code[..., 0] | (code[..., 1] << 4)).astype(np.uint8)
    sf = (exp + 127).astype(np.uint32)
    words = sf[:, 0] | (sf[:, 1] << 8) | (sf[:, 2] << 16) | (sf[:, 3] << 24)
    return packed, words.astype(np.uint32)


def build_case(rng, batch, contexts, epb, pad=0, spread=1.0):
    max_ctx = max(max(contexts), 1)
    pages_per = -(-max_ctx // epb)
    num_blocks = batch * pages_per + 3
    stride = epb * 68 + pad
    pages = rng.integers(0, 256, (num_blocks, stride)).astype(np.uint8)          # unused entries hold garbage
    table = np.full((batch, pages_per + 2), -7, np.int32)                        # unused slots hold an invalid page
    perm = rng.permutation(num_blocks)
    q = rng.standard_normal((batch, 64, 128)) * spread
    q_p, q_w = quantize_mxfp4(q.reshape(-1, 128))
    for b in range(batch):
        table[b, :pages_per] = perm[b * pages_per:(b + 1) * pages_per]
        n = contexts[b]
        scale = np.exp(rng.standard_normal((n, 1)) * spread)                     # rows of very different magnitude
        k_p, k_w = quantize_mxfp4(rng.standard_normal((n, 128)) * scale)
        t = np.arange(n)
        pg, off = table[b, t // epb], t % epb
        pages[pg[:, None], (off * 64)[:, None] + np.arange(64)[None, :]] = k_p
        pages[pg[:, None], (epb * 64 + off * 4)[:, None] + np.arange(4)[None, :]] = k_w.view(np.uint8).reshape(n, 4)
    weights = rng.standard_normal((batch, 64)).astype(np.float32)
    return dict(q=q_p.reshape(batch, 64, 64), q_sf=q_w.reshape(batch, 64).view(np.int32), pages=pages, weights=weights,
                context_lens=np.asarray(contexts, np.int32), block_table=table, epb=epb)


def run(wuda, c, columns):
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    logits = torch.full((len(c["context_lens"]), columns), float("-inf"), dtype=torch.float32, device="cuda")
    status = wuda.device_status_word()
    status.zero_()
    out = wuda.mqa_logits_fp4_decode_out(t(c["q"]).view(torch.int8), t(c["q_sf"]), t(c["pages"]), t(c["weights"]),
                                         t(c["context_lens"]), t(c["block_table"]), logits, columns, int(c["epb"]),
                                         status_word=status)
    torch.cuda.synchronize()
    assert out is logits
    return logits.cpu().numpy(), int(status.item())


def check(got, ref):
    valid = np.isfinite(ref)
    assert np.array_equal(np.isfinite(got), valid)          # nothing at or beyond a request's context is written
    assert np.all(got[~valid] == -np.inf)
    rms = np.sqrt(np.mean(ref[valid].astype(np.float64) ** 2)) if valid.any() else 0.0
    assert np.all(np.abs(got[valid] - ref[valid]) <= 1e-4 * np.abs(ref[valid]) + 1e-5 * rms)


def test_golden(wuda):
    g = load_golden("mqa_logits_fp4.npz")
    got, status = run(wuda, g, g["logits"].shape[1])
    assert status == 0
    check(got, g["logits"])


@pytest.mark.parametrize("batch,contexts,epb,pad", [
    (4, [1000, 37, 128, 1], 64, 0),          # ragged: several tiles, less than a tile, exactly one, one token
    (2, [700, 0], 32, 16),                   # a request without context; 32-entry pages with padded stride
    (3, [513, 129, 640], 128, 0),            # 128-entry pages, tile boundaries + 1
    (1, [4096], 64, 48),
    (2, [1025, 300], 256, 0),                # 256-entry pages: one page per item of the paged kernel
    (3, [257, 256, 255], 64, 0),             # around the paged kernel's item of 256 tokens
    (2, [333, 50], 16, 0),                   # page sizes the paged kernel does not take: the gather kernel
    (2, [500, 97], 48, 16),
])
def test_against_oracle(wuda, batch, contexts, epb, pad):
    rng = np.random.default_rng(batch * 101 + epb)
    c = build_case(rng, batch, contexts, epb, pad, spread=2.0)
    columns = -(-max(contexts) // 128) * 128 + 64
    got, status = run(wuda, c, columns)
    assert status == 0
    check(got, oracle.mqa_logits_fp4(c["q"], c["q_sf"], c["pages"], c["weights"], c["context_lens"], c["block_table"],
                                     epb, columns))


def test_many_items_per_sm(wuda):
    """Half a million tokens: every CTA of the persistent grid walks more items than it has key stages, crosses
    requests inside its range, and the ring's phases flip."""
    rng = np.random.default_rng(77)
    contexts = [40000, 33333, 50001, 256, 47000, 1, 65536, 30000, 52000, 44444, 61000, 38000, 0, 45678]
    c = build_case(rng, len(contexts), contexts, 64)
    columns = 65536
    got, status = run(wuda, c, columns)
    assert status == 0
    check(got, oracle.mqa_logits_fp4(c["q"], c["q_sf"], c["pages"], c["weights"], c["context_lens"], c["block_table"],
                                     64, columns))


def test_context_beyond_the_logits_row_is_cut_and_reported(wuda):
    rng = np.random.default_rng(10)
    c = build_case(rng, 2, [700, 300], 64)
    ref = oracle.mqa_logits_fp4(c["q"], c["q_sf"], c["pages"], c["weights"], c["context_lens"], c["block_table"], 64,
                                768)[:, :512]            # the first request's 700 tokens are cut to the 512 of a logits row
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    logits = torch.full((3, 512), float("-inf"), dtype=torch.float32, device="cuda")   # a guard row behind
    status = wuda.device_status_word()
    status.zero_()
    wuda.mqa_logits_fp4_decode_out(t(c["q"]).view(torch.int8), t(c["q_sf"]), t(c["pages"]), t(c["weights"]),
                                   t(c["context_lens"]), t(c["block_table"]), logits[:2], 512, 64, status_word=status)
    torch.cuda.synchronize()
    got = logits.cpu().numpy()
    assert int(status.item()) == 111
    assert np.all(got[2] == -np.inf)                      # nothing behind the last row
    check(got[:2], ref)


def test_reference_call_form_fills_the_tail(wuda):
    rng = np.random.default_rng(8)
    c = build_case(rng, 2, [300, 70], 64)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    got = wuda.mqa_logits_fp4_decode(t(c["q"]).view(torch.int8), t(c["q_sf"]), t(c["pages"]), t(c["weights"]),
                                     t(c["context_lens"]), t(c["block_table"]), 320, torch.float32,
                                     kv_entries_per_block=64, kv_block_stride_bytes=c["pages"].shape[1])
    torch.cuda.synchronize()
    assert tuple(got.shape) == (2, 320)
    check(got.cpu().numpy(), oracle.mqa_logits_fp4(c["q"], c["q_sf"], c["pages"], c["weights"], c["context_lens"],
                                                   c["block_table"], 64, 320))


def test_bad_page_index_is_reported(wuda):
    rng = np.random.default_rng(9)
    c = build_case(rng, 1, [200], 64)
    c["block_table"][0, 1] = 10 ** 6
    got, status = run(wuda, c, 256)
    assert status == 110 and np.all(np.isfinite(got[0, :200]))
