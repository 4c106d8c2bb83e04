"""GPU parity of the indexer's FP4 producers (through the C ABI): the indexer-q post (RoPE, Hadamard-128, MXFP4)
and the FP4 form of the indexer compressor, against the CPU oracle and the fixtures made with the reference's torch
twins, and the whole FP4 path - producers into the MXFP4 logits - against the oracle's logits.
The query tail is correctly rounded operations only: bytes identical to the oracle's.  The compressor contains
expf: >= 99.5 % identical bytes.  Against the twins the bar is the reference's own (cosine > 0.999, scales equal in
> 98 % of the blocks): they multiply by the Hadamard matrix and round e2m1 ties down."""
import numpy as np
import pytest
import torch

import oracle
from conftest import load_golden

pytestmark = pytest.mark.gpu


def cu(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def from_u16(a):
    return torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).cuda().view(torch.bfloat16)


def cosine(a, b):
    a, b = a.astype(np.float64).ravel(), b.astype(np.float64).ravel()
    return float(a @ b / np.sqrt((a @ a) * (b @ b)))


def rope_tables(max_pos):
    ang = np.outer(np.arange(max_pos, dtype=np.float32), (1.0 / (10000.0 ** (np.arange(32) / 32.0))).astype(np.float32))
    return np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)


def test_index_q_post_fp4_golden_and_oracle(wuda):
    g = load_golden("index_q_post_fp4.npz")
    iq = from_u16(g["iq"])
    q4, sf = wuda.idx_postprocess(iq, cu(g["q_pos"]), cu(g["cos"]), cu(g["sin"]))
    torch.cuda.synchronize()
    got_q, got_sf = q4.view(torch.uint8).cpu().numpy(), sf.cpu().numpy().view(np.uint32)
    oq, osf = oracle.index_q_post_fp4(g["iq"], g["q_pos"], g["cos"], g["sin"])
    assert np.array_equal(got_sf, osf)
    assert np.array_equal(got_q, oq)                                  # correctly rounded operations only: exact
    tokens, heads = got_sf.shape
    deq = oracle.dequant_mxfp4(got_q.reshape(-1, 64), got_sf.reshape(-1)).reshape(tokens, heads, 128)
    scale = np.ldexp(1.0, got_sf.view(np.uint8).reshape(tokens, heads, 4).astype(np.int32) - 127)
    assert cosine(deq, g["deq"]) > 0.999 and np.mean(scale == g["sf"]) > 0.98      # the reference test's own bar
    # strided input: a slice of the projection output
    wide = torch.zeros(iq.size(0), 4096 + heads * 128, dtype=torch.bfloat16, device="cuda")
    wide[:, :heads * 128] = iq.flatten(1)
    q2, s2 = wuda.idx_postprocess(wide[:, :heads * 128].unflatten(-1, (heads, 128)), cu(g["q_pos"]), cu(g["cos"]),
                                  cu(g["sin"]))
    torch.cuda.synchronize()
    assert torch.equal(q2, q4) and torch.equal(s2, sf)


@pytest.mark.parametrize("tokens,heads,seed", [(1, 64, 1), (64, 64, 2), (3, 5, 3), (128, 64, 4)])
def test_index_q_post_fp4_against_oracle(wuda, tokens, heads, seed):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((tokens, heads, 128)) * np.exp(rng.standard_normal((tokens, heads, 1)) * 3)
    x[0, 0, :32] = 0.0                                                # a block of zeros inside a live head
    iq = torch.from_numpy(x).bfloat16().cuda()
    cos, sin = rope_tables(512)
    q_pos = rng.integers(-2, 520, size=tokens).astype(np.int32)      # out-of-range positions are clamped
    q4, sf = wuda.idx_postprocess(iq, cu(q_pos), cu(cos), cu(sin))
    torch.cuda.synchronize()
    oq, osf = oracle.index_q_post_fp4(iq.cpu().view(torch.int16).numpy().view(np.uint16), q_pos, cos, sin)
    assert np.array_equal(sf.cpu().numpy().view(np.uint32), osf)
    assert np.array_equal(q4.view(torch.uint8).cpu().numpy(), oq)


def test_indexer_compressor_fp4_golden_and_oracle(wuda):
    g = load_golden("indexer_compressor_fp4.npz")
    rows = len(g["pos"])
    q4 = torch.full((rows, 64), 0xAB, dtype=torch.uint8, device="cuda")
    s4 = torch.full((rows, 4), 0xAB, dtype=torch.uint8, device="cuda")
    status = wuda.device_status_word()
    wuda.cache_writers_fp4(cu(g["pos"]), cu(g["cos"]), cu(g["sin"]), status_word=status,
                           indexer=dict(state=cu(g["state"]), state_row=cu(g["state_row"]), norm_w=cu(g["norm_w"]),
                                        q8=q4, s8=s4))
    torch.cuda.synchronize()
    assert status.item() == 0
    m = g["compress"]
    q, s = q4.cpu().numpy(), s4.cpu().numpy()
    assert (q[~m] == 0xAB).all() and (s[~m] == 0xAB).all()
    oq, os_ = oracle.indexer_compressor_fp4(g["state"], g["state_row"], g["pos"], g["norm_w"], g["cos"], g["sin"])
    assert np.mean(q == oq) >= 0.995 and np.mean(s == os_) >= 0.97
    words = s[m].astype(np.uint32) @ (1 << (8 * np.arange(4, dtype=np.uint32)))
    deq = oracle.dequant_mxfp4(q[m], words.astype(np.uint32))
    assert cosine(deq, g["deq"][m]) > 0.999 and np.mean(s[m] == g["s4"][m]) >= 0.95


@pytest.mark.parametrize("rows,ring,epb,pad", [(7, 8, 4, 128), (64, 8, 64, 0), (128, 16, 32, 16)])
def test_indexer_compressor_fp4_pool_against_oracle(wuda, rows, ring, epb, pad):
    rng = np.random.default_rng(rows)
    pos = rng.integers(3, 4000, size=rows).astype(np.int64)
    pos[: (rows + 1) // 2] |= 3
    cos, sin = rope_tables(4096)
    state = rng.normal(size=(rows, ring, 512)).astype(np.float32)
    state_row = (np.arange(rows) * ring + pos % ring).astype(np.int64)
    norm = (rng.random(128) + 0.5).astype(np.float32)
    pages = (rows + epb - 1) // epb + 2
    pool = np.full((pages, epb * 68 + pad), 0xA5, np.uint8)
    dst = rng.permutation(pages * epb)[:rows].astype(np.int64)
    dst[(pos + 1) % 4 != 0] = -1
    ref_pool = pool.copy()
    oq, os_ = oracle.indexer_compressor_fp4(state, state_row, pos, norm, cos, sin, pool=ref_pool, dst=dst, epb=epb)
    d_pool = cu(pool)
    q4 = torch.full((rows, 64), 0xAB, dtype=torch.uint8, device="cuda")
    s4 = torch.full((rows, 4), 0xAB, dtype=torch.uint8, device="cuda")
    status = wuda.device_status_word()
    wuda.cache_writers_fp4(cu(pos), cu(cos), cu(sin), status_word=status,
                           indexer=dict(state=cu(state), state_row=cu(state_row), norm_w=cu(norm), ring_entries=ring,
                                        pool=d_pool, dst=cu(dst), entries_per_block=epb, q8=q4, s8=s4))
    torch.cuda.synchronize()
    assert status.item() == 0
    got_pool = d_pool.cpu().numpy()
    changed = ref_pool != pool
    assert not np.any((got_pool != pool) & ~changed)                 # nothing outside the written records moves
    assert np.mean(got_pool == ref_pool) >= 1 - 5e-3
    assert np.mean(q4.cpu().numpy() == oq) >= 0.995 and np.mean(s4.cpu().numpy() == os_) >= 0.97


def test_fp4_producers_feed_the_fp4_logits(wuda):
    """What the FP4 compressor writes and the FP4 indexer-q post emits is what wuda_mqa_logits_fp4 reads: compress
    4 * T tokens of one request into T pool entries, transform a query, score."""
    rng = np.random.default_rng(78)
    tokens, epb, ring = 300, 64, 8
    pos = (np.arange(tokens) * 4 + 3).astype(np.int64)
    cos, sin = rope_tables(2048)
    state = rng.normal(size=(tokens, ring, 512)).astype(np.float32)
    state_row = (np.arange(tokens) * ring + pos % ring).astype(np.int64)
    norm = (rng.random(128) + 0.5).astype(np.float32)
    pages = 6
    table = rng.permutation(pages).astype(np.int32)
    dst = table[np.arange(tokens) // epb].astype(np.int64) * epb + np.arange(tokens) % epb
    pool = torch.zeros((pages, epb * 68), dtype=torch.uint8, device="cuda")
    wuda.cache_writers_fp4(cu(pos), cu(cos), cu(sin),
                           indexer=dict(state=cu(state), state_row=cu(state_row), norm_w=cu(norm), pool=pool, dst=cu(dst),
                                        entries_per_block=epb))
    iq = (torch.randn(1, 64, 128, device="cuda") * 2).bfloat16()
    q4, sf = wuda.idx_postprocess(iq, torch.tensor([1199], dtype=torch.int32, device="cuda"), cu(cos), cu(sin))
    w = torch.randn(1, 64, device="cuda") / 8
    ctx = torch.tensor([tokens], dtype=torch.int32, device="cuda")
    bt = cu(table[None, :])
    logits = torch.full((1, 512), float("-inf"), device="cuda")
    status = wuda.device_status_word()
    status.zero_()
    wuda.mqa_logits_fp4_decode_out(q4, sf, pool, w, ctx, bt, logits, 384, epb, status_word=status)
    torch.cuda.synchronize()
    assert status.item() == 0
    ref = oracle.mqa_logits_fp4(q4.view(torch.uint8).cpu().numpy(), sf.cpu().numpy(), pool.cpu().numpy(), w.cpu().numpy(),
                                ctx.cpu().numpy(), bt.cpu().numpy(), epb, 512)
    got = logits.cpu().numpy()
    v = np.isfinite(ref)
    assert np.array_equal(np.isfinite(got), v) and v.sum() == tokens
    rms = np.sqrt(np.mean(ref[v].astype(np.float64) ** 2))
    assert np.all(np.abs(got[v] - ref[v]) <= 1e-4 * np.abs(ref[v]) + 1e-5 * rms)
