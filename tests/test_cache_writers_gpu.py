"""GPU parity of the cache writers (indexer compressor, MAIN compressor, window KV; one launch,
through the C ABI) against the CPU oracle and the fixtures made with the reference's torch twins.
The only operation that is not correctly rounded on both sides is expf, so results are compared
byte for byte with a small allowance: >= 99.5 % identical bytes, scales identical or one
power of two / 2^-7 apart, bf16 values within one step."""
import numpy as np
import pytest
import torch

import oracle
from conftest import load_golden

pytestmark = pytest.mark.gpu


def cu(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a))
    return (t if dtype is None else t.to(dtype)).cuda()


def u16(t):
    return t.cpu().view(torch.int16).numpy().view(np.uint16)


def rope_tables(max_pos):
    ang = np.outer(np.arange(max_pos, dtype=np.float32), (1.0 / (10000.0 ** (np.arange(32) / 32.0))).astype(np.float32))
    return np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)


def close_bytes(got, ref, frac=0.995):
    assert got.shape == ref.shape
    assert np.mean(got == ref) >= frac, "only %.4f identical" % np.mean(got == ref)


def close_bf16(got, ref):
    d = np.abs(got.astype(np.int32) - ref.astype(np.int32))
    assert d.max() <= 1 and np.mean(d == 0) >= 0.995


def test_indexer_compressor_golden(wuda):
    g = load_golden("indexer_compressor_fp8.npz")
    rows = len(g["pos"])
    q8 = torch.full((rows, 128), 0xAB, dtype=torch.uint8, device="cuda")
    s8 = torch.full((rows,), -1.0, device="cuda")
    status = wuda.device_status_word()
    wuda.cache_writers_fp8(cu(g["pos"]), cu(g["cos"]), cu(g["sin"]), status_word=status,
                           indexer=dict(state=cu(g["state"]), state_row=cu(g["state_row"]), norm_w=cu(g["norm_w"]),
                                        q8=q8, s8=s8))
    torch.cuda.synchronize()
    assert status.item() == 0
    m = g["compress"]
    q, s = q8.cpu().numpy(), s8.cpu().numpy()
    assert (q[~m] == 0xAB).all() and (s[~m] == -1).all()
    close_bytes(q[m], g["q8"][m])
    assert np.allclose(s[m], g["scale"][m], rtol=2 ** -7)
    oq, os_ = oracle.indexer_compressor_fp8(g["state"], g["state_row"], g["pos"], g["norm_w"], g["cos"], g["sin"])
    close_bytes(q, oq, 0.999)
    assert np.mean(s == os_) >= 0.9


def test_main_compressor_golden(wuda):
    """The MAIN compressor against the fixture made from the reference's inline twin of the row
    (test/test_mqa_logits_fp4.py:772-791): state read-only, rows that do not compress untouched, scales equal,
    e4m3 codes those of the twin's values, rotary tail within one bf16 step.  The twin's own GPU gate is far
    looser (scale 1e-2, values 0.15, rope 0.05) because its kernel is built with fast-math."""
    g = load_golden("main_compressor_fp8.npz")
    rows = len(g["pos"])
    q8 = torch.full((rows, 448), 0xAB, dtype=torch.uint8, device="cuda")
    s8 = torch.full((rows, 7), -1.0, device="cuda")
    rope = torch.zeros((rows, 64), dtype=torch.bfloat16, device="cuda")
    state = cu(g["state"])
    before = state.clone()
    wuda.mqa_compressor_fp8_standalone(cu(g["pos"]), cu(g["norm_w"]), cu(g["cos"]), cu(g["sin"]), state,
                                       cu(g["state_row"]), 8, q8, s8, rope, 1e-6)
    torch.cuda.synchronize()
    assert torch.equal(state, before)
    m = g["compress"]
    q, s, r = q8.cpu().numpy(), s8.cpu().numpy(), u16(rope)
    assert (q[~m] == 0xAB).all() and (s[~m] == -1).all() and (r[~m] == 0).all()
    assert np.array_equal(s[m], g["scale"][m])
    want = oracle.e4m3_encode((g["values"][m].reshape(-1, 7, 64) / g["scale"][m][:, :, None]).reshape(-1, 448))
    close_bytes(q[m], want)
    close_bf16(r[m], g["rope"][m])


def test_window_kv_golden(wuda):
    g = load_golden("window_kv_fp8.npz")
    rows = len(g["pos"])
    q8 = torch.empty((rows, 448), dtype=torch.uint8, device="cuda")
    s8 = torch.empty((rows, 7), device="cuda")
    rope = torch.empty((rows, 64), dtype=torch.bfloat16, device="cuda")
    wuda.cache_writers_fp8(cu(g["pos"]), cu(g["cos"]), cu(g["sin"]),
                           window=dict(y=cu(g["y"]), norm_w=cu(g["norm_w"]), q8=q8, s8=s8, rope=rope))
    torch.cuda.synchronize()
    # every operation is correctly rounded on both sides and the sum of squares has one order
    oq, os_, orope = oracle.window_kv_fp8(g["y"], g["pos"], g["norm_w"], g["cos"], g["sin"])
    assert np.array_equal(q8.cpu().numpy(), oq)
    assert np.array_equal(s8.cpu().numpy(), os_)
    assert np.array_equal(u16(rope), orope)
    assert np.array_equal(s8.cpu().numpy(), g["s8"])
    close_bytes(q8.cpu().numpy(), g["q8"])
    close_bf16(u16(rope), g["rope"])


def make_step(rows, ring, seed, epb_idx=64, epb_cmp=64, epb_swa=256, pad=0):
    rng = np.random.default_rng(seed)
    pos = rng.integers(3, 4000, size=rows).astype(np.int64)
    pos[: (rows + 1) // 2] |= 3                                   # at least half the rows compress
    cos, sin = rope_tables(4096)
    case = dict(pos=pos, cos=cos, sin=sin, ring=ring)
    case["idx_state"] = rng.normal(size=(rows, ring, 512)).astype(np.float32)
    case["main_state"] = rng.normal(size=(rows, ring, 2048)).astype(np.float32)
    case["state_row"] = (np.arange(rows) * ring + pos % ring).astype(np.int64)
    case["idx_norm"] = (rng.random(128) + 0.5).astype(np.float32)
    case["main_norm"] = (rng.random(512) + 0.5).astype(np.float32)
    case["win_norm"] = (rng.random(512) + 0.5).astype(np.float32)
    case["y"] = (rng.normal(size=(rows, 512)) * rng.choice([0.01, 1, 30], size=(rows, 1))).astype(np.float32)
    for name, epb, rec in (("idx", epb_idx, 132), ("cmp", epb_cmp, 584), ("swa", epb_swa, 584)):
        pages = (rows + epb - 1) // epb + 2
        case[name + "_pool"] = np.full((pages, epb * rec + pad), 0xA5, np.uint8)
        case[name + "_dst"] = rng.permutation(pages * epb)[:rows].astype(np.int64)
        case[name + "_epb"] = epb
    case["idx_dst"][~((pos + 1) % 4 == 0)] = -1
    case["cmp_dst"][~((pos + 1) % 4 == 0)] = -1
    return case


def run_step(wuda, c, status=None):
    rows = len(c["pos"])
    d = dict(idx_pool=cu(c["idx_pool"]), cmp_pool=cu(c["cmp_pool"]), swa_pool=cu(c["swa_pool"]),
             idx_q8=torch.full((rows, 128), 0xAB, dtype=torch.uint8, device="cuda"),
             idx_s8=torch.full((rows,), -1.0, device="cuda"),
             main_q8=torch.full((rows, 448), 0xAB, dtype=torch.uint8, device="cuda"),
             main_s8=torch.full((rows, 7), -1.0, device="cuda"),
             main_rope=torch.zeros((rows, 64), dtype=torch.bfloat16, device="cuda"),
             win_q8=torch.empty((rows, 448), dtype=torch.uint8, device="cuda"),
             win_s8=torch.empty((rows, 7), device="cuda"),
             win_rope=torch.empty((rows, 64), dtype=torch.bfloat16, device="cuda"))
    row = cu(c["state_row"])
    wuda.cache_writers_fp8(
        cu(c["pos"]), cu(c["cos"]), cu(c["sin"]), status_word=status,
        indexer=dict(state=cu(c["idx_state"]), state_row=row, norm_w=cu(c["idx_norm"]), ring_entries=c["ring"],
                     pool=d["idx_pool"], dst=cu(c["idx_dst"]), entries_per_block=c["idx_epb"], q8=d["idx_q8"],
                     s8=d["idx_s8"]),
        main=dict(state=cu(c["main_state"]), state_row=row, norm_w=cu(c["main_norm"]), ring_entries=c["ring"],
                  pool=d["cmp_pool"], dst=cu(c["cmp_dst"]), entries_per_block=c["cmp_epb"], q8=d["main_q8"],
                  s8=d["main_s8"], rope=d["main_rope"]),
        window=dict(y=cu(c["y"]), norm_w=cu(c["win_norm"]), pool=d["swa_pool"], dst=cu(c["swa_dst"]),
                    entries_per_block=c["swa_epb"], q8=d["win_q8"], s8=d["win_s8"], rope=d["win_rope"]))
    torch.cuda.synchronize()
    return d


def oracle_step(c):
    o = {k: c[k].copy() for k in ("idx_pool", "cmp_pool", "swa_pool")}
    o["idx_q8"], o["idx_s8"] = oracle.indexer_compressor_fp8(
        c["idx_state"], c["state_row"], c["pos"], c["idx_norm"], c["cos"], c["sin"], pool=o["idx_pool"],
        dst=c["idx_dst"], epb=c["idx_epb"])
    o["main_q8"], o["main_s8"], o["main_rope"] = oracle.main_compressor_fp8(
        c["main_state"], c["state_row"], c["pos"], c["main_norm"], c["cos"], c["sin"], pool=o["cmp_pool"],
        dst=c["cmp_dst"], epb=c["cmp_epb"])
    o["win_q8"], o["win_s8"], o["win_rope"] = oracle.window_kv_fp8(
        c["y"], c["pos"], c["win_norm"], c["cos"], c["sin"], pool=o["swa_pool"], dst=c["swa_dst"], epb=c["swa_epb"])
    return o


@pytest.mark.parametrize("rows,ring,epbs,pad", [(1, 8, (64, 64, 256), 0), (7, 8, (4, 4, 8), 128),
                                                (64, 8, (64, 64, 256), 0), (128, 16, (16, 32, 64), 16),
                                                (37, 11, (64, 64, 256), 64)])
def test_all_three_writers_against_oracle(wuda, rows, ring, epbs, pad):
    c = make_step(rows, ring, rows * 31 + ring, *epbs, pad=pad)
    status = wuda.device_status_word()
    d = run_step(wuda, c, status)
    assert status.item() == 0
    o = oracle_step(c)
    m = (c["pos"] + 1) % 4 == 0
    for key in ("idx_q8", "main_q8"):
        got = d[key].cpu().numpy()
        assert (got[~m] == 0xAB).all()                                  # rows that do not compress: untouched
        close_bytes(got[m], o[key][m], 0.999)
    assert (d["idx_s8"].cpu().numpy()[~m] == -1).all() and (d["main_s8"].cpu().numpy()[~m] == -1).all()
    assert np.allclose(d["idx_s8"].cpu().numpy()[m], o["idx_s8"][m], rtol=2 ** -7)
    assert np.mean(d["main_s8"].cpu().numpy()[m] == o["main_s8"][m]) >= 0.99
    close_bf16(u16(d["main_rope"])[m], o["main_rope"][m])
    # the window writer has no transcendental: exact
    assert np.array_equal(d["win_q8"].cpu().numpy(), o["win_q8"])
    assert np.array_equal(d["win_s8"].cpu().numpy(), o["win_s8"])
    assert np.array_equal(u16(d["win_rope"]), o["win_rope"])
    assert np.array_equal(d["swa_pool"].cpu().numpy(), o["swa_pool"])   # records and canaries, byte for byte
    # pools: nothing outside the records written this step changes; inside them the bytes agree
    for key in ("idx_pool", "cmp_pool"):
        got, ref, rec = d[key].cpu().numpy(), o[key], _record_mask(c, key)
        assert not np.any((got != c[key]) & ~rec)
        assert np.mean(got[rec] == ref[rec]) >= 0.995


def _record_mask(c, key):
    """Bytes that belong to a record some row writes this step."""
    name = key.split("_")[0]
    pool = c[key]
    mask = np.zeros(pool.shape, bool)
    epb, rec, sc = c[name + "_epb"], (128, 4) if name == "idx" else (576, 7), None
    for dst in c[name + "_dst"]:
        if dst < 0:
            continue
        page, off = dst // epb, dst % epb
        mask[page, off * rec[0]:(off + 1) * rec[0]] = True
        stride = 4 if name == "idx" else 8
        mask[page, epb * rec[0] + off * stride: epb * rec[0] + off * stride + rec[1]] = True
    return mask


def test_compressed_indexer_entries_feed_the_logits_kernel(wuda):
    """What the indexer compressor writes is what wuda_mqa_logits_fp8 reads: compress 4*T tokens of one
    request into T pool entries, then score them."""
    rng = np.random.default_rng(77)
    tokens, epb = 96, 64
    c = make_step(tokens, 8, 5)
    c["pos"] = (np.arange(tokens) * 4 + 3).astype(np.int64)
    c["state_row"] = (np.arange(tokens) * 8 + c["pos"] % 8).astype(np.int64)
    pages = 4
    table = rng.permutation(pages).astype(np.int32)
    dst = (table[np.arange(tokens) // epb].astype(np.int64) * epb + np.arange(tokens) % epb)
    pool = torch.zeros((pages, epb * 132), dtype=torch.uint8, device="cuda")
    wuda.cache_writers_fp8(cu(c["pos"]), cu(c["cos"]), cu(c["sin"]),
                           indexer=dict(state=cu(c["idx_state"]), state_row=cu(c["state_row"]),
                                        norm_w=cu(c["idx_norm"]), pool=pool, dst=cu(dst), entries_per_block=epb))
    q = torch.randn(1, 64, 128, device="cuda").clamp(-448, 448).to(torch.float8_e4m3fn)
    w = torch.randn(1, 64, device="cuda") / 8
    ctx = torch.tensor([[tokens]], dtype=torch.int32, device="cuda")
    bt = cu(table[None, :])
    logits = torch.full((1, 256), float("-inf"), device="cuda")
    status = wuda.device_status_word()
    wuda.mqa_logits_fp8_decode_out(q, pool, w, ctx, bt, None, logits, epb, status_word=status)
    torch.cuda.synchronize()
    assert status.item() == 0
    ref = oracle.mqa_logits_fp8(q.view(torch.uint8).cpu().numpy(), pool.cpu().numpy(), w.cpu().numpy(),
                                ctx.cpu().numpy(), bt.cpu().numpy(), 1, epb, 256)
    got = logits.cpu().numpy()
    assert np.array_equal(np.isfinite(got), np.isfinite(ref)) and np.isfinite(got).sum() == tokens
    v = np.isfinite(ref)
    assert np.allclose(got[v], ref[v], rtol=1e-2, atol=1e-3 * np.abs(ref[v]).max())


def test_reports_bad_destination_and_state_row(wuda):
    c = make_step(8, 8, 3)
    c["pos"][:] = 7
    c["state_row"] = (np.arange(8) * 8 + 7).astype(np.int64)
    c["idx_dst"] = np.arange(8).astype(np.int64)
    c["cmp_dst"] = np.arange(8).astype(np.int64)
    c["idx_dst"][2] = c["idx_pool"].shape[0] * c["idx_epb"] + 5           # beyond the pool
    status = wuda.device_status_word()
    d = run_step(wuda, c, status)
    assert status.item() == 141
    assert (d["idx_q8"].cpu().numpy()[2] != 0xAB).any()                   # compact output still written
    c["idx_dst"][2] = 2
    c["state_row"][5] = 8 * 8 + 1                                         # beyond the state rings
    status.zero_()
    d = run_step(wuda, c, status)
    assert status.item() == 142
    assert (d["idx_q8"].cpu().numpy()[5] == 0xAB).all() and (d["main_q8"].cpu().numpy()[5] == 0xAB).all()


def test_standalone_main_compressor_signature(wuda):
    c = make_step(8, 8, 11)
    rows = 8
    q8 = torch.full((rows, 448), 0xAB, dtype=torch.uint8, device="cuda")
    s8 = torch.full((rows, 7), -1.0, device="cuda")
    rope = torch.zeros((rows, 64), dtype=torch.bfloat16, device="cuda")
    state = cu(c["main_state"])
    before = state.clone()
    wuda.mqa_compressor_fp8_standalone(cu(c["pos"]), cu(c["main_norm"]), cu(c["cos"]), cu(c["sin"]), state,
                                       cu(c["state_row"]), 8, q8, s8, rope, 1e-6)
    torch.cuda.synchronize()
    assert torch.equal(state, before)                                     # the state is read-only
    oq, os_, orope = oracle.main_compressor_fp8(c["main_state"], c["state_row"], c["pos"], c["main_norm"], c["cos"],
                                                c["sin"])
    close_bytes(q8.cpu().numpy(), oq, 0.999)


def test_rejects_bad_arguments(wuda):
    c = make_step(4, 8, 1)
    pos, cos, sin = cu(c["pos"]), cu(c["cos"]), cu(c["sin"])
    with pytest.raises(wuda.WudaError, match="no writer"):
        wuda.cache_writers_fp8(pos, cos, sin)
    with pytest.raises(wuda.WudaError, match="at least 8"):
        wuda.cache_writers_fp8(pos, cos, sin, indexer=dict(state=cu(c["idx_state"])[:, :4].contiguous(),
                                                           state_row=cu(c["state_row"]), norm_w=cu(c["idx_norm"])))
    with pytest.raises(wuda.WudaError, match="stride"):
        wuda.cache_writers_fp8(pos, cos, sin, window=dict(y=cu(c["y"]), norm_w=cu(c["win_norm"]),
                                                          pool=torch.zeros(2, 1000, dtype=torch.uint8, device="cuda"),
                                                          dst=cu(c["swa_dst"]), entries_per_block=256))
    with pytest.raises(wuda.WudaError, match="norm_w"):
        wuda.cache_writers_fp8(pos, cos, sin, window=dict(y=cu(c["y"]), norm_w=cu(c["idx_norm"])))
