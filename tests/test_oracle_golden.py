"""Pins the CPU oracle against fixtures produced by the reference's own Python
reference functions (tests/golden/make_golden.py) and against torch's number formats."""
import numpy as np
import pytest
import torch

import oracle
from conftest import load_golden


def test_e4m3_decode_matches_torch_for_all_256_codes():
    codes = np.arange(256, dtype=np.uint8)
    mine = oracle.e4m3_decode(codes)
    theirs = torch.from_numpy(codes).view(torch.float8_e4m3fn).float().numpy()
    assert np.array_equal(np.isnan(mine), np.isnan(theirs))
    ok = ~np.isnan(theirs)
    assert np.array_equal(mine[ok], theirs[ok])
    assert mine[0x7E] == 448.0 and mine[0x08] == 2.0 ** -6 and mine[0x01] == 2.0 ** -9


def test_e4m3_encode_matches_torch_round_to_nearest_even():
    rng = np.random.default_rng(5)
    x = rng.normal(size=200000).astype(np.float32) * rng.choice(
        [1e-4, 1e-3, 1e-2, 1, 10, 100], size=200000).astype(np.float32)
    x = np.clip(x, -448, 448)
    # exact midpoints between neighbouring codes exercise the ties-to-even rule
    grid = oracle.e4m3_decode(np.arange(0, 0x7E, dtype=np.uint8))
    mid = ((grid[:-1].astype(np.float64) + grid[1:]) / 2).astype(np.float32)
    x = np.concatenate([x, mid, -mid, grid, [0.0, 448.0, -448.0]]).astype(np.float32)
    mine = oracle.e4m3_encode(x)
    theirs = torch.from_numpy(x).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    same = (mine == theirs) | ((x == 0) & ((mine & 0x7F) == 0) & ((theirs & 0x7F) == 0))
    assert same.all(), x[~same][:8]


@pytest.mark.parametrize("name", ["mqa_logits_fp8_n1.npz", "mqa_logits_fp8_n2_epb32.npz"])
def test_mqa_logits_oracle_matches_reference_formula(name):
    g = load_golden(name)
    next_n, epb, stride = int(g["next_n"]), int(g["epb"]), int(g["logits_stride"])
    got = oracle.mqa_logits_fp8(g["q"], g["kv_pages"], g["weights"], g["context_lens"], g["block_table"],
                                next_n, epb, stride)
    exp = g["expected"]
    valid = np.isfinite(exp)
    # exactly the positions t < context are written
    assert np.array_equal(np.isfinite(got), valid)
    cols = np.arange(stride)[None, :]
    assert np.array_equal(valid, cols < g["context_lens"].reshape(-1)[:, None])
    # fp32 sums in a different order, and the scale applied after the head sum
    # instead of inside the dequantised key: 1e-4 relative to the row scale
    rms = np.sqrt(np.mean(exp[valid].astype(np.float64) ** 2))
    assert np.max(np.abs(got[valid] - exp[valid])) <= 1e-4 * rms


def test_mqa_logits_oracle_rejects_out_of_pool_page():
    g = load_golden("mqa_logits_fp8_n1.npz")
    bt = g["block_table"].copy()
    bt[0, 0] = g["kv_pages"].shape[0]
    with pytest.raises(ValueError):
        oracle.mqa_logits_fp8(g["q"], g["kv_pages"], g["weights"], g["context_lens"], bt, 1, 64,
                              int(g["logits_stride"]))


@pytest.mark.parametrize("name", ["topk_random.npz", "topk_ties.npz"])
def test_topk_oracle_matches_stable_argsort_and_page_transform(name):
    g = load_golden(name)
    pages, raw = oracle.topk(g["scores"], g["seq_lens"], g["page_table"], int(g["k"]), int(g["page_size"]))
    assert np.array_equal(raw, g["raw"])
    assert np.array_equal(pages, g["pages"])


def test_topk_oracle_trivial_rows():
    scores = np.random.default_rng(0).normal(size=(2, 256)).astype(np.float32)
    pt = np.arange(8, dtype=np.int32).reshape(2, 4) + 100
    pages, raw = oracle.topk(scores, np.array([5, 0], np.int32), pt, 16, 64)
    assert raw[0].tolist() == [0, 1, 2, 3, 4] + [-1] * 11
    assert raw[1].tolist() == [-1] * 16
    assert pages[0, :5].tolist() == [(100 << 6) + i for i in range(5)] and (pages[0, 5:] == -1).all()


def test_rmsnorm_oracle_matches_origin_model():
    g = load_golden("rmsnorm_7168.npz")
    got = oracle.rmsnorm_bf16(g["x"], g["gamma"], float(g["eps"]))
    assert np.array_equal(got, g["y"])


def test_rope_oracle_matches_origin_model_forward_and_inverse():
    g = load_golden("rope_192.npz")
    rows = {int(p): i for i, p in enumerate(g["table_rows"])}
    local_pos = np.array([rows[int(p)] for p in g["positions"]], np.int64)   # fixture stores only the used table rows
    fwd = oracle.rope_bf16(g["x"], local_pos, g["cos"], g["sin"], int(g["rope_dim"]))
    inv = oracle.rope_bf16(g["x"], local_pos, g["cos"], g["sin"], int(g["rope_dim"]), inverse=True)
    assert np.array_equal(fwd, g["y"]) and np.array_equal(inv, g["y_inverse"])
    # the first 128 dims of each head are untouched
    assert np.array_equal(fwd[..., :128], g["x"][..., :128])


def test_act_quant_oracle_matches_reference_pow2_twin():
    g = load_golden("act_quant_pow2_7168.npz")
    q, s = oracle.act_quant_fp8(g["x"], 128, round_scale=True)
    assert np.array_equal(s, g["scale"])
    assert np.array_equal(q, g["q"])


def test_act_quant_oracle_fp32_scales_round_trip():
    g = load_golden("act_quant_pow2_7168.npz")
    q, s = oracle.act_quant_fp8(g["x"], 128, round_scale=False)
    x = oracle.bf16_to_f32(g["x"]).reshape(6, -1, 128)
    amax = np.maximum(np.abs(x).max(-1), 1e-4).astype(np.float32)
    assert np.array_equal(s, amax * np.float32(1.0 / 448.0))
    deq = oracle.e4m3_decode(q).reshape(6, -1, 128) * s[..., None]
    assert np.max(np.abs(deq - x)) <= np.max(amax) / 448.0 * 16 * 1.01     # half a step of the top binade (step = 32 * scale)
    # every group's largest element maps to +-448 exactly
    assert np.all(np.abs(oracle.e4m3_decode(q).reshape(6, -1, 128)).max(-1)[amax > 1e-4] == 448.0)


def test_gemm_fp8_oracle_equals_dequantised_matmul():
    rng = np.random.default_rng(3)
    m, n, k = 5, 256, 384
    a = oracle.e4m3_encode(np.clip(rng.normal(size=(m, k)) * 100, -448, 448).astype(np.float32))
    b = oracle.e4m3_encode(np.clip(rng.normal(size=(n, k)) * 100, -448, 448).astype(np.float32))
    a_s = rng.uniform(0.5, 2, size=(m, k // 128)).astype(np.float32)
    b_s = rng.uniform(0.5, 2, size=(n // 128, k // 128)).astype(np.float32)
    got = oracle.gemm_fp8_blockscaled(a, a_s, b, b_s, out_bf16=False)
    ad = oracle.e4m3_decode(a).astype(np.float64) * np.repeat(a_s, 128, axis=1)
    bd = oracle.e4m3_decode(b).astype(np.float64) * np.repeat(np.repeat(b_s, 128, axis=0), 128, axis=1)
    ref = ad @ bd.T
    assert np.max(np.abs(got - ref)) <= 1e-5 * np.max(np.abs(ref))


def test_mhc_post_oracle_matches_reference_formula():
    """The reference's torch twin sums comb·residual first and adds post·x last; the oracle
    follows the reference kernel (product first, then four fmaf).  Both round once to bf16,
    so they agree to one bf16 step and are identical almost everywhere."""
    g = load_golden("mhc_post_7168.npz")
    got = oracle.mhc_post(g["x"], g["residual"], g["post"], g["comb"])
    d = np.abs(got.astype(np.int32) - g["out"].astype(np.int32))
    assert d.max() <= 1
    assert (d == 0).mean() >= 0.99
    # exact against a float64 evaluation rounded once, wherever that is not a near-tie
    x, res = oracle.bf16_to_f32(g["x"]).astype(np.float64), oracle.bf16_to_f32(g["residual"]).astype(np.float64)
    exact = np.einsum("mij,mih->mjh", g["comb"].astype(np.float64), res) + g["post"][..., None] * x[:, None, :]
    err = np.abs(oracle.bf16_to_f32(got) - exact)
    assert np.all(err <= np.abs(exact) * 2.0 ** -8 + 1e-6)


def test_indexer_compressor_oracle_matches_reference_twin():
    g = load_golden("indexer_compressor_fp8.npz")
    q8, scale = oracle.indexer_compressor_fp8(g["state"], g["state_row"], g["pos"], g["norm_w"], g["cos"], g["sin"])
    m = g["compress"]
    assert np.array_equal(m, (g["pos"] + 1) % 4 == 0) and m.sum() >= 8
    assert (q8[~m] == 0xAB).all() and (scale[~m] == -1).all()          # other rows are not touched
    # the twin forms softmax(score) * kv and sums; the oracle divides two running sums: the bf16
    # rounding that follows hides the difference almost always
    assert np.mean(q8[m] == g["q8"][m]) >= 0.995
    assert np.allclose(scale[m], g["scale"][m], rtol=2 ** -7)
    assert np.mean(scale[m] == g["scale"][m]) >= 0.9


def test_window_kv_oracle_matches_reference_twin():
    g = load_golden("window_kv_fp8.npz")
    q8, s8, rope = oracle.window_kv_fp8(g["y"], g["pos"], g["norm_w"], g["cos"], g["sin"])
    assert np.array_equal(s8, g["s8"])                                  # power-of-two scales: exact
    assert np.mean(q8 == g["q8"]) >= 0.995
    assert np.mean(rope == g["rope"]) >= 0.995
    assert np.abs(rope.astype(np.int32) - g["rope"].astype(np.int32)).max() <= 1


def test_main_compressor_oracle_structure():
    """No callable twin exists for the MAIN compressor (the reference checks it inline,
    test_mqa_logits_fp4.py:769-789); its two halves are the code pinned above: the window
    sum / norm / rotation of the indexer compressor at width 512 and the MODEL1 quantiser of
    the window writer.  Here: a float64 evaluation of the same formula, and the record layout."""
    rng = np.random.default_rng(9)
    rows, ring, epb = 8, 8, 4
    pos = np.arange(rows, dtype=np.int64)
    state = rng.normal(size=(rows, ring, 2048)).astype(np.float32)
    state_row = np.arange(rows) * ring + pos % ring
    norm = (rng.random(512) + 0.5).astype(np.float32)
    ang = np.outer(np.arange(16, dtype=np.float32), 1.0 / (10000.0 ** (np.arange(32) / 32.0))).astype(np.float32)
    cos, sin = np.cos(ang), np.sin(ang)
    stride = epb * 584 + 128
    pool = np.full((2, stride), 0xA5, np.uint8)
    q8, s8, rope = oracle.main_compressor_fp8(state, state_row, pos, norm, cos, sin, pool=pool,
                                              dst=np.arange(rows), epb=epb)
    for r in range(rows):
        page, off = pool[r // epb], r % epb
        body, sb = page[off * 576:(off + 1) * 576], page[epb * 576 + off * 8:epb * 576 + off * 8 + 8]
        if (pos[r] + 1) % 4:
            assert (q8[r] == 0xAB).all() and (s8[r] == -1).all() and (body == 0xA5).all() and (sb == 0xA5).all()
            continue
        assert np.array_equal(body[:448], q8[r]) and np.array_equal(body[448:].view(np.uint16), rope[r])
        assert np.array_equal(sb[:7], (np.log2(s8[r]) + 127).astype(np.uint8)) and sb[7] == 0xA5
        cur = int(state_row[r]) % ring
        perm = [(cur - 7 + k) % ring for k in range(8)]
        kv = np.stack([state[r, perm[k], (0 if k < 4 else 512):(512 if k < 4 else 1024)] for k in range(8)]).astype(np.float64)
        sc = np.stack([state[r, perm[k], 1024 + (0 if k < 4 else 512):1024 + (512 if k < 4 else 1024)] for k in range(8)]).astype(np.float64)
        e = np.exp(sc - sc.max(0))
        agg = (e * kv).sum(0) / e.sum(0)
        ro = agg / np.sqrt((agg * agg).mean() + 1e-6) * norm
        p = pos[r] - 3
        ev, od = ro[448::2].copy(), ro[449::2].copy()
        ro[448::2], ro[449::2] = ev * cos[p] - od * sin[p], ev * sin[p] + od * cos[p]
        deq = oracle.e4m3_decode(q8[r]).reshape(7, 64) * s8[r][:, None]
        assert np.all(np.abs(deq - ro[:448].reshape(7, 64)) <= s8[r][:, None] * 16 * 1.01 + np.abs(ro[:448].reshape(7, 64)) * 2 ** -6)
        mag = np.repeat(np.abs(ev) + np.abs(od), 2)                  # three bf16 roundings of the pair
        assert np.all(np.abs(oracle.bf16_to_f32(rope[r]) - ro[448:]) <= mag * 2 ** -6 + 1e-3)
    assert (pool[:, epb * 584:] == 0xA5).all()


def test_index_q_post_oracle_matches_reference_twin():
    g = load_golden("index_q_post_fp8.npz")
    q8, w = oracle.index_q_post_fp8(g["iq"], g["q_pos"], g["cos"], g["sin"], g["weights"])
    assert np.array_equal(q8, g["q8"])
    assert np.array_equal(w, g["w_folded"])
    assert (q8[0, 0] == 0).all() and w[0, 0] == g["weights"][0, 0] * np.float32(1e-12)


def _cosine(a, b):
    a, b = a.astype(np.float64).ravel(), b.astype(np.float64).ravel()
    return float(a @ b / np.sqrt((a @ a) * (b @ b)))


def test_index_q_post_fp4_oracle_matches_reference_twin():
    """The twin multiplies by the Hadamard matrix and rounds e2m1 ties down; the reference kernel (and the oracle)
    run fp32 butterflies and round ties to even, so the twin's own acceptance is the bar (cosine > 0.999, scales equal
    in > 98 % of the blocks: test/test_idx_post_fp4.py:40-66)."""
    g = load_golden("index_q_post_fp4.npz")
    q4, sf = oracle.index_q_post_fp4(g["iq"], g["q_pos"], g["cos"], g["sin"])
    tokens, heads = sf.shape
    deq = oracle.dequant_mxfp4(q4.reshape(-1, 64), sf.reshape(-1)).reshape(tokens, heads, 128)
    scale = np.ldexp(1.0, sf.view(np.uint8).reshape(tokens, heads, 4).astype(np.int32) - 127)
    assert np.mean(scale == g["sf"]) >= 0.99          # a bf16 rounding of the transform's output can tip a block's amax
    assert _cosine(deq, g["deq"]) > 0.999
    same_scale = np.repeat(scale == g["sf"], 32, axis=-1)
    assert np.mean(deq[same_scale] == g["deq"][same_scale]) >= 0.99       # the rest: ties and the bf16 rounding
    step = np.abs(deq - g["deq"]) / np.repeat(scale, 32, axis=-1)         # ... and never more than one code apart
    assert step[same_scale].max() <= 1.0
    assert (q4[0, 0] & 0x77 == 0).all() and sf[0, 0] == 0x02020202    # the all-zero head: zero codes; the kernel's floor
    # constant lies one ulp above 6 * 2^-126, so the exponent byte is 2 where the twin's clamp gives 1


def test_indexer_compressor_fp4_oracle_matches_reference_twin():
    g = load_golden("indexer_compressor_fp4.npz")
    q4, s4 = oracle.indexer_compressor_fp4(g["state"], g["state_row"], g["pos"], g["norm_w"], g["cos"], g["sin"])
    m = g["compress"]
    assert np.array_equal(m, (g["pos"] + 1) % 4 == 0) and m.sum() >= 8
    assert (q4[~m] == 0xAB).all() and (s4[~m] == 0xAB).all()           # other rows are not touched
    words = s4[m].astype(np.uint32) @ (1 << (8 * np.arange(4, dtype=np.uint32)))
    deq = oracle.dequant_mxfp4(q4[m], words.astype(np.uint32))
    assert np.mean(s4[m] == g["s4"][m]) >= 0.95
    assert _cosine(deq, g["deq"][m]) > 0.999


def test_query_rms_rope_oracle_against_the_two_pass_fixtures():
    """No twin of the fused query tail exists in the reference's tests; the oracle is held against
    the origin model's RMSNorm (fixture rmsnorm_7168) re-used on 512-wide rows: unit weight, so
    the not-rotated 448 columns must be the rounded x * rsqrt(mean x^2 + eps)."""
    rng = np.random.default_rng(4)
    x = oracle.f32_to_bf16(rng.normal(size=(3, 2, 512)).astype(np.float32))
    ang = np.outer(np.arange(32, dtype=np.float32), 1.0 / (10000.0 ** (np.arange(32) / 32.0))).astype(np.float32)
    out = oracle.query_rms_rope(x, [0, 7, 31], np.cos(ang), np.sin(ang), out_heads=4)
    assert np.array_equal(out[:, :2], out[:, 2:])
    normed = oracle.rmsnorm_bf16(x.reshape(-1, 512), np.ones(512, np.float32), 1e-6).reshape(3, 2, 512)
    d = np.abs(out[:, :2, :448].astype(np.int32) - normed[..., :448].astype(np.int32))
    assert d.max() <= 1 and np.mean(d == 0) >= 0.995
    assert np.array_equal(out[0, :, 448:], normed[0, :, 448:]) or d.max() <= 1   # position 0: no rotation
    xf = oracle.bf16_to_f32(x).astype(np.float64)
    y = xf / np.sqrt((xf * xf).mean(-1, keepdims=True) + 1e-6)
    ev, od = y[..., 448::2].copy(), y[..., 449::2].copy()
    c, s = np.cos(ang.astype(np.float64))[[0, 7, 31]][:, None], np.sin(ang.astype(np.float64))[[0, 7, 31]][:, None]
    y[..., 448::2], y[..., 449::2] = ev * c - od * s, ev * s + od * c
    assert np.all(np.abs(oracle.bf16_to_f32(out[:, :2]) - y) <= np.abs(y) * 2.0 ** -8 + 1e-6)


def test_mhc_pre_oracle_matches_reference_twin():
    import sys, os
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))
    from make_golden import mhc_pre_inputs
    g = load_golden("mhc_pre_7168.npz")
    x, weight, base, scale = mhc_pre_inputs()
    xu = x.view(torch.int16).numpy().view(np.uint16)
    assert abs(float(np.abs(weight).sum() + np.abs(xu.astype(np.float64)).sum() % 1e6) - float(g["input_checksum"])) < 1e-3
    o = oracle.mhc_pre(xu, weight, base, scale, np.full(7168, 0x3F80, np.uint16))
    # the reference's own gates (test_hc_fused_tc.py:172-177) are 2e-3 / 2e-3 / 5e-4; fp32 twins agree far closer
    for key, tol in (("pre", 2e-6), ("post", 2e-6), ("comb", 2e-6)):
        assert np.abs(o[key] - g[key]).max() <= tol, key
    got, ref = oracle.bf16_to_f32(o["collapsed"]), oracle.bf16_to_f32(g["collapsed"])
    assert np.mean(o["collapsed"] == g["collapsed"]) >= 0.999
    assert np.all(np.abs(got - ref) <= np.abs(ref) * 2.0 ** -7 + 1e-6)
    # doubly stochastic after the Sinkhorn iterations
    assert np.allclose(o["comb"].sum(1), 1, atol=1e-4) and np.allclose(o["comb"].sum(2), 1, atol=1e-4)
    # unit gamma: normed = collapsed * rsqrt(mean^2), and the quantised copy decodes back to it
    y = oracle.bf16_to_f32(o["collapsed"]).astype(np.float64)
    n = y / np.sqrt((y * y).mean(-1, keepdims=True) + 1e-6)
    assert np.all(np.abs(oracle.bf16_to_f32(o["normed"]) - n) <= np.abs(n) * 2.0 ** -8 + 1e-6)
    deq = oracle.e4m3_decode(o["xq"]).reshape(3, 56, 128) * o["xsf"][..., None]
    nb = oracle.bf16_to_f32(o["normed"]).reshape(3, 56, 128)
    assert np.all(np.abs(deq - nb) <= o["xsf"][..., None] * 16 * 1.01 + np.abs(nb) * 2.0 ** -4)
    assert np.all(np.log2(o["xsf"]) == np.round(np.log2(o["xsf"])))


def test_moe_route_oracle_matches_origin_gate():
    g = load_golden("moe_gate_256.npz")
    x, w = oracle.bf16_to_f32(g["x"]).astype(np.float64), oracle.bf16_to_f32(g["weight"]).astype(np.float64)
    logits = (x @ w.T).astype(np.float32)
    for code, name in enumerate(("softmax", "sigmoid", "sqrtsoftplus")):
        weights, indices = oracle.moe_route(logits, g["bias"], int(g["topk"]), code, float(g["route_scale"]))
        assert np.array_equal(indices, g["indices_" + name]), name
        assert np.abs(weights - g["weights_" + name]).max() <= 1e-6, name
        if code:
            assert np.allclose(weights.sum(1), float(g["route_scale"]), rtol=1e-5)
    # ties go to the lower expert; without a bias the choice follows the score itself
    flat = np.zeros((1, 40), np.float32)
    flat[0, [7, 3, 30]] = 1.0
    weights, indices = oracle.moe_route(flat, None, 5, 1, 1.0)
    assert indices[0].tolist() == [3, 7, 30, 0, 1]


def test_sparse_mla_oracle_matches_reference_twin():
    """ref_flash_attn over deq_model1_row records (window entries, then top-k entries, with the
    attention sink): the oracle sums in double, the twin in fp32."""
    g = load_golden("sparse_mla_h16.npz")
    got = oracle.sparse_mla(g["q"], (g["swa_pool"], int(g["swa_epb"]), g["swa_idx"], g["swa_len"]),
                            (g["cmp_pool"], int(g["cmp_epb"]), g["cmp_idx"], g["cmp_len"]), g["sink"], float(g["scale"]))
    assert np.max(np.abs(got - g["out"])) <= 2e-5 * np.max(np.abs(g["out"]))


def test_mqa_logits_fp4_oracle_matches_reference_twin():
    """MXFP4 indexer scores: inputs quantised and paged by the reference's own helpers, expected values from
    its torch twin over the dequantised operands."""
    g = load_golden("mqa_logits_fp4.npz")
    got = oracle.mqa_logits_fp4(g["q"], g["q_sf"], g["pages"], g["weights"], g["context_lens"], g["block_table"],
                                int(g["epb"]), g["logits"].shape[1])
    ref = g["logits"]
    valid = np.isfinite(ref)
    assert np.array_equal(np.isfinite(got), valid)
    assert np.max(np.abs(got[valid] - ref[valid])) <= 1e-5 * np.sqrt(np.mean(ref[valid].astype(np.float64) ** 2))


def test_query_rms_rope_oracle_matches_the_reference_twin():
    """Fixture from the reference's inline twin of the fused query tail (test_mqa_logits_fp4.py:404-413,
    restated in tests/golden/make_golden.py): bit-exact on both head layouts up to the twin's own libm
    (torch's rsqrt against 1/sqrt: the last bf16 bit of a few values)."""
    g = load_golden("query_rms_rope.npz")
    for name, out_heads in (("full", 8), ("half", 8)):
        got = oracle.query_rms_rope(g["x_" + name], g["positions"], g["cos"], g["sin"], out_heads=out_heads,
                                    eps=float(g["eps"]))
        want = g["out_" + name]
        d = np.abs(got.astype(np.int32) - want.astype(np.int32))
        assert d.max() <= 1 and np.mean(d == 0) >= 0.999, (name, int(d.max()), float(np.mean(d == 0)))


def test_main_compressor_oracle_matches_the_reference_twin():
    """Fixture from the reference's inline twin of the MAIN compressor row (test_mqa_logits_fp4.py:772-791):
    scales exact, e4m3 codes those of the twin's values, rotary tail within one bf16 step (the twin's own GPU
    check allows 1e-2 / 0.15 / 0.05 because its kernel is built with fast-math)."""
    g = load_golden("main_compressor_fp8.npz")
    q8, s8, rope = oracle.main_compressor_fp8(g["state"], g["state_row"], g["pos"], g["norm_w"], g["cos"], g["sin"])
    rows = np.nonzero(g["compress"])[0]
    assert len(rows) == 8
    for r in range(len(g["pos"])):
        if not g["compress"][r]:
            assert (q8[r] == 0xAB).all() and (s8[r] == -1).all()
    assert np.array_equal(s8[rows], g["scale"][rows])
    want_q = oracle.e4m3_encode((g["values"][rows].reshape(-1, 7, 64) / g["scale"][rows][:, :, None]).reshape(-1, 448))
    same = q8[rows] == want_q
    assert same.mean() >= 0.995, float(same.mean())
    deq = oracle.e4m3_decode(q8[rows]).reshape(-1, 7, 64) * s8[rows][:, :, None]
    assert np.all(np.abs(deq.reshape(-1, 448) - g["values"][rows]) <=
                  np.abs(g["values"][rows]) * 2.0 ** -3 + np.repeat(s8[rows], 64, axis=1) * 2.0 ** -9)
    d = np.abs(rope[rows].astype(np.int32) - g["rope"][rows].astype(np.int32))
    assert d.max() <= 1 and np.mean(d == 0) >= 0.99


@pytest.mark.parametrize("name", ["plain", "limit"])
def test_moe_block_oracle_matches_the_origin_module(name):
    """Fixture from the origin's MoE module (Gate, Experts, shared Expert, origin/model.py:546-644) on bf16
    weights: same experts selected, same routing weights, and the block output within two bf16 steps of the
    largest term (torch sums a projection in fp32, the oracle in double: single roundings differ)."""
    g = load_golden("moe_block_origin.npz")
    y, rw, idx = oracle.moe_block(g["x_" + name], g["gate_w_" + name], g["gate_bias_" + name], g["w1_" + name],
                                  g["w3_" + name], g["w2_" + name], int(g["topk"]), 2, float(g["route_scale"]),
                                  float(g["limit_" + name]))
    assert np.array_equal(np.sort(idx, axis=1), np.sort(g["indices_" + name], axis=1))
    order = np.argsort(idx, axis=1), np.argsort(g["indices_" + name], axis=1)
    assert np.allclose(np.take_along_axis(rw, order[0], 1), np.take_along_axis(g["weights_" + name], order[1], 1),
                       rtol=2e-6, atol=1e-7)
    got, want = oracle.bf16_to_f32(y), oracle.bf16_to_f32(g["y_" + name])
    assert np.all(np.abs(got - want) <= 2.0 ** -7 * np.abs(want) + 2.0 ** -8 * np.abs(want).max())
    assert np.mean(y == g["y_" + name]) >= 0.9


def test_fp4_gemm_oracle_matches_the_origin_lossless_cast_and_the_reference_dequantiser():
    """Fixture: weights quantised by the reference test's per_token_cast_to_fp4, dequantised by its
    cast_back_from_fp4, and cast to e4m3 with 128x128 scales by the origin's cast_e2m1fn_to_e4m3fn
    (origin/convert.py:20-52).  The oracle's FP8 x FP4 product must equal the product of the dequantised operands,
    and so must its FP8 product over the origin's lossless cast: nibble order, code table and the meaning of the
    scale bytes are the reference's."""
    g = load_golden("fp4_gemm.npz")
    ref = g["c"]
    rms = np.sqrt(np.mean(ref.astype(np.float64) ** 2))
    c4 = oracle.gemm_fp8_fp4(g["a"], g["a_s"], g["w4"], g["w_sf"], out_bf16=False)
    c8 = oracle.gemm_fp8_blockscaled(g["a"], g["a_s"], g["w8"], g["w8_scale"], out_bf16=False)
    assert np.all(np.abs(c4 - ref) <= 1e-6 * rms) and np.all(np.abs(c8 - ref) <= 1e-6 * rms)
    # the dequantised weights themselves: code table and scale bytes
    codes = np.stack([g["w4"] & 15, g["w4"] >> 4], -1).reshape(g["w_deq"].shape)
    table = np.array([0, .5, 1, 1.5, 2, 3, 4, 6, 0, -.5, -1, -1.5, -2, -3, -4, -6], np.float32)
    assert np.array_equal(table[codes] * np.repeat(np.exp2(g["w_sf"].astype(np.float32) - 127), 32, 1), g["w_deq"])
    # the oracle's quantiser on the values the reference's quantiser saw (bf16-representable): the same scale bytes
    # (2^ceil(log2(amax / 6))); the same codes except at exact rounding ties, which the test's bucketize sends down
    # and the hardware conversion the oracle follows to the even code
    oc, osf, _ = oracle.fp4_act_quant(oracle.f32_to_bf16(g["w"]))
    assert np.array_equal(osf, g["w_sf"])
    mine = np.stack([oc & 15, oc >> 4], -1).reshape(g["w"].shape)
    scaled = np.abs(g["w"]) / np.repeat(np.exp2(g["w_sf"].astype(np.float32) - 127), 32, 1)
    tie = np.isin(scaled, [0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0])
    mine = np.where((mine & 7) == 0, 0, mine)        # the hardware conversion keeps the sign of a zero, the test drops it
    assert np.array_equal(mine[~tie], codes[~tie]) and np.mean(mine == codes) > 0.98
    assert np.all((mine[tie] & 7).astype(int) - (codes[tie] & 7).astype(int) >= 0)
