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
