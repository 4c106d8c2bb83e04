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
