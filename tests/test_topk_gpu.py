"""GPU parity of the top-k selection + page transform (through the C ABI) against the
CPU oracle (stable arg-sort) and the golden fixtures.  Index work: bit-exact sets."""
import numpy as np
import pytest
import torch

import oracle
from conftest import load_golden

pytestmark = pytest.mark.gpu
PAGE = 64


def run(wuda, scores, seq_lens, page_table, k, rows_per_table_row=1):
    ds = torch.from_numpy(scores).cuda()
    dl = torch.from_numpy(np.asarray(seq_lens, np.int32)).cuda()
    dp = torch.from_numpy(page_table).cuda()
    raw = torch.full((scores.shape[0], k), -7, dtype=torch.int32, device="cuda")
    out = wuda.topk_v2(ds, dl, dp, k, PAGE, raw_indices=raw, rows_per_table_row=rows_per_table_row)
    torch.cuda.synchronize()
    return out.cpu().numpy(), raw.cpu().numpy()


def check(wuda, scores, seq_lens, page_table, k, rows_per_table_row=1):
    got_pages, got_raw = run(wuda, scores, seq_lens, page_table, k, rows_per_table_row)
    pt_rows = np.repeat(page_table, rows_per_table_row, axis=0)
    ref_pages, ref_raw = oracle.topk(scores, seq_lens, pt_rows, k, PAGE)
    bits = PAGE.bit_length() - 1
    for r in range(scores.shape[0]):
        n = int(seq_lens[r])
        if n <= k:   # trivial rows are position-exact
            assert np.array_equal(got_raw[r], ref_raw[r]), "row %d trivial" % r
        else:        # selected SET is exact (ties towards the lower index), order is free
            assert np.array_equal(np.sort(got_raw[r]), np.sort(ref_raw[r])), "row %d set differs" % r
        raw = got_raw[r].astype(np.int64)
        exp = np.where(raw < 0, -1, (pt_rows[r][np.maximum(raw, 0) >> bits].astype(np.int64) << bits)
                       | (np.maximum(raw, 0) & (PAGE - 1))).astype(np.int32)
        assert np.array_equal(got_pages[r], exp), "row %d page transform" % r


def make(rows, length, lens, tie_levels=0, seed=0):
    rng = np.random.default_rng(seed)
    scores = rng.normal(size=(rows, length)).astype(np.float32)
    if tie_levels:
        scores = rng.integers(0, tie_levels, size=(rows, length)).astype(np.float32)
    for r in range(rows):
        scores[r, lens[r]:] = -np.inf
    pages = max((length + PAGE - 1) // PAGE, 1)
    page_table = rng.integers(0, 1 << 20, size=(rows, pages), dtype=np.int32)
    return scores, np.asarray(lens, np.int32), page_table


@pytest.mark.parametrize("name", ["topk_random.npz", "topk_ties.npz"])
def test_golden_fixture(wuda, name):
    g = load_golden(name)
    got_pages, got_raw = run(wuda, g["scores"], g["seq_lens"], g["page_table"], int(g["k"]))
    for r in range(g["scores"].shape[0]):
        if g["seq_lens"][r] <= int(g["k"]):
            assert np.array_equal(got_raw[r], g["raw"][r]) and np.array_equal(got_pages[r], g["pages"][r])
        else:
            assert np.array_equal(np.sort(got_raw[r]), np.sort(g["raw"][r]))
            assert np.array_equal(np.sort(got_pages[r]), np.sort(g["pages"][r]))


@pytest.mark.parametrize("k", [13, 512, 2048])
@pytest.mark.parametrize("length", [2049, 4096, 12288, 16384, 40000, 65536])
def test_random_rows(wuda, k, length):
    lens = [length, max(length // 2, 1), min(k, length), min(k + 1, length), 1, 0, length - 1, length // 3 + 1]
    check(wuda, *make(len(lens), length, lens, seed=k + length), k)


@pytest.mark.parametrize("tie_levels", [1, 2, 7, 50])
def test_duplicate_heavy_rows_take_lowest_indices(wuda, tie_levels):
    lens = [30000, 12288, 65536, 2500]
    check(wuda, *make(4, 65536, lens, tie_levels=tie_levels, seed=tie_levels), 2048)
    check(wuda, *make(4, 65536, lens, tie_levels=tie_levels, seed=tie_levels + 100), 512)


@pytest.mark.parametrize("crowd,step", [(1500, 1.0 / 64), (300, 1.0 / 64), (2000, 1.0 / 1024), (1100, 0.0)])
def test_threshold_inside_a_crowded_bin(wuda, crowd, step):
    """Scores crowded into a narrow band around the k-th value (hundreds of candidates share the threshold's
    histogram bin, many of them equal): the band's members must still be ranked exactly - larger first, lower
    index first among equals.  Projection outputs of real layers look like this: tens of thousands in magnitude,
    a few binades wide, runs of exact zeros behind a ReLU."""
    rng = np.random.default_rng(crowd)
    rows, length, k = 6, 8192, 2048
    scores = (rng.normal(size=(rows, length)) * 3000.0).astype(np.float32)
    for r in range(rows):
        scores[r, rng.permutation(length)[:1000]] += 60000.0                  # 1000 clear winners
        where = rng.permutation(length)[:crowd + 600]
        band = 30000.0 + rng.integers(0, 256, size=where.size) * step          # the k-th value lies in here
        scores[r, where] = band.astype(np.float32)
    lens = [length] * rows
    pages = length // PAGE
    page_table = rng.integers(0, 1 << 20, size=(rows, pages), dtype=np.int32)
    check(wuda, scores, np.asarray(lens, np.int32), page_table, k)


@pytest.mark.parametrize("shape", ["log_uniform", "across_zero", "tiny_and_huge"])
def test_kth_value_binades_above_the_sampled_bound(wuda, shape):
    """Keys are sparse near zero: when the scores around the k-th value are spread over many binades, or the k-th
    value is a small positive number with negative scores right below it, the candidate bound found from the
    samples lies far from the k-th value in key space.  The selection among the candidates must not depend on
    that distance."""
    rng = np.random.default_rng(len(shape))
    rows, length, k = 5, 8192, 2048
    scores = np.empty((rows, length), np.float32)
    for r in range(rows):
        big = rng.uniform(100.0, 1000.0, size=2000)
        if shape == "log_uniform":
            rest = 10.0 ** rng.uniform(-6.0, 0.0, size=length - 2000) * rng.choice([-1.0, 1.0], size=length - 2000)
        elif shape == "across_zero":
            rest = rng.normal(-2.0, 1.0, size=length - 2000)
        else:
            rest = np.where(rng.random(length - 2000) < 0.02, rng.uniform(1e-30, 1e-20, size=length - 2000),
                            -rng.uniform(1e-3, 1e3, size=length - 2000))
        row = np.concatenate([big, rest]).astype(np.float32)
        scores[r] = row[rng.permutation(length)]
    pages = length // PAGE
    page_table = rng.integers(0, 1 << 20, size=(rows, pages), dtype=np.int32)
    check(wuda, scores, np.full(rows, length, np.int32), page_table, k)


def test_crowded_rows_cost_about_what_spread_rows_cost(wuda):
    """A selection whose cost grew with the square of the threshold bin's size would take twenty times longer on
    crowded rows than on normal ones; the bound here is loose (a factor of 4) and relative, so it holds at any clock."""
    rng = np.random.default_rng(5)
    rows, length, k = 64, 8192, 2048
    spread = rng.normal(size=(rows, length)).astype(np.float32)
    crowded = np.maximum(rng.normal(size=(rows, length)) - 0.4, 0).astype(np.float32)    # the k-th value is an exact zero
    crowded[:, ::3] = (30000.0 + rng.integers(0, 200, size=crowded[:, ::3].shape) / 64.0).astype(np.float32)
    seq = torch.full((rows,), length, dtype=torch.int32, device="cuda")
    table = torch.arange(rows * (length // PAGE), dtype=torch.int32, device="cuda").reshape(rows, -1)
    out = torch.empty(rows, k, dtype=torch.int32, device="cuda")

    def device_time(scores):
        d = torch.from_numpy(scores).cuda()
        graph = torch.cuda.CUDAGraph()
        wuda.topk_v2_transform(d, seq, table, out, PAGE)
        torch.cuda.synchronize()
        with torch.cuda.graph(graph):
            for _ in range(10):
                wuda.topk_v2_transform(d, seq, table, out, PAGE)
        best = 1e9
        for _ in range(5):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            graph.replay()
            e1.record()
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1))
        return best

    far = (10.0 ** rng.uniform(-6.0, 0.0, size=(rows, length)) * rng.choice([-1.0, 1.0], size=(rows, length))).astype(np.float32)
    far[:, :2000] = rng.uniform(100.0, 1000.0, size=(rows, 2000)).astype(np.float32)   # the bound falls binades below the k-th value
    t_spread, t_crowded, t_far = device_time(spread), device_time(crowded), device_time(far)
    assert t_crowded < 4.0 * t_spread, (t_crowded, t_spread)
    assert t_far < 2.5 * t_spread, (t_far, t_spread)


def test_special_values(wuda):
    rng = np.random.default_rng(9)
    scores = rng.normal(size=(3, 8192)).astype(np.float32)
    scores[0, ::3] = 0.0
    scores[0, 1::3] = -0.0          # equal to +0.0 for the selection
    scores[0, 2::3] = -np.abs(scores[0, 2::3])
    scores[1, :4000] = -np.inf      # rows whose tail of the selection is -inf
    scores[2] = np.float32(1e-42) * rng.integers(-5, 5, size=8192).astype(np.float32)   # subnormals
    pt = rng.integers(0, 1 << 20, size=(3, 128), dtype=np.int32)
    check(wuda, scores, np.array([8192, 8192, 8192], np.int32), pt, 2048)
    check(wuda, scores, np.array([8192, 5000, 8191], np.int32), pt, 4500)


def test_unaligned_row_stride_and_many_rows(wuda):
    rng = np.random.default_rng(4)
    rows, length = 333, 3001       # odd stride: rows are not 16-byte aligned
    scores = rng.normal(size=(rows, length)).astype(np.float32)
    lens = rng.integers(0, length + 1, size=rows).astype(np.int32)
    pt = rng.integers(0, 1 << 20, size=(rows, 47), dtype=np.int32)
    check(wuda, scores, lens, pt, 777)


def test_rows_sharing_a_page_table_row(wuda):
    scores, lens, _ = make(6, 5000, [5000, 4999, 3000, 2999, 100, 99], seed=2)
    pt = np.random.default_rng(1).integers(0, 1 << 20, size=(3, 79), dtype=np.int32)
    check(wuda, scores, lens, pt, 1024, rows_per_table_row=2)


def test_config1_shape_k2048(wuda):
    """128 rows of 16384..65536 fp32 scores with a heavy-tailed distribution like the
    indexer logits, k = 2048."""
    rng = np.random.default_rng(0xB201)
    rows, length = 128, 65536
    lens = rng.integers(16384, 65537, size=rows).astype(np.int32)
    scores = (rng.normal(size=(rows, length)) * rng.uniform(0.01, 0.1, size=(rows, length))).astype(np.float32)
    pt = rng.integers(0, 1 << 20, size=(rows, length // PAGE), dtype=np.int32)
    check(wuda, scores, lens, pt, 2048)


def test_bad_arguments(wuda):
    s = torch.zeros(2, 128, device="cuda")
    l = torch.tensor([128, 128], dtype=torch.int32, device="cuda")
    pt = torch.zeros(2, 2, dtype=torch.int32, device="cuda")
    with pytest.raises(RuntimeError):
        wuda.topk_v2(s, l, pt, 16, page_size=48)
    with pytest.raises(RuntimeError):
        wuda.topk_v2(s.double(), l, pt, 16)
    with pytest.raises(RuntimeError):
        wuda.topk_v2(s, l[:1], pt, 16)
