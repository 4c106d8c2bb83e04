"""The cache manager against a recorded run of the reference's KVCacheManager
(dsv4_megakernel/megakernel/test/kv_cache_manager.py) over a scripted request lifecycle:
every slot, position, state row, destination entry, block table, window index list and
pool geometry it hands out must be identical.  CPU only: the manager is host code."""
import gzip
import json
import os
import sys

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
from make_golden import kv_trace  # noqa: E402  (the recorder; needs no reference checkout)

from wuda_b200.kv_cache import KVCacheManager, WIN  # noqa: E402


def _traces():
    with gzip.open(os.path.join(HERE, "golden", "kv_cache_trace.json.gz"), "rt") as f:
        return json.load(f)


@pytest.mark.parametrize("n", [0, 1, 2])
def test_trace_equals_reference(n):
    t = _traces()[n]
    ops = [tuple(op) for op in t["ops"]]
    got = json.loads(json.dumps(kv_trace(KVCacheManager, t["config"], ops)))
    exp = t["expect"]
    assert got["geometry"] == exp["geometry"]
    assert got["shapes"] == exp["shapes"]
    assert len(got["events"]) == len(exp["events"])
    for i, (a, b) in enumerate(zip(got["events"], exp["events"])):
        assert a == b, "event %d differs" % i


def test_state_reset_and_slot_reuse():
    m = KVCacheManager(2, 8, 4, device="cpu")
    s = m.alloc_request()
    assert torch.all(m.main_state[s, :, :1024] == 0) and torch.all(m.main_state[s, :, 1024:] == float("-inf"))
    assert torch.all(m.idx_state[s, :, :256] == 0) and torch.all(m.idx_state[s, :, 256:] == float("-inf"))
    m.main_state[s].fill_(3.0)
    m.idx_state[s].fill_(3.0)
    m.free_request(s)
    assert m.alloc_request() == s                      # the freed slot comes back first ...
    assert torch.all(m.main_state[s, :, :1024] == 0)   # ... with its state reset
    assert torch.all(m.idx_state[s, :, 256:] == float("-inf"))


def test_step_destinations():
    m = KVCacheManager(1, 8, 4, device="cpu")
    s = m.alloc_request()
    for p in range(300):
        st = m.step_begin([s])
        assert st["pos"].tolist() == [p] and st["q_pos"].dtype == torch.int32
        assert st["main_state_row"].tolist() == [s * 8 + p % 8]
        page = m.block_table("swa", [s])[0, 0].item()
        assert st["swa_dst"].tolist() == [page * 256 + p % WIN]
        if (p + 1) % 4:
            assert st["idx_dst"].tolist() == [-1] and st["cmp_dst"].tolist() == [-1]
        else:
            ct = (p + 1) // 4 - 1
            assert st["idx_dst"].item() == m.block_table("idx", [s])[0, ct // 64].item() * 64 + ct % 64
            assert st["cmp_dst"].item() == m.block_table("cmp", [s])[0, ct // 64].item() * 64 + ct % 64
    assert m.n_compressed([s], [299]).tolist() == [75]
    idx, lens = m.swa_indices([s], [299], 128)
    assert lens.tolist() == [128] and sorted(idx[0, 0].tolist()) == list(range(page * 256, page * 256 + 128))
    idx, lens = m.swa_indices([s], [4], 128)
    assert lens.tolist() == [5] and idx[0, 0, 5:].eq(-1).all()


def test_argument_errors():
    with pytest.raises(ValueError):
        KVCacheManager(1, 4, 2, device="cpu", state_ring_entries=4)
    with pytest.raises(ValueError):
        KVCacheManager(1, 4, 2, device="cpu", idx_entries_per_block=0)
    with pytest.raises(ValueError):
        KVCacheManager(1, 4, 2, device="cpu", idx_block_stride_bytes=100)
    m = KVCacheManager(1, 4, 2, device="cpu", indexer_fp8=False)
    with pytest.raises(ValueError):
        m.indexer_cache_view()
    m.alloc_request()
    with pytest.raises(IndexError):
        m.alloc_request()                              # no free slot


def test_advance_equals_stepping():
    a = KVCacheManager(2, 64, 8, device="cpu")
    b = KVCacheManager(2, 64, 8, device="cpu")
    sa, sb = a.alloc_request(), b.alloc_request()
    for _ in range(1000):
        a.step_begin([sa])
    b.advance(sb, 1000)
    for _ in range(9):
        x, y = a.step_begin([sa]), b.step_begin([sb])
        for key in ("pos", "main_state_row", "idx_dst", "cmp_dst", "swa_dst"):
            assert x[key].tolist() == y[key].tolist()
        for name in ("swa", "cmp", "idx"):
            assert a.block_table(name, [sa]).tolist() == b.block_table(name, [sb]).tolist()
