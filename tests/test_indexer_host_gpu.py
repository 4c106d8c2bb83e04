"""The host-buffer form of the indexer step (wuda_indexer_plan_*, wuda_indexer_topk_host[_pages]) against the CPU
oracle: inputs in host memory, page-transformed top-k indices back in host memory; with a page list only the named
pages of the pool are uploaded and the rest stays as the device holds it."""
import numpy as np
import pytest
import torch

import oracle
from wuda_b200 import workloads

pytestmark = pytest.mark.gpu
K = 64


def reference(case):
    logits = oracle.mqa_logits_fp8(case["q"], case["kv_pages"], case["weights"], case["context_lens"], case["block_table"],
                                   case["next_n"], case["epb"], case["logits_stride"])
    table = np.repeat(case["block_table"], case["next_n"], axis=0)
    pages, _ = oracle.topk(logits, case["context_lens"].reshape(-1), table, K, case["epb"])
    return pages


def same_sets(got, ref):
    return np.array_equal(np.sort(got, axis=1), np.sort(ref, axis=1))


def make_plan(wuda, case):
    return wuda.IndexerHostPlan(case["batch"], case["next_n"], case["num_blocks"], case["epb"], case["page_stride"],
                                case["block_table"].shape[1], case["logits_stride"], K)


def run(plan, case, out, dirty=None):
    return plan.run(case["q"], case["kv_pages"], case["weights"], case["context_lens"], case["block_table"], out, case["batch"],
                    dirty_pages=dirty)


@pytest.mark.parametrize("next_n", [1, 2])
def test_whole_pool_upload_matches_the_oracle(wuda, next_n):
    case = workloads.make_mqa_case(6, next_n, 200, 1500, seed=21 + next_n)
    plan = make_plan(wuda, case)
    out = np.empty((case["batch"] * next_n, K), np.int32)
    run(plan, case, out)
    assert same_sets(out, reference(case))
    plan.close()


def test_only_listed_pages_are_uploaded(wuda):
    case = workloads.make_mqa_case(5, 1, 300, 1200, seed=33)
    plan = make_plan(wuda, case)
    out = np.empty((case["batch"], K), np.int32)
    run(plan, case, out)                                    # the pool is on the device now
    before = reference(case)
    assert same_sets(out, before)
    # the host rewrites the page that holds each request's newest tokens (large keys: they enter the top-k) ...
    epb = case["epb"]
    last = (case["context_lens"][:, -1] - 1) // epb
    dirty = case["block_table"][np.arange(case["batch"]), last].astype(np.int32)
    changed = dict(case, kv_pages=case["kv_pages"].copy())
    changed["kv_pages"][dirty, :epb * 128] = 0x7e           # +448 everywhere: with q ~ N(0, 1) some heads score high
    # ... and, without listing it, one more page, which therefore must NOT reach the device
    other = int(case["block_table"][0, 0])
    assert other not in dirty.tolist()
    on_device = dict(changed, kv_pages=changed["kv_pages"].copy())
    changed["kv_pages"][other, :epb * 128] = 0x7e
    run(plan, changed, out, dirty=np.sort(dirty))
    expected = reference(on_device)
    assert same_sets(out, expected)
    assert not same_sets(expected, before) and not same_sets(expected, reference(changed))
    # an empty list uploads nothing at all
    run(plan, dict(changed, kv_pages=np.zeros_like(changed["kv_pages"])), out, dirty=np.empty(0, np.int32))
    assert same_sets(out, expected)
    plan.close()


def test_a_page_outside_the_pool_is_refused(wuda):
    case = workloads.make_mqa_case(2, 1, 100, 200, seed=5)
    plan = make_plan(wuda, case)
    out = np.empty((case["batch"], K), np.int32)
    with pytest.raises(Exception, match="outside the pool"):
        run(plan, case, out, dirty=np.array([case["num_blocks"]], np.int32))
    plan.close()
