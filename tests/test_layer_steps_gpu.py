"""Several decode steps through the whole layer with the cache manager in the loop, in the shape of the
reference's own simulation (test/test_e2e_decode.py:1504-1526): 16 requests, 8 steps, one slot freed and
taken again at step 5 (its state rings re-initialised), an all-zero residual row on a compress step, fresh
random residual streams every step.  Per step the stages that carry state from one step to the next are held
against the CPU oracle on the layer's own device buffers (cache writers, indexer logits, top-k translation,
sparse attention); at the end two complete runs must agree in every bit of the outputs, the three pools and
both state rings - the reference's determinism gate (:1602-1628), which is what catches a race between the
forked cache writers, the query tail and the main chain."""
import numpy as np
import pytest
import torch

import oracle
from wuda_b200.layer_setup import build_random_layer

pytestmark = pytest.mark.gpu
SMALL = dict(topk=512, experts=32, inter=512, moe_topk=4)
BATCH, STEPS, REUSE_AT, ZERO_STEP, ZERO_ROW = 16, 8, 5, 3, 1


def u16(t):
    return t.cpu().view(torch.int16).numpy().view(np.uint16)


def check_step(layer, st, m):
    a, stage, cache = layer.attn, layer.attn.stage, layer.attn.cache
    w = {k: v.cpu().numpy() for k, v in stage.w.tensors.items() if k not in ("wq_b", "wq_b_scales")}
    pos = st["pos"].cpu().numpy()
    ring = cache.state_ring_entries
    rows = st["main_state_row"].cpu().numpy()
    got = dict(idx=cache.idx_pool.cpu().numpy(), cmp=cache.cmp_pool.cpu().numpy(), swa=cache.swa_pool.cpu().numpy())
    # cache writers: the records this step wrote, recomputed from the rings the front GEMM's epilogue filled
    want = {k: v.copy() for k, v in got.items()}
    fp4 = stage.indexer_fp4
    (oracle.indexer_compressor_fp4 if fp4 else oracle.indexer_compressor_fp8)(
        cache.idx_state.cpu().numpy().reshape(-1, ring, 512), rows, pos, w["idx_norm"], w["cos_table"], w["sin_table"],
        pool=want["idx"], dst=st["idx_dst"].cpu().numpy(), epb=cache.entries_per_block["idx"])
    oracle.main_compressor_fp8(cache.main_state.cpu().numpy().reshape(-1, ring, 2048), rows, pos, w["main_norm"], w["cos_table"],
                               w["sin_table"], pool=want["cmp"], dst=st["cmp_dst"].cpu().numpy(), epb=cache.entries_per_block["cmp"])
    oracle.window_kv_fp8(stage.win_y2[:m].cpu().numpy(), pos, w["win_norm"], w["cos_table"], w["sin_table"], pool=want["swa"],
                         dst=st["swa_dst"].cpu().numpy(), epb=cache.entries_per_block["swa"])
    assert np.array_equal(got["swa"], want["swa"])
    for name in ("idx", "cmp"):
        assert np.mean(got[name] == want[name]) >= 1 - 1e-5             # a handful of bytes may differ (expf)
    # indexer logits over the pool as it stands after the writers, top-k translated with the compressed pool's pages
    ncmp = stage.n_compressed[:m].cpu().numpy()
    assert np.array_equal(ncmp, (pos + 1) // 4)
    bt, cmp_bt = stage.block_table[:m].cpu().numpy(), stage.cmp_block_table[:m].cpu().numpy()
    logits = stage.logits[:m].cpu().numpy()
    valid = np.arange(stage.logits_stride)[None, :] < ncmp[:, None]
    if fp4:    # codes at the start of the iq buffer, the query's scale words where the folded weights would be
        heads = stage.w.index_heads
        q4 = stage.iq_fp8.view(-1)[:m * heads * 64].view(m, heads, 64).cpu().numpy()
        q_sf = stage.w_folded.view(torch.int32)[:m].cpu().numpy().view(np.uint32)
        ref_l = oracle.mqa_logits_fp4(q4, q_sf, got["idx"], stage.w64[:m].cpu().numpy(), ncmp, bt, cache.entries_per_block["idx"],
                                      stage.logits_stride)
        rel, floor = 1e-4, 1e-5
    else:
        ref_l = oracle.mqa_logits_fp8(stage.iq_fp8[:m].cpu().numpy(), got["idx"], stage.w_folded[:m].cpu().numpy(),
                                      ncmp.reshape(m, 1), bt, 1, cache.entries_per_block["idx"], stage.logits_stride)
        rel, floor = 1e-2, 1e-4
    if valid.any():
        rms = np.sqrt(np.mean(ref_l[valid].astype(np.float64) ** 2))
        assert np.all(np.abs(logits[valid] - ref_l[valid]) <= rel * np.abs(ref_l[valid]) + floor * rms + 1e-30)
    masked = np.where(valid, logits, -np.inf).astype(np.float32)
    ref_pages, _ = oracle.topk(masked, ncmp, cmp_bt, layer.attn.topk, cache.entries_per_block["cmp"])
    got_pages = stage.topk_indices[:m].cpu().numpy()
    for r in range(m):
        assert sorted(got_pages[r].tolist()) == sorted(ref_pages[r].tolist())
    # sparse attention over the window and the selected records
    swa = (got["swa"], cache.entries_per_block["swa"], a.swa_idx[:m].cpu().numpy(), a.swa_len[:m].cpu().numpy())
    cmp = (got["cmp"], cache.entries_per_block["cmp"], got_pages, a.cmp_len[:m].cpu().numpy())
    assert np.array_equal(swa[3], np.minimum(pos + 1, 128)) and np.array_equal(cmp[3], np.minimum(ncmp, layer.attn.topk))
    ref = oracle.sparse_mla(u16(stage.q_main[:m]), swa, cmp, a.w.attn_sink.cpu().numpy(), 512 ** -0.5)
    out = oracle.bf16_to_f32(u16(a.mla_out[:m])).astype(np.float64)
    assert np.all(np.abs(out - ref) <= np.abs(ref).max(axis=-1, keepdims=True) * 2.0 ** -7 + 1e-6)


def run_sim(check, native, indexer_fp4=False):
    layer, slots, _ = build_random_layer(BATCH, 1, seed=17, native=native, indexer_fp4=indexer_fp4, **SMALL)   # every request at position 0 next
    assert layer.attn.stage.indexer_fp4 == indexer_fp4
    cache = layer.attn.cache
    g = torch.Generator(device="cuda").manual_seed(42)
    finals = []
    for t in range(STEPS):
        if t == REUSE_AT:                              # slot lifecycle: state rings back to kv = 0 / score = -inf
            cache.free_request(slots[0])
            slots[0] = cache.alloc_request()
        hidden = (torch.randn(BATCH, 4, 7168, generator=g, device="cuda") * 0.1).bfloat16()
        if t == ZERO_STEP:
            hidden[ZERO_ROW].zero_()                   # an all-zero row on a compress step (position 3)
        st = layer.prepare(slots)
        if t == ZERO_STEP:
            assert (int(st["pos"][ZERO_ROW]) + 1) % 4 == 0
        if t == REUSE_AT:
            assert int(st["pos"][0]) == 0 and int(st["pos"][1]) == t
        out = layer.launch(hidden, BATCH)
        torch.cuda.synchronize()
        layer.check_status()
        assert bool(torch.isfinite(out.float()).all())
        if check:
            check_step(layer, st, BATCH)
        finals.append(out.clone())
    stage, b = layer.attn.stage, BATCH
    if native:
        mid = [layer.view("logits", torch.float32, b, stage.logits_stride), layer.view("q_main", torch.bfloat16, b, 128, 512),
               layer.view("mla_out", torch.bfloat16, b, 128, 512), layer.view("q_proj", torch.bfloat16, b, stage.w.n_total),
               layer.view("front_out", torch.bfloat16, b, 2048)]
    else:
        mid = [stage.logits, stage.q_main, layer.attn.mla_out, stage.y, layer.attn.front_out]
    # only the scored positions of a logits row are defined (the rest keeps whatever the buffer held)
    scored = torch.arange(stage.logits_stride, device="cuda")[None, :] < stage.n_compressed[:b, None]
    mid[0] = torch.where(scored, mid[0][:b], torch.zeros_like(mid[0][:b]))
    snap = finals + [cache.swa_pool.clone(), cache.cmp_pool.clone(), cache.idx_pool.clone(), cache.main_state.clone(),
                     cache.idx_state.clone()] + [t.clone() for t in mid]
    # the last step once more as a graph replay: same inputs, same rows and destinations, same bits
    layer.capture(hidden, BATCH)
    again = layer.replay()
    torch.cuda.synchronize()
    assert torch.equal(again, finals[-1])
    return snap


def test_eight_steps_with_slot_reuse_and_a_zero_row_then_the_same_again():
    first = run_sim(check=True, native=False)      # sequenced from Python, stage tensors held against the oracle
    second = run_sim(check=False, native=True)     # the library's own C++ sequence, one call per step
    third = run_sim(check=False, native=True)
    for a, b, c in zip(first, second, third):
        assert torch.equal(b.contiguous().view(torch.uint8), c.contiguous().view(torch.uint8))
    for a, b in zip(first, second):
        assert torch.equal(a.contiguous().view(torch.uint8), b.contiguous().view(torch.uint8))   # byte view: NaN-safe


def test_the_same_simulation_with_the_fp4_indexer():
    """The indexer in its FP4 form (Hadamard + MXFP4 query and keys, block-scaled logits) inside the whole layer: the
    Python sequence with the stage checks, then the library's own sequence, bit for bit the same."""
    first = run_sim(check=True, native=False, indexer_fp4=True)
    second = run_sim(check=False, native=True, indexer_fp4=True)
    for a, b in zip(first, second):
        assert torch.equal(a.contiguous().view(torch.uint8), b.contiguous().view(torch.uint8))
