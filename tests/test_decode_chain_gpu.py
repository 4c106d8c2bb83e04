"""The layer launch of the indexer half of a decode step (wuda_csa_decode_step through
wuda_b200.decode.CsaDecodeStage) checked stage by stage: every stage's GPU output is compared with
the CPU oracle applied to that stage's GPU inputs, over several steps of a small batch with the
cache manager handing out rows and destinations, first as eager launches and then as replays of
one captured CUDA graph."""
import numpy as np
import pytest
import torch

import oracle
from wuda_b200 import workloads
from wuda_b200.decode import CsaDecodeStage, CsaWeights
from wuda_b200.kv_cache import KVCacheManager

pytestmark = pytest.mark.gpu

Q_LORA, INDEX_HEADS, MAIN_HEADS, OUT_HEADS, TOPK = 256, 64, 2, 4, 48


def u16(t):
    return t.cpu().view(torch.int16).numpy().view(np.uint16)


def make_stage(batch, seed, cmp_epb=None, max_pages=8, fp4=False):
    g = torch.Generator().manual_seed(seed)
    n_total = INDEX_HEADS * 128 + MAIN_HEADS * 512
    w = torch.randn(n_total, Q_LORA, generator=g) * 0.05
    w8, ws = workloads.quantize_fp8_128x128(w)
    ang = torch.outer(torch.arange(4096, dtype=torch.float32), 1.0 / (10000.0 ** (torch.arange(32) / 32.0)))
    host = dict(wq_b=torch.from_numpy(w8), wq_b_scales=torch.from_numpy(ws), q_norm=torch.rand(Q_LORA, generator=g) + 0.5,
                idx_norm=torch.rand(128, generator=g) + 0.5, main_norm=torch.rand(512, generator=g) + 0.5,
                win_norm=torch.rand(512, generator=g) + 0.5, cos_table=torch.cos(ang).contiguous(),
                sin_table=torch.sin(ang).contiguous())
    weights = CsaWeights(index_heads=INDEX_HEADS, main_heads=MAIN_HEADS, out_heads=OUT_HEADS,
                         **{k: v.cuda() for k, v in host.items()})
    extra = {} if cmp_epb is None else dict(cmp_entries_per_block=cmp_epb)
    if fp4:
        extra["indexer_fp8"] = False      # the indexer pool holds MXFP4 records: the step takes its FP4 forms
    cache = KVCacheManager(batch + 1, 64, max_pages, device="cuda", **extra)
    cache._pools["cmp"].take()   # the compressed-KV pool numbers its pages one off the indexer pool's
    stage = CsaDecodeStage(weights, cache, batch, topk=TOPK)
    return stage, cache, {k: v.numpy() for k, v in host.items()}, g


def fast_forward(cache, slots, tokens, gen):
    """Advances the requests without running kernels and fills the indexer entries they would have
    written with random keys (finite e4m3 codes) and scales."""
    for s, n in zip(slots, tokens):
        for _ in range(n):
            cache.step_begin([s])
    pool = cache.idx_pool
    epb = cache.entries_per_block["idx"]
    if not cache.indexer_fp8:             # MXFP4 records: any codes, exponent bytes around one
        pool[:, :epb * 64] = torch.randint(0, 256, (pool.size(0), epb * 64), generator=gen, dtype=torch.uint8).cuda()
        pool[:, epb * 64:epb * 68] = torch.randint(120, 131, (pool.size(0), epb * 4), generator=gen, dtype=torch.uint8).cuda()
        return
    keys = torch.randint(0, 0x7E, (pool.size(0), epb * 128), generator=gen, dtype=torch.uint8)
    keys |= (torch.randint(0, 2, keys.shape, generator=gen, dtype=torch.uint8) << 7)
    scales = torch.rand(pool.size(0), epb, generator=gen) * 0.09 + 0.01
    pool[:, :epb * 128] = keys.cuda()
    pool[:, epb * 128:epb * 132] = scales.view(torch.uint8).cuda()


def check_step(stage, cache, host, st, m, before):
    """`before` holds copies of the pools taken before the step."""
    assert int(stage.status.item()) == 0
    pos = st["pos"].cpu().numpy()
    cos, sin = host["cos_table"], host["sin_table"]
    # 1 q RMSNorm + power-of-two quantisation
    normed = oracle.rmsnorm_bf16(u16(stage.q_raw[:m]), host["q_norm"], 1e-6)
    ref_q, ref_s = oracle.act_quant_fp8(normed, 128, round_scale=True)
    q8, qs = stage.q_fp8[:m].cpu().numpy(), stage.q_scales[:m].cpu().numpy()
    assert np.mean(q8 == ref_q) >= 0.995 and np.mean(qs == ref_s) >= 0.99
    # 2 projection, on the GPU's own quantised activations
    y = u16(stage.y[:m])
    ref_y = oracle.gemm_fp8_blockscaled(q8, qs, host["wq_b"], host["wq_b_scales"])
    yf, rf = oracle.bf16_to_f32(y), oracle.bf16_to_f32(ref_y)
    assert np.all(np.abs(yf - rf) <= 1e-2 * np.abs(rf) + 1e-3 * np.abs(rf).max())
    n_index = INDEX_HEADS * 128
    # 3 query RMSNorm + RoPE, 4 indexer-q post: exact on the GPU's y
    ref_qm = oracle.query_rms_rope(y[:, n_index:].reshape(m, MAIN_HEADS, 512), pos, cos, sin, out_heads=OUT_HEADS)
    assert np.array_equal(u16(stage.q_main[:m]), ref_qm)
    fp4 = stage.indexer_fp4
    if fp4:    # codes at the start of the iq buffer, the scale words where the folded weights would be
        q4 = stage.iq_fp8.view(-1)[:m * INDEX_HEADS * 64].view(m, INDEX_HEADS, 64).cpu().numpy()
        q_sf = stage.w_folded.view(torch.int32)[:m].cpu().numpy().view(np.uint32)
        ref_q4, ref_sf = oracle.index_q_post_fp4(y[:, :n_index].reshape(m, INDEX_HEADS, 128), pos.astype(np.int32), cos, sin)
        assert np.array_equal(q4, ref_q4) and np.array_equal(q_sf, ref_sf)
    else:
        ref_iq, ref_w = oracle.index_q_post_fp8(y[:, :n_index].reshape(m, INDEX_HEADS, 128), pos.astype(np.int32), cos,
                                                sin, stage.w64[:m].cpu().numpy())
        assert np.array_equal(stage.iq_fp8[:m].cpu().numpy(), ref_iq)
        assert np.array_equal(stage.w_folded[:m].cpu().numpy(), ref_w)
    # 5 cache writers
    ring = cache.state_ring_entries
    pools = {k: v.copy() for k, v in before.items()}
    rows = st["main_state_row"].cpu().numpy()
    (oracle.indexer_compressor_fp4 if fp4 else oracle.indexer_compressor_fp8)(
        cache.idx_state.cpu().numpy().reshape(-1, ring, 512), rows, pos, host["idx_norm"], cos, sin, pool=pools["idx"],
        dst=st["idx_dst"].cpu().numpy(), epb=cache.entries_per_block["idx"])
    oracle.main_compressor_fp8(cache.main_state.cpu().numpy().reshape(-1, ring, 2048), rows, pos, host["main_norm"], cos,
                               sin, pool=pools["cmp"], dst=st["cmp_dst"].cpu().numpy(),
                               epb=cache.entries_per_block["cmp"])
    oracle.window_kv_fp8(stage.win_y2[:m].cpu().numpy(), pos, host["win_norm"], cos, sin, pool=pools["swa"],
                         dst=st["swa_dst"].cpu().numpy(), epb=cache.entries_per_block["swa"])
    got = dict(idx=cache.idx_pool.cpu().numpy(), cmp=cache.cmp_pool.cpu().numpy(), swa=cache.swa_pool.cpu().numpy())
    assert np.array_equal(got["swa"], pools["swa"])
    for name in ("idx", "cmp"):
        changed = pools[name] != before[name]
        assert not np.any((got[name] != before[name]) & ~changed)       # nothing outside the written records moves
        assert np.mean(got[name] == pools[name]) >= 1 - 1e-5          # a handful of bytes may differ (expf)
    # 6 logits over the GPU's pool with the GPU's q, 7 top-k over the GPU's logits
    ncmp = stage.n_compressed[:m].cpu().numpy()
    assert np.array_equal(ncmp, (pos + 1) // 4)
    bt, cmp_bt = stage.block_table[:m].cpu().numpy(), stage.cmp_block_table[:m].cpu().numpy()
    assert not np.array_equal(bt, cmp_bt)    # the two pools number their pages differently here
    logits = stage.logits[:m].cpu().numpy()
    valid = np.arange(stage.logits_stride)[None, :] < ncmp[:, None]
    assert np.all(np.isfinite(logits[valid]))
    if fp4:
        ref_l = oracle.mqa_logits_fp4(q4, q_sf, got["idx"], stage.w64[:m].cpu().numpy(), ncmp, bt,
                                      cache.entries_per_block["idx"], stage.logits_stride)
        rms = np.sqrt(np.mean(ref_l[valid].astype(np.float64) ** 2))
        assert np.all(np.abs(logits[valid] - ref_l[valid]) <= 1e-4 * np.abs(ref_l[valid]) + 1e-5 * rms)
    else:
        ref_l = oracle.mqa_logits_fp8(stage.iq_fp8[:m].cpu().numpy(), got["idx"], stage.w_folded[:m].cpu().numpy(),
                                      ncmp.reshape(m, 1), bt, 1, cache.entries_per_block["idx"], stage.logits_stride)
        rms = np.sqrt(np.mean(ref_l[valid].astype(np.float64) ** 2))
        assert np.all(np.abs(logits[valid] - ref_l[valid]) <= 1e-2 * np.abs(ref_l[valid]) + 1e-4 * rms)
    masked = np.where(valid, logits, -np.inf).astype(np.float32)
    # positions are translated with the pages of the compressed-KV pool, which the attention reads
    ref_pages, ref_raw = oracle.topk(masked, ncmp, cmp_bt, TOPK, cache.entries_per_block["cmp"])
    got_pages, got_raw = stage.topk_indices[:m].cpu().numpy(), stage.topk_raw[:m].cpu().numpy()
    for r in range(m):
        assert sorted(got_raw[r].tolist()) == sorted(ref_raw[r].tolist())
        assert sorted(got_pages[r].tolist()) == sorted(ref_pages[r].tolist())


@pytest.mark.parametrize("cmp_epb,max_pages,fp4", [(None, 8, False), (32, 16, False), (None, 8, True)])
def test_steps_eager_then_graph(wuda, cmp_epb, max_pages, fp4):
    """The second case gives the compressed-KV pool pages half the size of the indexer pool's: the
    top-k positions must be translated with the compressed pool's page size, the logits read with
    the indexer pool's.  The third runs the FP4 form of the indexer (Hadamard + MXFP4 query and keys)."""
    batch = 5
    stage, cache, host, gen = make_stage(batch, 1234, cmp_epb, max_pages, fp4)
    assert stage.indexer_fp4 == fp4
    if cmp_epb is not None:
        assert cache.entries_per_block["cmp"] == cmp_epb != cache.entries_per_block["idx"]
    slots = [cache.alloc_request() for _ in range(batch)]
    fast_forward(cache, slots, [397, 802, 1, 530, 1199], gen)
    graph = None
    for step in range(9):
        m = batch
        st = stage.prepare(slots)
        stage.q_raw[:m] = (torch.randn(m, Q_LORA, generator=gen) * 2).bfloat16().cuda()
        stage.w64[:m] = (torch.randn(m, INDEX_HEADS, generator=gen) / 8).cuda()
        stage.win_y2[:m] = torch.randn(m, 512, generator=gen).cuda()
        # what the front GEMM publishes: this token's fresh state-ring entries
        rows = st["main_state_row"]
        cache.main_state.view(-1, 2048)[rows] = torch.randn(m, 2048, generator=gen).cuda()
        cache.idx_state.view(-1, 512)[rows] = torch.randn(m, 512, generator=gen).cuda()
        stage.logits.fill_(float("-inf"))
        before = dict(idx=cache.idx_pool.cpu().numpy(), cmp=cache.cmp_pool.cpu().numpy(), swa=cache.swa_pool.cpu().numpy())
        if step < 4:
            stage.launch(m)
        else:
            if graph is None:
                graph = stage.capture(m)          # runs the step itself (eagerly, then once more while capturing)
            stage.replay()
        torch.cuda.synchronize()
        check_step(stage, cache, host, st, m, before)
    assert graph is not None


def test_rejects_bad_arguments(wuda):
    stage, cache, host, gen = make_stage(2, 5)
    with pytest.raises(ValueError):
        stage.prepare([])
    with pytest.raises(wuda.WudaError, match=r"m must be"):
        stage.launch(0)
