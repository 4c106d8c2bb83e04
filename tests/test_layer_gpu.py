"""The attention half-layer as one launch sequence (wuda_b200.layer.AttentionHalfLayer): the stages are
tested one by one elsewhere; here the glue is - that every stage reads what the stage before wrote.  The
sparse attention is recomputed by the CPU oracle from the chain's own device buffers (the query the chain
normalised, the cache pools its writers filled, the top-k entries it translated with the compressed-KV
page table), and a replay of the captured CUDA graph must reproduce the eager pass bit for bit."""
import numpy as np
import pytest
import torch

import oracle
from wuda_b200 import o_proj
from wuda_b200.decode import CsaWeights
from wuda_b200.kv_cache import KVCacheManager
from wuda_b200.layer import AttentionHalfLayer, HalfLayerWeights

pytestmark = pytest.mark.gpu

HIDDEN, Q_LORA, INDEX_HEADS, MAIN_HEADS, TOPK = 7168, 1536, 64, 128, 512


def u16(t):
    return t.cpu().view(torch.int16).numpy().view(np.uint16)


def build(batch, contexts):
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(21)
    rnd8 = lambda *s: torch.randint(0, 0x7E, s, generator=g, dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn)
    sc = lambda *s: torch.rand(s, generator=g, device=dev) * 1e-3 + 1e-4
    n_total = INDEX_HEADS * 128 + MAIN_HEADS * 512
    ang = torch.outer(torch.arange(8192, dtype=torch.float32), 1.0 / (10000.0 ** (torch.arange(32) / 32.0))).to(dev)
    cos, sin = torch.cos(ang).contiguous(), torch.sin(ang).contiguous()
    csa = CsaWeights(rnd8(n_total, Q_LORA), sc(n_total // 128, Q_LORA // 128), torch.rand(Q_LORA, generator=g, device=dev) + 0.5,
                     torch.rand(128, generator=g, device=dev) + 0.5, torch.rand(512, generator=g, device=dev) + 0.5,
                     torch.rand(512, generator=g, device=dev) + 0.5, cos, sin, index_heads=INDEX_HEADS, main_heads=MAIN_HEADS)
    hw = HalfLayerWeights(
        hc_weight=torch.randn(24, 4 * HIDDEN, generator=g, device=dev) * 0.01, hc_base=torch.zeros(24, device=dev),
        hc_scale=torch.ones(3, device=dev), attn_norm=torch.ones(HIDDEN, dtype=torch.bfloat16, device=dev),
        front_w8=rnd8(2048, HIDDEN), front_w8_scales=sc(16, HIDDEN // 128),
        front_w16=(torch.randn(2624, HIDDEN, generator=g, device=dev) * 0.02).bfloat16(),
        ape=torch.randn(4, 1024, generator=g, device=dev), idx_ape=torch.randn(4, 256, generator=g, device=dev),
        o_proj=o_proj.OProjWeights(rnd8(16, 1024, 4096), sc(16 * 8, 32), rnd8(HIDDEN, 16384), sc(56, 128)),
        attn_sink=torch.randn(MAIN_HEADS, generator=g, device=dev))
    cache = KVCacheManager(batch + 1, 40, 12, device=dev)
    cache._pools["cmp"].take()            # the compressed-KV pool numbers its pages one off the indexer pool's
    slots = [cache.alloc_request() for _ in range(batch)]
    for s, n in zip(slots, contexts):
        cache.advance(s, n - 1)
    # the entries earlier steps would have written: random finite indexer keys and MODEL1 records
    epb = cache.entries_per_block["idx"]
    pool = cache.idx_pool
    pool[:, :epb * 128] = torch.randint(0, 0x7E, (pool.size(0), epb * 128), generator=g, dtype=torch.uint8, device=dev)
    pool[:, epb * 128:epb * 132] = (torch.rand(pool.size(0), epb, generator=g, device=dev) * 0.09 + 0.01).view(torch.uint8)
    for name in ("swa", "cmp"):
        data, e = cache._pools[name].data, cache.entries_per_block[name]
        body = torch.randint(0, 256, (data.size(0), e, 576), generator=g, device=dev, dtype=torch.int32)
        body = torch.where((body & 0x7f) == 0x7f, body & 0x80, body)
        body[..., 449::2] = (body[..., 449::2] & 0x80) | 0x3e | (body[..., 449::2] & 1)     # bf16 high bytes: |x| < 1
        data[:, :e * 576] = body.to(torch.uint8).reshape(data.size(0), e * 576)
        sb = torch.zeros(data.size(0), e, 8, dtype=torch.uint8, device=dev)
        sb[..., :7] = torch.randint(115, 122, (data.size(0), e, 7), generator=g, device=dev).to(torch.uint8)
        data[:, e * 576:e * 584] = sb.reshape(data.size(0), e * 8)
    cache.main_state.normal_(generator=g)
    cache.idx_state.normal_(generator=g)
    layer = AttentionHalfLayer(csa, hw, cache, batch, topk=TOPK)
    x = torch.randn(batch, 4, HIDDEN, generator=g, device=dev).bfloat16()
    return layer, cache, slots, x


def test_half_layer_stages_feed_each_other():
    batch, contexts = 3, [700, 131, 2900]       # one request whose compressed history exceeds the top-k
    layer, cache, slots, x = build(batch, contexts)
    layer.prepare(slots)
    out = layer.launch(x, batch).clone()
    torch.cuda.synchronize()
    layer.check_status()
    assert tuple(out.shape) == (batch, 4, HIDDEN) and bool(torch.isfinite(out.float()).all())
    st = layer.stage
    ncmp = st.n_compressed[:batch].cpu().numpy()
    assert np.array_equal(ncmp, np.asarray(contexts) // 4)
    # the attention read the chain's query, the pools after this step's cache writers, the translated top-k
    swa = (cache.swa_pool.cpu().numpy(), cache.entries_per_block["swa"], layer.swa_idx[:batch].cpu().numpy(),
           layer.swa_len[:batch].cpu().numpy())
    cmp = (cache.cmp_pool.cpu().numpy(), cache.entries_per_block["cmp"], st.topk_indices[:batch].cpu().numpy(),
           layer.cmp_len[:batch].cpu().numpy())
    assert np.array_equal(swa[3], np.minimum(np.asarray(contexts), 128))
    assert np.array_equal(cmp[3], np.minimum(ncmp, TOPK))
    ref = oracle.sparse_mla(u16(st.q_main[:batch]), swa, cmp, layer.w.attn_sink.cpu().numpy(), 512 ** -0.5)
    got = oracle.bf16_to_f32(u16(layer.mla_out[:batch])).astype(np.float64)
    row_max = np.abs(ref).max(axis=-1, keepdims=True)
    assert np.all(np.abs(got - ref) <= row_max * 2.0 ** -7 + 1e-6)
    # the translated entries are the compressed-KV pool's pages of the request, not the indexer pool's
    bt = st.cmp_block_table[:batch].cpu().numpy()
    for b in range(batch):
        pages = set((cmp[2][b, :cmp[3][b]] // 64).tolist())
        assert pages <= set(bt[b].tolist())
    # the captured graph reproduces the eager pass (same inputs, same state rows, same destinations)
    layer.capture(x, batch)
    again = layer.replay()
    torch.cuda.synchronize()
    layer.check_status()
    assert torch.equal(out, again)
