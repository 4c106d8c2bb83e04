"""A random-init decode layer at the model's geometry (hidden 7168, q_lora 1536, 64 index heads x 128,
128 query heads x 512, 16 output groups x 1024, compress ratio 4, window 128, 256 routed NVFP4 experts of
intermediate 2048 with top-8 routing, one FP8 shared expert), for the benchmarks and the layer tests.

All random draws are made for the whole layer from one seed and then cut to what a rank holds, so that a
tensor-parallel pair and a single GPU see the same weights, caches and inputs.
"""
import torch

from . import moe, o_proj
from .decode import CsaWeights
from .kv_cache import KVCacheManager
from .layer import AttentionHalfLayer, DecoderLayer, FfnWeights, HalfLayerWeights

HIDDEN, Q_LORA, INDEX_HEADS, MAIN_HEADS, GROUPS = 7168, 1536, 64, 128, 16


def model1_pool(pages, epb, seed, device="cuda"):
    """uint8 [pages, stride] pool of random MODEL1 records (finite e4m3, exponents near 0, small bf16)."""
    g = torch.Generator(device=device).manual_seed(seed)
    stride = -(-epb * 584 // 576) * 576
    pool = torch.zeros(pages, stride, dtype=torch.uint8, device=device)
    body = torch.randint(0, 256, (pages, epb, 576), generator=g, device=device, dtype=torch.int32)
    body = torch.where((body & 0x7f) == 0x7f, body & 0x80, body)
    body[..., 449::2] = (body[..., 449::2] & 0x80) | 0x3e | (body[..., 449::2] & 1)   # bf16 high bytes: |x| in [0.1, 0.6)
    pool[:, :epb * 576] = body.to(torch.uint8).reshape(pages, epb * 576)
    sb = torch.zeros(pages, epb, 8, dtype=torch.uint8, device=device)
    sb[..., :7] = torch.randint(115, 122, (pages, epb, 7), generator=g, device=device).to(torch.uint8)
    pool[:, epb * 576:epb * 584] = sb.reshape(pages, epb * 8)
    return pool


def _fp8_weight(g, n, k, device, pow2=True):
    """Random e4m3 bytes of moderate magnitude (exponent field <= 8: |w| <= 3.75) with both signs, and
    128x128 block scales around 1e-2, so that a K = 7168 product stays O(1); with pow2 the scales are rounded to
    powers of two, the form the reference's checkpoints hold (UE8M0)."""
    b = torch.randint(0, 0x48, (n, k), generator=g, dtype=torch.uint8, device=device)
    sign = torch.randint(0, 2, (n, k), generator=g, dtype=torch.uint8, device=device) << 7
    scales = torch.rand(((n + 127) // 128, k // 128), generator=g, device=device) * 1e-2 + 5e-3
    if pow2:
        scales = torch.exp2(torch.log2(scales).round())
    return (b | sign).view(torch.float8_e4m3fn), scales


def build_random_layer(batch, context, topk=2048, rank=0, world=1, tp_link=None, ep_link=None, seed=11,
                       experts=256, inter=2048, moe_topk=8, device="cuda", peer_wait_ms=2000, native=True, pow2_scales=True,
                       indexer_fp4=False):
    """Returns (layer, slots, hidden_states): a DecoderLayer whose requests all stand at position context - 1
    (the timed token), the request slots, and bf16 [batch, 4, hidden] residual streams.  world = 2 builds what
    rank `rank` of a tensor-parallel pair holds and needs both links.  pow2_scales: FP8 weight scales are powers
    of two (as in the reference's checkpoints) and the projections that gain from it apply them in the tensor core.
    indexer_fp4: the indexer pool holds MXFP4 records and the step takes the FP4 forms of the indexer's kernels."""
    if world not in (1, 2) or (world == 2 and (tp_link is None or ep_link is None)):
        raise ValueError("world must be 1, or 2 with both links")
    dev = device
    g = torch.Generator(device=dev).manual_seed(seed)
    hidden = HIDDEN
    heads = MAIN_HEADS // world
    rnd = lambda *s, scale=1.0: torch.randn(*s, generator=g, device=dev) * scale
    n_index = INDEX_HEADS * 128
    # ---- attention half
    wq_b, wq_b_s = _fp8_weight(g, n_index + MAIN_HEADS * 512, Q_LORA, dev, pow2_scales)
    ang = torch.outer(torch.arange(65536, dtype=torch.float32), 1.0 / (10000.0 ** (torch.arange(32) / 32.0))).to(dev)
    cos, sin = torch.cos(ang).contiguous(), torch.sin(ang).contiguous()
    norms = [torch.rand(n, generator=g, device=dev) + 0.5 for n in (Q_LORA, 128, 512, 512)]
    if world == 2:
        lo = n_index + rank * heads * 512
        rows = torch.cat([torch.arange(n_index, device=dev), torch.arange(lo, lo + heads * 512, device=dev)])
        wq_b = wq_b.view(torch.uint8)[rows].contiguous().view(torch.float8_e4m3fn)
        wq_b_s = wq_b_s[torch.cat([torch.arange(n_index // 128, device=dev),
                                   torch.arange(lo // 128, (lo + heads * 512) // 128, device=dev)])].contiguous()
    csa = CsaWeights(wq_b, wq_b_s, *norms, cos, sin, index_heads=INDEX_HEADS, main_heads=heads, scales_pow2=pow2_scales)
    front_w8, front_w8_s = _fp8_weight(g, 2048, hidden, dev, pow2_scales)
    wo_a, wo_a_s = _fp8_weight(g, GROUPS * 1024, 4096, dev, pow2_scales)
    wo_b, wo_b_s = _fp8_weight(g, hidden, GROUPS * 1024, dev, pow2_scales)
    sink = rnd(MAIN_HEADS)
    if world == 2:
        gpr = GROUPS // 2
        wo_a = wo_a.view(torch.uint8)[rank * gpr * 1024:(rank + 1) * gpr * 1024].contiguous().view(torch.float8_e4m3fn)
        wo_a_s = wo_a_s[rank * gpr * 8:(rank + 1) * gpr * 8].contiguous()
        kh = GROUPS * 1024 // 2
        wo_b = wo_b.view(torch.uint8)[:, rank * kh:(rank + 1) * kh].contiguous().view(torch.float8_e4m3fn)
        wo_b_s = wo_b_s[:, rank * kh // 128:(rank + 1) * kh // 128].contiguous()
        sink = sink[rank * heads:(rank + 1) * heads].contiguous()
    hw = HalfLayerWeights(
        hc_weight=rnd(24, 4 * hidden, scale=0.01), hc_base=torch.zeros(24, device=dev), hc_scale=torch.ones(3, device=dev),
        attn_norm=(rnd(hidden, scale=0.1) + 1.0).bfloat16(), front_w8=front_w8, front_w8_scales=front_w8_s,
        front_w16=rnd(2624, hidden, scale=0.02).bfloat16(), ape=rnd(4, 1024), idx_ape=rnd(4, 256),
        o_proj=o_proj.OProjWeights(wo_a.view(GROUPS // world, 1024, 4096), wo_a_s, wo_b, wo_b_s, scales_pow2=pow2_scales),
        attn_sink=sink)
    # ---- caches: every request stands one token before `context`
    pages_per_req = (context // 4 + 63) // 64 + 1
    cache = KVCacheManager(batch, batch * pages_per_req + batch, pages_per_req, device=dev, indexer_fp8=not indexer_fp4)
    slots = [cache.alloc_request() for _ in range(batch)]
    for s_ in slots:
        cache.advance(s_, context - 1)
    epb = cache.entries_per_block["idx"]
    pool = cache.idx_pool
    if indexer_fp4:   # any e2m1 codes, exponent bytes around one
        pool[:, :epb * 64] = torch.randint(0, 256, (pool.size(0), epb * 64), generator=g, dtype=torch.uint8, device=dev)
        pool[:, epb * 64:epb * 68] = torch.randint(120, 131, (pool.size(0), epb * 4), generator=g, dtype=torch.uint8, device=dev)
    else:
        pool[:, :epb * 128] = torch.randint(0, 0x7E, (pool.size(0), epb * 128), generator=g, dtype=torch.uint8, device=dev)
        pool[:, epb * 128:epb * 132] = (torch.rand(pool.size(0), epb, generator=g, device=dev) * 0.09 + 0.01).view(torch.uint8)
    cache.main_state.normal_(generator=g)
    cache.idx_state.normal_(generator=g)
    for i, name in enumerate(("swa", "cmp")):   # attention caches: random finite records instead of a fresh pool's zeros
        data = cache._pools[name].data
        epb_m = cache.entries_per_block[name]
        data[:, :epb_m * 584] = model1_pool(data.size(0), epb_m, seed + 5 + i, dev)[:, :epb_m * 584]
    attention = AttentionHalfLayer(csa, hw, cache, batch, topk=topk, tp_link=tp_link)
    # ---- feed-forward half
    gate_w = rnd(experts, hidden, scale=0.05).bfloat16()
    w13, w13_s = _fp8_weight(g, 2 * inter, hidden, dev, pow2_scales)      # rows [0, inter) = w1 (gate), [inter, 2*inter) = w3 (up)
    w2, w2_s = _fp8_weight(g, hidden, inter, dev, pow2_scales)
    all_experts = moe.RandomRoutedExperts(experts, inter, hidden, device=dev, seed=seed + 1)
    first = 0
    if world == 2:
        ih = inter // 2
        rows = torch.cat([torch.arange(rank * ih, (rank + 1) * ih, device=dev),
                          torch.arange(inter + rank * ih, inter + (rank + 1) * ih, device=dev)])
        w13 = w13.view(torch.uint8)[rows].contiguous().view(torch.float8_e4m3fn)
        w13_s = w13_s[torch.cat([torch.arange(rank * ih // 128, (rank + 1) * ih // 128, device=dev),
                                 torch.arange((inter + rank * ih) // 128, (inter + (rank + 1) * ih) // 128, device=dev)])].contiguous()
        w2 = w2.view(torch.uint8)[:, rank * ih:(rank + 1) * ih].contiguous().view(torch.float8_e4m3fn)
        w2_s = w2_s[:, rank * ih // 128:(rank + 1) * ih // 128].contiguous()
        per = experts // 2
        first = rank * per
        all_experts.dev = {k: v[first:first + per].clone() for k, v in all_experts.dev.items()}
        all_experts.experts = per
        torch.cuda.empty_cache()
    ffn = FfnWeights(hc_weight=rnd(24, 4 * hidden, scale=0.01), hc_base=torch.zeros(24, device=dev),
                     hc_scale=torch.ones(3, device=dev), ffn_norm=(rnd(hidden, scale=0.1) + 1.0).bfloat16(),
                     gate_weight=gate_w, gate_bias=torch.zeros(experts, device=dev), routed=all_experts,
                     shared=moe.SharedExpert(w13, w13_s, w2, w2_s), experts_total=experts, expert_first=first,
                     topk=moe_topk, route_scale=2.5)
    layer = DecoderLayer(attention, ffn, batch, ep_link=ep_link, peer_wait_ms=peer_wait_ms, native=native)
    x = rnd(batch, 4, hidden).bfloat16()
    return layer, slots, x


def layer_weight_bytes(world=1, experts_active=None, experts=256, inter=2048):
    """Bytes of weights one rank streams per layer pass (FP8 / BF16 / NVFP4 as stored), for roofline figures:
    replicated mixes and front projection, this rank's share of the q / output projections and of the shared
    expert, and `experts_active` routed experts (default: all of the rank's)."""
    hidden = HIDDEN
    n_q = INDEX_HEADS * 128 + MAIN_HEADS * 512 // world
    attn = (2 * 24 * 4 * hidden * 4 + 2048 * hidden + 2624 * hidden * 2 + n_q * Q_LORA + GROUPS // world * 1024 * 4096
            + hidden * GROUPS * 1024 // world)
    shared = 3 * hidden * inter // world
    per_expert = 3 * (hidden * inter // 2 + hidden * inter // 16)
    gate = experts * hidden * 2
    active = experts // world if experts_active is None else experts_active
    return attn + shared + gate + active * per_expert
