"""Per-operator timing tables for the rows of the hot path that bench.py (the indexer
step) does not cover.  Device time with CUDA events over CUDA-graph replays, cold L2
between launches is not forced: weights (>= 15 MB) are re-streamed from HBM every launch
because consecutive launches use different weight buffers that together exceed L2.

    python -m wuda_b200.benchmarks gemm_fp8
    python -m wuda_b200.benchmarks gemm_fp8_pow2                   (power-of-two scales applied inside the tensor core)
    python -m wuda_b200.benchmarks gemm_fp8_fp4                    (FP8 activations x FP4 weights: the origin's fp4_gemm)
    python -m wuda_b200.benchmarks gemm_nvfp4
    python -m wuda_b200.benchmarks norm_rope_quant
    python -m wuda_b200.benchmarks csa_chain                       (layer launch of the indexer half-step)
    python -m wuda_b200.benchmarks csa_chain_fp4                   (the same with the indexer in its FP4 form)
    python -m wuda_b200.benchmarks csa_chain_launches              (three eager steps, for an ncu launch list)
    python -m wuda_b200.benchmarks attention_half_layer            (every built stage of the half-layer, one graph)
    python -m wuda_b200.benchmarks attention_half_layer_launches   (three eager passes, for an ncu launch list)
    python -m wuda_b200.benchmarks moe_experts                     (router + routed NVFP4 experts of one MoE block)
    python -m wuda_b200.benchmarks moe_experts_launches            (two eager passes, for an ncu launch list)
    python -m wuda_b200.benchmarks topk                            (top-2048 over L2-resident rows: the layer's and the bench's shapes)
    python -m wuda_b200.benchmarks mqa_fp4                         (MXFP4 paged MQA logits)
    python -m wuda_b200.benchmarks mqa_fp4_launches                (three eager launches at batch 64 x 32768, for ncu)
    python -m wuda_b200.benchmarks sparse_mla                      (sparse MLA decode attention, window 128 + top-2048)
    python -m wuda_b200.benchmarks sparse_mla_launches             (three eager launches of a small case, for ncu)
    python -m wuda_b200.benchmarks one gemm_fp8 64 24576 7168      (a few launches of one shape, for ncu)
    python -m wuda_b200.benchmarks layer                          (the whole decode layer, one graph: tok/s/GPU)
    python -m wuda_b200.benchmarks layer_launches                 (two eager passes of the layer, for an ncu launch list)
    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 -m wuda_b200.benchmarks layer_tp2
    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 -m wuda_b200.benchmarks tp2
    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 -m wuda_b200.benchmarks moe_ep2
"""
import json
import os
import sys

import numpy as np
import torch

import wuda_b200 as wuda
from wuda_b200 import workloads
from wuda_b200.layer_setup import model1_pool

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), float(p["bf16_tflops"]), "measured"
    except Exception:
        return 6650.0, 1590.0, "fallback"


def time_graph(fn, reps=20, inner=10):
    """Mean device time (us) of one call of fn, from graphs of `inner` calls."""
    fn()
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            for _ in range(inner):
                fn()
    torch.cuda.synchronize()
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / (reps * inner)


def gemm_fp8(pow2=False):
    hbm, tf, kind = peaks()
    print("block-scaled FP8 GEMM%s, bf16 out; peaks (%s): %.0f GB/s HBM, %.0f TFLOP/s dense bf16 (fp8 nominal = 2x)"
          % (" with power-of-two scales applied in the tensor core" if pow2 else "", kind, hbm, tf))
    print("%6s %6s %6s %9s %9s %8s %9s %8s" % ("M", "N", "K", "us", "GB/s", "of HBM", "TFLOP/s", "of 2xbf16"))
    shapes = ((24576, 7168), (7168, 16384), (2112, 7168), (4096, 7168)) + (((73728, 1536),) if pow2 else ())
    for n, k in shapes:
        for m in (1, 8, 32, 64, 128, 256):
            # enough distinct weight buffers that a launch never finds its weights in the 126 MB L2
            copies = max(2, int(300e6 // (n * k)) + 1)
            cases = [workloads.make_gemm_fp8_case(m, n, k, seed=7)]
            a = torch.from_numpy(cases[0]["a"]).cuda().view(torch.float8_e4m3fn)
            a_s = torch.from_numpy(cases[0]["a_s"]).cuda()
            w0 = torch.from_numpy(cases[0]["w"]).cuda()
            ws = [w0.clone().view(torch.float8_e4m3fn) for _ in range(copies)]
            w_s = torch.from_numpy(cases[0]["w_s"]).cuda()
            if pow2:
                a_s, w_s = torch.exp2(torch.log2(a_s).round()), torch.exp2(torch.log2(w_s).round())
            out = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
            state = {"i": 0}

            def fn():
                wuda.fp8_gemm(a, a_s, ws[state["i"] % copies], w_s, out=out, pow2_scales=pow2)
                state["i"] += 1

            us = time_graph(fn, reps=10, inner=copies * 2)
            by = workloads.gemm_fp8_algorithmic_bytes(m, n, k)
            gbs = by / us / 1e3
            tfl = 2.0 * m * n * k / us / 1e6
            print("%6d %6d %6d %9.1f %9.0f %7.1f%% %9.1f %7.1f%%" % (m, n, k, us, gbs, 100 * gbs / hbm, tfl, 100 * tfl / (2 * tf)))
            del ws


def gemm_fp8_fp4():
    """FP8 activations x FP4 weights (the origin's fp4_gemm).  Operands are random bytes made on the device (every
    byte pattern is a valid e2m1 pair; e4m3 bytes avoid the two NaN codes); results are checked by the tests."""
    hbm, tf, kind = peaks()
    print("FP8 x FP4 GEMM (e8m0 scales per 32 weights), bf16 out; peaks (%s): %.0f GB/s HBM, %.0f TFLOP/s dense bf16" % (kind, hbm, tf))
    print("%6s %6s %6s %9s %9s %8s" % ("M", "N", "K", "us", "GB/s", "of HBM"))
    gen = torch.Generator(device="cuda").manual_seed(7)
    for n, k in ((24576, 7168), (7168, 16384), (4096, 7168), (7168, 2048)):
        copies = max(2, int(300e6 // (n * k // 2)) + 1)
        ws = [torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, device="cuda", generator=gen) for _ in range(copies)]
        w_sf = torch.randint(118, 126, (n, k // 32), dtype=torch.uint8, device="cuda", generator=gen)
        for m in (1, 8, 32, 64, 128, 256):
            a = torch.randint(0, 0x78, (m, k), dtype=torch.uint8, device="cuda", generator=gen).view(torch.float8_e4m3fn)
            a_s = torch.exp2(torch.randint(-4, 4, (m, k // 128), device="cuda", generator=gen).float())
            out = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
            state = {"i": 0}

            def fn():
                wuda.fp4_gemm(a, a_s, ws[state["i"] % copies], w_sf, out=out)
                state["i"] += 1

            us = time_graph(fn, reps=10, inner=copies * 2)
            by = n * k // 2 + n * k // 32 + m * k + m * (k // 128) * 4 + m * n * 2
            gbs = by / us / 1e3
            print("%6d %6d %6d %9.1f %9.0f %7.1f%%" % (m, n, k, us, gbs, 100 * gbs / hbm))
        del ws


def gemm_nvfp4():
    hbm, tf, kind = peaks()
    print("NVFP4 block-scaled GEMM, bf16 out; peaks (%s): %.0f GB/s HBM, %.0f TFLOP/s dense bf16 (fp4 nominal = 4x)" % (kind, hbm, tf))
    print("%6s %6s %6s %9s %9s %8s %9s %8s" % ("M", "N", "K", "us", "GB/s", "of HBM", "TFLOP/s", "of 4xbf16"))
    for n, k in ((24576, 7168), (7168, 16384), (2112, 7168), (4096, 7168)):
        base = workloads.make_gemm_nvfp4_case(128, n, k, seed=7)
        t = lambda x: torch.from_numpy(x).cuda()
        copies = max(2, int(300e6 // (n * k // 2)) + 1)
        ws = [t(base["w"]).clone() for _ in range(copies)]
        w_sf = t(base["w_sf_packed"])
        for m in (1, 8, 32, 64, 128):
            a = t(np.ascontiguousarray(base["a"][:m]))
            a_sf = t(workloads.pack_nvfp4_scales(base["a_sf"][:m]))
            out = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
            state = {"i": 0}

            def fn():
                wuda.nvfp4_gemm(a, a_sf, base["a_gs"], ws[state["i"] % copies], w_sf, base["w_gs"], out=out)
                state["i"] += 1

            us = time_graph(fn, reps=10, inner=copies * 2)
            by = workloads.gemm_nvfp4_algorithmic_bytes(m, n, k)
            gbs = by / us / 1e3
            tfl = 2.0 * m * n * k / us / 1e6
            print("%6d %6d %6d %9.1f %9.0f %7.1f%% %9.1f %7.1f%%" % (m, n, k, us, gbs, 100 * gbs / hbm, tfl, 100 * tfl / (4 * tf)))
        del ws


def norm_rope_quant():
    hbm, _, kind = peaks()
    print("fused RMSNorm+quant and RoPE+quant; HBM peak (%s) %.0f GB/s" % (kind, hbm))
    for tokens in (1, 64, 256):
        g = torch.Generator().manual_seed(1)
        x = torch.randn(tokens, 7168, generator=g).bfloat16().cuda()
        gamma = torch.ones(7168).bfloat16().cuda()
        us = time_graph(lambda: wuda.rmsnorm_quant(x, gamma, 1e-6))
        by = tokens * 7168 * 2 + 14336 + tokens * 7168 * 3 + tokens * 56 * 4
        print("rmsnorm_quant tokens %4d: %7.2f us %7.0f GB/s" % (tokens, us, by / us / 1e3))
        proj = torch.randn(tokens, 128, 192, generator=g).bfloat16().cuda()
        pos = torch.randint(0, 65536, (tokens,), generator=g).cuda()
        freqs = 1.0 / (10000 ** (torch.arange(0, 64, 2, dtype=torch.float32) / 64))
        ang = torch.outer(torch.arange(65536).float(), freqs)
        cos, sin = ang.cos().cuda().contiguous(), ang.sin().cuda().contiguous()
        us = time_graph(lambda: wuda.rope_quant(proj, pos, cos, sin, 64))
        by = tokens * 24576 * 2 + tokens * 8 + tokens * 24576 + tokens * 192 * 4
        print("rope_quant    tokens %4d: %7.2f us %7.0f GB/s" % (tokens, us, by / us / 1e3))
    # FP4 quantisation (the origin's fp4_act_quant): the indexer's keys in place, and a weight matrix larger than L2
    for rows, cols, inplace in ((64, 7168, False), (64 * 128, 128, True), (24576, 7168, False)):
        copies = 1 if rows * cols < (1 << 24) else 3
        xs = [torch.randn(rows, cols, device="cuda").bfloat16() for _ in range(copies)]
        state = {"i": 0}

        def fn():
            wuda.fp4_act_quant(xs[state["i"] % copies], 32, inplace)
            state["i"] += 1

        us = time_graph(fn, inner=copies * 2)
        by = rows * cols * (4 if inplace else 2) + (0 if inplace else rows * cols * 17 // 32)
        print("fp4_act_quant %6d x %5d%s: %7.2f us %7.0f GB/s = %.2f of HBM" %
              (rows, cols, " in place" if inplace else "         ", us, by / us / 1e3, by / us / 1e3 / hbm))


def tp2():
    """Run under torch.distributed.run with two ranks: wo_b-shaped GEMM (N 7168, K 16384 split in two)
    with the fused all-reduce, next to the same local GEMM without any exchange."""
    import torch.distributed as dist
    rank = int(os.environ["RANK"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("gloo")
    hbm, _, kind = peaks()
    for m in (1, 32, 64, 128):
        n, k = 7168, 16384
        case = workloads.make_gemm_fp8_case(m, n, k // 2, seed=11 + rank)
        a = torch.from_numpy(case["a"]).cuda().view(torch.float8_e4m3fn)
        a_s, w_s = torch.from_numpy(case["a_s"]).cuda(), torch.from_numpy(case["w_s"]).cuda()
        copies = 6
        ws = [torch.from_numpy(case["w"]).cuda().view(torch.float8_e4m3fn).clone() for _ in range(copies)]
        out = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
        link = wuda.TP2Link(m, n)
        status = wuda.device_status_word()
        state = {"i": 0}

        def fused():
            link.fp8_gemm(a, a_s, ws[state["i"] % copies], w_s, out=out, status_word=status)
            state["i"] += 1

        def local():
            wuda.fp8_gemm(a, a_s, ws[state["i"] % copies], w_s, out=out)
            state["i"] += 1

        def timed(fn, iters=60):
            for _ in range(5):
                fn()
            dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(iters):
                fn()
            e1.record()
            torch.cuda.synchronize()
            t = torch.tensor([e0.elapsed_time(e1) * 1e3 / iters], dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item())

        t_local = timed(local)
        t_fused = timed(fused)
        by = workloads.gemm_fp8_algorithmic_bytes(m, n, k // 2)
        link_bytes = m * n * 4
        bound = max(by / (hbm * 1e3), link_bytes / (770.0 * 1e3))
        if rank == 0:
            print("M %4d: local GEMM %6.1f us, fused GEMM+all-reduce %6.1f us (status %d); roofline max(HBM %.1f us, NVLink %.1f us) "
                  "-> %.0f%% of it; %.1f MB over the link per rank" %
                  (m, t_local, t_fused, int(status.item()), by / (hbm * 1e3), link_bytes / 770e3, 100 * bound / t_fused,
                   link_bytes / 1e6))
        dist.barrier()
        link.close()
    dist.destroy_process_group()


def csa_chain(batch=64, context=32768, topk=2048, reps=30, launches_only=0, indexer_fp4=False):
    """The layer launch of the indexer half of a decode step (wuda_csa_decode_step, seven kernels in
    one CUDA graph) at the model's geometry: q_lora 1536, 64 index heads, 128 main heads, `batch`
    requests at `context` tokens.  L2 is flushed before every timed replay.  indexer_fp4: the indexer
    in its FP4 form (Hadamard + MXFP4 query and keys, 68-byte records)."""
    from wuda_b200.decode import CsaDecodeStage, CsaWeights
    from wuda_b200.kv_cache import KVCacheManager
    hbm, tf, kind = peaks()
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(7)
    q_lora, ih, mh = 1536, 64, 128
    n_total = ih * 128 + mh * 512
    w8 = torch.randint(0, 0x7E, (n_total, q_lora), generator=g, dtype=torch.uint8, device=dev)
    ws = torch.rand((n_total // 128, q_lora // 128), generator=g, device=dev) * 1e-3 + 1e-4
    ang = torch.outer(torch.arange(65536, dtype=torch.float32), 1.0 / (10000.0 ** (torch.arange(32) / 32.0))).to(dev)
    weights = CsaWeights(w8, ws, torch.rand(q_lora, generator=g, device=dev) + 0.5,
                         torch.rand(128, generator=g, device=dev) + 0.5, torch.rand(512, generator=g, device=dev) + 0.5,
                         torch.rand(512, generator=g, device=dev) + 0.5, torch.cos(ang).contiguous(),
                         torch.sin(ang).contiguous(), index_heads=ih, main_heads=mh)
    pages_per_req = (context // 4 + 63) // 64 + 1
    cache = KVCacheManager(batch, batch * pages_per_req + batch, pages_per_req, device=dev, indexer_fp8=not indexer_fp4)
    stage = CsaDecodeStage(weights, cache, batch, topk=topk)
    slots = [cache.alloc_request() for _ in range(batch)]
    for s in slots:
        cache.advance(s, context - 1)               # the timed token is the one at position context - 1
    epb = cache.entries_per_block["idx"]
    pool = cache.idx_pool
    if indexer_fp4:
        pool[:, :epb * 64] = torch.randint(0, 256, (pool.size(0), epb * 64), generator=g, dtype=torch.uint8, device=dev)
        pool[:, epb * 64:epb * 68] = torch.randint(120, 131, (pool.size(0), epb * 4), generator=g, dtype=torch.uint8, device=dev)
    else:
        pool[:, :epb * 128] = torch.randint(0, 0x7E, (pool.size(0), epb * 128), generator=g, dtype=torch.uint8, device=dev)
        pool[:, epb * 128:epb * 132] = (torch.rand(pool.size(0), epb, generator=g, device=dev) * 0.09 + 0.01).view(torch.uint8)
    cache.main_state.normal_(generator=g)
    cache.idx_state.normal_(generator=g)
    st = stage.prepare(slots)
    assert int(st["pos"][0]) == context - 1 and int(st["idx_dst"][0]) >= 0
    stage.q_raw.normal_(generator=g)
    stage.w64.normal_(generator=g)
    stage.win_y2.normal_(generator=g)
    if launches_only:
        for _ in range(launches_only):
            stage.launch(batch)
        torch.cuda.synchronize()
        stage.check_status()
        print("csa_chain: %d eager steps done" % launches_only)
        return
    stage.capture(batch)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    total = 0.0
    for i in range(reps + 3):
        flush.fill_(i & 0xff)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        stage.replay()
        e1.record()
        torch.cuda.synchronize()
        if i >= 3:
            total += e0.elapsed_time(e1) * 1e3
    stage.check_status()
    us = total / reps
    ncmp = int(stage.n_compressed[0])
    bytes_step = (n_total * q_lora + batch * ncmp * (68 if indexer_fp4 else 132) + 2 * batch * ncmp * 4 + batch * n_total * 2 * 2
                  + batch * mh * 512 * 2)
    print("indexer half of a decode step%s: batch %d, context %d (%d indexer entries / request), top-%d" %
          (" (FP4 indexer)" if indexer_fp4 else "", batch, context, ncmp, topk))
    print("  %.1f us per step (L2 flushed before each) = %.0f tokens/s for this stage chain; %.1f MB algorithmic "
          "-> %.0f GB/s = %.2f of %s HBM peak" % (us, batch / us * 1e6, bytes_step / 1e6, bytes_step / us / 1e3,
                                                   bytes_step / us / 1e3 / hbm, kind))


def attention_half_layer(batch=64, context=32768, topk=2048, reps=30, launches_only=0):
    """Every built stage of the attention half-layer in order, one CUDA graph: mHC pre -> front mixed
    GEMM + FRONT-EMIT -> indexer half-step (q norm/quant, q projection, tails, cache writers, MQA
    logits, top-k) -> sparse MLA attention over the window and the top-k compressed records ->
    inverse RoPE + quant, grouped wo_a, quant, wo_b -> mHC post.  Model geometry (hidden 7168,
    128 heads of 512, 16 output groups), random weights, L2 flushed before every timed replay."""
    from wuda_b200 import o_proj
    from wuda_b200.decode import CsaDecodeStage, CsaWeights
    from wuda_b200.kv_cache import KVCacheManager
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(11)
    hidden, q_lora, ih, mh = 7168, 1536, 64, 128
    rnd8 = lambda *s: torch.randint(0, 0x7E, s, generator=g, dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn)
    sc = lambda *s: torch.rand(s, generator=g, device=dev) * 1e-3 + 1e-4
    n_total = ih * 128 + mh * 512
    ang = torch.outer(torch.arange(65536, dtype=torch.float32), 1.0 / (10000.0 ** (torch.arange(32) / 32.0))).to(dev)
    cos, sin = torch.cos(ang).contiguous(), torch.sin(ang).contiguous()
    weights = CsaWeights(rnd8(n_total, q_lora), sc(n_total // 128, q_lora // 128),
                         torch.rand(q_lora, generator=g, device=dev) + 0.5, torch.rand(128, generator=g, device=dev) + 0.5,
                         torch.rand(512, generator=g, device=dev) + 0.5, torch.rand(512, generator=g, device=dev) + 0.5,
                         cos, sin, index_heads=ih, main_heads=mh)
    pages_per_req = (context // 4 + 63) // 64 + 1
    cache = KVCacheManager(batch, batch * pages_per_req + batch, pages_per_req, device=dev)
    slots = [cache.alloc_request() for _ in range(batch)]
    for s_ in slots:
        cache.advance(s_, context - 1)
    epb = cache.entries_per_block["idx"]
    pool = cache.idx_pool
    pool[:, :epb * 128] = torch.randint(0, 0x7E, (pool.size(0), epb * 128), generator=g, dtype=torch.uint8, device=dev)
    pool[:, epb * 128:epb * 132] = (torch.rand(pool.size(0), epb, generator=g, device=dev) * 0.09 + 0.01).view(torch.uint8)
    cache.main_state.normal_(generator=g)
    cache.idx_state.normal_(generator=g)
    # weights of the other stages
    from wuda_b200.layer import AttentionHalfLayer, HalfLayerWeights
    hw = HalfLayerWeights(
        hc_weight=torch.randn(24, 4 * hidden, generator=g, device=dev) * 0.01, hc_base=torch.zeros(24, device=dev),
        hc_scale=torch.ones(3, device=dev), attn_norm=torch.ones(hidden, dtype=torch.bfloat16, device=dev),
        front_w8=rnd8(2048, hidden), front_w8_scales=sc(16, hidden // 128),
        front_w16=(torch.randn(2624, hidden, generator=g, device=dev) * 0.02).bfloat16(),
        ape=torch.randn(4, 1024, generator=g, device=dev), idx_ape=torch.randn(4, 256, generator=g, device=dev),
        o_proj=o_proj.OProjWeights(rnd8(16, 1024, 4096), sc(16 * 8, 32), rnd8(hidden, 16384), sc(56, 128)),
        attn_sink=torch.randn(mh, generator=g, device=dev))
    x_hidden = torch.randn(batch, 4, hidden, generator=g, device=dev).bfloat16()
    for name in ("swa", "cmp"):   # attention caches: random finite records instead of the zeros of a fresh pool
        data = cache._pools[name].data
        epb_m = cache.entries_per_block[name]
        data[:, :epb_m * 584] = model1_pool(data.size(0), epb_m, 5)[:, :epb_m * 584]
    half_layer = AttentionHalfLayer(weights, hw, cache, batch, topk=topk)
    stage = half_layer.stage
    half_layer.prepare(slots)
    layer = lambda: half_layer.launch(x_hidden, batch)

    if launches_only:
        for _ in range(launches_only):
            layer()
        torch.cuda.synchronize()
        stage.check_status()
        print("attention_half_layer: %d eager passes done" % launches_only)
        return
    layer()
    torch.cuda.synchronize()
    stage.check_status()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        layer()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    total = 0.0
    for i in range(reps + 3):
        flush.fill_(i & 0xff)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        graph.replay()
        e1.record()
        torch.cuda.synchronize()
        if i >= 3:
            total += e0.elapsed_time(e1) * 1e3
    stage.check_status()
    us = total / reps
    wbytes = 24 * 4 * hidden * 4 + 2048 * hidden + 2624 * hidden * 2 + n_total * q_lora + 16 * 1024 * 4096 + hidden * 16384
    print("attention half-layer: batch %d, context %d, window 128 + top-%d" % (batch, context, topk))
    print("  %.1f us per pass (one graph, L2 flushed before each); weights streamed %.1f MB + %.1f MB of indexer keys"
          % (us, wbytes / 1e6, batch * (context // 4) * 132 / 1e6))


def moe_experts(tokens=64, topk=8, experts=256, dim=7168, inter=2048, reps=10, launches_only=0):
    """Router + routed experts of one MoE block at the model's geometry (256 NVFP4 experts, top-8,
    intermediate 2048): gate projection, routing, dispatch, gather-quantisation, grouped w1|w3 GEMM,
    SwiGLU + quantisation, grouped w2 GEMM, combine - nine launches in one CUDA graph.  The weights of
    the active experts (about 220 of 256 at batch 64) are far larger than L2, so no flush is needed."""
    from wuda_b200 import moe
    hbm, tf, kind = peaks()
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(3)
    w = moe.RandomRoutedExperts(experts, inter, dim)
    runner = moe.MoERunner(w, tokens, topk)
    x = torch.randn(tokens, dim, generator=g, device=dev).bfloat16()
    gate_w = (torch.randn(experts, dim, generator=g, device=dev) * 0.05).bfloat16()
    bias = torch.zeros(experts, device=dev)
    logits = torch.empty(tokens, experts, device=dev)
    y = torch.empty(tokens, dim, dtype=torch.bfloat16, device=dev)

    def step():
        rw, idx = wuda.moe_gate(x, gate_w, bias, "sqrtsoftplus", 2.5, topk, logits=logits)
        runner.forward(x, rw, idx, y=y)
        return idx

    idx = step()
    torch.cuda.synchronize()
    assert int(runner.status.item()) == 0
    if launches_only:
        for _ in range(launches_only - 1):
            step()
        torch.cuda.synchronize()
        print("moe_experts: %d eager passes done" % launches_only)
        return
    active = int(torch.unique(idx).numel())
    groups = int(runner.num_groups.item())
    us = time_graph(step, reps=reps, inner=1)
    per_expert = 2 * inter * dim // 2 + 2 * inter * dim // 16 + dim * inter // 2 + dim * inter // 16
    wbytes = active * per_expert
    print("MoE router + routed experts: %d tokens x top-%d of %d experts (%d active, %d row groups)" %
          (tokens, topk, experts, active, groups))
    print("  %.1f us per block; %.2f GB of expert weights streamed -> %.0f GB/s = %.2f of %s HBM peak" %
          (us, wbytes / 1e9, wbytes / us / 1e3, wbytes / us / 1e3 / hbm, kind))


def moe_ep2(tokens=64, topk=8, experts=256, dim=7168, inter=2048, iters=20):
    """Run under torch.distributed.run with two ranks: router + routed experts of one MoE block with the
    256 experts split over the two ranks and the combine step exchanging fp32 rows over NVLink peer
    memory; time per block = max over ranks of the device time."""
    import torch.distributed as dist
    from wuda_b200 import moe
    rank = int(os.environ["RANK"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("gloo")
    hbm, _, kind = peaks()
    half = experts // 2
    g = torch.Generator(device="cuda").manual_seed(3)          # the same tokens and gate on both ranks
    x = torch.randn(tokens, dim, generator=g, device="cuda").bfloat16()
    gate_w = (torch.randn(experts, dim, generator=g, device="cuda") * 0.05).bfloat16()
    bias = torch.zeros(experts, device="cuda")
    logits = torch.empty(tokens, experts, device="cuda")
    y = torch.empty(tokens, dim, dtype=torch.bfloat16, device="cuda")
    w = moe.RandomRoutedExperts(half, inter, dim, seed=10 + rank)
    link = moe.EP2Link(tokens, dim)
    runner = moe.MoERunner(w, tokens, topk, expert_first=rank * half, experts_total=experts, link=link)

    def step():
        rw, idx = wuda.moe_gate(x, gate_w, bias, "sqrtsoftplus", 2.5, topk, logits=logits)
        runner.forward(x, rw, idx, y=y)
        return idx

    for _ in range(3):
        idx = step()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        step()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) * 1e3 / iters], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    mine = (idx >= rank * half) & (idx < (rank + 1) * half)
    active = torch.tensor([int(torch.unique(idx[mine]).numel())], dtype=torch.float64)
    both = [torch.zeros(1, dtype=torch.float64) for _ in range(2)]
    dist.all_gather(both, active)
    status = int(runner.status.item())
    if rank == 0:
        per_expert = 2 * inter * dim // 2 + 2 * inter * dim // 16 + dim * inter // 2 + dim * inter // 16
        most = max(float(b.item()) for b in both)
        print("MoE block on two expert-parallel ranks: %d tokens x top-%d of %d experts (%d + %d active), status %d" %
              (tokens, topk, experts, int(both[0].item()), int(both[1].item()), status))
        print("  %.1f us per block (eager launches, max over ranks); the busier rank streams %.2f GB -> %.0f GB/s = %.2f of "
              "%s HBM peak; %.1f MB over the link per rank" %
              (float(t.item()), most * per_expert / 1e9, most * per_expert / float(t.item()) / 1e3,
               most * per_expert / float(t.item()) / 1e3 / hbm, kind, tokens * dim * 4 / 1e6))
    dist.barrier()
    link.close()
    dist.destroy_process_group()


def topk(k=2048):
    """Top-k selection + page transform over rows that were just written (L2-resident), CUDA-graph replays:
    64 rows of 8192 scores (the layer at 32 K context), 64 rows of 16384, and 128 rows of 16384..65536 scores
    (the benchmark step's shape)."""
    hbm, _, kind = peaks()
    g = torch.Generator(device="cuda").manual_seed(1)
    for rows, lo, hi in ((64, 8192, 8192), (64, 16384, 16384), (128, 16384, 65536)):
        lens = torch.randint(lo, hi + 1, (rows,), generator=g, device="cuda", dtype=torch.int32)
        stride = (hi + 255) // 256 * 256
        scores = torch.randn(rows, stride, generator=g, device="cuda")
        table = torch.arange(rows * (stride // 64), device="cuda", dtype=torch.int32).view(rows, -1)
        out = torch.empty(rows, k, dtype=torch.int32, device="cuda")
        us = time_graph(lambda: wuda.topk_v2_transform(scores, lens, table, out, 64), reps=20, inner=10)
        by = int(lens.sum()) * 4 + rows * k * 4
        print("top-%d of %3d rows x %5d..%5d scores: %6.2f us  (%.1f MB read once -> %.0f GB/s, %.2f of %s HBM peak; "
              "the rows are L2-resident)" % (k, rows, lo, hi, us, by / 1e6, by / us / 1e3, by / us / 1e3 / hbm, kind))


def mqa_fp4(batches=(64, 128), contexts=(8192, 32768), launches_only=0):
    """MXFP4 paged MQA logits (68 bytes per token): identity page tables, random codes and scale bytes."""
    hbm, _, kind = peaks()
    print("MXFP4 paged MQA logits, 64 heads x 128; HBM peak (%s) %.0f GB/s" % (kind, hbm))
    for batch in batches:
        for ctx in contexts:
            g = torch.Generator(device="cuda").manual_seed(ctx)
            epb, pages_per = 64, ctx // 64
            pages = torch.randint(0, 256, (batch * pages_per, epb * 68), generator=g, dtype=torch.uint8, device="cuda")
            pages[:, epb * 64:] = torch.randint(120, 130, (batch * pages_per, epb * 4), generator=g, dtype=torch.uint8,
                                                device="cuda")
            q = torch.randint(0, 256, (batch, 64, 64), generator=g, dtype=torch.uint8, device="cuda").view(torch.int8)
            q_sf = torch.randint(120, 130, (batch, 64, 4), generator=g, dtype=torch.uint8, device="cuda").view(torch.int32)
            weights = torch.randn(batch, 64, generator=g, device="cuda")
            lens = torch.full((batch,), ctx, dtype=torch.int32, device="cuda")
            table = torch.arange(batch * pages_per, dtype=torch.int32, device="cuda").view(batch, pages_per)
            logits = torch.empty(batch, ctx, device="cuda")
            status = wuda.device_status_word()
            fn = lambda: wuda.mqa_logits_fp4_decode_out(q, q_sf.view(batch, 64), pages, weights, lens, table, logits, ctx,
                                                        status_word=status)
            if launches_only:
                for _ in range(launches_only):
                    fn()
                torch.cuda.synchronize()
                print("ran %d launches at batch %d, context %d (status %d)" % (launches_only, batch, ctx, int(status.item())))
                continue
            us = time_graph(fn, reps=10, inner=5)
            assert int(status.item()) == 0
            by = batch * ctx * 68 + batch * ctx * 4
            print("batch %3d ctx %6d: %7.1f us  %6.0f GB/s = %.2f of peak (%.0f MB of pages)" %
                  (batch, ctx, us, by / us / 1e3, by / us / 1e3 / hbm, batch * ctx * 68 / 1e6))


def sparse_mla(batches=(4, 16, 64, 128), heads=128, window=128, topk=2048, context=32768, launches_only=0):
    """Sparse MLA decode attention: per request `window` sliding-window records and `topk` of the
    context / 4 compressed records, gathered by index from pools that exceed L2."""
    hbm, tf, kind = peaks()
    print("sparse MLA decode, heads %d, window %d + top-%d of %d compressed; peaks (%s) %.0f GB/s, %.0f TFLOP/s bf16"
          % (heads, window, topk, context // 4, kind, hbm, tf))
    print("%6s %9s %11s %9s %12s %9s" % ("batch", "us", "TFLOP/s", "of peak", "gather GB/s", "of peak"))
    for batch in batches:
        ncmp = context // 4
        cmp_pages = batch * ncmp // 64
        swa = model1_pool(batch, 256, 1)
        cmp = model1_pool(cmp_pages, 64, 2)
        view = lambda t, epb: t.as_strided((t.size(0), epb, 1, 584), (t.size(1), 584, 584, 1))
        g = torch.Generator().manual_seed(batch)
        swa_idx = torch.stack([torch.randperm(256, generator=g)[:window] + 256 * b for b in range(batch)]).int().cuda()
        cmp_idx = torch.stack([torch.randperm(ncmp, generator=g)[:topk] + ncmp * b for b in range(batch)]).int().cuda()
        swa_len = torch.full((batch,), window, dtype=torch.int32).cuda()
        cmp_len = torch.full((batch,), topk, dtype=torch.int32).cuda()
        q = torch.randn(batch, heads, 512, generator=g).bfloat16().cuda()
        sink = torch.randn(heads, generator=g).cuda()
        out = torch.empty_like(q)
        status = wuda.device_status_word()
        fn = lambda: wuda.sparse_mla_decode(q, view(swa, 256), swa_idx, swa_len, view(cmp, 64), cmp_idx, cmp_len, sink,
                                            512 ** -0.5, out=out, status_word=status)
        if launches_only:
            for _ in range(launches_only):
                fn()
            torch.cuda.synchronize()
            print("ran %d launches at batch %d (status %d)" % (launches_only, batch, int(status.item())))
            continue
        us = time_graph(fn, reps=10, inner=5)
        assert int(status.item()) == 0
        keys = batch * (window + topk)
        flops = keys * heads * 512 * 2 * 2            # Q K^T and P V, each once
        gathered = keys * 584
        print("%6d %9.1f %11.1f %8.1f%% %12.0f %8.1f%%" % (batch, us, flops / us / 1e6, flops / us / 1e6 / tf * 100,
                                                         gathered / us / 1e3, gathered / us / 1e3 / hbm * 100))


def pair_sync(group):
    """Both ranks of a pair have finished their set-up before either starts a call that waits for the other:
    the exchange kernels bound their waits, and set-up times differ by more than that bound."""
    import torch.distributed as dist
    torch.cuda.synchronize()
    if group is not None:
        dist.barrier(group=group)


def time_replays(replay, reps, group=None, flush=None):
    """Device time (us) of replay(), timed with CUDA events around each call on the current stream; with a
    process group, the ranks start each call together (host barrier) and the MEDIAN over the calls of the per-call
    MAX over ranks is returned (a call in which one rank's host leaves the barrier late makes its peer's kernel wait
    for it: with eight processes on one host such calls happen, and a mean would report the host, not the GPUs).
    Without a group: the mean.  `flush` (a buffer larger than L2) is rewritten before every call when given."""
    import torch.distributed as dist
    times = []
    for i in range(reps + 3):
        if flush is not None:
            flush.fill_(i & 0xff)
        if group is not None:
            torch.cuda.synchronize()
            dist.barrier(group=group)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        replay()
        e1.record()
        torch.cuda.synchronize()
        if i >= 3:
            times.append(e0.elapsed_time(e1) * 1e3)
    t = torch.tensor(times, dtype=torch.float64)
    if group is not None:
        if dist.get_backend(group) == "nccl":
            t = t.cuda()
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
        return float(t.median().item())
    return float(t.mean().item())


def tp2_gemm_leg(group, pair_rank, m=64, n=7168, k=16384, reps=30, seed=1234):
    """The wo_b projection of a tensor-parallel pair (K split in two, all-reduce fused into the GEMM epilogue
    over NVLink peer memory) as CUDA-graph replays, next to the same local GEMM without the exchange.
    Returns the timings and what the caller needs to check the result: the full synthetic case (identical on
    both ranks) and this rank's bf16 output as uint16."""
    hbm, _, kind = peaks()
    case = workloads.make_gemm_fp8_case(m, n, k, seed=seed)
    kl = k // 2
    sl, sb = slice(pair_rank * kl, (pair_rank + 1) * kl), slice(pair_rank * kl // 128, (pair_rank + 1) * kl // 128)
    t = lambda x: torch.from_numpy(np.ascontiguousarray(x)).cuda()
    a, w = t(case["a"][:, sl]).view(torch.float8_e4m3fn), t(case["w"][:, sl]).view(torch.float8_e4m3fn)
    a_s, w_s = t(case["a_s"][:, sb]), t(case["w_s"][:, sb])
    copies = 4                                    # rotate weight buffers: 4 x 59 MB exceed the L2
    ws = [w] + [w.clone() for _ in range(copies - 1)]
    out = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    link = wuda.TP2Link(m, n, group=group, device_sequence=True)
    status = wuda.device_status_word()

    def graph_of(fn):
        pair_sync(group)
        fn(ws[0])
        torch.cuda.synchronize()
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                for i in range(copies):
                    fn(ws[i])
        torch.cuda.synchronize()
        return g

    g_fused = graph_of(lambda wt: link.fp8_gemm(a, a_s, wt, w_s, out=out, status_word=status))
    g_local = graph_of(lambda wt: wuda.fp8_gemm(a, a_s, wt, w_s, out=out))
    t_local = time_replays(g_local.replay, reps, group) / copies
    t_fused = time_replays(g_fused.replay, reps, group) / copies
    got = out.cpu().view(torch.int16).numpy().view(np.uint16)       # last replay ends on ws[copies-1] == the same weights
    by = workloads.gemm_fp8_algorithmic_bytes(m, n, kl)
    link_bytes = m * n * 4
    bound_us = max(by / (hbm * 1e3), link_bytes / (770.0 * 1e3))
    res = dict(shape=[m, n, k], gemm_allreduce_us=t_fused, local_gemm_us=t_local, nvlink_bytes=link_bytes,
               hbm_bytes=by, roofline_us=bound_us, roofline_frac=bound_us / t_fused, status=int(status.item()),
               launch="CUDA-graph replays, call sequence numbered on the device")
    torch.cuda.synchronize()
    link.close()
    return res, case, got


def ep2_combine_leg(group, pair_rank, tokens=64, topk=8, experts=256, dim=7168, inter=2048, reps=10):
    """Router + routed experts of one MoE block with the experts split over a pair of ranks and the combine step
    exchanging fp32 partial rows over NVLink peer memory, as CUDA-graph replays.  Returns timings, this rank's
    output (uint16 bits of the bf16 rows) and its local fp32 partial sums for the caller's check."""
    from wuda_b200 import moe
    hbm, _, kind = peaks()
    half = experts // 2
    g = torch.Generator(device="cuda").manual_seed(3)          # the same tokens and gate on both ranks
    x = torch.randn(tokens, dim, generator=g, device="cuda").bfloat16()
    gate_w = (torch.randn(experts, dim, generator=g, device="cuda") * 0.05).bfloat16()
    bias = torch.zeros(experts, device="cuda")
    logits = torch.empty(tokens, experts, device="cuda")
    y = torch.empty(tokens, dim, dtype=torch.bfloat16, device="cuda")
    w = moe.RandomRoutedExperts(half, inter, dim, seed=10 + pair_rank)
    link = moe.EP2Link(tokens, dim, group=group, device_sequence=True)
    runner = moe.MoERunner(w, tokens, topk, expert_first=pair_rank * half, experts_total=experts, link=link)
    state = {}

    def step():
        rw, idx = wuda.moe_gate(x, gate_w, bias, "sqrtsoftplus", 2.5, topk, logits=logits)
        runner.forward(x, rw, idx, y=y)
        state["idx"] = idx

    pair_sync(group)
    step()
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            step()
    torch.cuda.synchronize()
    us = time_replays(graph.replay, reps, group)
    idx = state["idx"]
    mine = (idx >= pair_rank * half) & (idx < (pair_rank + 1) * half)
    active = int(torch.unique(idx[mine]).numel())
    # this rank's partial: fp32 sum of its experts' bf16 rows per token, in the kernel's order (pair order)
    rows = runner.pair_row[:tokens].long()
    out = runner.out.float()
    part = torch.zeros(tokens, dim, device="cuda")
    for j in range(topk):
        r = rows[:, j]
        part = part + torch.where((r >= 0)[:, None], out[r.clamp_min(0)], torch.zeros_like(part))
    per_expert = 2 * inter * dim // 2 + 2 * inter * dim // 16 + dim * inter // 2 + dim * inter // 16
    res = dict(tokens=tokens, experts=experts, active_experts=active, block_us=us, expert_bytes=active * per_expert,
               hbm_frac=active * per_expert / us / 1e3 / hbm, nvlink_bytes=tokens * dim * 4, status=int(runner.status.item()),
               launch="one CUDA graph per block, call sequence numbered on the device")
    got = y.cpu().view(torch.int16).numpy().view(np.uint16)
    part = part.cpu().numpy()
    torch.cuda.synchronize()
    link.close()
    return res, got, part


def layer_leg(batch=64, context=32768, topk=2048, reps=20, group=None, pair_rank=0, launches_only=0):
    """The whole decode layer (attention half + MoE half) of `batch` requests at `context` tokens as one CUDA
    graph, on one GPU (group None) or on a tensor-parallel pair; decode tokens/s/GPU = batch / (t * ranks).
    Returns (result dict, output of the last pass as a CPU tensor)."""
    from wuda_b200 import moe
    from wuda_b200.layer_setup import build_random_layer, layer_weight_bytes
    hbm, _, kind = peaks()
    world = 1 if group is None else 2
    tp_link = ep_link = None
    if world == 2:
        tp_link = wuda.TP2Link(batch, 7168, group=group, device_sequence=True)
        ep_link = moe.EP2Link(batch, 7168, group=group, device_sequence=True)
    layer, slots, x = build_random_layer(batch, context, topk=topk, rank=pair_rank, world=world, tp_link=tp_link,
                                         ep_link=ep_link)
    layer.prepare(slots)
    if launches_only:
        for _ in range(launches_only):
            layer.launch(x, batch)
        torch.cuda.synchronize()
        layer.check_status()
        print("layer: %d eager passes done" % launches_only)
        return None, None
    pair_sync(group)
    layer.capture(x, batch)
    us = time_replays(layer.replay, reps, group)
    layer.check_status()
    pair_sync(group)
    out = layer.replay()
    torch.cuda.synchronize()
    idx = layer.route_indices
    per = layer.ffn.routed.experts
    mine = (idx >= layer.ffn.expert_first) & (idx < layer.ffn.expert_first + per)
    active = int(torch.unique(idx[mine]).numel())
    ncmp = context // 4
    wbytes = layer_weight_bytes(world, experts_active=active)
    cache_bytes = batch * ncmp * 132 + batch * (128 + min(topk, ncmp)) * 584
    res = dict(batch=batch, context=context, ranks=world, layer_us=us, tok_s_per_gpu=batch / (us * 1e-6) / world,
               weight_bytes_per_rank=wbytes, cache_bytes_per_rank=cache_bytes, active_experts_this_rank=active,
               hbm_floor_us=(wbytes + cache_bytes) / (hbm * 1e3), hbm_frac=(wbytes + cache_bytes) / (hbm * 1e3) / us,
               launch="one CUDA graph per layer pass; weights streamed per pass (%.1f GB) exceed the L2" % (wbytes / 1e9),
               status=0)
    result = out.float().cpu()
    if tp_link is not None:
        torch.cuda.synchronize()
        tp_link.close()
        ep_link.close()
    return res, result


def layer(batch=64, context=32768):
    res, _ = layer_leg(batch, context)
    print("decode layer, batch %d, context %d, one GPU: %.1f us per pass = %.0f tokens/s/GPU; %.2f GB of weights + %.0f MB of "
          "cache records streamed = %.2f of the HBM floor (%.1f us)" %
          (batch, context, res["layer_us"], res["tok_s_per_gpu"], res["weight_bytes_per_rank"] / 1e9,
           res["cache_bytes_per_rank"] / 1e6, res["hbm_frac"], res["hbm_floor_us"]))


def layer_tp2(batch=64, context=32768):
    """Run under torch.distributed.run with two ranks."""
    import torch.distributed as dist
    rank = int(os.environ["RANK"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("gloo")
    group = dist.new_group([0, 1])
    res, _ = layer_leg(batch, context, group=group, pair_rank=rank)
    if rank == 0:
        print("decode layer, batch %d, context %d, tensor-parallel pair: %.1f us per pass = %.0f tokens/s/GPU; this rank "
              "streams %.2f GB of weights = %.2f of its HBM floor (%.1f us)" %
              (batch, context, res["layer_us"], res["tok_s_per_gpu"], res["weight_bytes_per_rank"] / 1e9, res["hbm_frac"],
               res["hbm_floor_us"]))
    dist.barrier()
    dist.destroy_process_group()


def one(kind, m, n, k, launches=5):
    """A few eager launches of one GEMM shape (profiler captures)."""
    t = lambda x: torch.from_numpy(np.ascontiguousarray(x)).cuda()
    if kind in ("gemm_fp8", "gemm_fp8_pow2"):
        c = workloads.make_gemm_fp8_case(m, n, k, seed=7)
        a, w = t(c["a"]).view(torch.float8_e4m3fn), t(c["w"]).view(torch.float8_e4m3fn)
        a_s, w_s = t(c["a_s"]), t(c["w_s"])
        if kind == "gemm_fp8_pow2":
            a_s, w_s = torch.exp2(torch.log2(a_s).round()), torch.exp2(torch.log2(w_s).round())
        fn = lambda: wuda.fp8_gemm(a, a_s, w, w_s, pow2_scales=kind == "gemm_fp8_pow2")
    elif kind == "fp4_act_quant":          # m rows of n values (k unused)
        xs = [torch.randn(m, n, device="cuda").bfloat16() for _ in range(launches)]
        state = {"i": 0}

        def fn():
            wuda.fp4_act_quant(xs[state["i"] % launches])
            state["i"] += 1
    elif kind == "gemm_fp8_fp4":
        gen = torch.Generator(device="cuda").manual_seed(7)
        a = torch.randint(0, 0x78, (m, k), dtype=torch.uint8, device="cuda", generator=gen).view(torch.float8_e4m3fn)
        a_s = torch.exp2(torch.randint(-4, 4, (m, k // 128), device="cuda", generator=gen).float())
        # a different weight buffer per launch, together larger than L2
        ws = [torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, device="cuda", generator=gen) for _ in range(launches)]
        w_sf = torch.randint(118, 126, (n, k // 32), dtype=torch.uint8, device="cuda", generator=gen)
        state = {"i": 0}

        def fn():
            wuda.fp4_gemm(a, a_s, ws[state["i"] % launches], w_sf)
            state["i"] += 1
    else:
        c = workloads.make_gemm_nvfp4_case(m, n, k, seed=7)
        a, w, a_sf, w_sf = t(c["a"]), t(c["w"]), t(c["a_sf_packed"]), t(c["w_sf_packed"])
        fn = lambda: wuda.nvfp4_gemm(a, a_sf, c["a_gs"], w, w_sf, c["w_gs"])
    for _ in range(launches):
        fn()
    torch.cuda.synchronize()
    print("ran %d launches of %s M=%d N=%d K=%d" % (launches, kind, m, n, k))


KINDS = {"topk": topk, "gemm_fp8": gemm_fp8, "gemm_fp8_pow2": lambda: gemm_fp8(pow2=True), "gemm_nvfp4": gemm_nvfp4, "gemm_fp8_fp4": gemm_fp8_fp4, "norm_rope_quant": norm_rope_quant, "tp2": tp2, "moe_ep2": moe_ep2, "mqa_fp4": mqa_fp4, "mqa_fp4_launches": lambda: mqa_fp4(batches=(64,), contexts=(32768,), launches_only=3),
         "sparse_mla": sparse_mla, "sparse_mla_launches": lambda: sparse_mla(batches=(32,), launches_only=3),
         "csa_chain": csa_chain, "csa_chain_fp4": lambda: csa_chain(indexer_fp4=True),
         "csa_chain_launches": lambda: csa_chain(launches_only=3),
         "attention_half_layer": attention_half_layer, "moe_experts": moe_experts,
         "layer": layer, "layer_tp2": layer_tp2, "layer_launches": lambda: layer_leg(launches_only=2),
         "moe_experts_launches": lambda: moe_experts(launches_only=2),
         "attention_half_layer_launches": lambda: attention_half_layer(launches_only=3)}


if __name__ == "__main__":
    which = sys.argv[1] if len(sys.argv) > 1 else "gemm_fp8"
    if which == "one":
        one(sys.argv[2], int(sys.argv[3]), int(sys.argv[4]), int(sys.argv[5]))
        sys.exit(0)
    KINDS[which]()
