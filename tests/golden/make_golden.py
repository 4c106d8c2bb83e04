"""Generates the golden fixtures in this directory by running the REFERENCE's own
Python reference functions (imported from a checkout of guluguluhhhh/wuda) on small
seeded inputs.  The fixtures store inputs and expected outputs, so the tests need
neither the checkout nor this script.

    python tests/golden/make_golden.py /path/to/reference [golden_<name> ...]

Functions used (paths inside the reference repository):
  dsv4_megakernel/megakernel/test/test_mqa_logits_fp4.py  ref_fp8_mqa_logits (:207-218); quantize_fp4 (:222-227),
                                                           build_paged_cache (:235-262) for the FP4 form
  dsv4_megakernel/megakernel/test/test_topk_v2.py         ref_page_transform (:86-94) and the
                                                           stable-argsort rule (:116)
  dsv4_megakernel/megakernel/test/test_e2e_decode.py      ref_mhc_post (:423-426), ref_flash_attn
                                                           (:377-392) over deq_model1_row (:346-356)
  dsv4_megakernel/megakernel/test/test_wq_b_fp8_gemm.py   ref_comp_step (:550-586, both forms), ref_win_step
                                                           (:646-665), ref_idx_fp8_chain (:184-196) and
                                                           ref_idx_chain (:161-182, the FP4 form)
  dsv4_megakernel/megakernel/test/test_hc_fused_tc.py     hc_reference (:115-136)
  dsv4_megakernel/origin/model.py                         Gate.forward (:563-584); Gate, Expert, MoE (:546-644) for
                                                           the whole MoE block on bf16 weights
  dsv4_megakernel/megakernel/test/kv_cache_manager.py     KVCacheManager (:53-257), run on the CPU
The first two are written for device="cuda"; they are run here on the CPU by mapping that one
keyword to "cpu", which changes no arithmetic.

Two of the reference's twins are not callable: they stand inline in GPU tests.  Their formulas are restated
here, statement by statement, and run on seeded CPU inputs:
  dsv4_megakernel/megakernel/test/test_mqa_logits_fp4.py:404-413   query RMSNorm + RoPE (golden_query_rms_rope)
  dsv4_megakernel/megakernel/test/test_mqa_logits_fp4.py:772-791   MAIN compressor row (golden_main_compressor)
"""
import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
from wuda_b200 import workloads  # noqa: E402


class _CpuTorch:
    """Proxy of the torch module that sends device='cuda' factory calls to the CPU."""

    def __init__(self):
        self._t = torch

    def __getattr__(self, name):
        attr = getattr(self._t, name)
        if callable(attr) and name in ("arange", "full", "zeros", "ones", "empty", "tensor", "randn",
                                       "randint", "rand", "randperm", "full_like"):
            def wrapped(*a, **k):
                if k.get("device") == "cuda":
                    k["device"] = "cpu"
                return attr(*a, **k)
            return wrapped
        return attr


def _load(ref_root, rel, name):
    path = os.path.join(ref_root, rel)
    sys.path.insert(0, os.path.dirname(path))
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    mod.torch = _CpuTorch()
    return mod


def logical_keys(case, b):
    """Dequantised keys of request b in token order: (e4m3 bytes as fp32 [T,128], scales [T])."""
    epb, ctx = case["epb"], int(case["ctx"][b])
    pages = case["block_table"][b, :(ctx + epb - 1) // epb]
    pg = case["kv_pages"][pages]
    k8 = pg[:, :epb * 128].reshape(-1, 128)[:ctx]
    sc = pg[:, epb * 128:epb * 132].copy().view(np.float32).reshape(-1)[:ctx]
    kf = torch.from_numpy(k8.copy()).view(torch.float8_e4m3fn).float()
    return kf, torch.from_numpy(sc.copy())


def golden_mqa(ref_mqa, name, **kw):
    case = workloads.make_mqa_case(**kw)
    rows = case["batch"] * case["next_n"]
    expected = np.full((rows, case["logits_stride"]), -np.inf, np.float32)
    q = torch.from_numpy(case["q"]).view(torch.float8_e4m3fn)
    w = torch.from_numpy(case["weights"])
    for b in range(case["batch"]):
        kf, sc = logical_keys(case, b)
        kv = kf * sc[:, None]                      # dequantised keys, fp32
        r0 = b * case["next_n"]
        qb = q[r0:r0 + case["next_n"]]
        ke = torch.from_numpy(case["context_lens"][b].astype(np.int64))
        ks = torch.zeros_like(ke)
        out = ref_mqa.ref_fp8_mqa_logits(qb, kv, w[r0:r0 + case["next_n"]], ks, ke)
        expected[r0:r0 + case["next_n"], :kv.shape[0]] = out.numpy()
    arrays = {k: case[k] for k in ("q", "kv_pages", "weights", "context_lens", "block_table", "ctx")}
    np.savez_compressed(os.path.join(HERE, name), expected=expected, next_n=case["next_n"], epb=case["epb"],
                        logits_stride=case["logits_stride"], **arrays)
    print(name, expected.shape, "finite:", int(np.isfinite(expected).sum()))


def golden_mqa_fp4(ref_mqa):
    """MXFP4 indexer scores: the reference's quantiser (quantize_fp4), page builder (build_paged_cache, shuffled
    pages) and torch twin (ref_fp8_mqa_logits over the dequantised values), all run on the CPU."""
    torch.manual_seed(31)
    batch, tokens, epb = 3, 384, 64
    q = torch.randn(batch, 64, 128).bfloat16()
    kv = torch.randn(batch, tokens, 128).bfloat16()
    weights = torch.randn(batch, 64)
    q_p, q_sf, q_sim = ref_mqa.quantize_fp4(q, 128)
    kv_p, kv_sf, kv_sim = ref_mqa.quantize_fp4(kv, 128)
    stride = epb * 68 + 48
    fused, table = ref_mqa.build_paged_cache(kv_p.view(-1, 64), kv_sf.view(-1), batch, tokens, shuffle=True,
                                             entries_per_block=epb, block_stride_bytes=stride)
    ctx = [384, 201, 1]
    rows = []
    for b in range(batch):
        ks, ke = torch.zeros(1, dtype=torch.int32), torch.full((1,), ctx[b], dtype=torch.int32)
        rows.append(ref_mqa.ref_fp8_mqa_logits(q_sim.view(batch, 64, 128)[b:b + 1], kv_sim.view(batch, tokens, 128)[b],
                                               weights[b:b + 1], ks, ke)[0])
    np.savez_compressed(os.path.join(HERE, "mqa_logits_fp4.npz"), q=q_p.view(batch, 64, 64).numpy().view(np.uint8),
                        q_sf=q_sf.view(batch, 64).numpy(), pages=fused.numpy(), weights=weights.numpy(),
                        context_lens=np.asarray(ctx, np.int32), block_table=table.numpy(), epb=np.int32(epb),
                        logits=torch.stack(rows).float().numpy())
    print("mqa_logits_fp4.npz", batch, tokens)


def golden_topk(ref_topk, name, rows, length, k, lens, tie_levels, seed):
    g = torch.Generator().manual_seed(seed)
    scores = torch.randn(rows, length, generator=g)
    if tie_levels > 0:
        scores = torch.randint(0, tie_levels, (rows, length), generator=g).float()
    for r in range(rows):
        scores[r, lens[r]:] = float("-inf")
    page_size = ref_topk.PAGE_SIZE
    num_pages = (length + page_size - 1) // page_size
    page_table = torch.randint(0, 1 << 20, (rows, max(num_pages, 1)), generator=g, dtype=torch.int32)
    raw = torch.full((rows, k), -1, dtype=torch.int32)
    pages = torch.full((rows, k), -1, dtype=torch.int32)
    for r in range(rows):
        n = lens[r]
        if n <= k:
            raw[r, :n] = torch.arange(n, dtype=torch.int32)
        else:
            raw[r] = torch.argsort(-scores[r, :n], stable=True)[:k].int()
        pages[r] = ref_topk.ref_page_transform(page_table[r], raw[r]).int()
    np.savez_compressed(os.path.join(HERE, name), scores=scores.numpy(), seq_lens=np.asarray(lens, np.int32),
                        page_table=page_table.numpy(), raw=raw.numpy(), pages=pages.numpy(), k=k,
                        page_size=page_size)
    print(name, raw.shape)


def _u16(t):
    return t.view(torch.int16).numpy().view(np.uint16).copy()


def golden_norm_rope_quant(ref_root):
    """RMSNorm and RoPE from the origin model (dsv4_megakernel/origin/model.py:183-196,
    232-244), power-of-two 1x128 FP8 quantisation from the reference's torch twin
    quant_act_fp8 (dsv4_megakernel/megakernel/test/test_front_mixed_gemm.py:75-83)."""
    model = _load(ref_root, "dsv4_megakernel/origin/model.py", "ref_origin_model")
    model.torch = torch          # the origin model needs the real module (nn.Module subclasses)
    g = torch.Generator().manual_seed(31)
    x = torch.randn(5, 7168, generator=g).bfloat16()
    gamma = (1 + 0.1 * torch.randn(7168, generator=g)).bfloat16()
    norm = model.RMSNorm(7168, 1e-6)
    norm.weight.data = gamma.float()
    y = norm(x)
    np.savez_compressed(os.path.join(HERE, "rmsnorm_7168.npz"), x=_u16(x), gamma=_u16(gamma), eps=1e-6, y=_u16(y))
    print("rmsnorm_7168.npz", tuple(y.shape))

    tokens, heads, head_dim, rope_dim = 4, 8, 192, 64
    xr = torch.randn(tokens, heads, head_dim, generator=g).bfloat16()
    pos = torch.tensor([0, 3, 4097, 65535])
    freqs = 1.0 / (10000 ** (torch.arange(0, rope_dim, 2, dtype=torch.float32) / rope_dim))
    ang = torch.outer(torch.arange(65536).float(), freqs)
    cis = torch.polar(torch.ones_like(ang), ang)
    fwd = xr.clone()
    model.apply_rotary_emb(fwd.view(1, tokens, heads, head_dim)[..., -rope_dim:], cis[pos])
    inv = xr.clone()
    model.apply_rotary_emb(inv.view(1, tokens, heads, head_dim)[..., -rope_dim:], cis[pos], inverse=True)
    np.savez_compressed(os.path.join(HERE, "rope_192.npz"), x=_u16(xr), positions=pos.numpy(),
                        cos=ang.cos()[pos.unique()].numpy(), sin=ang.sin()[pos.unique()].numpy(),
                        table_rows=pos.unique().numpy(), rope_dim=rope_dim, y=_u16(fwd), y_inverse=_u16(inv))
    print("rope_192.npz", tuple(fwd.shape))

    front = _load(ref_root, "dsv4_megakernel/megakernel/test/test_front_mixed_gemm.py", "ref_front")
    front.torch = torch
    xq = (torch.randn(6, front.K, generator=g) * 0.1).bfloat16()
    xq[0, :128] = 0                                   # an all-zero group: amax clamps at 1e-4
    q, exp = front.quant_act_fp8(xq)
    np.savez_compressed(os.path.join(HERE, "act_quant_pow2_7168.npz"), x=_u16(xq), q=q.view(torch.uint8).numpy(),
                        scale=torch.pow(2.0, exp.float() - 127.0).numpy())
    print("act_quant_pow2_7168.npz", tuple(q.shape))


def golden_mhc_post(ref_root):
    """The torch twin of the mHC post mix on seeded inputs of the model's width."""
    e2e = _load(ref_root, "dsv4_megakernel/megakernel/test/test_e2e_decode.py", "ref_e2e")
    e2e.torch = torch
    g = torch.Generator().manual_seed(41)
    m, hidden = 3, 7168
    x = torch.randn(m, hidden, generator=g).bfloat16()
    res = torch.randn(m, 4, hidden, generator=g).bfloat16()
    post = torch.rand(m, 4, generator=g) * 2
    comb = torch.softmax(torch.randn(m, 4, 4, generator=g), dim=-1)
    out = e2e.ref_mhc_post(x, res, post, comb)
    np.savez_compressed(os.path.join(HERE, "mhc_post_7168.npz"), x=_u16(x), residual=_u16(res), post=post.numpy(),
                        comb=comb.numpy(), out=_u16(out))
    print("mhc_post_7168.npz", tuple(out.shape))


def model1_pool(g, pages, epb):
    """A pool of random MODEL1 records: finite e4m3 bytes, scale exponents near 0, bf16 rotary values."""
    stride = -(-epb * 584 // 576) * 576
    pool = torch.zeros(pages, stride, dtype=torch.uint8)
    body = torch.randint(0, 256, (pages, epb, 448), generator=g, dtype=torch.int64)
    body = torch.where((body & 0x7f) == 0x7f, body & 0x80, body).to(torch.uint8)   # no NaN patterns
    rope = (torch.randn(pages, epb, 64, generator=g) * 0.7).bfloat16().view(torch.uint8).view(pages, epb, 128)
    pool[:, :epb * 576] = torch.cat([body, rope], dim=-1).reshape(pages, epb * 576)
    sb = torch.zeros(pages, epb, 8, dtype=torch.uint8)
    sb[..., :7] = torch.randint(115, 122, (pages, epb, 7), generator=g).to(torch.uint8)
    pool[:, epb * 576:epb * 584] = sb.reshape(pages, epb * 8)
    return pool


def golden_sparse_mla(ref_root):
    """ref_flash_attn over records dequantised by deq_model1_row: window entries, then top-k entries."""
    e2e = _load(ref_root, "dsv4_megakernel/megakernel/test/test_e2e_decode.py", "ref_e2e")
    e2e.torch = torch
    e2e.DEV = "cpu"
    g = torch.Generator().manual_seed(83)
    batch, heads = 3, 16
    swa_epb, cmp_epb, swa_cap, cmp_cap = 256, 64, 128, 160
    swa_pool, cmp_pool = model1_pool(g, 2, swa_epb), model1_pool(g, 5, cmp_epb)
    swa_len, cmp_len = [128, 37, 0], [160, 75, 9]
    swa_idx = torch.full((batch, swa_cap), -1, dtype=torch.int32)
    cmp_idx = torch.full((batch, cmp_cap), -1, dtype=torch.int32)
    for b in range(batch):
        swa_idx[b, :swa_len[b]] = torch.randperm(2 * swa_epb, generator=g)[:swa_len[b]].int()
        cmp_idx[b, :cmp_len[b]] = torch.randperm(5 * cmp_epb, generator=g)[:cmp_len[b]].int()
    q = (torch.randn(batch, heads, 512, generator=g) * 1.5).bfloat16()
    sink = torch.randn(heads, generator=g)
    scale = 512 ** -0.5
    outs = []
    for b in range(batch):
        sw = [e2e.deq_model1_row(swa_pool, int(i) // swa_epb, int(i) % swa_epb, swa_epb) for i in swa_idx[b, :swa_len[b]]]
        cm = [e2e.deq_model1_row(cmp_pool, int(i) // cmp_epb, int(i) % cmp_epb, cmp_epb) for i in cmp_idx[b, :cmp_len[b]]]
        sw = torch.stack(sw) if sw else torch.zeros(0, 512)
        cm = torch.stack(cm) if cm else torch.zeros(0, 512)
        outs.append(e2e.ref_flash_attn(q[b].float(), sw, cm, scale, sink))
    out = torch.stack(outs)
    np.savez_compressed(os.path.join(HERE, "sparse_mla_h16.npz"), q=_u16(q), swa_pool=swa_pool.numpy(),
                        cmp_pool=cmp_pool.numpy(), swa_idx=swa_idx.numpy(), cmp_idx=cmp_idx.numpy(),
                        swa_len=np.asarray(swa_len, np.int32), cmp_len=np.asarray(cmp_len, np.int32),
                        sink=sink.numpy(), scale=np.float32(scale), swa_epb=np.int32(swa_epb), cmp_epb=np.int32(cmp_epb),
                        out=out.numpy())
    print("sparse_mla_h16.npz", tuple(out.shape))


def golden_cache_writers(ref_root):
    """Indexer compressor (FP8 form) and window-KV torch twins on seeded state rings."""
    wqb = _load(ref_root, "dsv4_megakernel/megakernel/test/test_wq_b_fp8_gemm.py", "ref_wqb")
    wqb.torch = torch
    g = torch.Generator().manual_seed(61)
    max_pos = 64
    ang = torch.outer(torch.arange(max_pos, dtype=torch.float32), 1.0 / (10000.0 ** (torch.arange(32) / 32.0)))
    cos, sin = torch.cos(ang).contiguous(), torch.sin(ang).contiguous()

    rows = 12
    pos = torch.tensor([3, 7, 11, 12, 15, 19, 23, 30, 31, 35, 47, 59])
    state = torch.randn(rows, 8, 512, generator=g)
    state[0, 4:, :256], state[0, 4:, 256:] = 0.0, float("-inf")     # a fresh request: entries 4..7 never written
    state[1, :, 256:] *= 8.0                                        # peaked softmax
    state_row = torch.arange(rows) * 8 + pos % 8
    norm_w = torch.rand(128, generator=g) + 0.5
    q, scale, mask = wqb.ref_comp_step(state, state_row, pos, norm_w, cos, sin, fp8=True)
    np.savez_compressed(os.path.join(HERE, "indexer_compressor_fp8.npz"), state=state.numpy(), pos=pos.numpy(),
                        state_row=state_row.numpy(), norm_w=norm_w.numpy(), cos=cos.numpy(), sin=sin.numpy(),
                        q8=q.view(torch.uint8).numpy(), scale=scale.numpy(), compress=mask.numpy())
    print("indexer_compressor_fp8.npz", int(mask.sum()), "compress rows of", rows)

    tokens, heads = 5, 64
    iq = (torch.randn(tokens, heads, 128, generator=g) * torch.rand(tokens, heads, 1, generator=g) * 4).bfloat16()
    iq[0, 0] = 0                                                      # an all-zero head: the 1e-12 clamp
    w = torch.randn(tokens, heads, generator=g) / 8
    qpos = torch.tensor([0, 1, 13, 40, 63], dtype=torch.int32)
    q, wf = wqb.ref_idx_fp8_chain(iq, w, qpos.long(), cos, sin)
    np.savez_compressed(os.path.join(HERE, "index_q_post_fp8.npz"), iq=_u16(iq), weights=w.numpy(), q_pos=qpos.numpy(),
                        cos=cos.numpy(), sin=sin.numpy(), q8=q.view(torch.uint8).numpy(), w_folded=wf.numpy())
    print("index_q_post_fp8.npz", tuple(q.shape))

    rows = 6
    y = torch.randn(rows, 512, generator=g) * torch.tensor([1.0, 0.01, 30.0, 1.0, 1e-4, 3.0]).view(rows, 1)
    wpos = torch.tensor([0, 1, 17, 33, 62, 63])
    wnorm = torch.rand(512, generator=g) + 0.5
    q8, s8, rope = wqb.ref_win_step(y, wpos, wnorm, cos, sin)
    np.savez_compressed(os.path.join(HERE, "window_kv_fp8.npz"), y=y.numpy(), pos=wpos.numpy(), norm_w=wnorm.numpy(),
                        cos=cos.numpy(), sin=sin.numpy(), q8=q8.view(torch.uint8).numpy(), s8=s8.numpy(),
                        rope=_u16(rope))
    print("window_kv_fp8.npz", tuple(q8.shape))


def golden_fp4_producers(ref_root):
    """The FP4 form of the indexer's producers: the torch twins ref_idx_chain (query: RoPE, Hadamard-128, MXFP4) and
    ref_comp_step with fp8=False (compressed key).  The twins return the dequantised values and the scales."""
    wqb = _load(ref_root, "dsv4_megakernel/megakernel/test/test_wq_b_fp8_gemm.py", "ref_wqb")
    wqb.torch = torch
    g = torch.Generator().manual_seed(67)
    max_pos = 64
    ang = torch.outer(torch.arange(max_pos, dtype=torch.float32), 1.0 / (10000.0 ** (torch.arange(32) / 32.0)))
    cos, sin = torch.cos(ang).contiguous(), torch.sin(ang).contiguous()

    tokens, heads = 6, 64
    iq = (torch.randn(tokens, heads, 128, generator=g) * torch.rand(tokens, heads, 1, generator=g) * 4).bfloat16()
    iq[0, 0] = 0                                                      # an all-zero head: the scale's lower clamp
    qpos = torch.tensor([0, 1, 13, 40, 62, 63], dtype=torch.int32)
    deq, sf = wqb.ref_idx_chain(iq.float().view(tokens, -1), qpos.long(), cos, sin)
    np.savez_compressed(os.path.join(HERE, "index_q_post_fp4.npz"), iq=_u16(iq), q_pos=qpos.numpy(), cos=cos.numpy(),
                        sin=sin.numpy(), deq=deq.numpy(), sf=sf.numpy())
    print("index_q_post_fp4.npz", tuple(deq.shape))

    rows = 12
    pos = torch.tensor([3, 7, 11, 12, 15, 19, 23, 30, 31, 35, 47, 59])
    state = torch.randn(rows, 8, 512, generator=g)
    state[0, 4:, :256], state[0, 4:, 256:] = 0.0, float("-inf")     # a fresh request: entries 4..7 never written
    state[1, :, 256:] *= 8.0                                        # peaked softmax
    state_row = torch.arange(rows) * 8 + pos % 8
    norm_w = torch.rand(128, generator=g) + 0.5
    deq, s4, mask = wqb.ref_comp_step(state, state_row, pos, norm_w, cos, sin, fp8=False)
    np.savez_compressed(os.path.join(HERE, "indexer_compressor_fp4.npz"), state=state.numpy(), pos=pos.numpy(),
                        state_row=state_row.numpy(), norm_w=norm_w.numpy(), cos=cos.numpy(), sin=sin.numpy(),
                        deq=deq.numpy(), s4=s4.numpy(), compress=mask.numpy())
    print("indexer_compressor_fp4.npz", int(mask.sum()), "compress rows of", rows)


def mhc_pre_inputs(seed=71, m=3, hidden=7168):
    """Seeded inputs of the mHC-pre fixture (regenerated by the tests: 2.75 MB of weights are not
    stored).  numpy's PCG64 stream is stable across versions; the fixture carries a checksum."""
    rng = np.random.default_rng(seed)
    x = torch.from_numpy(rng.standard_normal((m, 4, hidden), dtype=np.float32)).bfloat16()
    weight = rng.standard_normal((24, 4 * hidden), dtype=np.float32) * np.float32(0.01)
    base = rng.standard_normal(24, dtype=np.float32) * np.float32(0.1)
    scale = np.array([1.0, 0.7, 1.3], np.float32)
    return x, weight, base, scale


def golden_mhc_pre(ref_root):
    hc = _load(ref_root, "dsv4_megakernel/megakernel/test/test_hc_fused_tc.py", "ref_hc")
    hc.torch = torch
    x, weight, base, scale = mhc_pre_inputs()
    collapsed, pre, post, comb = hc.hc_reference(x, torch.from_numpy(weight), torch.from_numpy(base),
                                                 torch.from_numpy(scale))
    check = float(np.abs(weight).sum() + np.abs(_u16(x).astype(np.float64)).sum() % 1e6)
    np.savez_compressed(os.path.join(HERE, "mhc_pre_7168.npz"), collapsed=_u16(collapsed), pre=pre.numpy(),
                        post=post.numpy(), comb=comb.numpy(), input_checksum=check)
    print("mhc_pre_7168.npz", tuple(collapsed.shape))


def golden_moe_gate(ref_root):
    """The origin's Gate on seeded inputs, once per score function, with and without a bias."""
    import types
    model = _load(ref_root, "dsv4_megakernel/origin/model.py", "ref_origin_model_gate")
    model.torch = torch
    g = torch.Generator().manual_seed(81)
    tokens, dim, experts, topk = 7, 256, 256, 8
    x = torch.randn(tokens, dim, generator=g).bfloat16()
    w = (torch.randn(experts, dim, generator=g) * 0.08).bfloat16()
    bias = torch.randn(experts, generator=g) * 0.05
    out = dict(x=_u16(x), weight=_u16(w), bias=bias.numpy(), route_scale=2.5, topk=topk)
    for name in ("softmax", "sigmoid", "sqrtsoftplus"):
        args = types.SimpleNamespace(dim=dim, n_activated_experts=topk, score_func=name, route_scale=2.5,
                                     n_hash_layers=0, n_routed_experts=experts, vocab_size=16)
        gate = model.Gate(1, args)
        gate.weight.data = w.float()
        gate.bias.data = bias.clone()
        weights, indices = gate(x.float())
        out["weights_" + name], out["indices_" + name] = weights.detach().numpy(), indices.numpy().astype(np.int32)
    np.savez_compressed(os.path.join(HERE, "moe_gate_256.npz"), **out)
    print("moe_gate_256.npz", tuple(weights.shape))


def golden_query_rms_rope():
    """The inline twin of the fused query tail (test_mqa_logits_fp4.py:404-413): per head row of 512,
    x * rsqrt(mean x^2 + eps) without a weight, the last 64 dims rotated in interleaved pairs at the token's
    position, one rounding to bf16 at the end; input_heads 64 repeats the heads to 128 (here 4 -> 8)."""
    g = torch.Generator().manual_seed(91)
    batch, eps, max_pos = 5, 1e-6, 64
    ang = torch.outer(torch.arange(max_pos, dtype=torch.float32), 1.0 / (10000.0 ** (torch.arange(32) / 32.0)))
    cos_tab, sin_tab = torch.cos(ang).contiguous(), torch.sin(ang).contiguous()
    positions = torch.tensor([0, 1, 17, 40, 63])
    out = dict(cos=cos_tab.numpy(), sin=sin_tab.numpy(), positions=positions.numpy(), eps=eps)
    for name, input_heads, out_heads in (("full", 8, 8), ("half", 4, 8)):
        query_x = (torch.randn(batch, input_heads, 512, generator=g) *
                   torch.tensor([1.0, 0.02, 30.0, 1.0, 5.0]).view(batch, 1, 1)).bfloat16()
        source = query_x if input_heads == out_heads else query_x.repeat(1, out_heads // input_heads, 1)
        source_f = source.float()
        ref = source_f * torch.rsqrt(source_f.square().mean(-1, keepdim=True) + eps)
        even, odd = ref[..., 448::2].clone(), ref[..., 449::2].clone()
        cos = cos_tab[positions, None, :]
        sin = sin_tab[positions, None, :]
        ref[..., 448::2] = even * cos - odd * sin
        ref[..., 449::2] = even * sin + odd * cos
        out["x_" + name], out["out_" + name] = _u16(query_x), _u16(ref.bfloat16())
    np.savez_compressed(os.path.join(HERE, "query_rms_rope.npz"), **out)
    print("query_rms_rope.npz", tuple(out["out_half"].shape))


def golden_main_compressor():
    """The inline twin of the MAIN compressor row (test_mqa_logits_fp4.py:772-791): softmax-weighted sum over
    the eight ring rows that end at the current one (rows 0..3 of the window read columns [0, 512), rows 4..7
    columns [512, 1024) of the kv and score halves), bf16, RMSNorm(512) with an fp32 weight, bf16, RoPE of the
    last 64 dims at position pos + 1 - 4, and the power-of-two scale per 64 of the first 448 values.  Stored:
    the twin's pre-quantisation values, its scales and its rotary tail."""
    g = torch.Generator().manual_seed(93)
    B, S = 10, 64
    ang = torch.outer(torch.arange(S, dtype=torch.float32), 1.0 / (10000.0 ** (torch.arange(32) / 32.0)))
    cos_tab, sin_tab = torch.cos(ang).contiguous(), torch.sin(ang).contiguous()
    pos = torch.tensor([3, 4, 7, 11, 15, 19, 30, 31, 47, 63])
    comp_state = torch.randn(B, 8, 2048, generator=g)
    comp_state[2, :, 1024:] *= 6.0                                    # a peaked softmax
    comp_state[3] *= torch.tensor(0.01)                               # small values: the 1e-4 scale floor
    comp_norm = torch.rand(512, generator=g) + 0.5
    state_rows = torch.arange(B) * 8 + pos % 8
    idx = torch.arange(512)
    blk_all, scale_all, rope_all = torch.zeros(B, 448), torch.full((B, 7), -1.0), torch.zeros(B, 64)
    mask = torch.zeros(B, dtype=torch.bool)
    for m in range(B):
        p = int(pos[m])
        if (p + 1) % 4 != 0:
            continue
        mask[m] = True
        current = int(state_rows[m]) % 8
        perm = [(current - 7 + r) % 8 for r in range(8)]
        kv0, sc0 = comp_state[m, :, :1024], comp_state[m, :, 1024:]
        col = torch.stack([idx if r < 4 else idx + 512 for r in range(8)])
        sc8 = torch.gather(sc0[perm], 1, col)
        kv8 = torch.gather(kv0[perm], 1, col)
        e = torch.exp(sc8 - sc8.max(0).values)
        agg = (e * kv8).sum(0) / e.sum(0)
        vb = agg.bfloat16().float()
        rms = torch.rsqrt((vb * vb).sum() / 512.0 + 1e-6)
        ro = (vb * rms * comp_norm).bfloat16().float()
        ri = p + 1 - 4
        ev, ov = ro[448::2].clone(), ro[449::2].clone()
        ro[448::2] = (ev * cos_tab[ri] - ov * sin_tab[ri]).bfloat16().float()
        ro[449::2] = (ev * sin_tab[ri] + ov * cos_tab[ri]).bfloat16().float()
        blk = ro[:448].view(7, 64)
        scale_ref = torch.pow(2.0, (blk.abs().max(1).values / 448.0).clamp_min(1e-4).log2().ceil())
        blk_all[m], scale_all[m], rope_all[m] = ro[:448], scale_ref, ro[448:]
    np.savez_compressed(os.path.join(HERE, "main_compressor_fp8.npz"), state=comp_state.numpy(), pos=pos.numpy(),
                        state_row=state_rows.numpy(), norm_w=comp_norm.numpy(), cos=cos_tab.numpy(), sin=sin_tab.numpy(),
                        values=blk_all.numpy(), scale=scale_all.numpy(), rope=_u16(rope_all.bfloat16()),
                        compress=mask.numpy())
    print("main_compressor_fp8.npz", int(mask.sum()), "compress rows of", B)


def golden_moe_block(ref_root):
    """The origin's MoE module (Gate + routed Experts + shared Expert, origin/model.py:546-644) on bf16
    weights, world_size 1, run on the CPU: the block structure (selection with a bias, weights without it,
    fp32 accumulation over experts, the shared expert added last, one cast at the end) that the NVFP4 / FP8
    arithmetic of this library is laid over.  The weights are exactly representable in bf16."""
    import types
    model = _load(ref_root, "dsv4_megakernel/origin/model.py", "ref_origin_model_moe")
    model.torch = torch
    g = torch.Generator().manual_seed(97)
    tokens, dim, inter, experts, topk = 9, 256, 256, 8, 3
    out = {}
    for name, limit in (("plain", 0.0), ("limit", 1.5)):
        args = types.SimpleNamespace(dim=dim, moe_inter_dim=inter, n_routed_experts=experts, n_shared_experts=1,
                                     n_activated_experts=topk, score_func="sqrtsoftplus", route_scale=2.5, n_hash_layers=0,
                                     vocab_size=16, expert_dtype=None, swiglu_limit=limit)
        with model.set_dtype(torch.bfloat16):
            block = model.MoE(1, args)
        bf = lambda *s, scale: (torch.randn(*s, generator=g) * scale).bfloat16()
        block.gate.weight.data = bf(experts, dim, scale=0.08).float()
        block.gate.bias.data = torch.randn(experts, generator=g) * 0.05
        w1, w3, w2 = bf(experts + 1, inter, dim, scale=0.08), bf(experts + 1, inter, dim, scale=0.08), bf(experts + 1, dim, inter, scale=0.08)
        for e, mod in enumerate(list(block.experts) + [block.shared_experts]):
            mod.w1.weight.data, mod.w3.weight.data, mod.w2.weight.data = w1[e].clone(), w3[e].clone(), w2[e].clone()
        x = (torch.randn(tokens, dim, generator=g) * 1.5).bfloat16()
        with torch.no_grad():
            y = block(x.view(1, tokens, dim), torch.zeros(1, tokens, dtype=torch.long)).view(tokens, dim)
            weights, indices = block.gate(x, None)
        out.update({"x_" + name: _u16(x), "gate_w_" + name: _u16(block.gate.weight.data.bfloat16()),
                    "gate_bias_" + name: block.gate.bias.data.numpy(), "w1_" + name: _u16(w1), "w3_" + name: _u16(w3),
                    "w2_" + name: _u16(w2), "y_" + name: _u16(y), "indices_" + name: indices.numpy().astype(np.int32),
                    "weights_" + name: weights.float().numpy(), "limit_" + name: limit})
    np.savez_compressed(os.path.join(HERE, "moe_block_origin.npz"), topk=topk, route_scale=2.5, **out)
    print("moe_block_origin.npz", tuple(y.shape))


KV_TRACE_CONFIGS = [
    dict(capacity=5, pages_per_pool=96, max_pages_per_req=12),
    dict(capacity=5, pages_per_pool=96, max_pages_per_req=12, state_ring_entries=16),
    dict(capacity=4, pages_per_pool=400, max_pages_per_req=40, swa_entries_per_block=64,
         cmp_entries_per_block=32, idx_entries_per_block=16),
]


def kv_trace(manager_cls, config, ops):
    """Replays a scripted request lifecycle on a cache manager and records everything it hands
    out.  `ops` is a list of ("alloc",), ("free", live index) and ("step", [live indices])."""
    m = manager_cls(device="cpu", **config)
    live, out = [], []
    for op in ops:
        if op[0] == "alloc":
            live.append(m.alloc_request())
            out.append(["alloc", live[-1]])
        elif op[0] == "free":
            slot = live.pop(op[1])
            m.free_request(slot)
            out.append(["free", slot])
        else:
            slots = [live[i] for i in op[1]]
            st = m.step_begin(slots)
            pos = st["pos"].tolist()
            swa, swa_len = m.swa_indices(slots, pos, 128)
            out.append(["step", {
                "slots": slots, "pos": pos, "q_pos": st["q_pos"].tolist(),
                "main_state_row": st["main_state_row"].tolist(), "idx_state_row": st["idx_state_row"].tolist(),
                "idx_dst": st["idx_dst"].tolist(), "cmp_dst": st["cmp_dst"].tolist(), "swa_dst": st["swa_dst"].tolist(),
                "block_table": {n: m.block_table(n, slots).tolist() for n in ("swa", "cmp", "idx")},
                "swa_indices": swa.tolist(), "swa_lens": swa_len.tolist(),
                "n_compressed": m.n_compressed(slots, pos).tolist()}])
    geometry = {n: m.geometry(n) for n in ("swa", "cmp", "idx")}
    shapes = {"main_state": list(m.main_state.shape), "idx_state": list(m.idx_state.shape),
              "swa_pool": list(m.swa_pool.shape), "cmp_pool": list(m.cmp_pool.shape), "idx_pool": list(m.idx_pool.shape),
              "cmp_view": [list(m.model1_cache_view("cmp").shape), list(m.model1_cache_view("cmp").stride())],
              "idx_view": [list(m.indexer_cache_view().shape), list(m.indexer_cache_view().stride())]}
    return {"events": out, "geometry": geometry, "shapes": shapes}


def kv_script(seed, capacity, steps):
    import random
    rnd = random.Random(seed)
    live, ops = 0, []
    for _ in range(steps):
        r = rnd.random()
        if live == 0 or (r < 0.05 and live < capacity):
            ops.append(("alloc",))
            live += 1
        elif r < 0.07:
            ops.append(("free", rnd.randrange(live)))
            live -= 1
            if live == 0:
                continue
        chosen = [i for i in range(live) if rnd.random() < 0.9] or [0]
        ops.append(("step", chosen))
    return ops


def golden_fp4_gemm(ref_root):
    """FP8 activations x FP4 weights.  The weights are quantised by the reference test's per_token_cast_to_fp4 (e2m1,
    one ue8m0 scale per 32), turned into the origin's lossless e4m3 form with 128x128 scales by its own
    cast_e2m1fn_to_e4m3fn (origin/convert.py:20-52: this is what fixes the nibble order, the code table and the
    meaning of the scale bytes), and dequantised by the test's cast_back_from_fp4; the activations by quant_act_fp8
    with power-of-two scales.  Expected output: the double-precision product of the dequantised operands."""
    ref_mqa = _load(ref_root, "dsv4_megakernel/megakernel/test/test_mqa_logits_fp4.py", "ref_mqa_fp4gemm")
    conv = _load(ref_root, "dsv4_megakernel/origin/convert.py", "ref_origin_convert")
    conv.torch = torch
    g = torch.Generator().manual_seed(97)
    m, n, k = 24, 256, 512
    w = (torch.randn(n, k, generator=g) * 0.05 * torch.exp(torch.randn(n, 1, generator=g) * 0.7)).bfloat16().float()
    packed, sf_words = ref_mqa.per_token_cast_to_fp4(w.float(), use_ue8m0=True, gran_k=32, use_packed_ue8m0=True)
    sf_bytes = sf_words.contiguous().view(torch.uint8).view(n, k // 32)
    w_deq = ref_mqa.cast_back_from_fp4(packed, sf_words)
    scale_f = (sf_bytes.to(torch.int32) << 23).view(torch.float32)
    w8, w8_scale = conv.cast_e2m1fn_to_e4m3fn(packed.contiguous(), scale_f)
    x = torch.randn(m, k, generator=g).bfloat16()
    xb = x.view(m, k // 128, 128).float()
    amax = xb.abs().amax(-1).clamp_min(1e-4)
    a_s = torch.exp2(torch.ceil(torch.log2(amax / 448.0)))
    a8 = (xb / a_s[..., None]).to(torch.float8_e4m3fn)
    a_deq = (a8.float() * a_s[..., None]).view(m, k)
    c = a_deq.double() @ w_deq.double().T
    np.savez_compressed(os.path.join(HERE, "fp4_gemm.npz"), a=a8.view(m, k).view(torch.uint8).numpy(), a_s=a_s.numpy(),
                        w4=packed.view(torch.uint8).numpy(), w_sf=sf_bytes.numpy(),
                        w8=w8.view(torch.uint8).numpy(), w8_scale=w8_scale.float().numpy(), w_deq=w_deq.numpy(), w=w.numpy(),
                        c=c.float().numpy())
    print("fp4_gemm.npz", m, n, k)


def golden_kv_cache(ref_root):
    import gzip
    import json
    ref = _load(ref_root, "dsv4_megakernel/megakernel/test/kv_cache_manager.py", "ref_kv_cache")
    ref.torch = torch
    traces = []
    for n, config in enumerate(KV_TRACE_CONFIGS):
        ops = kv_script(50 + n, config["capacity"], 420)
        traces.append({"config": config, "ops": ops, "expect": kv_trace(ref.KVCacheManager, config, ops)})
    with gzip.open(os.path.join(HERE, "kv_cache_trace.json.gz"), "wt") as f:
        json.dump(traces, f)
    print("kv_cache_trace.json.gz", sum(len(t["ops"]) for t in traces), "ops")


def main():
    if len(sys.argv) < 2 and "WUDA_REFERENCE_ROOT" not in os.environ:
        sys.exit("usage: make_golden.py <path to a checkout of the reference>  (or set WUDA_REFERENCE_ROOT)")
    ref_root = sys.argv[1] if len(sys.argv) > 1 else os.environ["WUDA_REFERENCE_ROOT"]
    only = set(sys.argv[2:])          # optional: names of single generators, e.g. `golden_moe_block`
    if only:
        for name in sorted(only):
            fn = globals()[name]
            fn(ref_root) if fn.__code__.co_argcount else fn()
        return
    tdir = "dsv4_megakernel/megakernel/test"
    ref_mqa = _load(ref_root, tdir + "/test_mqa_logits_fp4.py", "ref_mqa")
    golden_mqa(ref_mqa, "mqa_logits_fp8_n1.npz", batch=3, next_n=1, ctx_lo=1, ctx_hi=400, epb=64, seed=11)
    golden_mqa(ref_mqa, "mqa_logits_fp8_n2_epb32.npz", batch=2, next_n=2, ctx_lo=60, ctx_hi=300, epb=32,
               seed=12, page_pad=128)
    golden_mqa_fp4(ref_mqa)
    ref_topk = _load(ref_root, tdir + "/test_topk_v2.py", "ref_topk")
    golden_topk(ref_topk, "topk_random.npz", 3, 3000, 512, [3000, 2100, 300], 0, 21)
    golden_topk(ref_topk, "topk_ties.npz", 2, 4096, 1024, [4096, 2500], 7, 22)
    golden_norm_rope_quant(ref_root)
    golden_mhc_post(ref_root)
    golden_kv_cache(ref_root)
    golden_cache_writers(ref_root)
    golden_fp4_producers(ref_root)
    golden_mhc_pre(ref_root)
    golden_moe_gate(ref_root)
    golden_sparse_mla(ref_root)
    golden_query_rms_rope()
    golden_main_compressor()
    golden_moe_block(ref_root)
    golden_fp4_gemm(ref_root)


if __name__ == "__main__":
    main()
