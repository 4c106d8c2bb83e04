"""numpy-facing wrappers around liboracle.so (the plain-C oracle).

TEST INFRASTRUCTURE: the checker for parity tests and the timed CPU baseline, never a
code path of the product.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")


def build(force=False):
    """Compile oracle.c with gcc (make). The CPU flags are -march=native, so the library
    is rebuilt on the machine that runs it when it is stale or was built elsewhere."""
    src = os.path.join(_HERE, "oracle.c")
    stale = (not os.path.exists(_LIB_PATH)) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src)
    if force or stale:
        subprocess.check_call(["make", "-s", "-B", "-C", _HERE, "liboracle.so"])
    return _LIB_PATH


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        try:
            _lib = ctypes.CDLL(_LIB_PATH)
        except OSError:
            build(force=True)
            _lib = ctypes.CDLL(_LIB_PATH)
        _declare(_lib)
    return _lib


def _declare(l):
    c = ctypes
    l.oracle_e4m3_decode.argtypes = [c.c_void_p, c.c_void_p, c.c_int64]
    l.oracle_e4m3_encode.argtypes = [c.c_void_p, c.c_void_p, c.c_int64]
    l.oracle_mqa_logits_fp8.argtypes = [c.c_void_p] * 6 + [c.c_int] * 4 + [c.c_int64, c.c_int, c.c_int64]
    l.oracle_mqa_logits_fp8.restype = c.c_int
    l.oracle_topk.argtypes = [c.c_void_p] * 5 + [c.c_int, c.c_int64, c.c_int64, c.c_int, c.c_int]
    l.oracle_topk.restype = c.c_int
    l.oracle_num_threads.restype = c.c_int
    l.oracle_set_num_threads.argtypes = [c.c_int]
    l.oracle_rmsnorm_bf16.argtypes = [c.c_void_p, c.c_void_p, c.c_int, c.c_float, c.c_void_p, c.c_int, c.c_int]
    l.oracle_act_quant_fp8.argtypes = [c.c_void_p, c.c_void_p, c.c_void_p, c.c_int, c.c_int, c.c_int, c.c_int]
    l.oracle_rope_bf16.argtypes = [c.c_void_p, c.c_void_p, c.c_void_p, c.c_void_p, c.c_int, c.c_int, c.c_int,
                                   c.c_int, c.c_int]
    l.oracle_mhc_post.argtypes = [c.c_void_p] * 5 + [c.c_int, c.c_int]
    vp, i64 = c.c_void_p, c.c_int64
    l.oracle_indexer_compressor_fp8.argtypes = [vp, vp, c.c_int, vp, vp, vp, vp, c.c_int, c.c_float, vp, vp, c.c_int,
                                                i64, vp, vp, c.c_int]
    l.oracle_main_compressor_fp8.argtypes = [vp, vp, c.c_int, vp, vp, vp, vp, c.c_int, c.c_float, vp, vp, c.c_int,
                                             i64, vp, vp, vp, c.c_int]
    l.oracle_window_kv_fp8.argtypes = [vp, vp, vp, vp, vp, c.c_int, c.c_float, vp, vp, c.c_int, i64, vp, vp, vp,
                                       c.c_int]
    l.oracle_index_q_post_fp8.argtypes = [vp, i64, vp, vp, vp, c.c_int, vp, vp, vp, c.c_int, c.c_int]
    l.oracle_index_q_post_fp4.argtypes = [vp, i64, vp, vp, vp, c.c_int, vp, vp, c.c_int, c.c_int]
    l.oracle_indexer_compressor_fp4.argtypes = [vp, vp, c.c_int, vp, vp, vp, vp, c.c_int, c.c_float, vp, vp, c.c_int,
                                                i64, vp, vp, c.c_int]
    l.oracle_query_rms_rope.argtypes = [vp, i64, vp, vp, vp, c.c_int, vp, c.c_int, c.c_int, c.c_int, c.c_float]
    l.oracle_mhc_pre.argtypes = [vp, vp, vp, vp, vp, c.c_float, c.c_float, c.c_float, vp, vp, vp, vp, vp, vp, vp,
                                 c.c_int, c.c_int]
    l.oracle_sparse_mla.argtypes = [vp, vp, i64, c.c_int, vp, vp, c.c_int, vp, i64, c.c_int, vp, vp, c.c_int, vp,
                                    c.c_float, vp, c.c_int, c.c_int]
    l.oracle_moe_route.argtypes = [vp, vp, vp, vp, c.c_int, c.c_int, c.c_int, c.c_int, c.c_float]
    l.oracle_gemm_nvfp4.argtypes = [c.c_void_p, c.c_void_p, c.c_float, c.c_void_p, c.c_void_p, c.c_float, c.c_void_p,
                                    c.c_int, c.c_int, c.c_int, c.c_int]
    l.oracle_gemm_fp8_blockscaled.argtypes = [c.c_void_p, c.c_void_p, c.c_void_p, c.c_void_p, c.c_void_p,
                                              c.c_int, c.c_int, c.c_int, c.c_int]
    l.oracle_gemm_fp8_fp4.argtypes = [vp, vp, vp, vp, vp, c.c_int, c.c_int, c.c_int, c.c_int]
    l.oracle_fp4_act_quant.argtypes = [vp, i64, c.c_int, vp, vp, vp]
    l.oracle_head_ssq.argtypes = [vp, i64, vp]


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p) if a is not None else None


def _c(a, dtype):
    a = np.ascontiguousarray(a, dtype=dtype)
    return a


def num_threads():
    return int(lib().oracle_num_threads())


def set_num_threads(n=None):
    """Use n threads in the oracle's parallel loops (default: every core this process may run on),
    whatever OMP_NUM_THREADS said when the library was loaded.  Returns the count now in force."""
    if n is None:
        n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    lib().oracle_set_num_threads(int(n))
    return num_threads()


def e4m3_decode(u8):
    u8 = _c(u8, np.uint8)
    out = np.empty(u8.shape, np.float32)
    lib().oracle_e4m3_decode(_p(u8), _p(out), u8.size)
    return out


def e4m3_encode(f32):
    f32 = _c(f32, np.float32)
    out = np.empty(f32.shape, np.uint8)
    lib().oracle_e4m3_encode(_p(f32), _p(out), f32.size)
    return out


def mqa_logits_fp8(q, kv_pages, weights, context_lens, block_table, next_n, epb, logits_stride,
                   fill=-np.inf):
    """q uint8 [rows,64,128]; kv_pages uint8 [num_blocks, stride]; weights f32 [rows,64];
    context_lens int32 [batch, next_n]; block_table int32 [batch, P].  Returns
    fp32 [rows, logits_stride] pre-filled with `fill` (only t < context is written)."""
    q = _c(q, np.uint8)
    kv_pages = _c(kv_pages, np.uint8)
    weights = _c(weights, np.float32)
    context_lens = _c(context_lens, np.int32).reshape(-1, next_n)
    block_table = _c(block_table, np.int32)
    batch = context_lens.shape[0]
    rows = batch * next_n
    assert q.shape == (rows, 64, 128) and weights.shape == (rows, 64)
    logits = np.full((rows, logits_stride), fill, np.float32)
    rc = lib().oracle_mqa_logits_fp8(_p(q), _p(kv_pages), _p(weights), _p(context_lens), _p(block_table),
                                     _p(logits), batch, next_n, kv_pages.shape[0], epb,
                                     kv_pages.shape[1], block_table.shape[1], logits_stride)
    if rc != 0:
        raise ValueError("oracle_mqa_logits_fp8: block table entry outside the pool (rc=%d)" % rc)
    return logits


def topk(scores, seq_lens, page_table, k, page_size=64):
    """Returns (page_indices, raw_indices), int32 [rows, k], descending score order,
    ties by lower index."""
    scores = _c(scores, np.float32)
    seq_lens = _c(seq_lens, np.int32)
    page_table = _c(page_table, np.int32)
    rows = scores.shape[0]
    out = np.empty((rows, k), np.int32)
    raw = np.empty((rows, k), np.int32)
    rc = lib().oracle_topk(_p(scores), _p(seq_lens), _p(page_table), _p(out), _p(raw), rows,
                           scores.shape[1], page_table.shape[1], k, page_size)
    if rc != 0:
        raise ValueError("oracle_topk: page_size must be a power of two")
    return out, raw


def rmsnorm_bf16(x_bf16, gamma, eps=1e-6):
    """x: uint16 view of bf16 [rows, dim]; gamma fp32 [dim] or uint16 (bf16) [dim]. Returns uint16 (bf16)."""
    x = _c(x_bf16, np.uint16)
    is_bf16 = np.asarray(gamma).dtype == np.uint16
    g = _c(gamma, np.uint16 if is_bf16 else np.float32)
    y = np.empty_like(x)
    lib().oracle_rmsnorm_bf16(_p(x), _p(g), int(is_bf16), eps, _p(y), x.shape[0], x.shape[1])
    return y


def act_quant_fp8(x_bf16, block=128, round_scale=False):
    """x: uint16 view of bf16 [rows, dim]. Returns (e4m3 bytes [rows, dim], fp32 scales [rows, dim/block])."""
    x = _c(x_bf16, np.uint16)
    y = np.empty(x.shape, np.uint8)
    s = np.empty((x.shape[0], x.shape[1] // block), np.float32)
    lib().oracle_act_quant_fp8(_p(x), _p(y), _p(s), x.shape[0], x.shape[1], block, int(round_scale))
    return y, s


def rope_bf16(x_bf16, positions, cos_t, sin_t, rope_dim, inverse=False):
    """x: uint16 view of bf16 [tokens, heads, head_dim]; rotates the last rope_dim dims. Returns a copy."""
    x = _c(x_bf16, np.uint16).copy()
    pos = _c(positions, np.int64)
    cos_t, sin_t = _c(cos_t, np.float32), _c(sin_t, np.float32)
    lib().oracle_rope_bf16(_p(x), _p(pos), _p(cos_t), _p(sin_t), x.shape[0], x.shape[1], x.shape[2], rope_dim,
                           int(inverse))
    return x


def mhc_post(x_bf16, res_bf16, post, comb):
    """x uint16 (bf16) [M,H], res uint16 [M,4,H], post fp32 [M,4], comb fp32 [M,4,4] -> uint16 [M,4,H]."""
    x, res = _c(x_bf16, np.uint16), _c(res_bf16, np.uint16)
    post, comb = _c(post, np.float32), _c(comb, np.float32)
    out = np.empty_like(res)
    lib().oracle_mhc_post(_p(x), _p(res), _p(post), _p(comb), _p(out), x.shape[0], x.shape[1])
    return out


def _pool_args(pool, dst, epb):
    if pool is None:
        return None, None, 1, 0
    assert pool.dtype == np.uint8 and pool.ndim == 2 and pool.flags.c_contiguous
    return pool, _c(dst, np.int64), int(epb), pool.shape[1]


def indexer_compressor_fp8(state, state_row, pos, norm_w, cos_t, sin_t, eps=1e-6, pool=None, dst=None, epb=64):
    """state fp32 [blocks, ring, 512].  Returns (q8 [rows,128] uint8, scale [rows] fp32); rows that do not
    compress keep the fill (0xAB / -1).  `pool` (uint8 [pages, stride]) is written in place."""
    state = _c(state, np.float32)
    rows = len(pos)
    q8, s8 = np.full((rows, 128), 0xAB, np.uint8), np.full(rows, -1.0, np.float32)
    pool, dst, epb, stride = _pool_args(pool, dst, epb)
    sr, ps = _c(state_row, np.int64), _c(pos, np.int64)
    nw, ct, st = _c(norm_w, np.float32), _c(cos_t, np.float32), _c(sin_t, np.float32)
    lib().oracle_indexer_compressor_fp8(_p(state), _p(sr), state.shape[1], _p(ps), _p(nw), _p(ct), _p(st), ct.shape[0],
                                        eps, _p(pool), _p(dst), epb, stride, _p(q8), _p(s8), rows)
    return q8, s8


def main_compressor_fp8(state, state_row, pos, norm_w, cos_t, sin_t, eps=1e-6, pool=None, dst=None, epb=64):
    """state fp32 [blocks, ring, 2048].  Returns (q8 [rows,448], s8 [rows,7], rope uint16 [rows,64])."""
    state = _c(state, np.float32)
    rows = len(pos)
    q8, s8 = np.full((rows, 448), 0xAB, np.uint8), np.full((rows, 7), -1.0, np.float32)
    rope = np.zeros((rows, 64), np.uint16)
    pool, dst, epb, stride = _pool_args(pool, dst, epb)
    sr, ps = _c(state_row, np.int64), _c(pos, np.int64)
    nw, ct, st = _c(norm_w, np.float32), _c(cos_t, np.float32), _c(sin_t, np.float32)
    lib().oracle_main_compressor_fp8(_p(state), _p(sr), state.shape[1], _p(ps), _p(nw), _p(ct), _p(st), ct.shape[0], eps,
                                     _p(pool), _p(dst), epb, stride, _p(q8), _p(s8), _p(rope), rows)
    return q8, s8, rope


def window_kv_fp8(y, pos, norm_w, cos_t, sin_t, eps=1e-6, pool=None, dst=None, epb=256):
    """y fp32 [rows,512].  Returns (q8 [rows,448], s8 [rows,7], rope uint16 [rows,64])."""
    y = _c(y, np.float32)
    rows = y.shape[0]
    q8, s8 = np.empty((rows, 448), np.uint8), np.empty((rows, 7), np.float32)
    rope = np.empty((rows, 64), np.uint16)
    pool, dst, epb, stride = _pool_args(pool, dst, epb)
    ps = _c(pos, np.int64)
    nw, ct, st = _c(norm_w, np.float32), _c(cos_t, np.float32), _c(sin_t, np.float32)
    lib().oracle_window_kv_fp8(_p(y), _p(ps), _p(nw), _p(ct), _p(st), ct.shape[0], eps, _p(pool), _p(dst), epb, stride,
                               _p(q8), _p(s8), _p(rope), rows)
    return q8, s8, rope


def index_q_post_fp8(x_bf16, q_pos, cos_t, sin_t, weights=None):
    """x uint16 (bf16) [tokens, heads, 128] -> (q8 uint8 [tokens, heads, 128], weights * scale [tokens, heads])."""
    x = _c(x_bf16, np.uint16)
    tokens, heads = x.shape[0], x.shape[1]
    ct, st = _c(cos_t, np.float32), _c(sin_t, np.float32)
    q8, w = np.empty((tokens, heads, 128), np.uint8), np.empty((tokens, heads), np.float32)
    wt = None if weights is None else _c(weights, np.float32)
    lib().oracle_index_q_post_fp8(_p(x), heads * 128, _p(_c(q_pos, np.int32)), _p(ct), _p(st), ct.shape[0], _p(wt),
                                  _p(q8), _p(w), tokens, heads)
    return q8, w


def index_q_post_fp4(x_bf16, q_pos, cos_t, sin_t):
    """x uint16 (bf16) [tokens, heads, 128] -> (packed e2m1 uint8 [tokens, heads, 64], scale words uint32
    [tokens, heads]): RoPE on the last 64, Hadamard-128, one power-of-two scale per 32 values."""
    x = _c(x_bf16, np.uint16)
    tokens, heads = x.shape[0], x.shape[1]
    ct, st = _c(cos_t, np.float32), _c(sin_t, np.float32)
    q4, sf = np.empty((tokens, heads, 64), np.uint8), np.empty((tokens, heads), np.uint32)
    lib().oracle_index_q_post_fp4(_p(x), heads * 128, _p(_c(q_pos, np.int32)), _p(ct), _p(st), ct.shape[0], _p(q4),
                                  _p(sf), tokens, heads)
    return q4, sf


def indexer_compressor_fp4(state, state_row, pos, norm_w, cos_t, sin_t, eps=1e-6, pool=None, dst=None, epb=64):
    """The FP4 form of the indexer compressor.  Returns (packed e2m1 [rows, 64] uint8, exponent bytes [rows, 4]
    uint8); rows that do not compress keep the fill (0xAB).  `pool` (uint8 [pages, stride], 68 bytes per entry)
    is written in place."""
    state = _c(state, np.float32)
    rows = len(pos)
    q4, s4 = np.full((rows, 64), 0xAB, np.uint8), np.full((rows, 4), 0xAB, np.uint8)
    pool, dst, epb, stride = _pool_args(pool, dst, epb)
    sr, ps = _c(state_row, np.int64), _c(pos, np.int64)
    nw, ct, st = _c(norm_w, np.float32), _c(cos_t, np.float32), _c(sin_t, np.float32)
    lib().oracle_indexer_compressor_fp4(_p(state), _p(sr), state.shape[1], _p(ps), _p(nw), _p(ct), _p(st), ct.shape[0],
                                        eps, _p(pool), _p(dst), epb, stride, _p(q4), _p(s4), rows)
    return q4, s4


def query_rms_rope(x_bf16, positions, cos_t, sin_t, out_heads=None, eps=1e-6):
    """x uint16 (bf16) [tokens, heads, 512] -> uint16 [tokens, out_heads, 512]."""
    x = _c(x_bf16, np.uint16)
    tokens, heads = x.shape[0], x.shape[1]
    out_heads = out_heads or heads
    ct, st = _c(cos_t, np.float32), _c(sin_t, np.float32)
    out = np.empty((tokens, out_heads, 512), np.uint16)
    lib().oracle_query_rms_rope(_p(x), heads * 512, _p(_c(positions, np.int64)), _p(ct), _p(st), ct.shape[0], _p(out),
                                tokens, heads, out_heads, eps)
    return out


def mhc_pre(hidden_bf16, weight, base, scale, gamma_bf16=None, hc_eps=1e-6, rms_eps=1e-6, norm_eps=1e-6):
    """hidden uint16 (bf16) [M,4,D], weight fp32 [24,4D].  Returns a dict: pre, post [M,4], comb [M,4,4],
    collapsed uint16 [M,D] and, with gamma, normed uint16 [M,D], xq uint8 [M,D], xsf fp32 [M,D/128]."""
    x = _c(hidden_bf16, np.uint16)
    m, _, d = x.shape
    w, b, sc = _c(weight, np.float32), _c(base, np.float32), _c(scale, np.float32)
    out = dict(pre=np.empty((m, 4), np.float32), post=np.empty((m, 4), np.float32),
               comb=np.empty((m, 4, 4), np.float32), collapsed=np.empty((m, d), np.uint16))
    g = None
    if gamma_bf16 is not None:
        g = _c(gamma_bf16, np.uint16)
        out.update(normed=np.empty((m, d), np.uint16), xq=np.empty((m, d), np.uint8),
                   xsf=np.empty((m, d // 128), np.float32))
    lib().oracle_mhc_pre(_p(x), _p(w), _p(b), _p(sc), _p(g), hc_eps, rms_eps, norm_eps, _p(out["pre"]), _p(out["post"]),
                         _p(out["comb"]), _p(out["collapsed"]), _p(out.get("normed")), _p(out.get("xq")),
                         _p(out.get("xsf")), m, d)
    return out


def sparse_mla(q_bf16, swa, cmp, sink, scale):
    """q uint16 [batch, heads, 512]; swa / cmp = None or (pool uint8 [pages, stride], entries_per_block,
    indices int32 [batch, capacity], lengths int32 [batch]).  Returns fp32 [batch, heads, 512]."""
    q = _c(q_bf16, np.uint16)
    batch, heads = q.shape[0], q.shape[1]

    def unpack(t):
        if t is None:
            return None, 0, 1, None, None, 0
        pool, epb, idx, lens = t
        assert pool.dtype == np.uint8 and pool.ndim == 2 and pool.flags.c_contiguous
        idx = _c(idx, np.int32).reshape(batch, -1)
        return pool, pool.shape[1], int(epb), idx, _c(lens, np.int32), idx.shape[1]

    sp, ss, se, si, sl, sc = unpack(swa)
    cp, cs, ce, ci, cl, cc = unpack(cmp)
    sink = _c(sink, np.float32) if sink is not None else None
    out = np.zeros((batch, heads, 512), np.float32)
    lib().oracle_sparse_mla(_p(q), _p(sp), ss, se, _p(si), _p(sl), sc, _p(cp), cs, ce, _p(ci), _p(cl), cc, _p(sink),
                            float(scale), _p(out), batch, heads)
    return out


E2M1_VALUES = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0])


def dequant_mxfp4(packed_u8, scale_words):
    """packed uint8 [..., 64] (two e2m1 per byte, low nibble first) with uint32 [...] scale words (four ue8m0
    bytes, byte g scales values [32g, 32g+32)) -> float64 [..., 128], as cast_back_from_fp4 of
    dsv4_megakernel/megakernel/test/test_mqa_logits_fp4.py:103-115."""
    p = np.asarray(packed_u8, np.uint8)
    v = np.empty(p.shape[:-1] + (128,), np.float64)
    v[..., 0::2] = E2M1_VALUES[p & 15]
    v[..., 1::2] = E2M1_VALUES[p >> 4]
    w = np.asarray(scale_words).astype(np.uint32)
    e = np.stack([(w >> (8 * g)) & 255 for g in range(4)], axis=-1).astype(np.int64)      # [..., 4]
    return v * np.repeat(np.ldexp(1.0, e - 127), 32, axis=-1)


def mqa_logits_fp4(q, q_sf, kv_pages, weights, context_lens, block_table, epb, columns):
    """logits[b, t] = sum_h w[b, h] relu(q[b, h] . k[t]) over dequantised MXFP4 operands (the twin
    ref_fp8_mqa_logits, test_mqa_logits_fp4.py:207-218), t < context; -inf elsewhere.  Test infrastructure."""
    q = np.asarray(q).view(np.uint8)
    batch = q.shape[0]
    qf = dequant_mxfp4(q, np.asarray(q_sf).view(np.uint32).reshape(batch, 64))
    out = np.full((batch, columns), -np.inf, np.float32)
    for b in range(batch):
        n = int(context_lens[b])
        if n == 0:
            continue
        t = np.arange(n)
        page, off = np.asarray(block_table)[b, t // epb], t % epb
        keys = kv_pages[page[:, None], (off * 64)[:, None] + np.arange(64)[None, :]]
        sw = kv_pages[page[:, None], (epb * 64 + off * 4)[:, None] + np.arange(4)[None, :]].copy().view(np.uint32)[:, 0]
        kf = dequant_mxfp4(keys, sw)                                         # [n, 128]
        score = np.maximum(qf[b] @ kf.T, 0.0)                                # [64, n]
        out[b, :n] = (np.asarray(weights, np.float64)[b][:, None] * score).sum(0)
    return out


def gemm_bf16(a_bf16, w_bf16):
    """a uint16 (bf16) [M,K], w uint16 [N,K] -> float64 [M,N] (products of bf16 values are exact in
    fp32; the sum is taken in double so that any fp32 summation order can be held against it)."""
    a = bf16_to_f32(_c(a_bf16, np.uint16)).astype(np.float64)
    w = bf16_to_f32(_c(w_bf16, np.uint16)).astype(np.float64)
    return a @ w.T


def front_emit(y8_bf16, y16, pos, main_state, ape, main_row, idx_state, idx_ape, idx_row):
    """FRONT-EMIT scatter after dsv4_megakernel/megakernel/include/front_mixed_gemm.cuh:390-425 and
    test/test_wq_b_fp8_gemm.py:539-547.  States are modified in place; returns (win_y2, w64)."""
    y16 = _c(y16, np.float32)
    pos = np.asarray(pos, np.int64)
    win = bf16_to_f32(_c(y8_bf16, np.uint16)[:, 1536:2048]).copy()
    w64 = bf16_to_f32(f32_to_bf16(y16[:, 2560:2624]))
    ms, isr = main_state.reshape(-1, 2048), idx_state.reshape(-1, 512)
    for t in range(len(pos)):
        ph = int(pos[t]) % 4
        if main_row[t] >= 0:
            ms[main_row[t], :1024] = y16[t, :1024]
            ms[main_row[t], 1024:] = y16[t, 1024:2048] + ape[ph]
        if idx_row[t] >= 0:
            isr[idx_row[t], :256] = y16[t, 2048:2304]
            isr[idx_row[t], 256:] = y16[t, 2304:2560] + idx_ape[ph]
    return win, w64


def moe_route(logits, bias, k, score_func, route_scale=1.0):
    """logits fp32 [tokens, experts] -> (weights fp32 [tokens, k], indices int32 [tokens, k]);
    score_func 0 softmax, 1 sigmoid, 2 sqrt(softplus)."""
    lg = _c(logits, np.float32)
    b = None if bias is None else _c(bias, np.float32)
    w = np.empty((lg.shape[0], k), np.float32)
    idx = np.empty((lg.shape[0], k), np.int32)
    lib().oracle_moe_route(_p(lg), _p(b), _p(w), _p(idx), lg.shape[0], lg.shape[1], k, score_func, route_scale)
    return w, idx


E2M1_BOUNDS = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], np.float32)


def quantize_nvfp4_rows(x, gs):
    """fp32 [R, K] -> (packed e2m1 uint8 [R, K/2], ue4m3 scale bytes [R, K/16]) with a GIVEN tensor scale:
    sf = e4m3(min(amax/6/gs, 448)), q = e2m1(x / (sf*gs)), ties to the smaller magnitude (the rule of
    dsv4_megakernel/origin/convert.py:11-14 and megakernel/test/test_mqa_logits_fp4.py:69-115)."""
    x = np.ascontiguousarray(x, np.float32)
    r, k = x.shape
    v = x.reshape(r, k // 16, 16)
    gs = np.float32(gs)
    want = np.minimum(np.abs(v).max(-1) / np.float32(6.0) / gs, np.float32(448.0)).astype(np.float32)
    sf = e4m3_encode(want)
    d = e4m3_decode(sf).astype(np.float32)
    denom = (d * gs).astype(np.float32)[..., None]
    with np.errstate(divide="ignore", invalid="ignore"):
        scaled = np.where(d[..., None] > 0, v / denom, np.float32(0)).astype(np.float32)
    idx = np.searchsorted(E2M1_BOUNDS, np.minimum(np.abs(scaled), np.float32(6.0)), side="left").astype(np.uint8)
    code = idx | (((scaled < 0) & (idx != 0)).astype(np.uint8) << 3)
    code = code.reshape(r, k // 2, 2)
    return ((code[:, :, 0] & 15) | (code[:, :, 1] << 4)).astype(np.uint8), sf.reshape(r, k // 16)


def moe_dispatch(indices, experts):
    """indices int32 [tokens, k] -> (group_expert list, row_token [groups*16], pair_row [tokens, k]): pairs sorted
    by expert, stable in flat order, every expert padded to groups of 16 rows."""
    idx = np.asarray(indices, np.int32)
    flat = idx.reshape(-1)
    group_expert, row_token, pair_row = [], [], np.full(flat.shape, -1, np.int32)
    for e in range(experts):
        members = np.nonzero(flat == e)[0]
        if len(members) == 0:
            continue
        base = len(row_token)
        groups = (len(members) + 15) // 16
        group_expert += [e] * groups
        row_token += [int(p) // idx.shape[1] for p in members] + [-1] * (groups * 16 - len(members))
        pair_row[members] = base + np.arange(len(members))
    return np.array(group_expert, np.int32), np.array(row_token, np.int32), pair_row.reshape(idx.shape)


def moe_swiglu(h_bf16, row_weight, limit):
    """h uint16 (bf16) [R, 2I] = gate | up -> uint16 (bf16) [R, I] of weight * silu(min(gate, L)) * clamp(up, +-L)."""
    h = bf16_to_f32(_c(h_bf16, np.uint16))
    inter = h.shape[1] // 2
    gate, up = h[:, :inter].copy(), h[:, inter:].copy()
    if limit > 0:
        up = np.clip(up, -np.float32(limit), np.float32(limit))
        gate = np.minimum(gate, np.float32(limit))
    silu = (gate / (np.float32(1) + np.exp(-gate, dtype=np.float32))).astype(np.float32)
    return f32_to_bf16((np.asarray(row_weight, np.float32)[:, None] * (silu * up).astype(np.float32)).astype(np.float32))


def moe_block(x_bf16, gate_w_bf16, gate_bias, w1_bf16, w3_bf16, w2_bf16, k, score_func=2, route_scale=1.0,
              swiglu_limit=0.0, shared=True):
    """The structure of the origin's MoE.forward (dsv4_megakernel/origin/model.py:629-644) with Gate.forward
    (:563-584) and Expert.forward (:596-606) on bf16 weights, in numpy: router on fp32 copies (the bias shifts the
    selection, not the weights), every selected expert's bf16 projections w1 / w3 -> fp32 SwiGLU (clamped when
    swiglu_limit > 0) times the routing weight -> bf16 -> w2 -> bf16, summed over a token's experts in fp32 in
    expert order; the shared expert (last entry of w1 / w3 / w2 when `shared`) is added to that sum and the
    result is cast to bf16 once.  All tensors are uint16 bf16 bit patterns; w* are [E(+1), out, in].
    Returns (y uint16 [tokens, dim], routing weights fp32 [tokens, k], indices int32 [tokens, k])."""
    x = bf16_to_f32(_c(x_bf16, np.uint16))
    gw = bf16_to_f32(_c(gate_w_bf16, np.uint16))
    w1, w3, w2 = (bf16_to_f32(_c(w, np.uint16)) for w in (w1_bf16, w3_bf16, w2_bf16))
    experts = gw.shape[0]
    logits = (x.astype(np.float64) @ gw.astype(np.float64).T).astype(np.float32)
    rw, idx = moe_route(logits, gate_bias, k, score_func, route_scale)

    def lin(v, w):      # F.linear on bf16 operands: fp32 (here: double) sum, one rounding to bf16
        return bf16_to_f32(f32_to_bf16((v.astype(np.float64) @ w.astype(np.float64).T).astype(np.float32)))

    def expert(e, rows, weight):
        gate, up = lin(x[rows], w1[e]), lin(x[rows], w3[e])
        if swiglu_limit > 0:
            up = np.clip(up, -np.float32(swiglu_limit), np.float32(swiglu_limit))
            gate = np.minimum(gate, np.float32(swiglu_limit))
        h = (gate / (np.float32(1) + np.exp(-gate, dtype=np.float32))).astype(np.float32) * up
        if weight is not None:
            h = weight[:, None] * h
        return lin(bf16_to_f32(f32_to_bf16(h.astype(np.float32))), w2[e])

    y = np.zeros_like(x)
    for e in range(experts):
        rows, slot = np.nonzero(idx == e)
        if len(rows):
            y[rows] += expert(e, rows, rw[rows, slot])
    if shared:
        y = y + expert(experts, np.arange(x.shape[0]), None)
    return f32_to_bf16(y.astype(np.float32)), rw, idx


def gemm_fp8_blockscaled(a, a_s, b, b_s, out_bf16=True):
    """a e4m3 bytes [M,K], a_s fp32 [M,K/128], b e4m3 bytes [N,K], b_s fp32 [N/128,K/128].
    Returns uint16 (bf16) or fp32 [M,N]."""
    a, b = _c(a, np.uint8), _c(b, np.uint8)
    a_s, b_s = _c(a_s, np.float32), _c(b_s, np.float32)
    m, k = a.shape
    n = b.shape[0]
    c = np.empty((m, n), np.uint16 if out_bf16 else np.float32)
    lib().oracle_gemm_fp8_blockscaled(_p(a), _p(a_s), _p(b), _p(b_s), _p(c), m, n, k, int(out_bf16))
    return c


def gemm_fp8_fp4(a, a_s, b_packed, b_sf, out_bf16=True):
    """a e4m3 bytes [M,K], a_s fp32 [M,K/128], b_packed e2m1 pairs [N,K/2] (lower index in the low nibble), b_sf
    exponent bytes [N,K/32].  Returns uint16 (bf16) or fp32 [M,N]: the origin's fp4_gemm (origin/kernel.py:441-536)."""
    a, b, b_sf = _c(a, np.uint8), _c(b_packed, np.uint8), _c(b_sf, np.uint8)
    a_s = _c(a_s, np.float32)
    m, k = a.shape
    n = b.shape[0]
    c = np.empty((m, n), np.uint16 if out_bf16 else np.float32)
    lib().oracle_gemm_fp8_fp4(_p(a), _p(a_s), _p(b), _p(b_sf), _p(c), m, n, k, int(out_bf16))
    return c


def fp4_act_quant(x_bf16):
    """x uint16 (bf16) [rows, cols] -> (packed e2m1 uint8 [rows, cols/2], exponent bytes uint8 [rows, cols/32],
    dequantised bf16 uint16 [rows, cols]): the origin's fp4_act_quant in both forms (origin/kernel.py:126-200)."""
    x = _c(x_bf16, np.uint16)
    rows, cols = x.shape
    codes, scales = np.empty((rows, cols // 2), np.uint8), np.empty((rows, cols // 32), np.uint8)
    deq = np.empty((rows, cols), np.uint16)
    lib().oracle_fp4_act_quant(_p(x), rows, cols, _p(codes), _p(scales), _p(deq))
    return codes, scales, deq


def head_ssq(y_bf16):
    """y uint16 (bf16) [..., heads, 512] -> fp32 [..., heads] sums of squares in the reference kernel's order."""
    y = _c(y_bf16, np.uint16)
    out = np.empty(y.shape[:-1], np.float32)
    lib().oracle_head_ssq(_p(y), out.size, _p(out))
    return out


def hc_split_sinkhorn(mixes, hc_scale, hc_base, iters=20, eps=1e-6):
    """The origin's hc_split_sinkhorn (origin/kernel.py:355-436) in fp32 numpy, hc_mult = 4: mixes [n, 24] ->
    (pre [n, 4], post [n, 4], comb [n, 4, 4])."""
    f = np.float32
    mixes, sc, base = _c(mixes, f).reshape(-1, 24), _c(hc_scale, f), _c(hc_base, f)
    eps = f(eps)
    sig = lambda v: (f(1) / (f(1) + np.exp(-v, dtype=f))).astype(f)
    pre = sig(mixes[:, :4] * sc[0] + base[:4]) + eps
    post = f(2) * sig(mixes[:, 4:8] * sc[1] + base[4:8])
    c = (mixes[:, 8:] * sc[2] + base[8:]).reshape(-1, 4, 4).astype(f)
    c = np.exp(c - c.max(-1, keepdims=True), dtype=f)
    c = (c / c.sum(-1, keepdims=True, dtype=f) + eps).astype(f)
    c = (c / (c.sum(-2, keepdims=True, dtype=f) + eps)).astype(f)
    for _ in range(iters - 1):
        c = (c / (c.sum(-1, keepdims=True, dtype=f) + eps)).astype(f)
        c = (c / (c.sum(-2, keepdims=True, dtype=f) + eps)).astype(f)
    return pre.astype(f), post.astype(f), c


def bf16_to_f32(u16):
    return (np.asarray(u16, np.uint16).astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16(x):
    """Round-to-nearest-even fp32 -> bf16 bit patterns (finite inputs)."""
    b = np.ascontiguousarray(x, np.float32).view(np.uint32)
    return ((b + 0x7FFF + ((b >> 16) & 1)) >> 16).astype(np.uint16)


def gemm_nvfp4(a, a_sf, a_gs, w, w_sf, w_gs, out_bf16=True):
    """a packed e2m1 [M,K/2], a_sf ue4m3 bytes [M,K/16], a_gs fp32; w [N,K/2], w_sf [N,K/16], w_gs.
    Returns uint16 (bf16) or fp32 [M,N]."""
    a, w = _c(a, np.uint8), _c(w, np.uint8)
    a_sf, w_sf = _c(a_sf, np.uint8), _c(w_sf, np.uint8)
    m, k = a.shape[0], a.shape[1] * 2
    n = w.shape[0]
    c = np.empty((m, n), np.uint16 if out_bf16 else np.float32)
    lib().oracle_gemm_nvfp4(_p(a), _p(a_sf), float(a_gs), _p(w), _p(w_sf), float(w_gs), _p(c), m, n, k, int(out_bf16))
    return c
