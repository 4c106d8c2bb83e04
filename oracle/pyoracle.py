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


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p) if a is not None else None


def _c(a, dtype):
    a = np.ascontiguousarray(a, dtype=dtype)
    return a


def num_threads():
    return int(lib().oracle_num_threads())


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
