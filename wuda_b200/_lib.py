"""ctypes binding of libwuda_b200.so (the C ABI declared in include/wuda_b200.h).

The library must exist: there is no fallback path.  Importing this module on a machine
where the library has not been built raises ImportError with the build command.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libwuda_b200.so")

if not os.path.exists(LIB_PATH):
    raise ImportError(
        "wuda_b200: %s is missing. Build it with `python -m wuda_b200.build` "
        "(needs nvcc); there is no fallback implementation." % LIB_PATH)

lib = ctypes.CDLL(LIB_PATH)

c_int, c_i64, c_vp, c_float = ctypes.c_int, ctypes.c_int64, ctypes.c_void_p, ctypes.c_float



class CompressorBundle(ctypes.Structure):
    """wuda_compressor_bundle"""
    _fields_ = [("state", c_vp), ("state_row", c_vp), ("norm_w", c_vp), ("state_rows_total", c_i64),
                ("ring_entries", c_int), ("entries_per_block", c_int), ("num_blocks", c_int), ("reserved", c_int),
                ("block_stride_bytes", c_i64), ("pool", c_vp), ("dst", c_vp), ("q8", c_vp), ("s8", c_vp),
                ("rope", c_vp)]


class WindowBundle(ctypes.Structure):
    """wuda_window_bundle"""
    _fields_ = [("y", c_vp), ("norm_w", c_vp), ("entries_per_block", c_int), ("num_blocks", c_int),
                ("block_stride_bytes", c_i64), ("pool", c_vp), ("dst", c_vp), ("q8", c_vp), ("s8", c_vp),
                ("rope", c_vp)]


class CacheWriters(ctypes.Structure):
    """wuda_cache_writers"""
    _fields_ = [("pos", c_vp), ("cos_table", c_vp), ("sin_table", c_vp), ("max_pos", c_int), ("eps", c_float),
                ("indexer", CompressorBundle), ("main", CompressorBundle), ("window", WindowBundle)]


# name -> (restype, argtypes); mirrors include/wuda_b200.h one to one.
SIGNATURES = {
    "wuda_version": (c_int, []),
    "wuda_last_error": (ctypes.c_char_p, []),
    "wuda_num_sms": (c_int, []),
    "wuda_mqa_logits_fp8": (c_int, [c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_int, c_int, c_int, c_int,
                                    c_i64, c_int, c_i64, c_vp, c_vp]),
    "wuda_indexer_plan_create": (c_int, [ctypes.POINTER(c_vp), c_int, c_int, c_int, c_int, c_i64, c_int, c_i64, c_int]),
    "wuda_indexer_plan_destroy": (c_int, [c_vp]),
    "wuda_indexer_topk_host": (c_int, [c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_int, c_vp]),
    "wuda_rmsnorm_quant_fp8": (c_int, [c_vp, c_i64, c_vp, c_int, c_float, c_vp, c_vp, c_vp, c_int, c_int, c_int, c_vp]),
    "wuda_rope_quant_fp8": (c_int, [c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_int, c_int, c_int, c_int, c_int,
                                    c_int, c_int, c_vp]),
    "wuda_cache_writers_fp8": (c_int, [ctypes.POINTER(CacheWriters), c_int, c_vp, c_vp]),
    "wuda_index_q_post_fp8": (c_int, [c_vp, c_i64, c_vp, c_vp, c_vp, c_int, c_vp, c_vp, c_vp, c_int, c_int, c_vp]),
    "wuda_query_rms_rope": (c_int, [c_vp, c_i64, c_vp, c_vp, c_vp, c_int, c_vp, c_int, c_int, c_int, c_float, c_vp]),
    "wuda_mhc_post": (c_int, [c_vp, c_vp, c_vp, c_vp, c_vp, c_int, c_int, c_vp]),
    "wuda_gemm_fp8_scratch_bytes": (c_i64, [c_int, c_int]),
    "wuda_gemm_fp8_blockscaled": (c_int, [c_vp, c_vp, c_vp, c_vp, c_vp, c_int, c_int, c_int, c_vp, c_i64, c_vp, c_vp]),
    "wuda_gemm_fp8_blockscaled_noalloc": (c_int, [c_vp, c_vp, c_vp, c_vp, c_vp, c_int, c_int, c_int, c_vp, c_vp]),
    "wuda_tp2_inbox_bytes": (c_i64, [c_int, c_int]),
    "wuda_tp2_alloc": (c_int, [c_i64, ctypes.POINTER(c_vp), c_vp]),
    "wuda_tp2_open": (c_int, [c_vp, ctypes.POINTER(c_vp)]),
    "wuda_tp2_close": (c_int, [c_vp]),
    "wuda_tp2_free": (c_int, [c_vp]),
    "wuda_gemm_fp8_blockscaled_tp2": (c_int, [c_vp, c_vp, c_vp, c_vp, c_vp, c_int, c_int, c_int, c_vp, c_i64, c_vp,
                                              c_vp, c_int, c_int, c_vp, c_vp]),
    "wuda_gemm_nvfp4_scratch_bytes": (c_i64, [c_int, c_int]),
    "wuda_gemm_nvfp4": (c_int, [c_vp, c_vp, c_float, c_vp, c_vp, c_float, c_vp, c_int, c_int, c_int, c_vp, c_i64,
                                c_vp, c_vp]),
    "wuda_topk": (c_int, [c_vp, c_vp, c_vp, c_vp, c_vp, c_int, c_i64, c_i64, c_int, c_int, c_int, c_vp]),
}

for _name, (_res, _args) in SIGNATURES.items():
    _fn = getattr(lib, _name)  # AttributeError here = header and library disagree
    _fn.restype = _res
    _fn.argtypes = _args

WUDA_OK = 0
STATUS_NAMES = {0: "WUDA_OK", 1: "WUDA_ERR_INVALID_ARGUMENT", 2: "WUDA_ERR_UNSUPPORTED",
                3: "WUDA_ERR_CUDA", 4: "WUDA_ERR_NO_DEVICE", 5: "WUDA_ERR_DEVICE_STATUS"}


class WudaError(RuntimeError):
    """A C-ABI call returned a non-zero status (the reference raises RuntimeError from
    TORCH_CHECK in the same situations)."""

    def __init__(self, status, message):
        super().__init__("%s: %s" % (STATUS_NAMES.get(status, status), message))
        self.status = status


def check(status):
    if status != WUDA_OK:
        raise WudaError(status, lib.wuda_last_error().decode())
