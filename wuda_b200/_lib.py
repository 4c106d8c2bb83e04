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


class CsaWeights(ctypes.Structure):
    """wuda_csa_weights"""
    _fields_ = [("wq_b", c_vp), ("wq_b_scales", c_vp), ("q_norm", c_vp), ("idx_norm", c_vp), ("main_norm", c_vp),
                ("win_norm", c_vp), ("cos_table", c_vp), ("sin_table", c_vp), ("max_pos", c_int), ("q_lora", c_int),
                ("index_heads", c_int), ("main_heads", c_int), ("out_heads", c_int), ("eps", c_float), ("scales_pow2", c_int)]


class CsaCaches(ctypes.Structure):
    """wuda_csa_caches"""
    _fields_ = [("idx_state", c_vp), ("main_state", c_vp), ("state_rows_total", c_i64), ("ring_entries", c_int),
                ("idx_entries_per_block", c_int), ("cmp_entries_per_block", c_int), ("swa_entries_per_block", c_int),
                ("idx_num_blocks", c_int), ("cmp_num_blocks", c_int), ("swa_num_blocks", c_int), ("idx_fp4", c_int),
                ("idx_block_stride_bytes", c_i64), ("cmp_block_stride_bytes", c_i64), ("swa_block_stride_bytes", c_i64),
                ("idx_pool", c_vp), ("cmp_pool", c_vp), ("swa_pool", c_vp)]


class CsaStep(ctypes.Structure):
    """wuda_csa_step"""
    _fields_ = [("q_raw", c_vp), ("q_raw_stride", c_i64), ("w64", c_vp), ("win_y2", c_vp), ("pos", c_vp),
                ("q_pos", c_vp), ("main_state_row", c_vp), ("idx_state_row", c_vp), ("idx_dst", c_vp), ("cmp_dst", c_vp),
                ("swa_dst", c_vp), ("idx_block_table", c_vp), ("cmp_block_table", c_vp), ("n_compressed", c_vp), ("block_table_stride", c_int),
                ("topk", c_int), ("logits_stride", c_i64), ("logits", c_vp), ("topk_indices", c_vp), ("topk_raw", c_vp),
                ("q_main_out", c_vp)]


class CsaWorkspace(ctypes.Structure):
    """wuda_csa_workspace"""
    _fields_ = [("q_fp8", c_vp), ("q_scales", c_vp), ("y", c_vp), ("iq_fp8", c_vp), ("w_folded", c_vp),
                ("gemm_scratch", c_vp), ("gemm_scratch_bytes", c_i64), ("status_word", c_vp)]


class SparseMlaArgs(ctypes.Structure):
    """wuda_sparse_mla_args"""
    _fields_ = [("q", c_vp), ("swa_pool", c_vp), ("swa_stride", c_i64), ("swa_indices", c_vp), ("swa_lengths", c_vp),
                ("cmp_pool", c_vp), ("cmp_stride", c_i64), ("cmp_indices", c_vp), ("cmp_lengths", c_vp),
                ("attn_sink", c_vp), ("out", c_vp), ("workspace", c_vp), ("workspace_bytes", c_i64),
                ("swa_pages", ctypes.c_int32), ("swa_entries_per_block", ctypes.c_int32), ("swa_capacity", ctypes.c_int32),
                ("cmp_pages", ctypes.c_int32), ("cmp_entries_per_block", ctypes.c_int32), ("cmp_capacity", ctypes.c_int32),
                ("batch", ctypes.c_int32), ("heads", ctypes.c_int32), ("softmax_scale", c_float)]


class LayerWeights(ctypes.Structure):
    """wuda_layer_weights"""
    _fields_ = ([("csa", CsaWeights)] +
                [(n, c_vp) for n in ("attn_hc_weight", "attn_hc_base", "attn_hc_scale", "attn_norm", "front_w8",
                                     "front_w8_scales", "front_w16", "ape", "idx_ape", "wo_a", "wo_a_scales", "wo_b",
                                     "wo_b_scales", "attn_sink", "ffn_hc_weight", "ffn_hc_base", "ffn_hc_scale", "ffn_norm",
                                     "gate_weight", "gate_bias", "w13", "w13_sf", "w13_gs", "w2", "w2_sf", "w2_gs",
                                     "shared_w13", "shared_w13_scales", "shared_w2", "shared_w2_scales")] +
                [(n, c_int) for n in ("hidden", "o_groups", "experts_total", "expert_first", "experts_local", "moe_topk",
                                      "score_func", "inter", "shared_inter")] +
                [(n, c_float) for n in ("route_scale", "swiglu_limit", "act_scale_in", "act_scale_mid", "softmax_scale",
                                        "hc_eps", "rms_eps", "norm_eps")] +
                [("fp8_scales_pow2", c_int)])


class LayerState(ctypes.Structure):
    """wuda_layer_state"""
    _fields_ = [("caches", CsaCaches), ("workspace", c_vp), ("workspace_bytes", c_i64), ("tp_my_inbox", c_vp),
                ("tp_peer_inbox", c_vp), ("ep_my_inbox", c_vp), ("ep_peer_inbox", c_vp), ("ep_tokens_max", c_int),
                ("peer_wait_ms", c_int), ("m_max", c_int), ("reserved", c_int), ("status_word", c_vp)]


class LayerStep(ctypes.Structure):
    """wuda_layer_step"""
    _fields_ = ([(n, c_vp) for n in ("hidden_in", "hidden_out", "pos", "q_pos", "main_state_row", "idx_state_row", "idx_dst",
                                     "cmp_dst", "swa_dst", "idx_block_table", "cmp_block_table", "n_compressed",
                                     "swa_indices", "swa_lengths", "cmp_lengths")] +
                [("block_table_stride", c_int), ("topk", c_int), ("window", c_int), ("reserved", c_int),
                 ("logits_stride", c_i64)])


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
    "wuda_indexer_topk_host_pages": (c_int, [c_vp, c_vp, c_vp, c_vp, c_int, c_vp, c_vp, c_vp, c_vp, c_vp, c_int, c_vp]),
    "wuda_rmsnorm_quant_fp8": (c_int, [c_vp, c_i64, c_vp, c_int, c_float, c_vp, c_vp, c_vp, c_int, c_int, c_int, c_vp]),
    "wuda_rope_quant_fp8": (c_int, [c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_int, c_int, c_int, c_int, c_int,
                                    c_int, c_int, c_vp]),
    "wuda_cache_writers_fp8": (c_int, [ctypes.POINTER(CacheWriters), c_int, c_vp, c_vp]),
    "wuda_cache_writers_fp4": (c_int, [ctypes.POINTER(CacheWriters), c_int, c_vp, c_vp]),
    "wuda_index_q_post_fp4": (c_int, [c_vp, c_i64, c_vp, c_vp, c_vp, c_int, c_vp, c_vp, c_int, c_int, c_vp]),
    "wuda_index_q_post_fp8": (c_int, [c_vp, c_i64, c_vp, c_vp, c_vp, c_int, c_vp, c_vp, c_vp, c_int, c_int, c_vp]),
    "wuda_query_rms_rope": (c_int, [c_vp, c_i64, c_vp, c_vp, c_vp, c_int, c_vp, c_int, c_int, c_int, c_float, c_vp]),
    "wuda_csa_decode_step": (c_int, [ctypes.POINTER(CsaWeights), ctypes.POINTER(CsaCaches), ctypes.POINTER(CsaStep),
                                     ctypes.POINTER(CsaWorkspace), c_int, c_vp]),
    "wuda_mqa_logits_fp4": (c_int, [c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_int, c_int, c_int, c_int, c_i64, c_int,
                                    c_i64, c_vp, c_vp]),
    "wuda_sparse_mla_workspace_bytes": (c_i64, [c_int, c_int, c_int]),
    "wuda_sparse_mla_decode": (c_int, [ctypes.POINTER(SparseMlaArgs), c_vp, c_vp]),
    "wuda_mhc_pre_workspace_bytes": (c_i64, [c_int, c_int]),
    "wuda_mhc_pre": (c_int, [c_vp, c_vp, c_vp, c_vp, c_vp, c_float, c_float, c_float, c_vp, c_vp, c_vp, c_vp, c_vp,
                             c_vp, c_vp, c_vp, c_i64, c_int, c_int, c_vp]),
    "wuda_mhc_pre_mix": (c_int, [c_vp, c_vp, c_vp, c_i64, c_int, c_int, c_vp]),
    "wuda_mhc_pre_finish": (c_int, [c_vp, c_vp, c_int, c_vp, c_vp, c_vp, c_float, c_float, c_float, c_vp, c_vp, c_vp, c_vp,
                                    c_vp, c_vp, c_vp, c_vp, c_int, c_int, c_vp]),
    "wuda_mhc_tail": (c_int, [c_vp, c_vp, c_vp, c_float, c_vp, c_vp, c_int, c_vp]),
    "wuda_gemm_bf16_scratch_bytes": (c_i64, [c_int, c_int]),
    "wuda_gemm_bf16": (c_int, [c_vp, c_vp, c_vp, c_int, c_int, c_int, c_int, c_vp, c_i64, c_vp, c_vp]),
    "wuda_front_emit": (c_int, [c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_i64, c_int, c_vp,
                                c_vp]),
    "wuda_gemm_fp8_grouped": (c_int, [c_vp, c_vp, c_vp, c_vp, c_vp, c_int, c_int, c_int, c_int, c_vp, c_i64, c_vp, c_vp]),
    "wuda_gemm_fp8_grouped_pow2": (c_int, [c_vp, c_vp, c_vp, c_vp, c_vp, c_int, c_int, c_int, c_int, c_vp, c_i64, c_vp, c_vp]),
    "wuda_gemm_fp8_blockscaled_pow2": (c_int, [c_vp, c_vp, c_vp, c_vp, c_vp, c_int, c_int, c_int, c_vp, c_i64, c_vp, c_vp]),
    "wuda_gemm_fp8_fp4_pow2": (c_int, [c_vp, c_vp, c_vp, c_vp, c_vp, c_int, c_int, c_int, c_vp, c_i64, c_vp, c_vp]),
    "wuda_fp4_act_quant": (c_int, [c_vp, c_i64, c_vp, c_vp, c_int, c_i64, c_int, c_vp]),
    "wuda_head_ssq": (c_int, [c_vp, c_i64, c_vp, c_i64, c_int, c_vp]),
    "wuda_hc_split_sinkhorn": (c_int, [c_vp, c_vp, c_vp, c_float, c_vp, c_vp, c_vp, c_i64, c_vp]),
    "wuda_moe_route": (c_int, [c_vp, c_vp, c_vp, c_vp, c_int, c_int, c_int, c_int, c_float, c_vp]),
    "wuda_moe_max_groups": (c_int, [c_int, c_int, c_int]),
    "wuda_moe_dispatch": (c_int, [c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_int, c_int, c_int, c_int, c_vp, c_vp]),
    "wuda_moe_dispatch_range": (c_int, [c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_int, c_int, c_int, c_int, c_int, c_int,
                                        c_vp, c_vp]),
    "wuda_moe_ep2_inbox_bytes": (c_i64, [c_int, c_int]),
    "wuda_moe_combine_ep2": (c_int, [c_vp, c_vp, c_vp, c_vp, c_int, c_int, c_int, c_vp, c_vp, c_int, c_int, c_int, c_vp,
                                     c_vp]),
    "wuda_moe_gather_quant_nvfp4": (c_int, [c_vp, c_vp, c_vp, c_vp, c_float, c_int, c_int, c_int, c_vp]),
    "wuda_gemm_nvfp4_grouped": (c_int, [c_vp, c_vp, c_float, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_int, c_int, c_int,
                                        c_int, c_vp, c_i64, c_vp, c_vp]),
    "wuda_moe_swiglu_quant_nvfp4": (c_int, [c_vp, c_vp, c_vp, c_vp, c_vp, c_float, c_float, c_int, c_int, c_int, c_vp]),
    "wuda_moe_combine": (c_int, [c_vp, c_vp, c_vp, c_vp, c_int, c_int, c_int, c_vp]),
    "wuda_swiglu_quant_fp8": (c_int, [c_vp, c_vp, c_vp, c_vp, c_int, c_int, c_float, c_int, c_vp]),
    "wuda_mhc_post": (c_int, [c_vp, c_vp, c_vp, c_vp, c_vp, c_int, c_int, c_vp]),
    "wuda_gemm_fp8_scratch_bytes": (c_i64, [c_int, c_int]),
    "wuda_gemm_fp8_blockscaled": (c_int, [c_vp, c_vp, c_vp, c_vp, c_vp, c_int, c_int, c_int, c_vp, c_i64, c_vp, c_vp]),
    "wuda_gemm_sm_limit": (c_int, [c_int]),
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
    "wuda_layer_workspace_bytes": (c_i64, [ctypes.POINTER(LayerWeights), c_int, c_int, c_i64, c_int]),
    "wuda_layer_workspace_offset": (c_i64, [ctypes.POINTER(LayerWeights), c_int, c_int, c_i64, c_int, ctypes.c_char_p]),
    "wuda_layer_decode": (c_int, [ctypes.POINTER(LayerWeights), ctypes.POINTER(LayerState), ctypes.POINTER(LayerStep),
                                  c_int, c_vp]),
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
