"""Host-side mirror of the reference's operator interface.

Each function keeps the name, argument order and argument meaning of the PyTorch
extension function it replaces (dsv4_megakernel/megakernel/kernels/*.cu, one
PYBIND11_MODULE per file) and forwards to the C ABI.  Arguments are validated the way
the reference's TORCH_CHECK blocks do and failures raise RuntimeError before anything is
launched.  Work is enqueued on torch's current CUDA stream.
"""
import ctypes

import torch

from . import _lib
from ._lib import WudaError, check, lib

__all__ = ["mqa_logits_fp4_decode_out", "mqa_logits_fp4_decode", "mqa_logits_fp8_decode_out", "fp8_paged_mqa_logits", "topk_v2", "topk_v2_transform",
           "IndexerHostPlan", "sparse_mla_decode", "flash_mla_with_kvcache", "device_status_word", "num_sms", "rmsnorm_quant", "act_quant", "rope_quant",
           "rmsnorm_rope_out", "mhc_post_out", "mhc_pre", "moe_gate", "bf16_gemm", "front_mixed_gemm", "idx_postprocess_fp8", "idx_postprocess", "cache_writers_fp8", "cache_writers_fp4", "mqa_compressor_fp8_standalone", "fp8_gemm", "TP2Link", "exchange_handles", "nvfp4_gemm",
           "fp4_gemm", "fp4_act_quant", "hc_split_sinkhorn", "head_ssq_standalone", "idx_postprocess_standalone",
           "idx_postprocess_fp8_standalone", "mqa_compressor_standalone", "mqa_compressor_paged", "topk_v2_plan"]

NUM_INDEX_HEADS = 64
INDEX_HEAD_DIM = 128


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _require(cond, msg):
    if not cond:
        raise WudaError(1, msg)


def num_sms():
    n = lib.wuda_num_sms()
    if n < 0:
        check(-n)
    return n


def device_status_word(device=None):
    """A zeroed int32 scalar on the device for the kernels' status reports."""
    return torch.zeros(1, dtype=torch.int32, device=device or "cuda")


def mqa_logits_fp8_decode_out(q, kv_cache, weights, context_lens, block_table, schedule_meta, logits,
                              kv_entries_per_block=64, kv_block_stride_bytes=0, num_kv_stages=0,
                              comp_eps=1e-6, *, next_n=1, status_word=None, pdl=False):
    """Paged FP8 MQA logits written into `logits` (caller-owned, never allocates).

    Mirrors mqa_logits_fp8_decode_out (kernels/mqa_logits_fp8.cu:388-526):
      q [R,64,128] float8_e4m3fn, kv_cache uint8 [num_blocks, stride] (epb x 128 key
      bytes then epb fp32 scales per page), weights fp32 [R,64], context_lens int32
      [B] / [B,1] / [B,next_n], block_table int32 [B,max_pages], logits fp32 [>=R, L].
    `schedule_meta` and `num_kv_stages` are accepted for signature compatibility and
    ignored: tiles are scheduled inside the kernel and the stage count follows shared
    memory.  `next_n` (keyword, default 1 as in the reference) is the number of query
    rows per request; rows b*next_n .. b*next_n+next_n-1 share block_table[b].
    Positions t >= context are not written.
    """
    _require(q.is_cuda and q.is_contiguous() and q.dtype == torch.float8_e4m3fn and q.dim() == 3
             and q.size(1) == NUM_INDEX_HEADS and q.size(2) == INDEX_HEAD_DIM,
             "q must be contiguous CUDA FP8 [R,64,128]")
    rows = q.size(0)
    _require(next_n >= 1 and rows % next_n == 0, "rows must be a multiple of next_n")
    batch = rows // next_n
    _require(weights.is_cuda and weights.is_contiguous() and weights.dtype == torch.float32
             and tuple(weights.shape) == (rows, NUM_INDEX_HEADS),
             "weights must be contiguous CUDA FP32 [R,64]")
    _require(context_lens.is_cuda and context_lens.is_contiguous() and context_lens.dtype == torch.int32
             and context_lens.numel() == rows,
             "context_lens must be contiguous CUDA int32 with one entry per row")
    _require(block_table.is_cuda and block_table.is_contiguous() and block_table.dtype == torch.int32
             and block_table.dim() == 2 and block_table.size(0) == batch,
             "block_table must be contiguous CUDA int32 [B,max_pages]")
    _require(logits.is_cuda and logits.dtype == torch.float32 and logits.dim() == 2
             and logits.size(0) >= rows and logits.stride(1) == 1,
             "logits must be CUDA FP32 [>=R, L] with unit inner stride")
    _require(kv_cache.is_cuda and kv_cache.is_contiguous() and kv_cache.dtype == torch.uint8
             and kv_cache.dim() == 2, "kv_cache must be contiguous CUDA uint8 physical pages")
    if kv_block_stride_bytes == 0:
        kv_block_stride_bytes = kv_cache.size(1)
    _require(kv_cache.size(1) == kv_block_stride_bytes, "invalid FP8 KV page stride")
    check(lib.wuda_mqa_logits_fp8(
        q.data_ptr(), kv_cache.data_ptr(), weights.data_ptr(), context_lens.data_ptr(),
        block_table.data_ptr(), logits.data_ptr(), batch, next_n, kv_cache.size(0),
        int(kv_entries_per_block), int(kv_block_stride_bytes), block_table.size(1),
        logits.stride(0), status_word.data_ptr() if status_word is not None else None, _stream()))
    return logits


def fp8_paged_mqa_logits(q, kv_cache, weights, context_lens, block_table, schedule_meta, max_context_len,
                         kv_entries_per_block=64, status_word=None):
    """Allocating form with deep_gemm.fp8_paged_mqa_logits' shape conventions as the
    reference calls it (test/test_mqa_logits_fp4.py:518-522): q [B, next_n, 64, 128],
    returns fp32 [B*next_n, max_context_len], -inf beyond each row's context."""
    _require(q.dim() == 4, "q must be [B, next_n, 64, 128]")
    b, next_n = q.size(0), q.size(1)
    stride = (max_context_len + 255) // 256 * 256
    logits = torch.full((b * next_n, stride), float("-inf"), dtype=torch.float32, device=q.device)
    mqa_logits_fp8_decode_out(q.reshape(b * next_n, q.size(2), q.size(3)), kv_cache, weights,
                              context_lens, block_table, schedule_meta, logits, kv_entries_per_block,
                              next_n=next_n, status_word=status_word)
    return logits[:, :max_context_len]


def mqa_logits_fp4_decode_out(q, sf_q, kv_cache, weights, context_lens, block_table, logits, max_context_len=None,
                              kv_entries_per_block=64, kv_block_stride_bytes=0, *, status_word=None):
    """The FP4 indexer scores with the reference's argument order (kernels/mqa_logits_fp4.cu:474-650): q int8
    [B, 64, 64] packed e2m1, sf_q int32 [B, 64] (four ue8m0 bytes), kv_cache uint8 [num_blocks, stride] of fused
    pages (keys, then scale words), weights fp32 [B, 64], context_lens int32 [B], block_table int32 [B, pages],
    logits fp32 [B, >= max_context_len]; only t < context is written."""
    _require(q.is_cuda and q.is_contiguous() and q.element_size() == 1 and q.dim() == 3 and q.shape[1:] == (64, 64),
             "q must be contiguous CUDA int8 [B, 64, 64]")
    b = q.size(0)
    _require(sf_q.is_cuda and sf_q.is_contiguous() and sf_q.dtype == torch.int32 and sf_q.numel() == b * 64,
             "sf_q must be contiguous CUDA int32 [B, 64]")
    _require(kv_cache.is_cuda and kv_cache.is_contiguous() and kv_cache.dtype == torch.uint8 and kv_cache.dim() == 2,
             "kv_cache must be contiguous CUDA uint8 [num_blocks, stride]")
    _require(kv_block_stride_bytes in (0, kv_cache.size(1)), "kv_block_stride_bytes must match kv_cache")
    _f32(weights, "weights")
    _require(weights.numel() == b * 64, "weights must be [B, 64]")
    _require(context_lens.is_cuda and context_lens.dtype == torch.int32 and context_lens.numel() == b and
             context_lens.is_contiguous(), "context_lens must be contiguous CUDA int32 [B]")
    _require(block_table.is_cuda and block_table.dtype == torch.int32 and block_table.dim() == 2 and
             block_table.size(0) == b and block_table.stride(1) == 1, "block_table must be CUDA int32 [B, pages]")
    _require(logits.is_cuda and logits.dtype == torch.float32 and logits.dim() == 2 and logits.size(0) >= b and
             logits.stride(1) == 1, "logits must be CUDA fp32 [>= B, columns]")
    max_ctx = int(max_context_len) if max_context_len is not None else min(logits.size(1),
                                                                            block_table.size(1) * kv_entries_per_block)
    _require(max_ctx <= logits.size(1), "logits has fewer columns than max_context_len")
    check(lib.wuda_mqa_logits_fp4(q.data_ptr(), sf_q.data_ptr(), kv_cache.data_ptr(), weights.data_ptr(),
                                  context_lens.data_ptr(), block_table.data_ptr(), logits.data_ptr(), b, max_ctx,
                                  kv_cache.size(0), int(kv_entries_per_block), kv_cache.size(1),
                                  block_table.stride(0) if b > 1 else block_table.size(1),    # (one row: any stride)
                                  logits.stride(0) if logits.size(0) > 1 else logits.size(1), _ptr(status_word), _stream()))
    return logits


def mqa_logits_fp4_decode(q, sf_q, kv_cache, weights, context_lens, block_table, max_context_len,
                          out_dtype=torch.float32, kv_entries_per_block=64, kv_block_stride_bytes=0):
    """The allocating form (kernels/mqa_logits_fp4.cu:652-700): returns fp32 [B, max_context_len] with -inf
    at and beyond each request's context."""
    _require(out_dtype == torch.float32, "only fp32 logits are implemented")
    logits = torch.full((q.size(0), int(max_context_len)), float("-inf"), dtype=torch.float32, device=q.device)
    return mqa_logits_fp4_decode_out(q, sf_q, kv_cache, weights, context_lens, block_table, logits, max_context_len,
                                     kv_entries_per_block, kv_block_stride_bytes)


def topk_v2_transform(scores, seq_lens, page_table, page_indices, page_size=64, metadata=None,
                      raw_indices=None, *, rows_per_table_row=1):
    """Top-k indices of each row of `scores` written into `page_indices` [rows, k]
    after the page-table transform (kernels/topk_v2.cu:348-423).  `metadata` (the
    reference's plan tensor) is accepted and ignored.  Never allocates.
    `rows_per_table_row` (keyword, default 1 as in the reference) lets the next_n score
    rows of one request share that request's page-table row."""
    _require(scores.is_cuda and scores.dtype == torch.float32 and scores.dim() == 2 and scores.stride(1) == 1,
             "scores must be CUDA FP32 [rows, L] with unit inner stride")
    rows = scores.size(0)
    _require(seq_lens.is_cuda and seq_lens.is_contiguous() and seq_lens.dtype == torch.int32
             and seq_lens.numel() == rows, "seq_lens must be contiguous CUDA int32 [rows]")
    _require(page_table.is_cuda and page_table.is_contiguous() and page_table.dtype == torch.int32
             and page_table.dim() == 2 and page_table.size(0) * rows_per_table_row == rows,
             "page_table must be contiguous CUDA int32 [rows / rows_per_table_row, pages]")
    _require(page_indices.is_cuda and page_indices.is_contiguous() and page_indices.dtype == torch.int32
             and page_indices.dim() == 2 and page_indices.size(0) == rows,
             "page_indices must be contiguous CUDA int32 [rows, k]")
    k = page_indices.size(1)
    if raw_indices is not None:
        _require(raw_indices.is_cuda and raw_indices.is_contiguous() and raw_indices.dtype == torch.int32
                 and tuple(raw_indices.shape) == (rows, k), "raw_indices must be contiguous CUDA int32 [rows, k]")
    check(lib.wuda_topk(scores.data_ptr(), seq_lens.data_ptr(), page_table.data_ptr(), page_indices.data_ptr(),
                        raw_indices.data_ptr() if raw_indices is not None else None, rows, scores.stride(0),
                        page_table.stride(0), int(rows_per_table_row), k, int(page_size), _stream()))
    return page_indices


def topk_v2_plan(seq_lens, metadata, static_cluster_threshold=0):
    """The reference's plan call (kernels/topk_v2.cu:329-345) checks its arguments and fills `metadata` int32
    [B + 1, 2] with the rows it gives to clusters.  The kernel of this library decides that per row at launch and
    needs no plan: the arguments are checked the same way and `metadata` is left as it is."""
    _require(seq_lens.is_cuda and seq_lens.is_contiguous() and seq_lens.dtype == torch.int32,
             "seq_lens must be CUDA i32 [B]")
    _require(metadata.is_cuda and metadata.is_contiguous() and metadata.dtype == torch.int32
             and metadata.numel() == 2 * (seq_lens.numel() + 1), "metadata must be CUDA i32 [B+1, 2]")


def topk_v2(scores, seq_lens, page_table, topk, page_size=64, raw_indices=None, *, rows_per_table_row=1):
    """Allocating form (kernels/topk_v2.cu:428-439): returns page_indices int32 [rows, topk]."""
    out = torch.empty((scores.size(0), int(topk)), dtype=torch.int32, device=scores.device)
    return topk_v2_transform(scores, seq_lens, page_table, out, page_size, None, raw_indices,
                             rows_per_table_row=rows_per_table_row)


class IndexerHostPlan:
    """Host-buffer indexer step (wuda_indexer_plan_* / wuda_indexer_topk_host): inputs are
    numpy arrays or CPU torch tensors (page-locked for full copy bandwidth), the result is
    written into a caller-owned host int32 array [rows, k]."""

    def __init__(self, max_batch, next_n, num_blocks, entries_per_block, page_stride_bytes,
                 block_table_stride, logits_stride, k):
        import ctypes
        self._h = ctypes.c_void_p()
        check(lib.wuda_indexer_plan_create(ctypes.byref(self._h), max_batch, next_n, num_blocks,
                                           entries_per_block, page_stride_bytes, block_table_stride,
                                           logits_stride, k))
        self.next_n, self.k = next_n, k

    @staticmethod
    def _ptr(a):
        if a is None:
            return None
        return a.data_ptr() if isinstance(a, torch.Tensor) else a.ctypes.data

    def run(self, q, kv_pages, weights, context_lens, block_table, page_indices_out, batch, logits_out=None,
            stream=None, dirty_pages=None):
        """dirty_pages (host int32 array of page numbers, or None): with a list only those pages of kv_pages are
        uploaded, the rest of the pool is what earlier calls left on the device; None uploads the whole pool."""
        s = _stream() if stream is None else stream
        if dirty_pages is None:
            check(lib.wuda_indexer_topk_host(self._h, self._ptr(q), self._ptr(kv_pages), self._ptr(weights),
                                             self._ptr(context_lens), self._ptr(block_table),
                                             self._ptr(page_indices_out), self._ptr(logits_out), batch, s))
        else:
            n = int(dirty_pages.numel() if isinstance(dirty_pages, torch.Tensor) else dirty_pages.size)
            check(lib.wuda_indexer_topk_host_pages(self._h, self._ptr(q), self._ptr(kv_pages), self._ptr(dirty_pages), n,
                                                   self._ptr(weights), self._ptr(context_lens), self._ptr(block_table),
                                                   self._ptr(page_indices_out), self._ptr(logits_out), batch, s))
        return page_indices_out

    def close(self):
        if self._h:
            lib.wuda_indexer_plan_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def rmsnorm_quant(x, gamma, eps=1e-6, *, quant=True, scale_fmt=None, return_bf16=True):
    """RMSNorm(gamma, eps) of a bf16 [rows, dim] tensor and, in the same pass, its 1x128
    FP8 quantisation.  Returns (y_bf16 or None, y_fp8 or None, scales or None).
    scale_fmt: None = fp32 amax/448 scales, anything else = power-of-two scales, as the
    origin's act_quant (origin/kernel.py:105-125).  gamma None = no normalisation."""
    _require(x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 2 and x.stride(1) == 1,
             "x must be CUDA bf16 [rows, dim] with unit inner stride")
    rows, dim = x.shape
    if gamma is not None:
        _require(gamma.is_cuda and gamma.is_contiguous() and gamma.numel() == dim
                 and gamma.dtype in (torch.float32, torch.bfloat16), "gamma must be CUDA fp32 or bf16 [dim]")
    y16 = torch.empty((rows, dim), dtype=torch.bfloat16, device=x.device) if return_bf16 else None
    y8 = torch.empty((rows, dim), dtype=torch.float8_e4m3fn, device=x.device) if quant else None
    sc = torch.empty((rows, dim // 128), dtype=torch.float32, device=x.device) if quant else None
    check(lib.wuda_rmsnorm_quant_fp8(x.data_ptr(), x.stride(0), gamma.data_ptr() if gamma is not None else None,
                                     int(gamma is not None and gamma.dtype == torch.bfloat16), float(eps),
                                     y16.data_ptr() if y16 is not None else None,
                                     y8.data_ptr() if y8 is not None else None,
                                     sc.data_ptr() if sc is not None else None, rows, dim,
                                     0 if scale_fmt is None else 1, _stream()))
    return y16, y8, sc


def act_quant(x, block_size=128, scale_fmt=None):
    """Block-wise FP8 quantisation with the origin's signature (origin/kernel.py:105):
    returns (y float8_e4m3fn, scales fp32 [..., N/128])."""
    _require(block_size == 128, "block_size must be 128")
    shape = x.shape
    _, y8, sc = rmsnorm_quant(x.reshape(-1, shape[-1]), None, quant=True, scale_fmt=scale_fmt, return_bf16=False)
    return y8.view(shape), sc.view(*shape[:-1], shape[-1] // 128)


def rope_quant(x, positions, cos_table, sin_table, rope_dim, *, inverse=False, quant=True, scale_fmt=None,
               return_bf16=False):
    """Partial RoPE of bf16 [tokens, heads, head_dim] (last rope_dim dims of each head) and,
    in the same pass, 1x128 FP8 quantisation of the flat row.  Returns (y_bf16 or None,
    y_fp8 [tokens, heads*head_dim] or None, scales or None)."""
    _require(x.is_cuda and x.is_contiguous() and x.dtype == torch.bfloat16 and x.dim() == 3,
             "x must be contiguous CUDA bf16 [tokens, heads, head_dim]")
    tokens, heads, head_dim = x.shape
    _require(positions.is_cuda and positions.is_contiguous() and positions.dtype == torch.int64
             and positions.numel() == tokens, "positions must be contiguous CUDA int64 [tokens]")
    _require(cos_table.is_cuda and cos_table.is_contiguous() and cos_table.dtype == torch.float32
             and cos_table.dim() == 2 and cos_table.size(1) == rope_dim // 2 and sin_table.shape == cos_table.shape
             and sin_table.is_cuda and sin_table.is_contiguous() and sin_table.dtype == torch.float32,
             "cos/sin tables must be contiguous CUDA fp32 [max_pos, rope_dim/2]")
    width = heads * head_dim
    y16 = torch.empty_like(x) if return_bf16 else None
    y8 = torch.empty((tokens, width), dtype=torch.float8_e4m3fn, device=x.device) if quant else None
    sc = torch.empty((tokens, width // 128), dtype=torch.float32, device=x.device) if quant else None
    check(lib.wuda_rope_quant_fp8(x.data_ptr(), positions.data_ptr(), cos_table.data_ptr(), sin_table.data_ptr(),
                                  y16.data_ptr() if y16 is not None else None,
                                  y8.data_ptr() if y8 is not None else None,
                                  sc.data_ptr() if sc is not None else None, tokens, heads, head_dim, rope_dim,
                                  cos_table.size(0), int(inverse), 0 if scale_fmt is None else 1, _stream()))
    return y16, y8, sc


def mhc_pre(hidden, weight, base, scale, attn_norm_w=None, hc_eps=1e-6, rms_eps=1e-6, attn_norm_eps=1e-6,
            quant=True, workspace=None):
    """mHC pre of a half-layer (the reference's tf32_hc_prenorm_gemm + hc_reduce_fuse_out pair,
    test/test_hc_fused_tc.py:85-112): hidden bf16 [M, 4, D], weight fp32 [24, 4*D], base fp32 [24],
    scale fp32 [3], attn_norm_w bf16 [D] or None.  Returns a dict with pre, post [M,4], comb [M,4,4],
    collapsed bf16 [M,D] and, with attn_norm_w, normed bf16 [M,D] (+ xq e4m3 [M,D], xsf fp32 [M,D/128]
    when quant)."""
    _require(hidden.is_cuda and hidden.is_contiguous() and hidden.dtype == torch.bfloat16 and hidden.dim() == 3
             and hidden.size(1) == 4, "hidden must be contiguous CUDA bf16 [M, 4, D]")
    m, _, d = hidden.shape
    _require(_f32(weight, "weight").shape == (24, 4 * d), "weight must be fp32 [24, 4*D]")
    _require(_f32(base, "base").numel() == 24 and _f32(scale, "scale").numel() == 3, "base [24] and scale [3] are fp32")
    dev = hidden.device
    out = dict(pre=torch.empty(m, 4, device=dev), post=torch.empty(m, 4, device=dev), comb=torch.empty(m, 4, 4, device=dev),
               collapsed=torch.empty(m, d, dtype=torch.bfloat16, device=dev))
    if attn_norm_w is not None:
        _require(attn_norm_w.is_cuda and attn_norm_w.is_contiguous() and attn_norm_w.dtype == torch.bfloat16
                 and attn_norm_w.numel() == d, "attn_norm_w must be contiguous CUDA bf16 [D]")
        out["normed"] = torch.empty(m, d, dtype=torch.bfloat16, device=dev)
        if quant:
            out["xq"] = torch.empty(m, d, dtype=torch.float8_e4m3fn, device=dev)
            out["xsf"] = torch.empty(m, d // 128, device=dev)
    need = lib.wuda_mhc_pre_workspace_bytes(m, d)
    _require(need > 0, "unsupported M or D")
    if workspace is None:
        workspace = torch.empty(need, dtype=torch.uint8, device=dev)
    check(lib.wuda_mhc_pre(hidden.data_ptr(), weight.data_ptr(), base.data_ptr(), scale.data_ptr(), _ptr(attn_norm_w),
                           hc_eps, rms_eps, attn_norm_eps, out["pre"].data_ptr(), out["post"].data_ptr(),
                           out["comb"].data_ptr(), out["collapsed"].data_ptr(), _ptr(out.get("normed")),
                           _ptr(out.get("xq")), _ptr(out.get("xsf")), workspace.data_ptr(), workspace.numel(), m, d,
                           _stream()))
    return out


def mhc_post_out(attention_out, residual, post, comb, output):
    """output[m,j,:] = post[m,j] * attention_out[m,:] + sum_i comb[m,i,j] * residual[m,i,:], with
    the reference's signature and checks (kernels/mhc_post.cu:139-177): bf16 [M,7168] and
    [M,4,7168], fp32 [M,4] and [M,4,4], caller-owned bf16 output [M,4,7168], 1 <= M <= 128."""
    _require(attention_out.is_cuda and attention_out.is_contiguous() and attention_out.dtype == torch.bfloat16
             and attention_out.dim() == 2, "attention_out must be contiguous CUDA bf16 [M, hidden]")
    m, hidden = attention_out.shape
    _require(1 <= m <= 128, "M must be in [1, 128]")
    for name, t, dtype, shape in (("residual", residual, torch.bfloat16, (m, 4, hidden)),
                                  ("post", post, torch.float32, (m, 4)), ("comb", comb, torch.float32, (m, 4, 4)),
                                  ("output", output, torch.bfloat16, (m, 4, hidden))):
        _require(t.is_cuda and t.is_contiguous() and t.dtype == dtype and tuple(t.shape) == shape,
                 f"{name} must be contiguous CUDA {dtype} {list(shape)}")
    check(lib.wuda_mhc_post(attention_out.data_ptr(), residual.data_ptr(), post.data_ptr(), comb.data_ptr(),
                            output.data_ptr(), m, hidden, _stream()))
    return output


def _ptr(t):
    return t.data_ptr() if t is not None else None


_mla_workspace = {}   # per device: partial sums of split requests (grown on demand)


def _model1_pool(cache, name):
    """(pointer, page stride, pages, entries) of a MODEL1 pool given either as uint8 [pages, stride]
    with an explicit entry count, or as the strided [pages, entries, 1, 584] view the cache manager hands
    to the attention (kv_cache.KVCacheManager.model1_cache_view)."""
    _require(cache.is_cuda and cache.element_size() == 1 and cache.dim() == 4 and cache.size(3) == 584
             and cache.stride(3) == 1 and cache.stride(1) == 584,
             f"{name} must be a CUDA 1-byte [pages, entries, 1, 584] view of a MODEL1 pool")
    return cache.data_ptr(), cache.stride(0), cache.size(0), cache.size(1)


def sparse_mla_decode(q, swa_cache, swa_indices, swa_lengths, cmp_cache=None, cmp_indices=None, cmp_lengths=None,
                      attn_sink=None, softmax_scale=None, *, out=None, status_word=None, split=True):
    """Decode attention of q bf16 [batch, heads, 512] over gathered MODEL1 records: swa_lengths[b] entries of
    swa_indices[b] in swa_cache, then cmp_lengths[b] entries of cmp_indices[b] in cmp_cache (pool entry
    indices, negative = skipped), with the attention sink in the denominator.  Returns bf16
    [batch, heads, 512]."""
    _require(q.is_cuda and q.is_contiguous() and q.dtype == torch.bfloat16 and q.dim() == 3 and q.size(2) == 512,
             "q must be contiguous CUDA bf16 [batch, heads, 512]")
    batch, heads = q.size(0), q.size(1)
    a = _lib.SparseMlaArgs()
    a.q, a.batch, a.heads = q.data_ptr(), batch, heads
    a.softmax_scale = float(softmax_scale if softmax_scale is not None else 512 ** -0.5)
    for name, cache, idx, lens in (("swa", swa_cache, swa_indices, swa_lengths), ("cmp", cmp_cache, cmp_indices, cmp_lengths)):
        if cache is None:
            setattr(a, name + "_capacity", 0)
            continue
        ptr, stride, pages, entries = _model1_pool(cache, name + "_cache")
        _require(idx.is_cuda and idx.is_contiguous() and idx.dtype == torch.int32 and idx.numel() % max(batch, 1) == 0,
                 f"{name}_indices must be contiguous CUDA int32 [batch, capacity]")
        _require(lens.is_cuda and lens.is_contiguous() and lens.dtype == torch.int32 and lens.numel() == batch,
                 f"{name}_lengths must be contiguous CUDA int32 [batch]")
        setattr(a, name + "_pool", ptr)
        setattr(a, name + "_stride", stride)
        setattr(a, name + "_pages", pages)
        setattr(a, name + "_entries_per_block", entries)
        setattr(a, name + "_indices", idx.data_ptr())
        setattr(a, name + "_lengths", lens.data_ptr())
        setattr(a, name + "_capacity", idx.numel() // max(batch, 1))
    if attn_sink is not None:
        _require(attn_sink.is_cuda and attn_sink.is_contiguous() and attn_sink.dtype == torch.float32
                 and attn_sink.numel() == heads, "attn_sink must be contiguous CUDA fp32 [heads]")
        a.attn_sink = attn_sink.data_ptr()
    if out is None:
        out = torch.empty_like(q)
    _require(out.is_cuda and out.is_contiguous() and out.dtype == torch.bfloat16 and out.shape == q.shape,
             "out must be contiguous CUDA bf16 shaped like q")
    a.out = out.data_ptr()
    if split and batch > 0:   # small batches: several CTAs per request, merged by a second launch
        need = lib.wuda_sparse_mla_workspace_bytes(batch, heads, a.swa_capacity + a.cmp_capacity)
        _require(need >= 0, "wuda_sparse_mla_workspace_bytes rejected the shape")
        if need > 0:
            ws = _mla_workspace.get(q.device)
            if ws is None or ws.numel() < need:
                ws = _mla_workspace[q.device] = torch.empty(need, dtype=torch.uint8, device=q.device)
            a.workspace, a.workspace_bytes = ws.data_ptr(), need
    check(lib.wuda_sparse_mla_decode(ctypes.byref(a), _ptr(status_word), _stream()))
    return out


def flash_mla_with_kvcache(q, k_cache, block_table=None, cache_seqlens=None, head_dim_v=512,
                           tile_scheduler_metadata=None, num_splits=None, softmax_scale=None, causal=False,
                           is_fp8_kvcache=True, indices=None, topk_length=None, extra_k_cache=None,
                           extra_indices_in_kvcache=None, extra_topk_length=None, attn_sink=None):
    """The sparse FP8 decode call of the layer step with the keyword list it is made with at
    test/test_e2e_decode.py:719-728: q bf16 [batch, 1, heads, 512]; k_cache / extra_k_cache MODEL1 views;
    indices [batch, 1, topk] with topk_length [batch] for the first pool, extra_* for the second.  Only this
    form (sparse indices, FP8 records, one query token, value = key) is implemented; the scheduler metadata
    is accepted and ignored.  Returns (out bf16 [batch, 1, heads, 512], None)."""
    _require(is_fp8_kvcache and indices is not None and block_table is None and cache_seqlens is None and not causal,
             "only the sparse FP8 form (indices given, no block table, not causal) is implemented")
    _require(head_dim_v == 512 and q.dim() == 4 and q.size(1) == 1, "q must be [batch, 1, heads, 512] with head_dim_v 512")
    batch, heads = q.size(0), q.size(2)
    if topk_length is None:
        topk_length = torch.full((batch,), indices.size(-1), dtype=torch.int32, device=q.device)
    if extra_k_cache is not None and extra_topk_length is None:
        extra_topk_length = torch.full((batch,), extra_indices_in_kvcache.size(-1), dtype=torch.int32, device=q.device)
    out = sparse_mla_decode(q.view(batch, heads, 512), k_cache, indices.reshape(batch, -1), topk_length, extra_k_cache,
                            None if extra_k_cache is None else extra_indices_in_kvcache.reshape(batch, -1),
                            extra_topk_length, attn_sink, softmax_scale)
    return out.view(batch, 1, heads, 512), None


def _f32(t, name, last=None):
    _require(t.is_cuda and t.is_contiguous() and t.dtype == torch.float32 and (last is None or t.size(-1) == last),
             f"{name} must be contiguous CUDA fp32" + (f" [..., {last}]" if last else ""))
    return t


def _pool_fields(bundle, rows, name):
    pool, dst = bundle.get("pool"), bundle.get("dst")
    if pool is None:
        return dict(entries_per_block=1, num_blocks=1, block_stride_bytes=0, pool=None, dst=None)
    _require(pool.is_cuda and pool.dtype == torch.uint8 and pool.dim() == 2 and pool.stride(1) == 1,
             f"{name}: pool must be CUDA uint8 [pages, stride]")
    _require(dst is not None and dst.is_cuda and dst.is_contiguous() and dst.dtype == torch.int64
             and dst.numel() == rows, f"{name}: dst must be contiguous CUDA int64 [rows]")
    return dict(entries_per_block=int(bundle["entries_per_block"]), num_blocks=pool.size(0),
                block_stride_bytes=pool.stride(0), pool=pool.data_ptr(), dst=dst.data_ptr())


def _compact_fields(bundle, rows, name, nq, ns, with_rope, scale_dtype=torch.float32):
    q8, s8, rope = bundle.get("q8"), bundle.get("s8"), bundle.get("rope")
    if q8 is not None:
        _require(q8.is_cuda and q8.is_contiguous() and q8.element_size() == 1 and q8.numel() == rows * nq,
                 f"{name}: q8 must be contiguous CUDA 1-byte [rows, {nq}]")
    if s8 is not None:
        _require(s8.is_cuda and s8.is_contiguous() and s8.dtype == scale_dtype and s8.numel() == rows * ns,
                 f"{name}: s8 must be contiguous CUDA {scale_dtype} with {ns} per row")
    if rope is not None:
        _require(with_rope and rope.is_cuda and rope.is_contiguous() and rope.dtype == torch.bfloat16
                 and rope.numel() == rows * 64, f"{name}: rope must be contiguous CUDA bf16 [rows, 64]")
    return dict(q8=_ptr(q8), s8=_ptr(s8), rope=_ptr(rope))


def _compressor_bundle(bundle, rows, name, half, fp4=False):
    if bundle is None:
        return _lib.CompressorBundle()
    state = _f32(bundle["state"], name + ".state", 4 * half)
    ring = int(bundle.get("ring_entries", state.size(-2) if state.dim() == 3 else 8))
    row = bundle["state_row"]
    _require(row.is_cuda and row.is_contiguous() and row.dtype == torch.int64 and row.numel() == rows,
             f"{name}: state_row must be contiguous CUDA int64 [rows]")
    norm = _f32(bundle["norm_w"], name + ".norm_w", half)
    fields = dict(state=state.data_ptr(), state_row=row.data_ptr(), norm_w=norm.data_ptr(),
                  state_rows_total=state.numel() // (4 * half), ring_entries=ring)
    fields.update(_pool_fields(bundle, rows, name))
    if fp4:
        fields.update(_compact_fields(bundle, rows, name, 64, 4, False, torch.uint8))
    else:
        fields.update(_compact_fields(bundle, rows, name, 128 if half == 128 else 448, 1 if half == 128 else 7, half == 512))
    return _lib.CompressorBundle(**fields)


def cache_writers_fp8(pos, cos_table, sin_table, *, indexer=None, main=None, window=None, eps=1e-6, status_word=None,
                      indexer_fp4=False):
    """The indexer compressor, the MAIN compressor and the window-KV writer of one decode step in one
    launch (wuda_cache_writers_fp8; with indexer_fp4=True wuda_cache_writers_fp4: the indexer entry is an MXFP4
    record - Hadamard transform, 64 code bytes + 4 exponent bytes -, its compact outputs q8 uint8 [rows, 64] and
    s8 uint8 [rows, 4]).  Each writer is a dict or None:
      indexer / main: state fp32 [blocks, ring, 512 | 2048], state_row int64 [rows], norm_w fp32 [128 | 512],
                      optional pool uint8 [pages, stride] + dst int64 [rows] + entries_per_block,
                      optional compact outputs q8, s8 (and rope bf16 [rows,64] for main)
      window:         y fp32 [rows, 512], norm_w fp32 [512], the same optional pool and compact outputs
    Everything is caller-owned; nothing is allocated."""
    _require(pos.is_cuda and pos.is_contiguous() and pos.dtype == torch.int64 and pos.dim() == 1,
             "pos must be contiguous CUDA int64 [rows]")
    rows = pos.numel()
    _f32(cos_table, "cos_table", 32)
    _f32(sin_table, "sin_table", 32)
    _require(cos_table.shape == sin_table.shape and cos_table.dim() == 2, "cos/sin tables must both be [max_pos, 32]")
    args = _lib.CacheWriters(pos=pos.data_ptr(), cos_table=cos_table.data_ptr(), sin_table=sin_table.data_ptr(),
                             max_pos=cos_table.size(0), eps=float(eps))
    args.indexer = _compressor_bundle(indexer, rows, "indexer", 128, fp4=indexer_fp4)
    args.main = _compressor_bundle(main, rows, "main", 512)
    if window is not None:
        y = _f32(window["y"], "window.y", 512)
        _require(y.numel() == rows * 512, "window.y must be [rows, 512]")
        fields = dict(y=y.data_ptr(), norm_w=_f32(window["norm_w"], "window.norm_w", 512).data_ptr())
        fields.update(_pool_fields(window, rows, "window"))
        fields.update(_compact_fields(window, rows, "window", 448, 7, True))
        args.window = _lib.WindowBundle(**fields)
    entry = lib.wuda_cache_writers_fp4 if indexer_fp4 else lib.wuda_cache_writers_fp8
    check(entry(ctypes.byref(args), rows, _ptr(status_word), _stream()))


def cache_writers_fp4(pos, cos_table, sin_table, **kw):
    """cache_writers_fp8 with the indexer compressor in its FP4 form."""
    cache_writers_fp8(pos, cos_table, sin_table, indexer_fp4=True, **kw)


def mqa_compressor_fp8_standalone(cmp_pos, comp_norm, cos_tab, sin_tab, comp_state, comp_state_row,
                                  comp_state_ring_entries, comp_q8, comp_s8, comp_rope, comp_eps=1e-6):
    """The MAIN compressor on its own, with the reference's argument list
    (kernels/mqa_logits_fp8.cu:542-599): compact outputs only."""
    cache_writers_fp8(cmp_pos, cos_tab, sin_tab, eps=comp_eps,
                      main=dict(state=comp_state, state_row=comp_state_row, norm_w=comp_norm,
                                ring_entries=comp_state_ring_entries, q8=comp_q8, s8=comp_s8, rope=comp_rope))


def mqa_compressor_standalone(cmp_pos, comp_norm, cos_tab, sin_tab, comp_state, comp_state_row, comp_state_ring_entries,
                              comp_q8, comp_s8, comp_rope, eps=1e-6):
    """The same call under the name the FP4 logits module exports (kernels/mqa_logits_fp4.cu:653-680)."""
    rows = cmp_pos.numel()      # the reference takes int32 row numbers here; the writers take int64
    mqa_compressor_fp8_standalone(cmp_pos, comp_norm, cos_tab, sin_tab, comp_state,
                                  comp_state_row.reshape(-1)[:rows].to(torch.int64), comp_state_ring_entries, comp_q8,
                                  comp_s8, comp_rope, eps)


def mqa_compressor_paged(cmp_pos, comp_norm, cos_tab, sin_tab, comp_state, comp_state_row, comp_state_ring_entries,
                         cmp_cache, cmp_dst, cmp_entries_per_block, cmp_block_stride_bytes, eps=1e-6):
    """The MAIN compressor writing its 584-byte records straight into the pool's pages, with the reference's
    argument list and checks (kernels/mqa_logits_fp4.cu:681-750): cmp_cache uint8 pages of cmp_block_stride_bytes,
    cmp_dst[r] = the physical entry row r goes to (negative: nowhere)."""
    _require(cmp_entries_per_block > 0 and cmp_block_stride_bytes >= cmp_entries_per_block * 584
             and cmp_cache.is_cuda and cmp_cache.is_contiguous() and cmp_cache.dtype == torch.uint8
             and cmp_cache.numel() % cmp_block_stride_bytes == 0, "cmp_cache physical page geometry is invalid")
    _require(cmp_dst.is_cuda and cmp_dst.is_contiguous() and cmp_dst.numel() >= cmp_pos.numel(),
             "cmp_dst must be a contiguous CUDA integer tensor [>=B]")
    rows = cmp_pos.numel()      # the reference takes int32 row numbers and destinations; the writers take int64
    cache_writers_fp8(cmp_pos, cos_tab, sin_tab, eps=eps,
                      main=dict(state=comp_state, state_row=comp_state_row.reshape(-1)[:rows].to(torch.int64),
                                norm_w=comp_norm, ring_entries=comp_state_ring_entries,
                                pool=cmp_cache.view(-1, cmp_block_stride_bytes),
                                dst=cmp_dst.reshape(-1)[:rows].to(torch.int64),
                                entries_per_block=int(cmp_entries_per_block)))


def rmsnorm_rope_out(x, positions, cos_table, sin_table, out, input_heads=None, eps=1e-6, pdl=False, max_blocks=0):
    """Per-head RMSNorm (no gamma) + RoPE on the last 64 dims, bf16 -> bf16 in one pass with one
    rounding, with the reference's signature (kernels/rmsnorm_prod.cu:160-167).  `x` is
    [B, heads, 512] and may be a column slice of a wider projection output (row stride taken from
    the tensor); `out` is caller-owned [B, out_heads, 512], out head h reads head h % heads."""
    _require(x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 3 and x.size(2) == 512
             and x.stride(2) == 1 and x.stride(1) == 512, "x must be CUDA bf16 [B, heads, 512] with dense heads")
    b, heads, _ = x.shape
    _require(input_heads in (None, 0, heads), "input_heads must equal x.size(1)")
    _require(out.is_cuda and out.is_contiguous() and out.dtype == torch.bfloat16 and out.dim() == 3
             and out.size(0) == b and out.size(2) == 512 and out.size(1) % heads == 0,
             "out must be contiguous CUDA bf16 [B, k * heads, 512]")
    _require(positions.is_cuda and positions.is_contiguous() and positions.dtype == torch.int64
             and positions.numel() == b, "positions must be contiguous CUDA int64 [B]")
    _f32(cos_table, "cos_table", 32)
    _f32(sin_table, "sin_table", 32)
    check(lib.wuda_query_rms_rope(x.data_ptr(), x.stride(0), positions.data_ptr(), cos_table.data_ptr(),
                                  sin_table.data_ptr(), cos_table.size(0), out.data_ptr(), b, heads, out.size(1),
                                  float(eps), _stream()))
    return out


def idx_postprocess_fp8(iq, weights, q_pos, rope_cos, rope_sin, q_fp8=None, weights_out=None):
    """Indexer-q post, FP8 form (the reference's idx_postprocess_fp8_standalone,
    kernels/wq_b_fp8_gemm.cu:1368-1567): iq bf16 [M, heads, 128] (may be a column slice of the
    projection output), weights fp32 [M, heads] or None, q_pos int32 [M].  Returns
    (q e4m3 [M, heads, 128], weights * scale fp32 [M, heads])."""
    _require(iq.is_cuda and iq.dtype == torch.bfloat16 and iq.dim() == 3 and iq.size(2) == 128
             and iq.stride(2) == 1 and iq.stride(1) == 128, "iq must be CUDA bf16 [M, heads, 128] with dense heads")
    m, heads, _ = iq.shape
    _require(q_pos.is_cuda and q_pos.is_contiguous() and q_pos.dtype == torch.int32 and q_pos.numel() == m,
             "q_pos must be contiguous CUDA int32 [M]")
    if weights is not None:
        _require(weights.is_cuda and weights.is_contiguous() and weights.dtype == torch.float32
                 and weights.numel() == m * heads, "weights must be contiguous CUDA fp32 [M, heads]")
    _f32(rope_cos, "rope_cos", 32)
    _f32(rope_sin, "rope_sin", 32)
    if q_fp8 is None:
        q_fp8 = torch.empty((m, heads, 128), dtype=torch.float8_e4m3fn, device=iq.device)
    if weights_out is None:
        weights_out = torch.empty((m, heads), dtype=torch.float32, device=iq.device)
    _require(q_fp8.is_contiguous() and q_fp8.element_size() == 1 and q_fp8.numel() == m * heads * 128
             and weights_out.is_contiguous() and weights_out.dtype == torch.float32
             and weights_out.numel() == m * heads, "outputs must be contiguous [M, heads, 128] / fp32 [M, heads]")
    check(lib.wuda_index_q_post_fp8(iq.data_ptr(), iq.stride(0), q_pos.data_ptr(), rope_cos.data_ptr(),
                                    rope_sin.data_ptr(), rope_cos.size(0), _ptr(weights), q_fp8.data_ptr(),
                                    weights_out.data_ptr(), m, heads, _stream()))
    return q_fp8, weights_out


def idx_postprocess(iq, q_pos, rope_cos, rope_sin, iq_fp4=None, iq_sf=None):
    """Indexer-q post, FP4 form (the reference's idx_postprocess, kernels/idx_post_fp4.cu; device chain
    include/idx_post_fp4.cuh:79-224): iq bf16 [M, heads, 128] (may be a column slice of the projection output),
    q_pos int32 [M].  RoPE on the last 64 dims, Hadamard-128, MXFP4.  Returns (iq_fp4 int8 [M, heads, 64] packed
    e2m1, iq_sf int32 [M, heads] of four exponent bytes): the q / sf_q operands of mqa_logits_fp4_decode."""
    _require(iq.is_cuda and iq.dtype == torch.bfloat16 and iq.dim() == 3 and iq.size(2) == 128
             and iq.stride(2) == 1 and iq.stride(1) == 128, "iq must be CUDA bf16 [M, heads, 128] with dense heads")
    m, heads, _ = iq.shape
    _require(q_pos.is_cuda and q_pos.is_contiguous() and q_pos.dtype == torch.int32 and q_pos.numel() == m,
             "q_pos must be contiguous CUDA int32 [M]")
    _f32(rope_cos, "rope_cos", 32)
    _f32(rope_sin, "rope_sin", 32)
    if iq_fp4 is None:
        iq_fp4 = torch.empty((m, heads, 64), dtype=torch.int8, device=iq.device)
    if iq_sf is None:
        iq_sf = torch.empty((m, heads), dtype=torch.int32, device=iq.device)
    _require(iq_fp4.is_contiguous() and iq_fp4.element_size() == 1 and iq_fp4.numel() == m * heads * 64
             and iq_sf.is_contiguous() and iq_sf.element_size() == 4 and iq_sf.numel() == m * heads,
             "outputs must be contiguous 1-byte [M, heads, 64] / 4-byte [M, heads]")
    check(lib.wuda_index_q_post_fp4(iq.data_ptr(), iq.stride(0), q_pos.data_ptr(), rope_cos.data_ptr(),
                                    rope_sin.data_ptr(), rope_cos.size(0), iq_fp4.data_ptr(), iq_sf.data_ptr(), m, heads,
                                    _stream()))
    return iq_fp4, iq_sf


def idx_postprocess_standalone(iq_f32, q_pos, rope_cos, rope_sin):
    """idx_postprocess under the name the q-projection module exports (kernels/wq_b_fp8_gemm.cu:1474-1507): iq bf16
    [M, 64, 128] (an fp32 tensor is rounded to bf16 first, which is what the projection's epilogue would have
    stored).  Returns (iq_fp4 int8 [M, 64, 64], iq_sf int32 [M, 64])."""
    return idx_postprocess(iq_f32 if iq_f32.dtype == torch.bfloat16 else iq_f32.bfloat16(), q_pos, rope_cos, rope_sin)


def idx_postprocess_fp8_standalone(iq, weights, q_pos, rope_cos, rope_sin):
    """idx_postprocess_fp8 under the reference's export name (kernels/wq_b_fp8_gemm.cu:1509-1546).  Returns
    (q e4m3 [M, 64, 128], weights * scale fp32 [M, 64])."""
    return idx_postprocess_fp8(iq if iq.dtype == torch.bfloat16 else iq.bfloat16(), weights, q_pos, rope_cos, rope_sin)


def head_ssq_standalone(y, num_heads=None):
    """Per (row, head) sum of squares over the bf16 main q [M, heads * 512] -> fp32 [M, heads]
    (kernels/wq_b_fp8_gemm.cu:101-123, 1548-1566), in the reference kernel's summation order."""
    _require(y.is_cuda and y.dtype == torch.bfloat16 and y.dim() == 2 and y.stride(1) == 1 and y.size(1) % 512 == 0,
             "y must be CUDA bf16 [M, heads * 512] with unit inner stride")
    heads = y.size(1) // 512 if num_heads is None else int(num_heads)
    _require(heads * 512 <= y.size(1), "y has fewer than num_heads heads")
    ssq = torch.empty((y.size(0), heads), dtype=torch.float32, device=y.device)
    check(lib.wuda_head_ssq(y.data_ptr(), y.stride(0), ssq.data_ptr(), y.size(0), heads, _stream()))
    return ssq


def hc_split_sinkhorn(mixes, hc_scale, hc_base, hc_mult=4, sinkhorn_iters=20, eps=1e-6):
    """The origin's hc_split_sinkhorn (origin/kernel.py:430-436): mixes fp32 [b, s, 24] -> (pre [b, s, 4], post
    [b, s, 4], comb [b, s, 4, 4])."""
    _require(hc_mult == 4 and sinkhorn_iters == 20, "hc_mult 4 and 20 Sinkhorn iterations are what is built")
    _require(mixes.is_cuda and mixes.is_contiguous() and mixes.dtype == torch.float32 and mixes.size(-1) == 24,
             "mixes must be contiguous CUDA fp32 [..., 24]")
    _require(hc_scale.is_cuda and hc_scale.is_contiguous() and hc_scale.dtype == torch.float32 and hc_scale.numel() == 3
             and hc_base.is_cuda and hc_base.is_contiguous() and hc_base.dtype == torch.float32 and hc_base.numel() == 24,
             "hc_scale fp32 [3] and hc_base fp32 [24] must be contiguous CUDA tensors")
    lead = mixes.shape[:-1]
    pre, post = mixes.new_empty(*lead, 4), mixes.new_empty(*lead, 4)
    comb = mixes.new_empty(*lead, 4, 4)
    check(lib.wuda_hc_split_sinkhorn(mixes.data_ptr(), hc_scale.data_ptr(), hc_base.data_ptr(), float(eps), pre.data_ptr(),
                                     post.data_ptr(), comb.data_ptr(), mixes.numel() // 24, _stream()))
    return pre, post, comb


def fp4_act_quant(x, block_size=32, inplace=False):
    """Block-wise FP4 quantisation with the origin's signature (origin/kernel.py:186-200): returns (y
    float4_e2m1fn_x2 [..., N/2], scales float8_e8m0fnu [..., N/32]); inplace=True overwrites x with the
    dequantised values and returns it."""
    _require(block_size == 32, "block_size must be 32")
    _require(x.is_cuda and x.dtype == torch.bfloat16 and x.size(-1) % 32 == 0, "x must be CUDA bf16 [..., N], N % 32 == 0")
    n = x.size(-1)
    # rows of a wider matrix (a column slice with 16-byte aligned rows) are read and written where they are
    strided = x.dim() == 2 and x.stride(1) == 1 and x.stride(0) >= n and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0
    z = x if (strided or x.is_contiguous()) else x.contiguous()
    rows = z.numel() // n
    stride = z.stride(0) if strided else n
    if inplace:
        check(lib.wuda_fp4_act_quant(z.data_ptr(), stride, None, None, 1, rows, n, _stream()))
        if z.data_ptr() != x.data_ptr():
            x.copy_(z)
        return x
    y = torch.empty(*z.shape[:-1], n // 2, dtype=torch.uint8, device=x.device)
    sc = torch.empty(*z.shape[:-1], n // 32, dtype=torch.uint8, device=x.device)
    check(lib.wuda_fp4_act_quant(z.data_ptr(), stride, y.data_ptr(), sc.data_ptr(), 0, rows, n, _stream()))
    fp4 = getattr(torch, "float4_e2m1fn_x2", None)
    e8 = getattr(torch, "float8_e8m0fnu", None)
    return (y.view(fp4) if fp4 is not None else y), (sc.view(e8) if e8 is not None else sc)


def _scales_as_fp32(t, name):
    """fp32 scales as they are; float8_e8m0fnu (or raw exponent bytes) -> the fp32 power of two, exactly."""
    if t.dtype == torch.float32:
        return t
    _require(t.element_size() == 1, name + " must be fp32 or one exponent byte per scale")
    return (t.view(torch.uint8).to(torch.int32) << 23).view(torch.float32)


def fp4_gemm(a, a_s, b, b_s, scale_dtype=torch.float32, *, out=None, status_word=None):
    """C[M,N] = A_fp8[M,K] @ B_fp4[N,K]^T with the origin's signature (origin/kernel.py:518-536): a e4m3, a_s one
    POWER-OF-TWO scale per row and 128 K-elements (fp32 or float8_e8m0fnu: act_quant with scale_fmt "ue8m0"), b
    float4_e2m1fn_x2 [N, K/2], b_s float8_e8m0fnu [N, K/32].  bf16 output."""
    _require(a.is_cuda and a.is_contiguous() and a.dtype == torch.float8_e4m3fn, "a must be contiguous CUDA e4m3")
    _require(b.is_cuda and b.is_contiguous() and b.element_size() == 1 and b.dim() == 2,
             "b must be contiguous CUDA float4_e2m1fn_x2 (or bytes) [N, K/2]")
    k = a.size(-1)
    m = a.numel() // k
    n = b.size(0)
    _require(b.size(1) * 2 == k and k % 128 == 0, "a and b disagree on K, or K is not a multiple of 128")
    _require(a_s.is_cuda and a_s.is_contiguous() and a_s.numel() == m * (k // 128), "a_s must be contiguous CUDA [M, K/128]")
    _require(b_s.is_cuda and b_s.is_contiguous() and b_s.element_size() == 1 and tuple(b_s.shape) == (n, k // 32),
             "b_s must be contiguous CUDA float8_e8m0fnu (or bytes) [N, K/32]")
    a_sf = _scales_as_fp32(a_s, "a_s")
    if out is None:
        out = torch.empty(*a.shape[:-1], n, dtype=torch.bfloat16, device=a.device)
    need = lib.wuda_gemm_fp8_scratch_bytes(m, n)
    _require(need >= 0, "m must be in [1, 256]")
    scratch = _scratch_for(a.device, need)
    check(lib.wuda_gemm_fp8_fp4_pow2(a.data_ptr(), a_sf.data_ptr(), b.data_ptr(), b_s.data_ptr(), out.data_ptr(), m, n, k,
                                     scratch.data_ptr(), scratch.numel(),
                                     status_word.data_ptr() if status_word is not None else None, _stream()))
    return out


_gemm_scratch = {}


def _scratch_for(device, nbytes):
    """A zeroed scratch buffer per device, grown on demand (the GEMM leaves it zero)."""
    buf = _gemm_scratch.get(device)
    if buf is None or buf.numel() < nbytes:
        buf = torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _gemm_scratch[device] = buf
    return buf


def fp8_gemm(a, a_s, b, b_s, scale_dtype=torch.float32, *, out=None, status_word=None, pow2_scales=False):
    """C[M,N] = A[M,K] @ B[N,K]^T with 1x128 (A) and 128x128 (B) fp32 block scales, bf16
    output: the origin's fp8_gemm(a, a_s, b, b_s) (origin/kernel.py:257-273).  pow2_scales=True promises that
    every scale is a power of two (the reference's UE8M0 scales) and takes the kernel that applies them inside
    the tensor core."""
    if a_s.dtype != torch.float32 and b_s.dtype != torch.float32:    # float8_e8m0fnu scales: powers of two by type
        pow2_scales = True
    a_s, b_s = _scales_as_fp32(a_s, "a_s"), _scales_as_fp32(b_s, "b_s")
    _require(a.is_cuda and a.is_contiguous() and a.dtype == torch.float8_e4m3fn, "a must be contiguous CUDA e4m3")
    _require(b.is_cuda and b.is_contiguous() and b.dtype == torch.float8_e4m3fn and b.dim() == 2,
             "b must be contiguous CUDA e4m3 [N, K]")
    k = a.size(-1)
    m = a.numel() // k
    n = b.size(0)
    _require(b.size(1) == k, "a and b disagree on K")
    _require(a_s.is_cuda and a_s.is_contiguous() and a_s.dtype == torch.float32 and a_s.numel() == m * (k // 128),
             "a_s must be contiguous CUDA fp32 [M, K/128]")
    _require(b_s.is_cuda and b_s.is_contiguous() and b_s.dtype == torch.float32
             and tuple(b_s.shape) == ((n + 127) // 128, k // 128), "b_s must be contiguous CUDA fp32 [ceil(N/128), K/128]")
    if out is None:
        out = torch.empty(*a.shape[:-1], n, dtype=torch.bfloat16, device=a.device)
    need = lib.wuda_gemm_fp8_scratch_bytes(m, n)
    _require(need >= 0, "m must be in [1, 256]")
    scratch = _scratch_for(a.device, need)
    entry = lib.wuda_gemm_fp8_blockscaled_pow2 if pow2_scales else lib.wuda_gemm_fp8_blockscaled
    check(entry(a.data_ptr(), a_s.data_ptr(), b.data_ptr(), b_s.data_ptr(), out.data_ptr(), m, n, k, scratch.data_ptr(),
                scratch.numel(), status_word.data_ptr() if status_word is not None else None, _stream()))
    return out


def bf16_gemm(a, w, *, out=None, out_dtype=torch.bfloat16, status_word=None):
    """C[M,N] = A[M,K] @ W[N,K]^T on bf16 operands with fp32 accumulation; bf16 or fp32 output
    (the origin's `linear` on bf16 weights, origin/model.py:108-120)."""
    _require(a.is_cuda and a.is_contiguous() and a.dtype == torch.bfloat16, "a must be contiguous CUDA bf16")
    _require(w.is_cuda and w.is_contiguous() and w.dtype == torch.bfloat16 and w.dim() == 2,
             "w must be contiguous CUDA bf16 [N, K]")
    k = a.size(-1)
    m, n = a.numel() // k, w.size(0)
    _require(w.size(1) == k, "a and w disagree on K")
    if out is None:
        out = torch.empty(*a.shape[:-1], n, dtype=out_dtype, device=a.device)
    _require(out.is_contiguous() and out.dtype in (torch.bfloat16, torch.float32) and out.numel() == m * n,
             "out must be contiguous bf16 or fp32 [M, N]")
    need = lib.wuda_gemm_bf16_scratch_bytes(m, n)
    _require(need >= 0, "m must be in [1, 128]")
    scratch = _scratch_for(a.device, need)
    check(lib.wuda_gemm_bf16(a.data_ptr(), w.data_ptr(), out.data_ptr(), int(out.dtype == torch.float32), m, n, k,
                             scratch.data_ptr(), scratch.numel(), _ptr(status_word), _stream()))
    return out


def front_mixed_gemm(x, x_fp8, x_sf, w_bf16, w_fp8, w_sf, out, *, pos=None, main_state=None, ape=None,
                     main_state_row=None, idx_state=None, idx_state_row=None, idx_ape=None, win_y2=None, w64=None,
                     y16=None, status_word=None, sm_split=None):
    """The front projection of a decode step with its side-channel outputs, after the reference's
    front_mixed_gemm_csa_swapab (kernels/front_mixed_gemm_csa_swapab.cu:262-279):
    y[M, 4672] = x . [W8 (2048 rows, FP8 1x128 / 128x128 scales) | W16 (2624 rows, BF16)]^T.
    `out` bf16 [M, 2048] receives the FP8 segment (q_raw | win); the BF16 segment is produced in fp32
    (`y16` [M, 2624], allocated if not given) and scattered into the state rings, win_y2 and w64 when
    those are passed (all-or-none with pos).  Three launches: two GEMMs and the scatter.  sm_split = (SMs of the
    FP8 GEMM, SMs of the BF16 GEMM) launches them with the shares wuda_layer_decode gives them when it runs the two
    side by side, which makes the sums bit-identical to that call's."""
    m = x.size(0)
    _require(tuple(w_fp8.shape) == (2048, x.size(1)) and tuple(w_bf16.shape) == (2624, x.size(1)),
             "w_fp8 must be [2048, K] and w_bf16 [2624, K]")
    _require(out.is_cuda and out.is_contiguous() and out.dtype == torch.bfloat16 and tuple(out.shape) == (m, 2048),
             "out must be contiguous CUDA bf16 [M, 2048]")
    if y16 is None:
        y16 = torch.empty(m, 2624, dtype=torch.float32, device=x.device)
    try:
        if sm_split is not None:
            lib.wuda_gemm_sm_limit(int(sm_split[0]))
        fp8_gemm(x_fp8, x_sf, w_fp8, w_sf, out=out, status_word=status_word)
        if sm_split is not None:
            lib.wuda_gemm_sm_limit(int(sm_split[1]))
        bf16_gemm(x, w_bf16, out=y16, status_word=status_word)
    finally:
        if sm_split is not None:
            lib.wuda_gemm_sm_limit(0)
    if pos is not None:
        _require(pos.is_cuda and pos.is_contiguous() and pos.dtype == torch.int64 and pos.numel() == m,
                 "pos must be contiguous CUDA int64 [M]")
        rows_total = 0
        for state, width, row, table, tw in ((main_state, 2048, main_state_row, ape, 1024),
                                             (idx_state, 512, idx_state_row, idx_ape, 256)):
            if state is None:
                continue
            _f32(state, "state", width)
            _require(row is not None and row.is_cuda and row.is_contiguous() and row.dtype == torch.int64
                     and row.numel() == m, "state rows must be contiguous CUDA int64 [M]")
            _require(_f32(table, "ape").shape == (4, tw), "ape must be fp32 [4, %d]" % tw)
            total = state.numel() // width
            _require(rows_total in (0, total), "the two state rings must have the same number of rows")
            rows_total = total
        if win_y2 is not None:
            _require(_f32(win_y2, "win_y2", 512).numel() == m * 512, "win_y2 must be fp32 [M, 512]")
        if w64 is not None:
            _require(_f32(w64, "w64", 64).numel() == m * 64, "w64 must be fp32 [M, 64]")
        check(lib.wuda_front_emit(out.data_ptr(), y16.data_ptr(), pos.data_ptr(), _ptr(main_state), _ptr(ape),
                                  _ptr(main_state_row), _ptr(idx_state), _ptr(idx_ape), _ptr(idx_state_row),
                                  _ptr(win_y2), _ptr(w64), max(rows_total, 1), m, _ptr(status_word), _stream()))
    return out, y16


SCORE_FUNCS = {"softmax": 0, "sigmoid": 1, "sqrtsoftplus": 2}


def moe_gate(x, weight, bias=None, score_func="sqrtsoftplus", route_scale=1.0, topk=8, *, logits=None):
    """The origin's Gate.forward (origin/model.py:563-584) for score-routed layers: x bf16 [M, dim],
    gate weight bf16 [experts, dim], bias fp32 [experts] or None.  Returns (weights fp32 [M, topk],
    indices int32 [M, topk]).  Two launches: the projection (fp32 logits) and the router."""
    _require(score_func in SCORE_FUNCS, "score_func must be one of %s" % sorted(SCORE_FUNCS))
    m, experts = x.size(0), weight.size(0)
    if logits is None:
        logits = torch.empty(m, experts, dtype=torch.float32, device=x.device)
    bf16_gemm(x, weight, out=logits)
    if bias is not None:
        _require(_f32(bias, "bias").numel() == experts, "bias must be fp32 [experts]")
    w = torch.empty(m, topk, dtype=torch.float32, device=x.device)
    idx = torch.empty(m, topk, dtype=torch.int32, device=x.device)
    check(lib.wuda_moe_route(logits.data_ptr(), _ptr(bias), w.data_ptr(), idx.data_ptr(), m, experts, topk,
                             SCORE_FUNCS[score_func], float(route_scale), _stream()))
    return w, idx


def exchange_handles(my_handle, group=None):
    """Host-side bootstrap of the two-rank link: all-gathers the ranks' 64-byte IPC handles
    over torch.distributed (any backend) and returns the peer's.  Not on the hot path."""
    import torch.distributed as dist
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    _require(world == 2, "the link joins exactly two ranks")
    backend = dist.get_backend(group)
    device = "cuda" if backend == "nccl" else "cpu"
    mine = torch.tensor(list(my_handle), dtype=torch.uint8, device=device)
    both = [torch.zeros(64, dtype=torch.uint8, device=device) for _ in range(2)]
    dist.all_gather(both, mine, group=group)
    return bytes(both[1 - rank].cpu().tolist())


class TP2Link:
    """Exchange buffers of a two-rank tensor-parallel pair for fp8_gemm's fused all-reduce.

    link = TP2Link(max_m, n)           # allocates this rank's inbox, exchanges IPC handles
    y = link.fp8_gemm(a_local, a_s, w_local, w_s)   # == bf16(sum over ranks), on both ranks
    """

    def __init__(self, m, n, group=None, peer_handle=None, loopback=False, device_sequence=False):
        """device_sequence: the link numbers its calls on the device (both ranks must choose alike); needed
        when the call is captured into a CUDA graph and replayed."""
        import ctypes
        self.m, self.n, self.device_sequence = m, n, device_sequence
        self.nbytes = lib.wuda_tp2_inbox_bytes(m, n)
        _require(self.nbytes > 0, "unsupported (m, n) for the exchange buffer")
        self._local, self._peer = ctypes.c_void_p(), ctypes.c_void_p()
        handle = (ctypes.c_ubyte * 64)()
        check(lib.wuda_tp2_alloc(self.nbytes, ctypes.byref(self._local), handle))
        self.handle = bytes(handle)
        self.epoch = 0
        self._mute = None
        if loopback:
            # a peer that never answers: a second buffer on this GPU receives the pushes and
            # nothing ever raises the flags of the real inbox (tests of the time-out path)
            self._mute = ctypes.c_void_p()
            check(lib.wuda_tp2_alloc(self.nbytes, ctypes.byref(self._mute), (ctypes.c_ubyte * 64)()))
            self._peer = self._mute
            self._own_peer = False
        else:
            if peer_handle is None:
                peer_handle = exchange_handles(self.handle, group)
            buf = (ctypes.c_ubyte * 64).from_buffer_copy(peer_handle)
            check(lib.wuda_tp2_open(buf, ctypes.byref(self._peer)))
            self._own_peer = True

    def fp8_gemm(self, a, a_s, b, b_s, *, out=None, status_word=None, peer_wait_ms=2000):
        k = a.size(-1)
        m = a.numel() // k
        n = b.size(0)
        _require(m <= self.m and n == self.n, "shape outside what the link was created for")
        if out is None:
            out = torch.empty(*a.shape[:-1], n, dtype=torch.bfloat16, device=a.device)
        need = lib.wuda_gemm_fp8_scratch_bytes(m, n)
        scratch = _scratch_for(a.device, need)
        self.epoch += 1
        check(lib.wuda_gemm_fp8_blockscaled_tp2(a.data_ptr(), a_s.data_ptr(), b.data_ptr(), b_s.data_ptr(),
                                                out.data_ptr(), m, n, k, scratch.data_ptr(), scratch.numel(),
                                                self._local, self._peer, 0 if self.device_sequence else self.epoch,
                                                int(peer_wait_ms),
                                                status_word.data_ptr() if status_word is not None else None,
                                                _stream()))
        return out

    def close(self):
        if getattr(self, "_own_peer", False) and self._peer:
            lib.wuda_tp2_close(self._peer)
        self._peer = None
        if getattr(self, "_mute", None):
            lib.wuda_tp2_free(self._mute)
            self._mute = None
        if getattr(self, "_local", None):
            lib.wuda_tp2_free(self._local)
            self._local = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def nvfp4_gemm(a, a_sf_packed, a_global_scale, w, w_sf_packed, w_global_scale, *, out=None, status_word=None):
    """bf16 C[M,N] = NVFP4 A[M,K] @ W[N,K]^T: a, w packed e2m1 uint8 [rows, K/2]; *_sf_packed the
    ue4m3 block scales in tensor-core order (wuda_b200.workloads.pack_nvfp4_scales); one fp32
    scale per tensor."""
    _require(a.is_cuda and a.is_contiguous() and a.dtype == torch.uint8 and a.dim() == 2, "a must be CUDA uint8 [M, K/2]")
    _require(w.is_cuda and w.is_contiguous() and w.dtype == torch.uint8 and w.dim() == 2 and w.size(1) == a.size(1),
             "w must be CUDA uint8 [N, K/2]")
    m, k = a.size(0), a.size(1) * 2
    n = w.size(0)
    _require(a_sf_packed.is_cuda and a_sf_packed.dtype == torch.uint8
             and a_sf_packed.numel() == ((m + 127) // 128) * 128 * (k // 16), "a_sf_packed has the wrong size")
    _require(w_sf_packed.is_cuda and w_sf_packed.dtype == torch.uint8
             and w_sf_packed.numel() == ((n + 127) // 128) * 128 * (k // 16), "w_sf_packed has the wrong size")
    if out is None:
        out = torch.empty(m, n, dtype=torch.bfloat16, device=a.device)
    need = lib.wuda_gemm_nvfp4_scratch_bytes(m, n)
    _require(need >= 0, "m must be in [1, 256]")
    scratch = _scratch_for(a.device, need)
    check(lib.wuda_gemm_nvfp4(a.data_ptr(), a_sf_packed.data_ptr(), float(a_global_scale), w.data_ptr(),
                              w_sf_packed.data_ptr(), float(w_global_scale), out.data_ptr(), m, n, k,
                              scratch.data_ptr(), scratch.numel(),
                              status_word.data_ptr() if status_word is not None else None, _stream()))
    return out
