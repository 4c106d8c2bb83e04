"""Host-side driver of the indexer half of a decode step.

`CsaDecodeStage` owns the weights, the cache manager's pools and a fixed workspace, and issues
`wuda_csa_decode_step` (the C++ layer launch) for a batch of request slots.  It plays the part
of the reference's decode_step between the front GEMM and the sparse attention
(dsv4_megakernel/megakernel/test/test_e2e_decode.py:560-640) and, like it, can be captured into
a CUDA graph (:1347-1358): all per-step device inputs live in fixed buffers that `prepare()`
refills, so a captured step is replayed with new positions and destinations.
"""
import ctypes

import torch

from . import _lib
from ._lib import check, lib
from .kv_cache import KVCacheManager


def _ptr(t):
    return t.data_ptr() if t is not None else None


class CsaWeights:
    """Device weights of the stage.  wq_b is e4m3 [index_heads*128 + main_heads*512, q_lora] with
    fp32 128x128 block scales; the norm weights are fp32; the tables fp32 [max_pos, 32]."""

    def __init__(self, wq_b, wq_b_scales, q_norm, idx_norm, main_norm, win_norm, cos_table, sin_table,
                 index_heads=64, main_heads=128, out_heads=None, eps=1e-6, scales_pow2=False):
        """scales_pow2: every wq_b scale is a power of two (the reference's UE8M0 scales); the projection then runs on
        the GEMM that applies the scales inside the tensor core."""
        self.q_lora = wq_b.size(1)
        self.index_heads, self.main_heads = index_heads, main_heads
        self.out_heads = out_heads or main_heads
        self.eps = eps
        self.n_total = index_heads * 128 + main_heads * 512
        if wq_b.size(0) != self.n_total or wq_b.element_size() != 1:
            raise ValueError("wq_b must be 1-byte [index_heads*128 + main_heads*512, q_lora]")
        self.tensors = dict(wq_b=wq_b, wq_b_scales=wq_b_scales, q_norm=q_norm, idx_norm=idx_norm, main_norm=main_norm,
                            win_norm=win_norm, cos_table=cos_table, sin_table=sin_table)
        for name, t in self.tensors.items():
            if not (t.is_cuda and t.is_contiguous()) or (name != "wq_b" and t.dtype != torch.float32):
                raise ValueError(name + " must be a contiguous CUDA tensor (fp32 unless wq_b)")
        self.c = _lib.CsaWeights(max_pos=cos_table.size(0), q_lora=self.q_lora, index_heads=index_heads,
                                 main_heads=main_heads, out_heads=self.out_heads, eps=eps, scales_pow2=int(bool(scales_pow2)),
                                 **{k: t.data_ptr() for k, t in self.tensors.items()})


class CsaDecodeStage:
    def __init__(self, weights, cache, max_batch, topk=2048, max_compressed=None, device="cuda"):
        if not isinstance(cache, KVCacheManager):
            raise TypeError("cache must be a wuda_b200.kv_cache.KVCacheManager")
        if not 1 <= max_batch <= 128:
            raise ValueError("max_batch must be in [1, 128]")
        self.w, self.cache, self.max_batch, self.topk = weights, cache, max_batch, topk
        # A cache whose indexer pool holds MXFP4 records (KVCacheManager(indexer_fp8=False)) selects the FP4 form of
        # the step: Hadamard + MXFP4 indexer-q post and compressor, block-scaled logits.  iq_fp8 then receives the
        # packed codes and w_folded (viewed as int32) the query's scale words.
        self.indexer_fp4 = not cache.indexer_fp8
        if self.indexer_fp4 and weights.index_heads != 64:
            raise ValueError("the FP4 form of the indexer has 64 index heads")
        epb = cache.entries_per_block["idx"]
        max_compressed = max_compressed or cache.max_pages * epb
        self.logits_stride = (max_compressed + 255) // 256 * 256
        m, dev = max_batch, device
        i64 = lambda *s: torch.zeros(*s, dtype=torch.int64, device=dev)
        i32 = lambda *s: torch.zeros(*s, dtype=torch.int32, device=dev)
        # per-step inputs (fixed addresses: a captured step reads whatever prepare() put here)
        self.pos, self.q_pos = i64(m), i32(m)
        self.main_state_row, self.idx_state_row = i64(m), i64(m)
        self.idx_dst, self.cmp_dst, self.swa_dst = i64(m), i64(m), i64(m)
        self.block_table = i32(m, cache.max_pages)
        self.cmp_block_table = i32(m, cache.max_pages)
        self.n_compressed = i32(m)
        self.q_raw = torch.zeros(m, weights.q_lora, dtype=torch.bfloat16, device=dev)
        self.w64 = torch.zeros(m, weights.index_heads, dtype=torch.float32, device=dev)
        self.win_y2 = torch.zeros(m, 512, dtype=torch.float32, device=dev)
        # outputs
        self.logits = torch.full((m, self.logits_stride), float("-inf"), dtype=torch.float32, device=dev)
        self.topk_indices = torch.full((m, topk), -1, dtype=torch.int32, device=dev)
        self.topk_raw = torch.full((m, topk), -1, dtype=torch.int32, device=dev)
        self.q_main = torch.zeros(m, weights.out_heads, 512, dtype=torch.bfloat16, device=dev)
        # workspace
        self.q_fp8 = torch.zeros(m, weights.q_lora, dtype=torch.uint8, device=dev)
        self.q_scales = torch.zeros(m, weights.q_lora // 128, dtype=torch.float32, device=dev)
        self.y = torch.zeros(m, weights.n_total, dtype=torch.bfloat16, device=dev)
        self.iq_fp8 = torch.zeros(m, weights.index_heads, 128, dtype=torch.uint8, device=dev)
        self.w_folded = torch.zeros(m, weights.index_heads, dtype=torch.float32, device=dev)
        scratch_bytes = lib.wuda_gemm_fp8_scratch_bytes(m, weights.n_total)
        self.gemm_scratch = torch.zeros(scratch_bytes, dtype=torch.uint8, device=dev)
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        self._caches = _lib.CsaCaches(
            idx_state=cache.idx_state.data_ptr(), main_state=cache.main_state.data_ptr(),
            state_rows_total=cache.capacity * cache.state_ring_entries, ring_entries=cache.state_ring_entries,
            idx_entries_per_block=epb, cmp_entries_per_block=cache.entries_per_block["cmp"],
            swa_entries_per_block=cache.entries_per_block["swa"], idx_num_blocks=cache.idx_pool.size(0),
            cmp_num_blocks=cache.cmp_pool.size(0), swa_num_blocks=cache.swa_pool.size(0),
            idx_block_stride_bytes=cache.block_stride_bytes["idx"], cmp_block_stride_bytes=cache.block_stride_bytes["cmp"],
            swa_block_stride_bytes=cache.block_stride_bytes["swa"], idx_fp4=int(self.indexer_fp4),
            idx_pool=cache.idx_pool.data_ptr(),
            cmp_pool=cache.cmp_pool.data_ptr(), swa_pool=cache.swa_pool.data_ptr())
        self._ws = _lib.CsaWorkspace(q_fp8=self.q_fp8.data_ptr(), q_scales=self.q_scales.data_ptr(), y=self.y.data_ptr(),
                                     iq_fp8=self.iq_fp8.data_ptr(), w_folded=self.w_folded.data_ptr(),
                                     gemm_scratch=self.gemm_scratch.data_ptr(), gemm_scratch_bytes=scratch_bytes,
                                     status_word=self.status.data_ptr())
        self._graph, self._graph_m = None, 0

    # ---- host side of a step: positions, rows and destinations from the cache manager
    def prepare(self, slots):
        """Advances every request by one token and refills the per-step device buffers."""
        m = len(slots)
        if not 1 <= m <= self.max_batch:
            raise ValueError("batch of %d requests does not fit max_batch=%d" % (m, self.max_batch))
        st = self.cache.step_begin(slots)
        pos = st["pos"].tolist()
        self.pos[:m].copy_(st["pos"], non_blocking=True)
        self.q_pos[:m].copy_(st["q_pos"], non_blocking=True)
        self.main_state_row[:m].copy_(st["main_state_row"], non_blocking=True)
        self.idx_state_row[:m].copy_(st["idx_state_row"], non_blocking=True)
        for name in ("idx_dst", "cmp_dst", "swa_dst"):
            getattr(self, name)[:m].copy_(st[name], non_blocking=True)
        self.block_table[:m].copy_(self.cache.block_table("idx", slots), non_blocking=True)
        self.cmp_block_table[:m].copy_(self.cache.block_table("cmp", slots), non_blocking=True)
        self.n_compressed[:m].copy_(self.cache.n_compressed(slots, pos), non_blocking=True)
        return st

    def _step_struct(self, m):
        return _lib.CsaStep(
            q_raw=self.q_raw.data_ptr(), q_raw_stride=self.q_raw.stride(0), w64=self.w64.data_ptr(),
            win_y2=self.win_y2.data_ptr(), pos=self.pos.data_ptr(), q_pos=self.q_pos.data_ptr(),
            main_state_row=self.main_state_row.data_ptr(), idx_state_row=self.idx_state_row.data_ptr(),
            idx_dst=self.idx_dst.data_ptr(), cmp_dst=self.cmp_dst.data_ptr(), swa_dst=self.swa_dst.data_ptr(),
            idx_block_table=self.block_table.data_ptr(), cmp_block_table=self.cmp_block_table.data_ptr(),
            n_compressed=self.n_compressed.data_ptr(),
            block_table_stride=self.block_table.stride(0), topk=self.topk, logits_stride=self.logits_stride,
            logits=self.logits.data_ptr(), topk_indices=self.topk_indices.data_ptr(), topk_raw=self.topk_raw.data_ptr(),
            q_main_out=self.q_main.data_ptr())

    def launch(self, m):
        """Enqueues the seven kernels of the step for the first m rows of the step buffers."""
        step = self._step_struct(m)
        check(lib.wuda_csa_decode_step(ctypes.byref(self.w.c), ctypes.byref(self._caches), ctypes.byref(step),
                                       ctypes.byref(self._ws), m, torch.cuda.current_stream().cuda_stream))

    def capture(self, m):
        """Captures launch(m) into a CUDA graph after one eager call (kernel attributes are set on
        first use).  The eager call and the capture pass both run the step on the current buffers."""
        self.launch(m)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            self.launch(m)
        self._graph, self._graph_m = graph, m
        return graph

    def replay(self):
        self._graph.replay()

    def check_status(self):
        code = int(self.status.item())
        if code:
            raise _lib.WudaError(5, "device status %d" % code)
