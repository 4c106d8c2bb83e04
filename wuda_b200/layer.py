"""One decode layer as one launch sequence.

AttentionHalfLayer: what the reference's decode_step does between the residual streams going in and coming
out (dsv4_megakernel/megakernel/test/test_e2e_decode.py:475-800), with its CUDA-graph capture (:1347-1358):

    mHC pre -> front mixed GEMM + FRONT-EMIT -> indexer half-step (q norm / quant, merged q projection,
    query tails, cache writers, MQA logits, top-k) -> sparse MLA attention over the window and the top-k
    compressed records -> inverse RoPE + quant, grouped wo_a, quant, wo_b -> mHC post

DecoderLayer: the origin's Block.forward (dsv4_megakernel/origin/model.py:688-700) for one decode token per
request - the attention half above, then the feed-forward half

    mHC pre (ffn weights) + ffn RMSNorm -> router -> routed NVFP4 experts + shared expert -> mHC post

on one GPU or on a pair of tensor-parallel ranks.  On a pair every rank holds half of the query heads (its
columns of the q projection, its groups of wo_a, its K slice of wo_b, whose all-reduce is fused into the GEMM
epilogue over NVLink peer memory), half of the routed experts and half of the shared expert's intermediate
columns (the combine kernel exchanges the partial rows over peer memory); mHC mixes, the front projection,
the indexer and every cache writer are replicated, as in the reference's own two-rank geometry
(test/test_e2e_decode.py:162-167, 1446-1448).  No NCCL call is on the path.

Every stage is a C entry point of the library; these classes own the buffers between them, prepare the
per-step host arrays through the cache manager, and capture the sequence into one CUDA graph.
"""
from dataclasses import dataclass
from typing import Optional

import torch

import ctypes

from . import _lib, moe, o_proj, ops
from ._lib import check, lib
from .decode import CsaDecodeStage

WINDOW = 128


@dataclass
class HalfLayerWeights:
    """Weights of the stages around the indexer half-step (that one's are a decode.CsaWeights)."""
    hc_weight: torch.Tensor      # fp32 [24, 4*hidden]
    hc_base: torch.Tensor        # fp32 [24]
    hc_scale: torch.Tensor       # fp32 [3]
    attn_norm: torch.Tensor      # bf16 [hidden]
    front_w8: torch.Tensor       # e4m3 [2048, hidden]  (q_lora + indexer / compressor rows of the front GEMM)
    front_w8_scales: torch.Tensor
    front_w16: torch.Tensor      # bf16 [2624, hidden]
    ape: torch.Tensor            # fp32 [4, 1024]
    idx_ape: torch.Tensor        # fp32 [4, 256]
    o_proj: o_proj.OProjWeights
    attn_sink: torch.Tensor      # fp32 [heads]


class AttentionHalfLayer:
    def __init__(self, csa_weights, weights, cache, max_batch, topk=2048, softmax_scale=512 ** -0.5, tp_link=None):
        """tp_link (ops.TP2Link): this rank holds half of the heads - csa_weights projects only its main
        heads, weights.o_proj holds its wo_a groups and its K slice of wo_b - and wo_b sums over the pair."""
        self.sm_split = None      # (FP8, BF16) SM shares of the front projection, set by a DecoderLayer that mirrors the C++ call
        self.w, self.cache, self.max_batch, self.topk = weights, cache, max_batch, topk
        self.softmax_scale, self.tp_link = softmax_scale, tp_link
        self.stage = CsaDecodeStage(csa_weights, cache, max_batch, topk=topk)
        self.cos, self.sin = csa_weights.tensors["cos_table"], csa_weights.tensors["sin_table"]
        dev = weights.hc_weight.device
        hidden = weights.attn_norm.numel()
        self.hidden, self.heads = hidden, csa_weights.out_heads
        self.front_out = torch.empty(max_batch, weights.front_w8.size(0), dtype=torch.bfloat16, device=dev)
        self.y16 = torch.empty(max_batch, weights.front_w16.size(0), dtype=torch.float32, device=dev)
        self.mla_out = torch.empty(max_batch, self.heads, 512, dtype=torch.bfloat16, device=dev)
        self.pre_ws = torch.empty(lib.wuda_mhc_pre_workspace_bytes(max_batch, hidden), dtype=torch.uint8, device=dev)
        self.swa_idx = torch.full((max_batch, WINDOW), -1, dtype=torch.int32, device=dev)
        self.swa_len = torch.zeros(max_batch, dtype=torch.int32, device=dev)
        self.cmp_len = torch.zeros(max_batch, dtype=torch.int32, device=dev)
        self.stage.q_raw = self.front_out[:, :csa_weights.q_lora]       # the chain reads the q_lora columns in place
        self.status = self.stage.status
        self.out = None
        self._graph, self._graph_m, self._graph_x = None, 0, None

    def prepare(self, slots):
        """Host side of a step: positions, destinations, page tables, window entries (device copies only)."""
        st = self.stage.prepare(slots)
        m = len(slots)
        pos = st["pos"].tolist()
        idx, lens = self.cache.swa_indices(slots, pos, WINDOW)
        self.swa_idx[:m].copy_(idx.view(m, WINDOW), non_blocking=True)
        self.swa_len[:m].copy_(lens, non_blocking=True)
        self.cmp_len[:m].copy_(torch.clamp(self.stage.n_compressed[:m], max=self.topk), non_blocking=True)
        return st

    def launch(self, hidden_states, m):
        """hidden_states bf16 [m, 4, hidden] -> bf16 [m, 4, hidden]; all launches on the current stream."""
        w, st, cache = self.w, self.stage, self.cache
        pre = ops.mhc_pre(hidden_states, w.hc_weight, w.hc_base, w.hc_scale, w.attn_norm, workspace=self.pre_ws)
        ops.front_mixed_gemm(pre["normed"], pre["xq"], pre["xsf"], w.front_w16, w.front_w8, w.front_w8_scales,
                             self.front_out[:m], pos=st.pos[:m], main_state=cache.main_state, ape=w.ape,
                             main_state_row=st.main_state_row[:m], idx_state=cache.idx_state,
                             idx_state_row=st.idx_state_row[:m], idx_ape=w.idx_ape, win_y2=st.win_y2[:m], w64=st.w64[:m],
                             y16=self.y16[:m], status_word=self.status, sm_split=self.sm_split)
        st.launch(m)
        ops.sparse_mla_decode(st.q_main[:m], cache.model1_cache_view("swa"), self.swa_idx[:m], self.swa_len[:m],
                              cache.model1_cache_view("cmp"), st.topk_indices[:m], self.cmp_len[:m], w.attn_sink,
                              self.softmax_scale, out=self.mla_out[:m], status_word=self.status)
        self.out = o_proj.run_o_proj_mhc_post(self.mla_out[:m], st.pos[:m], self.cos, self.sin, hidden_states, pre["post"],
                                              pre["comb"], w.o_proj, tp_link=self.tp_link, status_word=self.status)
        return self.out

    def capture(self, hidden_states, m):
        """One eager pass (sizes the per-device scratch buffers), then the same pass as a CUDA graph that reads
        `hidden_states` in place; replay() returns the output tensor of the captured pass."""
        self.launch(hidden_states, m)
        torch.cuda.synchronize()
        self.check_status()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            out = self.launch(hidden_states, m)
        self._graph, self._graph_m, self._graph_x, self._graph_out = graph, m, hidden_states, out
        return graph

    def replay(self):
        self._graph.replay()
        return self._graph_out

    def check_status(self):
        self.stage.check_status()


@dataclass
class FfnWeights:
    """Weights of the feed-forward half: the ffn-side mHC mix, ffn_norm, the router and the experts this rank
    holds (origin/model.py:609-627, 661-676)."""
    hc_weight: torch.Tensor      # fp32 [24, 4*hidden]
    hc_base: torch.Tensor        # fp32 [24]
    hc_scale: torch.Tensor       # fp32 [3]
    ffn_norm: torch.Tensor       # bf16 [hidden]
    gate_weight: torch.Tensor    # bf16 [experts_total, hidden]
    gate_bias: Optional[torch.Tensor]   # fp32 [experts_total] or None
    routed: object               # moe.RoutedExperts / RandomRoutedExperts: this rank's experts
    shared: Optional[moe.SharedExpert]  # the shared expert (on a pair: this rank's half of its intermediate columns)
    experts_total: int = 256
    expert_first: int = 0        # index of this rank's first expert
    topk: int = 8
    score_func: str = "sqrtsoftplus"
    route_scale: float = 1.0


class DecoderLayer:
    """Block.forward for one decode token per request: hidden bf16 [m, 4, hidden] -> bf16 [m, 4, hidden].

    native=True (default): the launch sequence is the library's own C++ (wuda_layer_decode: one call per step,
    every intermediate tensor in one workspace).  native=False: the same entry points called one by one from
    Python, each stage's tensors at hand - the form the stage-level tests read.  Both give the same bits."""

    def __init__(self, attention, ffn, max_batch, ep_link=None, peer_wait_ms=2000, native=True):
        self.attn, self.ffn, self.max_batch, self.native = attention, ffn, max_batch, native
        self.ep_link, self.peer_wait_ms = ep_link, peer_wait_ms
        dev = ffn.hc_weight.device
        hidden = ffn.ffn_norm.numel()
        self.hidden = hidden
        self.out = torch.empty(max_batch, 4, hidden, dtype=torch.bfloat16, device=dev)
        self.route_indices = None
        self._graph = None
        if native:
            self._init_native(dev)
        else:
            self.runner = moe.MoERunner(ffn.routed, max_batch, ffn.topk, device=dev, expert_first=ffn.expert_first,
                                        experts_total=ffn.experts_total, link=ep_link, peer_wait_ms=peer_wait_ms)
            self.pre_ws = torch.empty(lib.wuda_mhc_pre_workspace_bytes(max_batch, hidden), dtype=torch.uint8, device=dev)
            self.gate_logits = torch.empty(max_batch, ffn.experts_total, dtype=torch.float32, device=dev)
            self.y = torch.empty(max_batch, hidden, dtype=torch.bfloat16, device=dev)
            # the SM shares the C++ sequence gives the GEMMs it runs side by side (wuda_b200/csrc/layer_decode.cu): with
            # them this Python-sequenced form adds in the same order and is bit-identical to it
            n = lib.wuda_num_sms()
            first = n * 5 // 16
            attention.sm_split = (first, n - first) if first > 8 else (n, n)
            self._shared_sms = n - 32 if n > 64 else n

    # ---- the C++ launch sequence
    def _init_native(self, dev):
        a, f, st = self.attn, self.ffn, self.attn.stage
        hw, routed, shared = a.w, f.routed, f.shared
        if shared is not None and float(shared.limit) != float(routed.swiglu_limit):
            raise ValueError("the shared and the routed experts must use one swiglu_limit")
        p = lambda t: t.data_ptr() if t is not None else None
        w = _lib.LayerWeights()
        w.csa = st.w.c
        w.attn_hc_weight, w.attn_hc_base, w.attn_hc_scale, w.attn_norm = p(hw.hc_weight), p(hw.hc_base), p(hw.hc_scale), p(hw.attn_norm)
        w.front_w8, w.front_w8_scales, w.front_w16 = p(hw.front_w8), p(hw.front_w8_scales), p(hw.front_w16)
        w.ape, w.idx_ape = p(hw.ape), p(hw.idx_ape)
        w.wo_a, w.wo_a_scales, w.wo_b, w.wo_b_scales = p(hw.o_proj.wo_a), p(hw.o_proj.wo_a_scale), p(hw.o_proj.wo_b), p(hw.o_proj.wo_b_scale)
        w.attn_sink = p(hw.attn_sink)
        w.ffn_hc_weight, w.ffn_hc_base, w.ffn_hc_scale, w.ffn_norm = p(f.hc_weight), p(f.hc_base), p(f.hc_scale), p(f.ffn_norm)
        w.gate_weight, w.gate_bias = p(f.gate_weight), p(f.gate_bias)
        d = routed.dev
        w.w13, w.w13_sf, w.w13_gs, w.w2, w.w2_sf, w.w2_gs = (p(d[k]) for k in ("w13", "w13_sf", "w13_gs", "w2", "w2_sf", "w2_gs"))
        if shared is not None:
            w.shared_w13, w.shared_w13_scales, w.shared_w2, w.shared_w2_scales = p(shared.w13), p(shared.w13_scale), p(shared.w2), p(shared.w2_scale)
            w.shared_inter = shared.inter
        w.hidden, w.o_groups = self.hidden, hw.o_proj.wo_a.size(0)
        w.experts_total, w.expert_first, w.experts_local = f.experts_total, f.expert_first, routed.experts
        w.moe_topk, w.score_func, w.inter = f.topk, ops.SCORE_FUNCS[f.score_func], routed.inter
        w.route_scale, w.swiglu_limit = float(f.route_scale), float(routed.swiglu_limit)
        w.act_scale_in, w.act_scale_mid = float(routed.act_scale_in), float(routed.act_scale_mid)
        w.softmax_scale = float(a.softmax_scale)
        w.hc_eps = w.rms_eps = w.norm_eps = 1e-6
        w.fp8_scales_pow2 = int(bool(hw.o_proj.scales_pow2))
        self._w = w
        self._geometry = (self.max_batch, a.topk, st.logits_stride, a.swa_idx.size(1))
        need = lib.wuda_layer_workspace_bytes(ctypes.byref(w), *self._geometry)
        if need <= 0:
            raise ValueError("wuda_layer_workspace_bytes refused the layer geometry")
        self.workspace = torch.zeros(need, dtype=torch.uint8, device=dev)
        s = _lib.LayerState()
        s.caches = st._caches
        s.workspace, s.workspace_bytes = self.workspace.data_ptr(), need
        if a.tp_link is not None:
            if not a.tp_link.device_sequence:
                raise ValueError("the tensor-parallel link must number its calls on the device (device_sequence=True)")
            s.tp_my_inbox, s.tp_peer_inbox = a.tp_link._local, a.tp_link._peer
        if self.ep_link is not None:
            if not self.ep_link.device_sequence:
                raise ValueError("the expert-parallel link must number its calls on the device (device_sequence=True)")
            s.ep_my_inbox, s.ep_peer_inbox, s.ep_tokens_max = self.ep_link._local, self.ep_link._peer, self.ep_link.max_tokens
        s.peer_wait_ms, s.m_max, s.status_word = int(self.peer_wait_ms), self.max_batch, st.status.data_ptr()
        self._s = s

    def view(self, name, dtype, *shape):
        """A stage's result inside the workspace of the native form (names: wuda_layer_workspace_offset)."""
        off = lib.wuda_layer_workspace_offset(ctypes.byref(self._w), *self._geometry, name.encode())
        if off < 0:
            raise KeyError(name)
        n = 1
        for d in shape:
            n *= d
        return self.workspace[off:off + n * torch.empty(0, dtype=dtype).element_size()].view(dtype).view(*shape)

    def _launch_native(self, hidden_states, m):
        a, st = self.attn, self.attn.stage
        if not (hidden_states.is_cuda and hidden_states.is_contiguous() and hidden_states.dtype == torch.bfloat16
                and tuple(hidden_states.shape) == (m, 4, self.hidden)):
            raise ValueError("hidden_states must be contiguous CUDA bf16 [m, 4, hidden]")
        t = _lib.LayerStep(
            hidden_in=hidden_states.data_ptr(), hidden_out=self.out.data_ptr(), pos=st.pos.data_ptr(), q_pos=st.q_pos.data_ptr(),
            main_state_row=st.main_state_row.data_ptr(), idx_state_row=st.idx_state_row.data_ptr(), idx_dst=st.idx_dst.data_ptr(),
            cmp_dst=st.cmp_dst.data_ptr(), swa_dst=st.swa_dst.data_ptr(), idx_block_table=st.block_table.data_ptr(),
            cmp_block_table=st.cmp_block_table.data_ptr(), n_compressed=st.n_compressed.data_ptr(),
            swa_indices=a.swa_idx.data_ptr(), swa_lengths=a.swa_len.data_ptr(), cmp_lengths=a.cmp_len.data_ptr(),
            block_table_stride=st.block_table.stride(0), topk=a.topk, window=a.swa_idx.size(1), logits_stride=st.logits_stride)
        check(lib.wuda_layer_decode(ctypes.byref(self._w), ctypes.byref(self._s), ctypes.byref(t), m,
                                    torch.cuda.current_stream().cuda_stream))
        self.route_indices = self.view("route_indices", torch.int32, self.max_batch, self.ffn.topk)[:m]
        return self.out[:m]

    def prepare(self, slots):
        return self.attn.prepare(slots)

    def launch_ffn(self, x, m):
        """The feed-forward half on the residual streams x bf16 [m, 4, hidden] (Python-sequenced form)."""
        f = self.ffn
        pre = ops.mhc_pre(x, f.hc_weight, f.hc_base, f.hc_scale, f.ffn_norm, quant=False, workspace=self.pre_ws)
        normed = pre["normed"]
        rw, idx = ops.moe_gate(normed, f.gate_weight, f.gate_bias, f.score_func, f.route_scale, f.topk,
                               logits=self.gate_logits[:m])
        self.route_indices = idx
        shared = None
        if f.shared is not None:   # on the SM share wuda_layer_decode gives the shared expert beside the router
            lib.wuda_gemm_sm_limit(self._shared_sms)
            try:
                shared = f.shared.forward(normed)
            finally:
                lib.wuda_gemm_sm_limit(0)
        y = self.runner.forward(normed, rw, idx, shared=shared, y=self.y[:m])
        return ops.mhc_post_out(y, x, pre["post"], pre["comb"], self.out[:m])

    def launch(self, hidden_states, m):
        if self.native:
            return self._launch_native(hidden_states, m)
        return self.launch_ffn(self.attn.launch(hidden_states, m), m)

    def capture(self, hidden_states, m):
        """One eager pass, then the same pass as a CUDA graph reading `hidden_states` in place.  On a pair of
        ranks both must call this (and later replay()) the same number of times: the exchange steps number
        their calls on the device."""
        self.launch(hidden_states, m)
        torch.cuda.synchronize()
        self.check_status()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            out = self.launch(hidden_states, m)
        self._graph, self._graph_out = graph, out
        return graph

    def replay(self):
        self._graph.replay()
        return self._graph_out

    def check_status(self):
        self.attn.check_status()
        if not self.native:
            code = int(self.runner.status.item())
            if code:
                raise _lib.WudaError(5, "device status %d in the MoE block" % code)
