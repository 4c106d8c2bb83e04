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

from . import moe, o_proj, ops
from ._lib import lib
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
                             y16=self.y16[:m], status_word=self.status)
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
    """Block.forward for one decode token per request: hidden bf16 [m, 4, hidden] -> bf16 [m, 4, hidden]."""

    def __init__(self, attention, ffn, max_batch, ep_link=None, peer_wait_ms=2000):
        self.attn, self.ffn, self.max_batch = attention, ffn, max_batch
        dev = ffn.hc_weight.device
        hidden = ffn.ffn_norm.numel()
        self.hidden = hidden
        self.runner = moe.MoERunner(ffn.routed, max_batch, ffn.topk, device=dev, expert_first=ffn.expert_first,
                                    experts_total=ffn.experts_total, link=ep_link, peer_wait_ms=peer_wait_ms)
        self.pre_ws = torch.empty(lib.wuda_mhc_pre_workspace_bytes(max_batch, hidden), dtype=torch.uint8, device=dev)
        self.gate_logits = torch.empty(max_batch, ffn.experts_total, dtype=torch.float32, device=dev)
        self.y = torch.empty(max_batch, hidden, dtype=torch.bfloat16, device=dev)
        self.out = torch.empty(max_batch, 4, hidden, dtype=torch.bfloat16, device=dev)
        self.route_indices = None
        self._graph = None

    def prepare(self, slots):
        return self.attn.prepare(slots)

    def launch_ffn(self, x, m):
        """The feed-forward half on the residual streams x bf16 [m, 4, hidden]."""
        f = self.ffn
        pre = ops.mhc_pre(x, f.hc_weight, f.hc_base, f.hc_scale, f.ffn_norm, quant=False, workspace=self.pre_ws)
        normed = pre["normed"]
        rw, idx = ops.moe_gate(normed, f.gate_weight, f.gate_bias, f.score_func, f.route_scale, f.topk,
                               logits=self.gate_logits[:m])
        self.route_indices = idx
        shared = f.shared.forward(normed) if f.shared is not None else None
        y = self.runner.forward(normed, rw, idx, shared=shared, y=self.y[:m])
        return ops.mhc_post_out(y, x, pre["post"], pre["comb"], self.out[:m])

    def launch(self, hidden_states, m):
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
        code = int(self.runner.status.item())
        if code:
            from ._lib import WudaError
            raise WudaError(5, "device status %d in the MoE block" % code)
