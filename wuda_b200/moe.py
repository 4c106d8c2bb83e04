"""Host-side driver of the routed experts of the MoE block (the origin's MoE / Expert modules,
dsv4_megakernel/origin/model.py:587-644): routing -> dispatch -> NVFP4 quantisation of the gathered
rows -> grouped w1|w3 GEMM -> SwiGLU + quantisation -> grouped w2 GEMM -> combine.  Every buffer is
allocated once; a forward pass is eight launches with no host synchronisation in between (the number
of row groups stays on the device), so it can be captured into a CUDA graph.
"""
import numpy as np
import ctypes

import torch

from . import ops, workloads
from ._lib import check, lib


class RoutedExperts:
    """NVFP4 weights of `experts` SwiGLU experts: w13 = [w1; w3] stacked ([2*inter, dim]) and w2
    ([dim, inter]) per expert, quantised here from fp32/bf16 tensors (set-up, not the hot path)."""

    def __init__(self, w1, w3, w2, act_scale_in, act_scale_mid, swiglu_limit=0.0, device="cuda"):
        experts, inter, dim = w1.shape
        if w3.shape != w1.shape or tuple(w2.shape) != (experts, dim, inter) or dim % 256 or inter % 256:
            raise ValueError("w1, w3 must be [E, inter, dim], w2 [E, dim, inter], dims multiples of 256")
        self.experts, self.inter, self.dim = experts, inter, dim
        self.act_scale_in, self.act_scale_mid, self.swiglu_limit = float(act_scale_in), float(act_scale_mid), float(swiglu_limit)
        q13, s13, g13, q2, s2, g2, raw13, raw2 = [], [], [], [], [], [], [], []
        for e in range(experts):
            q, sf, gs = workloads.quantize_nvfp4(torch.cat([w1[e], w3[e]]).float())
            q13.append(q), s13.append(workloads.pack_nvfp4_scales(sf)), g13.append(gs), raw13.append(sf)
            q, sf, gs = workloads.quantize_nvfp4(w2[e].float())
            q2.append(q), s2.append(workloads.pack_nvfp4_scales(sf)), g2.append(gs), raw2.append(sf)
        self.host = dict(w13=np.stack(q13), w13_sf=np.stack(s13), w13_gs=np.array(g13, np.float32), w2=np.stack(q2),
                         w2_sf=np.stack(s2), w2_gs=np.array(g2, np.float32))
        self.raw_scales = dict(w13=raw13, w2=raw2)          # unpacked scale bytes, kept for checks on the host
        self.dev = {k: torch.from_numpy(v).to(device) for k, v in self.host.items()}


class RandomRoutedExperts:
    """Random NVFP4 expert weights created on the device (benchmarks): packed e2m1 codes, ue4m3 scale
    bytes in a sane range, unit tensor scales.  Same attributes as RoutedExperts minus the host copies."""

    def __init__(self, experts, inter, dim, act_scale_in=1.0 / 448, act_scale_mid=1.0 / 448, swiglu_limit=0.0,
                 device="cuda", seed=1):
        self.experts, self.inter, self.dim = experts, inter, dim
        self.act_scale_in, self.act_scale_mid, self.swiglu_limit = act_scale_in, act_scale_mid, swiglu_limit
        g = torch.Generator(device=device).manual_seed(seed)
        rnd = lambda *s, hi=256: torch.randint(0, hi, s, generator=g, dtype=torch.uint8, device=device)
        self.dev = dict(
            w13=rnd(experts, 2 * inter, dim // 2), w13_sf=rnd(experts, (2 * inter // 128) * (dim // 256) * 2048, hi=0x30),
            w13_gs=torch.full((experts,), 1e-3, device=device),
            w2=rnd(experts, dim, inter // 2), w2_sf=rnd(experts, (dim // 128) * (inter // 256) * 2048, hi=0x30),
            w2_gs=torch.full((experts,), 1e-3, device=device))


class EP2Link:
    """Exchange buffers of two expert-parallel ranks for the combine step of the routed experts
    (the all-reduce site of MoE.forward, origin/model.py:641-642): each rank's inbox receives the peer's
    fp32 partial rows over NVLink peer memory.  Created like ops.TP2Link (the IPC handles travel over
    torch.distributed once); `loopback=True` makes the rank its own peer (one GPU: y = local + local),
    `mute=True` gives a peer that never answers (time-out path)."""

    def __init__(self, max_tokens, dim, group=None, peer_handle=None, loopback=False, mute=False, device_sequence=False):
        self.max_tokens, self.dim, self.device_sequence = max_tokens, dim, device_sequence
        self.nbytes = lib.wuda_moe_ep2_inbox_bytes(max_tokens, dim)
        if self.nbytes <= 0:
            raise ValueError("unsupported (max_tokens, dim) for the exchange buffer")
        self._local, self._peer, self._mute = ctypes.c_void_p(), ctypes.c_void_p(), None
        handle = (ctypes.c_ubyte * 64)()
        check(lib.wuda_tp2_alloc(self.nbytes, ctypes.byref(self._local), handle))
        self.handle, self.epoch, self._own_peer = bytes(handle), 0, False
        if mute:
            self._mute = ctypes.c_void_p()
            check(lib.wuda_tp2_alloc(self.nbytes, ctypes.byref(self._mute), (ctypes.c_ubyte * 64)()))
            self._peer = self._mute
        elif loopback:
            self._peer = self._local
        else:
            if peer_handle is None:
                peer_handle = ops.exchange_handles(self.handle, group)
            check(lib.wuda_tp2_open((ctypes.c_ubyte * 64).from_buffer_copy(peer_handle), ctypes.byref(self._peer)))
            self._own_peer = True

    def close(self):
        if self._own_peer and self._peer:
            lib.wuda_tp2_close(self._peer)
        self._peer, self._own_peer = None, False
        if self._mute:
            lib.wuda_tp2_free(self._mute)
            self._mute = None
        if self._local:
            lib.wuda_tp2_free(self._local)
            self._local = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class MoERunner:
    """Routed experts of one rank.  With expert parallelism the rank holds experts
    [expert_first, expert_first + weights.experts) of experts_total and `link` joins it to its peer."""

    def __init__(self, weights, max_tokens, topk, device="cuda", expert_first=0, experts_total=None, link=None,
                 peer_wait_ms=2000):
        self.w, self.max_tokens, self.topk = weights, max_tokens, topk
        self.expert_first, self.experts_total = expert_first, experts_total or weights.experts
        self.link, self.peer_wait_ms = link, peer_wait_ms
        self.max_groups = lib.wuda_moe_max_groups(max_tokens, topk, weights.experts)
        rows = self.max_groups * 16
        dev = device
        z = lambda *s, dtype=torch.uint8: torch.zeros(*s, dtype=dtype, device=dev)
        self.group_expert, self.num_groups = z(self.max_groups, dtype=torch.int32), z(1, dtype=torch.int32)
        self.row_token, self.row_weight = z(rows, dtype=torch.int32), z(rows, dtype=torch.float32)
        self.pair_row = z(max_tokens, topk, dtype=torch.int32)
        self.a1, self.a1_sf = z(rows, weights.dim // 2), z(self.max_groups, weights.dim // 256, 2048)
        self.h = z(rows, 2 * weights.inter, dtype=torch.bfloat16)
        self.a2, self.a2_sf = z(rows, weights.inter // 2), z(self.max_groups, weights.inter // 256, 2048)
        self.out = z(rows, weights.dim, dtype=torch.bfloat16)
        need = max(lib.wuda_gemm_nvfp4_scratch_bytes(16, 2 * weights.inter), lib.wuda_gemm_nvfp4_scratch_bytes(16, weights.dim))
        self.scratch = z(need)
        self.status = z(1, dtype=torch.int32)

    def forward(self, x, weights, indices, shared=None, y=None):
        """x bf16 [M, dim]; routing weights fp32 [M, k] and indices int32 [M, k] (ops.moe_gate);
        shared bf16 [M, dim] or None.  Returns y bf16 [M, dim]."""
        w, m = self.w, x.size(0)
        if m > self.max_tokens or indices.shape != (m, self.topk):
            raise ValueError("batch does not fit this runner")
        s = torch.cuda.current_stream().cuda_stream
        st = self.status.data_ptr()
        check(lib.wuda_moe_dispatch_range(indices.data_ptr(), weights.data_ptr(), self.group_expert.data_ptr(),
                                          self.num_groups.data_ptr(), self.row_token.data_ptr(), self.row_weight.data_ptr(),
                                          self.pair_row.data_ptr(), m, self.topk, w.experts, self.expert_first,
                                          self.experts_total, self.max_groups, st, s))
        check(lib.wuda_moe_gather_quant_nvfp4(x.data_ptr(), self.pair_row.data_ptr(), self.a1.data_ptr(), self.a1_sf.data_ptr(),
                                              w.act_scale_in, m, self.topk, w.dim, s))
        d = w.dev
        check(lib.wuda_gemm_nvfp4_grouped(self.a1.data_ptr(), self.a1_sf.data_ptr(), w.act_scale_in, d["w13"].data_ptr(),
                                          d["w13_sf"].data_ptr(), d["w13_gs"].data_ptr(), self.group_expert.data_ptr(),
                                          self.num_groups.data_ptr(), self.row_token.data_ptr(), self.h.data_ptr(), self.max_groups, w.experts,
                                          2 * w.inter, w.dim, self.scratch.data_ptr(), self.scratch.numel(), st, s))
        check(lib.wuda_moe_swiglu_quant_nvfp4(self.h.data_ptr(), self.pair_row.data_ptr(), weights.data_ptr(), self.a2.data_ptr(),
                                              self.a2_sf.data_ptr(), w.act_scale_mid, w.swiglu_limit, m, self.topk, w.inter, s))
        check(lib.wuda_gemm_nvfp4_grouped(self.a2.data_ptr(), self.a2_sf.data_ptr(), w.act_scale_mid, d["w2"].data_ptr(),
                                          d["w2_sf"].data_ptr(), d["w2_gs"].data_ptr(), self.group_expert.data_ptr(),
                                          self.num_groups.data_ptr(), self.row_token.data_ptr(), self.out.data_ptr(), self.max_groups, w.experts,
                                          w.dim, w.inter, self.scratch.data_ptr(), self.scratch.numel(), st, s))
        if y is None:
            y = torch.empty(m, w.dim, dtype=torch.bfloat16, device=x.device)
        shared_ptr = shared.data_ptr() if shared is not None else None
        if self.link is None:
            check(lib.wuda_moe_combine(self.out.data_ptr(), self.pair_row.data_ptr(), shared_ptr, y.data_ptr(), m, self.topk,
                                       w.dim, s))
        else:
            self.link.epoch += 1
            check(lib.wuda_moe_combine_ep2(self.out.data_ptr(), self.pair_row.data_ptr(), shared_ptr, y.data_ptr(), m,
                                           self.topk, w.dim, self.link._local, self.link._peer, self.link.max_tokens,
                                           0 if self.link.device_sequence else self.link.epoch, int(self.peer_wait_ms), st, s))
        return y


class SharedExpert:
    """The dense shared expert (Expert.forward, origin/model.py:587-606) on FP8 weights: w13 = [w1; w3]
    e4m3 [2*inter, dim] and w2 e4m3 [dim, inter] with fp32 128x128 block scales."""

    def __init__(self, w13, w13_scale, w2, w2_scale, swiglu_limit=0.0):
        self.w13, self.w13_scale, self.w2, self.w2_scale, self.limit = w13, w13_scale, w2, w2_scale, float(swiglu_limit)
        self.inter = w2.size(1)

    def forward(self, x):
        """x bf16 [M, dim] -> bf16 [M, dim]: quantise, w1|w3 GEMM, SwiGLU + quantise, w2 GEMM (four launches)."""
        x8, xs = ops.act_quant(x, 128, "ue8m0")
        h = ops.fp8_gemm(x8, xs, self.w13, self.w13_scale)
        m = x.size(0)
        a8 = torch.empty(m, self.inter, dtype=torch.float8_e4m3fn, device=x.device)
        a_s = torch.empty(m, self.inter // 128, dtype=torch.float32, device=x.device)
        check(lib.wuda_swiglu_quant_fp8(h.data_ptr(), None, a8.data_ptr(), a_s.data_ptr(), m, self.inter, self.limit, 1,
                                        torch.cuda.current_stream().cuda_stream))
        return ops.fp8_gemm(a8, a_s, self.w2, self.w2_scale)


def moe_block(x, gate_weight, gate_bias, routed, shared, score_func="sqrtsoftplus", route_scale=1.0):
    """One MoE block of the origin (MoE.forward, origin/model.py:620-644) on one rank: router, routed
    NVFP4 experts (a MoERunner), dense shared expert (a SharedExpert or None), sum in bf16."""
    w, idx = ops.moe_gate(x, gate_weight, gate_bias, score_func, route_scale, routed.topk)
    return routed.forward(x, w, idx, shared=shared.forward(x) if shared is not None else None)
