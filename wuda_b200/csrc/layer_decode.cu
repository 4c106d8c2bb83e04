// The whole decode layer as one C call: the launch sequence of the origin's Block.forward
// (dsv4_megakernel/origin/model.py:688-700) for one token per request, i.e. what the reference's
// decode_step (dsv4_megakernel/megakernel/test/test_e2e_decode.py:475-800) does for the attention half,
// followed by the feed-forward half the reference's megakernel does not have:
//
//   mHC pre (attention weights) + attention RMSNorm + FP8 quantisation
//   front projection (FP8 segment, BF16 segment) + FRONT-EMIT scatter into the state rings
//   indexer half-step (wuda_csa_decode_step: q norm / quant, merged q projection, query tails, cache
//       writers, paged MQA logits, top-k)
//   sparse MLA attention over the window and the selected compressed records
//   inverse RoPE + quantisation, grouped wo_a, quantisation, wo_b (on a pair: K-split with the all-reduce
//       fused into the epilogue over peer memory), mHC post
//   mHC pre (ffn weights) + ffn RMSNorm, router projection + routing
//   shared expert (quantise, w1|w3, SwiGLU + quantise, w2), routed NVFP4 experts (dispatch, gather +
//       quantise, grouped w1|w3, SwiGLU + quantise, grouped w2), combine (on a pair: with the exchange of
//       partial rows over peer memory), mHC post
//
// Host code only: every stage is one of the library's own entry points, called in order on the caller's
// stream (two stretches of independent work on a side stream forked from it and joined back, see Side below);
// nothing is allocated and nothing synchronises, so the call can be captured into a CUDA graph.
// All intermediate tensors live in one caller-provided workspace that this file lays out.
#include <cuda_runtime.h>

#include <cstdint>

#include "host.h"

namespace wuda {
namespace layer {

constexpr int kHeadDim = 512, kRopeDim = 64, kORank = 1024, kFront8 = 2048, kFront16 = 2624;

// Bump allocator over the workspace; with base == nullptr it only measures.
struct Carver {
    uint8_t* base;
    int64_t used = 0;
    explicit Carver(void* b) : base(static_cast<uint8_t*>(b)) {}
    template <typename T>
    T* take(int64_t count) {
        const int64_t at = used;
        used += (count * static_cast<int64_t>(sizeof(T)) + 255) / 256 * 256;
        return base ? reinterpret_cast<T*>(base + at) : nullptr;
    }
};

struct Buffers {
    // attention half
    uint8_t* pre_ws;
    float *a_pre, *a_post, *a_comb;
    uint16_t *a_normed;
    uint8_t* a_xq;
    float* a_xsf;
    uint16_t* front_out;
    float* y16;
    float *w64, *win_y2;
    uint8_t* q_fp8;
    float* q_scales;
    uint16_t* y;
    uint8_t* iq_fp8;
    float* w_folded;
    float* logits;
    int32_t *topk_indices, *topk_raw;
    uint16_t *q_main, *mla_out;
    uint8_t* mla_ws;
    int64_t mla_ws_bytes;
    uint8_t* o_fp8;
    float* o_scale;
    uint16_t* z;
    uint8_t* z_fp8;
    float* z_scale;
    uint16_t *projected, *attn_out;
    // feed-forward half
    float *f_pre, *f_post, *f_comb;
    uint16_t* f_normed;
    float* gate_logits;
    float* route_w;
    int32_t* route_idx;
    uint8_t* s_x8;
    float* s_xs;
    uint16_t* s_h;
    uint8_t* s_a8;
    float* s_as;
    uint16_t* s_out;
    int32_t *group_expert, *num_groups, *row_token, *pair_row;
    float* row_weight;
    uint8_t *a1, *a1_sf, *a2, *a2_sf;
    uint16_t *h, *r_out, *y_moe;
    uint8_t *gemm_scratch, *side_scratch, *nvfp4_scratch;
    int64_t gemm_scratch_bytes, nvfp4_scratch_bytes;
    int max_groups;
};

int64_t max64(int64_t a, int64_t b) { return a > b ? a : b; }

// Two places of the layer hold independent work whose GEMMs are bound by their fixed latencies (15-40 MB of
// weights each): the FP8 and the BF16 segment of the front projection, and the shared expert beside router
// projection / routing / dispatch / gather.  Each pair runs side by side - one part on a side stream forked from
// the caller's and joined back (under stream capture: parallel branches of the graph) - with the GEMMs kept to
// disjoint shares of the SMs (wuda_gemm_sm_limit); a GEMM launched on every SM would leave no room beside it.
// Stream and events are created once per device and never destroyed.
struct Side {
    bool ready = false;
    cudaStream_t stream = nullptr;
    cudaEvent_t fork[2] = {nullptr, nullptr}, done[2] = {nullptr, nullptr};
};

int side_of_current_device(Side** out) {
    static Side sides[16];
    int dev = 0;
    WUDA_CUDA(cudaGetDevice(&dev));
    WUDA_REQUIRE(dev >= 0 && dev < 16, "device ordinal %d is outside the 16 this library keeps state for", dev);
    Side& s = sides[dev];
    if (!s.ready) {
        WUDA_CUDA(cudaStreamCreateWithFlags(&s.stream, cudaStreamNonBlocking));
        for (cudaEvent_t* e : {&s.fork[0], &s.fork[1], &s.done[0], &s.done[1]})
            WUDA_CUDA(cudaEventCreateWithFlags(e, cudaEventDisableTiming));
        s.ready = true;
    }
    *out = &s;
    return WUDA_OK;
}

// SM shares (of the device's n): FP8 front segment 5/16 (its weights are 14.7 MB against the BF16 segment's
// 37.6 MB), BF16 segment the rest; the shared expert all but 32, which the router's small kernels keep.
int front8_sms(int n) { return n * 5 / 16 > 8 ? n * 5 / 16 : n; }
int front16_sms(int n) { return n * 5 / 16 > 8 ? n - n * 5 / 16 : n; }
int shared_sms(int n) { return n > 64 ? n - 32 : n; }

// Lays the buffers out for up to m rows; returns the bytes used, or -1 for a geometry an entry point refuses.
int64_t carve(const wuda_layer_weights* w, int m, int topk, int64_t logits_stride, int window, void* base, Buffers* b) {
    Carver c(base);
    const int hidden = w->hidden, heads = w->csa.out_heads;
    const int64_t pre_bytes = wuda_mhc_pre_workspace_bytes(m, hidden);
    if (pre_bytes < 0) return -1;
    b->pre_ws = c.take<uint8_t>(pre_bytes);
    b->a_pre = c.take<float>(m * 4), b->a_post = c.take<float>(m * 4), b->a_comb = c.take<float>(m * 16);
    b->a_normed = c.take<uint16_t>(static_cast<int64_t>(m) * hidden);
    b->a_xq = c.take<uint8_t>(static_cast<int64_t>(m) * hidden);
    b->a_xsf = c.take<float>(static_cast<int64_t>(m) * (hidden / 128));
    b->front_out = c.take<uint16_t>(static_cast<int64_t>(m) * kFront8);
    b->y16 = c.take<float>(static_cast<int64_t>(m) * kFront16);
    b->w64 = c.take<float>(static_cast<int64_t>(m) * w->csa.index_heads);
    b->win_y2 = c.take<float>(static_cast<int64_t>(m) * 512);
    const int n_q = w->csa.index_heads * 128 + w->csa.main_heads * kHeadDim;
    b->q_fp8 = c.take<uint8_t>(static_cast<int64_t>(m) * w->csa.q_lora);
    b->q_scales = c.take<float>(static_cast<int64_t>(m) * (w->csa.q_lora / 128));
    b->y = c.take<uint16_t>(static_cast<int64_t>(m) * n_q);
    b->iq_fp8 = c.take<uint8_t>(static_cast<int64_t>(m) * w->csa.index_heads * 128);
    b->w_folded = c.take<float>(static_cast<int64_t>(m) * w->csa.index_heads);
    b->logits = c.take<float>(static_cast<int64_t>(m) * logits_stride);
    b->topk_indices = c.take<int32_t>(static_cast<int64_t>(m) * topk);
    b->topk_raw = c.take<int32_t>(static_cast<int64_t>(m) * topk);
    b->q_main = c.take<uint16_t>(static_cast<int64_t>(m) * heads * kHeadDim);
    b->mla_out = c.take<uint16_t>(static_cast<int64_t>(m) * heads * kHeadDim);
    b->mla_ws_bytes = wuda_sparse_mla_workspace_bytes(m, heads, window + topk);
    if (b->mla_ws_bytes < 0) return -1;
    // a smaller batch is split over more CTAs and needs more room: size for the worst of 1..m requests
    for (int mm = 1; mm < m; mm *= 2) b->mla_ws_bytes = max64(b->mla_ws_bytes, wuda_sparse_mla_workspace_bytes(mm, heads, window + topk));
    b->mla_ws = c.take<uint8_t>(b->mla_ws_bytes);
    const int64_t o_width = static_cast<int64_t>(heads) * kHeadDim, z_width = static_cast<int64_t>(w->o_groups) * kORank;
    b->o_fp8 = c.take<uint8_t>(m * o_width);
    b->o_scale = c.take<float>(m * (o_width / 128));
    b->z = c.take<uint16_t>(m * z_width);
    b->z_fp8 = c.take<uint8_t>(m * z_width);
    b->z_scale = c.take<float>(m * (z_width / 128));
    b->projected = c.take<uint16_t>(static_cast<int64_t>(m) * hidden);
    b->attn_out = c.take<uint16_t>(static_cast<int64_t>(m) * 4 * hidden);
    b->f_pre = c.take<float>(m * 4), b->f_post = c.take<float>(m * 4), b->f_comb = c.take<float>(m * 16);
    b->f_normed = c.take<uint16_t>(static_cast<int64_t>(m) * hidden);
    b->gate_logits = c.take<float>(static_cast<int64_t>(m) * w->experts_total);
    b->route_w = c.take<float>(static_cast<int64_t>(m) * w->moe_topk);
    b->route_idx = c.take<int32_t>(static_cast<int64_t>(m) * w->moe_topk);
    const int si = w->shared_inter;
    b->s_x8 = c.take<uint8_t>(static_cast<int64_t>(m) * hidden);
    b->s_xs = c.take<float>(static_cast<int64_t>(m) * (hidden / 128));
    b->s_h = c.take<uint16_t>(static_cast<int64_t>(m) * 2 * si);
    b->s_a8 = c.take<uint8_t>(static_cast<int64_t>(m) * si);
    b->s_as = c.take<float>(static_cast<int64_t>(m) * (si > 0 ? si / 128 : 0));
    b->s_out = c.take<uint16_t>(static_cast<int64_t>(m) * hidden);
    b->max_groups = wuda_moe_max_groups(m, w->moe_topk, w->experts_local);
    if (b->max_groups < 1) return -1;
    const int64_t rows = static_cast<int64_t>(b->max_groups) * 16;
    b->group_expert = c.take<int32_t>(b->max_groups);
    b->num_groups = c.take<int32_t>(1);
    b->row_token = c.take<int32_t>(rows);
    b->row_weight = c.take<float>(rows);
    b->pair_row = c.take<int32_t>(static_cast<int64_t>(m) * w->moe_topk);
    b->a1 = c.take<uint8_t>(rows * (hidden / 2));
    b->a1_sf = c.take<uint8_t>(static_cast<int64_t>(b->max_groups) * (hidden / 256) * 2048);
    b->h = c.take<uint16_t>(rows * 2 * w->inter);
    b->a2 = c.take<uint8_t>(rows * (w->inter / 2));
    b->a2_sf = c.take<uint8_t>(static_cast<int64_t>(b->max_groups) * (w->inter / 256) * 2048);
    b->r_out = c.take<uint16_t>(rows * hidden);
    b->y_moe = c.take<uint16_t>(static_cast<int64_t>(m) * hidden);
    // one scratch for every FP8 / BF16 GEMM of the stream (their flags share one place), one for the grouped NVFP4 pair
    int64_t need = wuda_gemm_fp8_scratch_bytes(m, 128);
    need = max64(need, wuda_gemm_bf16_scratch_bytes(m, 128));
    if (need < 0) return -1;
    b->gemm_scratch_bytes = need;
    b->gemm_scratch = c.take<uint8_t>(need);
    b->side_scratch = c.take<uint8_t>(need);   // for the GEMMs that run beside others on the side stream
    b->nvfp4_scratch_bytes = wuda_gemm_nvfp4_scratch_bytes(16, 128);
    b->nvfp4_scratch = c.take<uint8_t>(b->nvfp4_scratch_bytes);
    return c.used;
}

}  // namespace layer
}  // namespace wuda

extern "C" int64_t wuda_layer_workspace_bytes(const wuda_layer_weights* w, int m_max, int topk, int64_t logits_stride,
                                              int window) {
    if (!w || m_max < 1 || m_max > 128 || topk < 1 || logits_stride < 1 || window < 0) return -1;
    wuda::layer::Buffers b;
    return wuda::layer::carve(w, m_max, topk, logits_stride, window, nullptr, &b);
}

#define WUDA_STAGE(call)                 \
    do {                                 \
        const int st__ = (call);         \
        if (st__ != WUDA_OK) return st__; \
    } while (0)

extern "C" int wuda_layer_decode(const wuda_layer_weights* w, const wuda_layer_state* s, const wuda_layer_step* t, int m,
                                 void* stream) {
    using namespace wuda;
    using namespace wuda::layer;
    clear_error();
    WUDA_REQUIRE(w && s && t, "weights, state and step must not be NULL");
    WUDA_REQUIRE(m >= 1 && m <= s->m_max && s->m_max <= 128, "m must be in [1, m_max] and m_max <= 128 (got %d, %d)", m, s->m_max);
    WUDA_REQUIRE(w->hidden % 128 == 0 && w->o_groups >= 1 && w->csa.out_heads % w->o_groups == 0,
                 "hidden must be a multiple of 128 and the heads a multiple of the output groups");
    WUDA_REQUIRE(t->hidden_in && t->hidden_out && t->hidden_in != t->hidden_out, "hidden_in and hidden_out are required and distinct");
    WUDA_REQUIRE((s->tp_my_inbox == nullptr) == (s->tp_peer_inbox == nullptr) && (s->ep_my_inbox == nullptr) == (s->ep_peer_inbox == nullptr),
                 "an exchange needs both inboxes");
    WUDA_REQUIRE(s->workspace && (reinterpret_cast<uintptr_t>(s->workspace) & 255u) == 0, "workspace must be 256-byte aligned");
    Buffers b;
    // the layout depends on m_max only, so that a smaller step finds every buffer where a captured graph expects it
    const int64_t need = carve(w, s->m_max, t->topk, t->logits_stride, t->window, s->workspace, &b);
    WUDA_REQUIRE(need >= 0, "unsupported layer geometry");
    WUDA_REQUIRE(s->workspace_bytes >= need, "workspace holds %lld bytes; %lld are needed (wuda_layer_workspace_bytes)",
                 static_cast<long long>(s->workspace_bytes), static_cast<long long>(need));
    const int hidden = w->hidden, heads = w->csa.out_heads;
    int32_t* status = s->status_word;
    const wuda_csa_caches& c = s->caches;

    // ---------------------------------------------------------------- attention half
    WUDA_STAGE(wuda_mhc_pre(t->hidden_in, w->attn_hc_weight, w->attn_hc_base, w->attn_hc_scale, w->attn_norm, w->hc_eps, w->rms_eps,
                            w->norm_eps, b.a_pre, b.a_post, b.a_comb, nullptr, b.a_normed, b.a_xq, b.a_xsf, b.pre_ws,
                            wuda_mhc_pre_workspace_bytes(s->m_max, hidden), m, hidden, stream));
    Side* side = nullptr;
    WUDA_STAGE(side_of_current_device(&side));
    cudaStream_t main_stream = static_cast<cudaStream_t>(stream);
    const int sms = wuda_num_sms();
    {   // the two segments of the front projection side by side; the fork is joined on every path
        WUDA_CUDA(cudaEventRecord(side->fork[0], main_stream));
        WUDA_CUDA(cudaStreamWaitEvent(side->stream, side->fork[0], 0));
        wuda_gemm_sm_limit(front16_sms(sms));
        int st = wuda_gemm_bf16(b.a_normed, w->front_w16, b.y16, 1, m, kFront16, hidden, b.side_scratch, b.gemm_scratch_bytes, status,
                                side->stream);
        WUDA_CUDA(cudaEventRecord(side->done[0], side->stream));
        wuda_gemm_sm_limit(front8_sms(sms));
        if (st == WUDA_OK)
            st = wuda_gemm_fp8_blockscaled(b.a_xq, b.a_xsf, w->front_w8, w->front_w8_scales, b.front_out, m, kFront8, hidden,
                                           b.gemm_scratch, b.gemm_scratch_bytes, status, stream);
        wuda_gemm_sm_limit(0);
        WUDA_CUDA(cudaStreamWaitEvent(main_stream, side->done[0], 0));
        if (st != WUDA_OK) return st;
    }
    WUDA_STAGE(wuda_front_emit(b.front_out, b.y16, t->pos, c.main_state, w->ape, t->main_state_row, c.idx_state, w->idx_ape,
                               t->idx_state_row, b.win_y2, b.w64, c.state_rows_total, m, status, stream));
    wuda_csa_step step = {};
    step.q_raw = b.front_out;                 // the q_lora columns of the front projection, read in place
    step.q_raw_stride = kFront8;
    step.w64 = b.w64;
    step.win_y2 = b.win_y2;
    step.pos = t->pos;
    step.q_pos = t->q_pos;
    step.main_state_row = t->main_state_row;
    step.idx_state_row = t->idx_state_row;
    step.idx_dst = t->idx_dst;
    step.cmp_dst = t->cmp_dst;
    step.swa_dst = t->swa_dst;
    step.idx_block_table = t->idx_block_table;
    step.cmp_block_table = t->cmp_block_table;
    step.n_compressed = t->n_compressed;
    step.block_table_stride = t->block_table_stride;
    step.topk = t->topk;
    step.logits_stride = t->logits_stride;
    step.logits = b.logits;
    step.topk_indices = b.topk_indices;
    step.topk_raw = b.topk_raw;
    step.q_main_out = b.q_main;
    wuda_csa_workspace ws = {};
    ws.q_fp8 = b.q_fp8;
    ws.q_scales = b.q_scales;
    ws.y = b.y;
    ws.iq_fp8 = b.iq_fp8;
    ws.w_folded = b.w_folded;
    ws.gemm_scratch = b.gemm_scratch;
    ws.gemm_scratch_bytes = b.gemm_scratch_bytes;
    ws.status_word = status;
    WUDA_STAGE(wuda_csa_decode_step(&w->csa, &c, &step, &ws, m, stream));

    wuda_sparse_mla_args a = {};
    a.q = b.q_main;
    a.swa_pool = c.swa_pool, a.swa_stride = c.swa_block_stride_bytes, a.swa_pages = c.swa_num_blocks;
    a.swa_entries_per_block = c.swa_entries_per_block;
    a.swa_indices = t->swa_indices, a.swa_lengths = t->swa_lengths, a.swa_capacity = t->window;
    a.cmp_pool = c.cmp_pool, a.cmp_stride = c.cmp_block_stride_bytes, a.cmp_pages = c.cmp_num_blocks;
    a.cmp_entries_per_block = c.cmp_entries_per_block;
    a.cmp_indices = b.topk_indices, a.cmp_lengths = t->cmp_lengths, a.cmp_capacity = t->topk;
    a.attn_sink = w->attn_sink;
    a.out = b.mla_out;
    a.batch = m, a.heads = heads;
    a.softmax_scale = w->softmax_scale;
    const int64_t mla_need = wuda_sparse_mla_workspace_bytes(m, heads, t->window + t->topk);
    if (mla_need > 0) a.workspace = b.mla_ws, a.workspace_bytes = mla_need;
    WUDA_STAGE(wuda_sparse_mla_decode(&a, status, stream));

    const int o_width = heads * kHeadDim, z_width = w->o_groups * kORank;
    WUDA_STAGE(wuda_rope_quant_fp8(b.mla_out, t->pos, w->csa.cos_table, w->csa.sin_table, nullptr, b.o_fp8, b.o_scale, m, heads,
                                   kHeadDim, kRopeDim, w->csa.max_pos, 1, 1, stream));
    WUDA_STAGE((w->fp8_scales_pow2 ? wuda_gemm_fp8_grouped_pow2 : wuda_gemm_fp8_grouped)(
        b.o_fp8, b.o_scale, w->wo_a, w->wo_a_scales, b.z, m, kORank, o_width / w->o_groups, w->o_groups, b.gemm_scratch,
        b.gemm_scratch_bytes, status, stream));
    WUDA_STAGE(wuda_rmsnorm_quant_fp8(b.z, z_width, nullptr, 0, 0.0f, nullptr, b.z_fp8, b.z_scale, m, z_width, 1, stream));
    if (s->tp_peer_inbox)
        WUDA_STAGE(wuda_gemm_fp8_blockscaled_tp2(b.z_fp8, b.z_scale, w->wo_b, w->wo_b_scales, b.projected, m, hidden, z_width,
                                                 b.gemm_scratch, b.gemm_scratch_bytes, s->tp_my_inbox, s->tp_peer_inbox, 0,
                                                 s->peer_wait_ms, status, stream));
    else
        WUDA_STAGE(wuda_gemm_fp8_blockscaled(b.z_fp8, b.z_scale, w->wo_b, w->wo_b_scales, b.projected, m, hidden, z_width,
                                             b.gemm_scratch, b.gemm_scratch_bytes, status, stream));
    WUDA_STAGE(wuda_mhc_post(b.projected, t->hidden_in, b.a_post, b.a_comb, b.attn_out, m, hidden, stream));

    // ---------------------------------------------------------------- feed-forward half
    WUDA_STAGE(wuda_mhc_pre(b.attn_out, w->ffn_hc_weight, w->ffn_hc_base, w->ffn_hc_scale, w->ffn_norm, w->hc_eps, w->rms_eps,
                            w->norm_eps, b.f_pre, b.f_post, b.f_comb, nullptr, b.f_normed, nullptr, nullptr, b.pre_ws,
                            wuda_mhc_pre_workspace_bytes(s->m_max, hidden), m, hidden, stream));
    // the shared expert on the side stream, beside router projection, routing, dispatch and gather
    const void* shared_rows = nullptr;
    if (w->shared_w13) {
        const int si = w->shared_inter;
        WUDA_CUDA(cudaEventRecord(side->fork[1], main_stream));
        WUDA_CUDA(cudaStreamWaitEvent(side->stream, side->fork[1], 0));
        wuda_gemm_sm_limit(shared_sms(sms));
        int st = wuda_rmsnorm_quant_fp8(b.f_normed, hidden, nullptr, 0, 0.0f, nullptr, b.s_x8, b.s_xs, m, hidden, 1, side->stream);
        if (st == WUDA_OK)
            st = wuda_gemm_fp8_blockscaled(b.s_x8, b.s_xs, w->shared_w13, w->shared_w13_scales, b.s_h, m, 2 * si, hidden,
                                           b.side_scratch, b.gemm_scratch_bytes, status, side->stream);
        if (st == WUDA_OK) st = wuda_swiglu_quant_fp8(b.s_h, nullptr, b.s_a8, b.s_as, m, si, w->swiglu_limit, 1, side->stream);
        if (st == WUDA_OK)
            st = wuda_gemm_fp8_blockscaled(b.s_a8, b.s_as, w->shared_w2, w->shared_w2_scales, b.s_out, m, hidden, si, b.side_scratch,
                                           b.gemm_scratch_bytes, status, side->stream);
        wuda_gemm_sm_limit(0);
        WUDA_CUDA(cudaEventRecord(side->done[1], side->stream));
        if (st != WUDA_OK) {
            WUDA_CUDA(cudaStreamWaitEvent(main_stream, side->done[1], 0));
            return st;
        }
        shared_rows = b.s_out;
    }
    int routed = wuda_gemm_bf16(b.f_normed, w->gate_weight, b.gate_logits, 1, m, w->experts_total, hidden, b.gemm_scratch,
                                b.gemm_scratch_bytes, status, stream);
    if (routed == WUDA_OK)
        routed = wuda_moe_route(b.gate_logits, w->gate_bias, b.route_w, b.route_idx, m, w->experts_total, w->moe_topk, w->score_func,
                                w->route_scale, stream);
    if (routed == WUDA_OK)
        routed = wuda_moe_dispatch_range(b.route_idx, b.route_w, b.group_expert, b.num_groups, b.row_token, b.row_weight, b.pair_row, m,
                                         w->moe_topk, w->experts_local, w->expert_first, w->experts_total, b.max_groups, status,
                                         stream);
    if (routed == WUDA_OK)
        routed = wuda_moe_gather_quant_nvfp4(b.f_normed, b.pair_row, b.a1, b.a1_sf, w->act_scale_in, m, w->moe_topk, hidden, stream);
    if (w->shared_w13) WUDA_CUDA(cudaStreamWaitEvent(main_stream, side->done[1], 0));   // join
    if (routed != WUDA_OK) return routed;
    WUDA_STAGE(wuda_gemm_nvfp4_grouped(b.a1, b.a1_sf, w->act_scale_in, w->w13, w->w13_sf, w->w13_gs, b.group_expert, b.num_groups, b.row_token, b.h,
                                       b.max_groups, w->experts_local, 2 * w->inter, hidden, b.nvfp4_scratch, b.nvfp4_scratch_bytes,
                                       status, stream));
    WUDA_STAGE(wuda_moe_swiglu_quant_nvfp4(b.h, b.pair_row, b.route_w, b.a2, b.a2_sf, w->act_scale_mid, w->swiglu_limit, m, w->moe_topk,
                                           w->inter, stream));
    WUDA_STAGE(wuda_gemm_nvfp4_grouped(b.a2, b.a2_sf, w->act_scale_mid, w->w2, w->w2_sf, w->w2_gs, b.group_expert, b.num_groups,
                                       b.row_token, b.r_out, b.max_groups, w->experts_local, hidden, w->inter, b.nvfp4_scratch,
                                       b.nvfp4_scratch_bytes, status, stream));
    if (s->ep_peer_inbox)
        WUDA_STAGE(wuda_moe_combine_ep2(b.r_out, b.pair_row, shared_rows, b.y_moe, m, w->moe_topk, hidden, s->ep_my_inbox,
                                        s->ep_peer_inbox, s->ep_tokens_max, 0, s->peer_wait_ms, status, stream));
    else
        WUDA_STAGE(wuda_moe_combine(b.r_out, b.pair_row, shared_rows, b.y_moe, m, w->moe_topk, hidden, stream));
    WUDA_STAGE(wuda_mhc_post(b.y_moe, b.attn_out, b.f_post, b.f_comb, t->hidden_out, m, hidden, stream));
    return WUDA_OK;
}

// Where a stage's result lies in the workspace, for callers (and tests) that read intermediate tensors:
// byte offset from the workspace base, or -1 for an unknown name.
extern "C" int64_t wuda_layer_workspace_offset(const wuda_layer_weights* w, int m_max, int topk, int64_t logits_stride, int window,
                                               const char* name) {
    using namespace wuda::layer;
    if (!w || !name || m_max < 1 || m_max > 128) return -1;
    Buffers b;
    uint8_t* const base = reinterpret_cast<uint8_t*>(static_cast<uintptr_t>(256));   // never dereferenced
    if (carve(w, m_max, topk, logits_stride, window, base, &b) < 0) return -1;
    struct Entry {
        const char* name;
        const void* ptr;
    } const table[] = {{"logits", b.logits},       {"topk_indices", b.topk_indices}, {"topk_raw", b.topk_raw},
                       {"q_main", b.q_main},       {"mla_out", b.mla_out},           {"attn_out", b.attn_out},
                       {"gate_logits", b.gate_logits}, {"route_indices", b.route_idx},  {"route_weights", b.route_w},
                       {"moe_out", b.y_moe},       {"front_out", b.front_out},       {"q_proj", b.y},
                       {"iq_fp8", b.iq_fp8},       {"w_folded", b.w_folded},         {"win_y2", b.win_y2},
                       {"w64", b.w64}};
    for (const Entry& e : table) {
        bool same = true;
        for (int i = 0; e.name[i] || name[i]; ++i)
            if (e.name[i] != name[i]) {
                same = false;
                break;
            }
        if (same) return static_cast<const uint8_t*>(e.ptr) - base;
    }
    return -1;
}
