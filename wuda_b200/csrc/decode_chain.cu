// Layer launch of the indexer half of a decode step: the reference's three consecutive stages
//   qnorm_quant + wq_b_proj_gemm_merged  (q RMSNorm + quant, q projection, indexer-q post,
//                                          indexer compressor, window KV)
//   mqa_logits_fp8_decode_out            (paged MQA logits, MAIN compressor, query RMSNorm + RoPE)
//   topk_v2                              (top-k + page-table transform)
// as they are called from decode_step (dsv4_megakernel/megakernel/test/test_e2e_decode.py:560-640),
// enqueued on one stream with no host synchronisation and no allocation, so a caller can capture
// the whole step into a CUDA graph once and replay it.  Everything here is host code: the step is
// seven launches of this library's kernels:
//   1 q RMSNorm + power-of-two 1x128 FP8 quantisation of q_raw
//   2 block-scaled FP8 GEMM with the merged [indexer heads | main heads] weight
//   3 query RMSNorm + RoPE of the main heads (reads the GEMM output in place)
//   4 indexer-q post (reads the GEMM output in place) -> FP8 q + folded head weights (FP4 form: Hadamard + MXFP4 q)
//   5 cache writers: the indexer entry of this step must be in the pool before 6 scores it
//   6 paged MQA logits over the indexer pool (FP8 records, or MXFP4 records with caches.idx_fp4)
//   7 top-k + page transform
// Only 1 -> 2 -> 4 -> 6 -> 7 is a chain.  5 needs nothing from 1-4 and 3 feeds nothing in 4-7, so
// they run on two side streams forked from and joined back into the caller's stream with events
// (5 joins before 6, 3 at the end).  Under stream capture the forks become parallel branches of the
// graph.  The side streams and events are created once per device and never destroyed.
#include "host.h"

namespace wuda {
namespace chain {

struct Side {
    bool ready = false;
    cudaStream_t writers = nullptr, query = nullptr;
    cudaEvent_t fork = nullptr, forked_gemm = nullptr, writers_done = nullptr, query_done = nullptr;
};

int side_of_current_device(Side** out) {
    static Side sides[16];
    int dev = 0;
    WUDA_CUDA(cudaGetDevice(&dev));
    WUDA_REQUIRE(dev >= 0 && dev < 16, "device ordinal %d is outside the 16 this library keeps state for", dev);
    Side& s = sides[dev];
    if (!s.ready) {
        WUDA_CUDA(cudaStreamCreateWithFlags(&s.writers, cudaStreamNonBlocking));
        WUDA_CUDA(cudaStreamCreateWithFlags(&s.query, cudaStreamNonBlocking));
        for (cudaEvent_t* e : {&s.fork, &s.forked_gemm, &s.writers_done, &s.query_done})
            WUDA_CUDA(cudaEventCreateWithFlags(e, cudaEventDisableTiming));
        s.ready = true;
    }
    *out = &s;
    return WUDA_OK;
}

}  // namespace chain
}  // namespace wuda

extern "C" int wuda_csa_decode_step(const wuda_csa_weights* w, const wuda_csa_caches* c, const wuda_csa_step* s,
                                    const wuda_csa_workspace* ws, int m, void* stream) {
    using namespace wuda;
    clear_error();
    WUDA_REQUIRE(w && c && s && ws, "weights, caches, step and workspace must not be NULL");
    WUDA_REQUIRE(m >= 1 && m <= 128, "m must be in [1, 128] (got %d)", m);
    WUDA_REQUIRE(w->q_lora >= 128 && w->q_lora % 128 == 0, "q_lora must be a positive multiple of 128");
    WUDA_REQUIRE(w->index_heads >= 1 && w->main_heads >= 1 && w->out_heads >= w->main_heads,
                 "index_heads, main_heads >= 1 and out_heads >= main_heads are required");
    WUDA_REQUIRE(ws->q_fp8 && ws->q_scales && ws->y && ws->iq_fp8 && ws->w_folded && ws->gemm_scratch,
                 "every workspace buffer is required");
    WUDA_REQUIRE(!c->idx_fp4 || w->index_heads == 64, "the FP4 form of the indexer has 64 index heads (got %d)",
                 w->index_heads);
    const int n_index = w->index_heads * 128, n_main = w->main_heads * 512;
    const int n_total = n_index + n_main;
    const char* y = static_cast<const char*>(ws->y);
    cudaStream_t main_stream = static_cast<cudaStream_t>(stream);
    chain::Side* side = nullptr;
    int st = chain::side_of_current_device(&side);
    if (st != WUDA_OK) return st;

    // ---- branch A (side stream): the cache writers, independent of the projection
    WUDA_CUDA(cudaEventRecord(side->fork, main_stream));
    WUDA_CUDA(cudaStreamWaitEvent(side->writers, side->fork, 0));
    wuda_cache_writers cw = {};
    cw.pos = s->pos;
    cw.cos_table = w->cos_table;
    cw.sin_table = w->sin_table;
    cw.max_pos = w->max_pos;
    cw.eps = w->eps;
    cw.indexer.state = c->idx_state;
    cw.indexer.state_row = s->idx_state_row;
    cw.indexer.norm_w = w->idx_norm;
    cw.indexer.state_rows_total = c->state_rows_total;
    cw.indexer.ring_entries = c->ring_entries;
    cw.indexer.entries_per_block = c->idx_entries_per_block;
    cw.indexer.num_blocks = c->idx_num_blocks;
    cw.indexer.block_stride_bytes = c->idx_block_stride_bytes;
    cw.indexer.pool = c->idx_pool;
    cw.indexer.dst = s->idx_dst;
    cw.main = cw.indexer;
    cw.main.state = c->main_state;
    cw.main.state_row = s->main_state_row;
    cw.main.norm_w = w->main_norm;
    cw.main.entries_per_block = c->cmp_entries_per_block;
    cw.main.num_blocks = c->cmp_num_blocks;
    cw.main.block_stride_bytes = c->cmp_block_stride_bytes;
    cw.main.pool = c->cmp_pool;
    cw.main.dst = s->cmp_dst;
    cw.window.y = s->win_y2;
    cw.window.norm_w = w->win_norm;
    cw.window.entries_per_block = c->swa_entries_per_block;
    cw.window.num_blocks = c->swa_num_blocks;
    cw.window.block_stride_bytes = c->swa_block_stride_bytes;
    cw.window.pool = c->swa_pool;
    cw.window.dst = s->swa_dst;
    const bool fp4 = c->idx_fp4 != 0;   // the indexer's FP4 form: Hadamard + MXFP4 query and keys, block-scaled logits
    int status = (fp4 ? wuda_cache_writers_fp4 : wuda_cache_writers_fp8)(&cw, m, ws->status_word, side->writers);
    WUDA_CUDA(cudaEventRecord(side->writers_done, side->writers));

    // ---- the chain on the caller's stream.  Every fork is joined on every path out of this function,
    // also after a refused launch, so that a stream capture in progress stays well formed.
    if (status == WUDA_OK)
        status = wuda_rmsnorm_quant_fp8(s->q_raw, s->q_raw_stride, w->q_norm, 0, w->eps, nullptr, ws->q_fp8, ws->q_scales,
                                        m, w->q_lora, 1, stream);
    if (status == WUDA_OK)
        status = (w->scales_pow2 ? wuda_gemm_fp8_blockscaled_pow2 : wuda_gemm_fp8_blockscaled)(
            ws->q_fp8, ws->q_scales, w->wq_b, w->wq_b_scales, ws->y, m, n_total, w->q_lora, ws->gemm_scratch, ws->gemm_scratch_bytes,
            ws->status_word, stream);
    // ---- branch B (side stream): the main heads' query tail, needed only by the attention that follows
    bool query_forked = false;
    if (status == WUDA_OK && s->q_main_out) {
        WUDA_CUDA(cudaEventRecord(side->forked_gemm, main_stream));
        WUDA_CUDA(cudaStreamWaitEvent(side->query, side->forked_gemm, 0));
        query_forked = true;
        status = wuda_query_rms_rope(y + static_cast<int64_t>(n_index) * 2, n_total, s->pos, w->cos_table, w->sin_table,
                                     w->max_pos, s->q_main_out, m, w->main_heads, w->out_heads, w->eps, side->query);
        WUDA_CUDA(cudaEventRecord(side->query_done, side->query));
    }
    if (status == WUDA_OK)
        status = fp4 ? wuda_index_q_post_fp4(y, n_total, s->q_pos, w->cos_table, w->sin_table, w->max_pos, ws->iq_fp8,
                                             ws->w_folded, m, w->index_heads, stream)
                     : wuda_index_q_post_fp8(y, n_total, s->q_pos, w->cos_table, w->sin_table, w->max_pos, s->w64,
                                             ws->iq_fp8, ws->w_folded, m, w->index_heads, stream);
    WUDA_CUDA(cudaStreamWaitEvent(main_stream, side->writers_done, 0));     // join A: the pool is written
    if (status == WUDA_OK) {
        if (fp4) {
            const int64_t by_table = static_cast<int64_t>(s->block_table_stride) * c->idx_entries_per_block;
            const int64_t cap = s->logits_stride < by_table ? s->logits_stride : by_table;
            status = wuda_mqa_logits_fp4(ws->iq_fp8, ws->w_folded, c->idx_pool, s->w64, s->n_compressed, s->idx_block_table,
                                         s->logits, m, static_cast<int>(cap < 0x7fffff00 ? cap : 0x7fffff00),
                                         c->idx_num_blocks, c->idx_entries_per_block, c->idx_block_stride_bytes,
                                         s->block_table_stride, s->logits_stride, ws->status_word, stream);
        } else {
            status = wuda_mqa_logits_fp8(ws->iq_fp8, c->idx_pool, ws->w_folded, s->n_compressed, s->idx_block_table,
                                         s->logits, m, 1, c->idx_num_blocks, c->idx_entries_per_block,
                                         c->idx_block_stride_bytes, s->block_table_stride, s->logits_stride,
                                         ws->status_word, stream);
        }
    }
    if (status == WUDA_OK)
        // the selected positions become entries of the pool the attention reads: the compressed-KV pool's page
        // table and page size when that table is given, else the indexer pool's
        status = wuda_topk(s->logits, s->n_compressed, s->cmp_block_table ? s->cmp_block_table : s->idx_block_table,
                           s->topk_indices, s->topk_raw, m, s->logits_stride, s->block_table_stride, 1, s->topk,
                           s->cmp_block_table ? c->cmp_entries_per_block : c->idx_entries_per_block, stream);
    if (query_forked) WUDA_CUDA(cudaStreamWaitEvent(main_stream, side->query_done, 0));   // join B
    return status;
}
