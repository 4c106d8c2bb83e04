/*
 * wuda_b200 — C ABI of the B200 (sm_100a) decode hot path.
 *
 * One shared library, plain pointers and sizes, no framework types.  Every pointer is a
 * DEVICE pointer unless its name ends in `_host`.  Every call enqueues work on `stream`
 * (a cudaStream_t passed as void*; NULL = the legacy default stream) and returns
 * without synchronising, except the `*_host` convenience calls, which copy from and to
 * host buffers and synchronise the stream before returning.
 *
 * Return value: WUDA_OK or a wuda_status.  Arguments are validated before anything is
 * launched; a failed call launches nothing.  The text of the last failure on the
 * calling thread is available from wuda_last_error().  Device-side problems (a wait
 * that ran out of time, a block-table entry outside the pool) never trap the GPU: the
 * kernel records a code (wuda_device_status) in the caller's `status_word` and ends.
 *
 * File:line citations name the interface of the reference (guluguluhhhh/wuda, paths
 * relative to dsv4_megakernel/megakernel/) that the entry point stands in for.
 */
#ifndef WUDA_B200_H_
#define WUDA_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum wuda_status {
    WUDA_OK = 0,
    WUDA_ERR_INVALID_ARGUMENT = 1, /* shape / alignment / range check failed            */
    WUDA_ERR_UNSUPPORTED = 2,      /* valid request outside what the kernels implement   */
    WUDA_ERR_CUDA = 3,             /* a CUDA runtime or driver call failed               */
    WUDA_ERR_NO_DEVICE = 4,        /* no sm_100 device / driver entry point unavailable  */
    WUDA_ERR_DEVICE_STATUS = 5     /* (host-buffer calls) the kernel reported a code     */
} wuda_status;

/* Codes a kernel may leave in `status_word` (0 = nothing to report). */
typedef enum wuda_device_status {
    WUDA_DEV_OK = 0,
    WUDA_DEV_TIMEOUT_FULL_Q = 101,
    WUDA_DEV_TIMEOUT_EMPTY_Q = 102,
    WUDA_DEV_TIMEOUT_FULL_KV = 103,
    WUDA_DEV_TIMEOUT_EMPTY_KV = 104,
    WUDA_DEV_TIMEOUT_FULL_TMEM = 105,
    WUDA_DEV_TIMEOUT_EMPTY_TMEM = 106,
    WUDA_DEV_BAD_PAGE_INDEX = 110, /* block_table entry outside [0, num_blocks): page 0 was read instead */
    WUDA_DEV_BAD_CONTEXT_LEN = 111, /* a context length beyond logits_stride or block_table_stride * entries_per_block
                                       was cut to that limit: nothing is written past a row of the logits */
    WUDA_DEV_TIMEOUT_GEMM_FULL = 121,
    WUDA_DEV_TIMEOUT_GEMM_EMPTY = 122,
    WUDA_DEV_TIMEOUT_GEMM_TMEM_FULL = 123,
    WUDA_DEV_TIMEOUT_GEMM_TMEM_EMPTY = 124,
    WUDA_DEV_SCALE_NOT_POW2 = 125, /* a scale given to a *_pow2 GEMM was not a power of two: it was truncated to one */
    WUDA_DEV_TIMEOUT_PEER_FLAG = 131,
    WUDA_DEV_BAD_DESTINATION = 141, /* cache destination outside the pool: that record was not written */
    WUDA_DEV_BAD_STATE_ROW = 142,   /* state_row outside the state rings: that row was skipped         */
    WUDA_DEV_BAD_EXPERT = 143,      /* expert index outside [0, experts): that pair was dropped        */
    WUDA_DEV_TIMEOUT_MLA_KEYS = 151,
    WUDA_DEV_TIMEOUT_MLA_SCORES = 152,
    WUDA_DEV_TIMEOUT_MLA_SCORES_READ = 153,
    WUDA_DEV_TIMEOUT_MLA_PROBS = 154,
    WUDA_DEV_TIMEOUT_MLA_OUTPUT = 155,
    WUDA_DEV_MLA_SCALE_RANGE = 156  /* a key's scale exponent outside [-15, 7] was clamped into that range */
} wuda_device_status;

/* Library version (major*10000 + minor*100 + patch). */
int wuda_version(void);
/* Message of the last non-OK return on this thread ("" if none). Never NULL. */
const char* wuda_last_error(void);
/* Number of SMs of the current device, or a negative wuda_status. */
int wuda_num_sms(void);

/* ------------------------------------------------------------------------------------
 * Paged FP8 MQA logits (the indexer score).
 *
 *   logits[r, t] = scale[t] * sum_h weights[r, h] * relu( sum_d q[r, h, d] * k[t, d] )
 *
 * for every row r = b * next_n + j and every token t < context_lens[b, j] of request b,
 * where token t lives in physical page block_table[b, t / entries_per_block] at slot
 * t % entries_per_block.  Positions t >= context_lens[b, j] are NOT written.  A negative context
 * length counts as 0; one beyond min(logits_stride, block_table_stride * entries_per_block) is cut
 * to that limit and reported as WUDA_DEV_BAD_CONTEXT_LEN (the reference checks neither).
 *
 * Stands in for mqa_logits_fp8_decode_out (kernels/mqa_logits_fp8.cu:388-526) without
 * its optional compressor / query tails, and for deep_gemm.fp8_paged_mqa_logits as
 * called at test/test_mqa_logits_fp4.py:518-522.  The reference's `schedule_meta`
 * tensor has no counterpart: the tile schedule is computed inside the kernel.
 *
 *   q             e4m3  [batch * next_n, 64, 128], contiguous, 16-byte aligned
 *   kv_pages      uint8 [num_blocks, page_stride_bytes]; a page is
 *                 entries_per_block x 128 e4m3 key bytes followed by entries_per_block
 *                 fp32 per-token scales (test/test_mqa_logits_fp4.py:443-474);
 *                 16-byte aligned, page_stride_bytes % 16 == 0 and >= epb * 132
 *   weights       fp32  [batch * next_n, 64] (per-head weight, q scale pre-folded)
 *   context_lens  int32 [batch, next_n] (for next_n == 1 this is the reference's [B] / [B,1])
 *   block_table   int32 [batch, block_table_stride]; rows of one request share it
 *   logits        fp32  [batch * next_n, logits_stride]
 *   next_n        1 or 2; entries_per_block 32, 64 or 128
 *   status_word   int32 on the device, nullable; see wuda_device_status
 */
int wuda_mqa_logits_fp8(const void* q, const void* kv_pages, const float* weights,
                        const int32_t* context_lens, const int32_t* block_table, float* logits,
                        int batch, int next_n, int num_blocks, int entries_per_block,
                        int64_t page_stride_bytes, int block_table_stride, int64_t logits_stride,
                        int32_t* status_word, void* stream);

/* ------------------------------------------------------------------------------------
 * Top-k index selection over the logits, then the page-table transform.
 *
 * For each row r: the indices of the k largest values of scores[r, 0 : seq_lens[r]],
 * in no particular order; equal values are resolved towards the lower index, so the
 * selected SET equals argsort(-scores, stable)[:k].  Rows with seq_lens[r] <= k yield
 * 0, 1, .., n-1 followed by -1.  Each selected index i is written as
 *     page_indices[r, j] = (page_table[r, i / page_size] * page_size) | (i % page_size)
 * (page_size a power of two; -1 stays -1); with page_table == NULL the raw index is
 * written.  raw_indices (nullable) receives the untransformed indices.
 *
 * Stands in for topk_v2 / topk_v2_transform (kernels/topk_v2.cu:329-439); the
 * reference's `metadata` plan tensor has no counterpart (no plan kernel is needed).
 *
 *   scores       fp32  [rows, score_stride]
 *   seq_lens     int32 [rows]
 *   page_table   int32 [rows / rows_per_table_row, page_table_stride], nullable; row r
 *                uses table row r / rows_per_table_row (1 = one table row per score
 *                row, as in the reference; next_n when the next_n rows of a request
 *                share the request's block table)
 *   page_indices int32 [rows, k];  raw_indices int32 [rows, k], nullable
 */
int wuda_topk(const float* scores, const int32_t* seq_lens, const int32_t* page_table,
              int32_t* page_indices, int32_t* raw_indices, int rows, int64_t score_stride,
              int64_t page_table_stride, int rows_per_table_row, int k, int page_size,
              void* stream);

/* ------------------------------------------------------------------------------------
 * RMSNorm + 1x128 FP8 quantisation in one pass over a bf16 row.
 *
 *   y = bf16( gamma * (x * rsqrt(mean(x^2) + eps)) )           (gamma == NULL: y = x)
 *   per 128 elements of y: amax = max(|y|, 1e-4); scale = amax / 448 (scale_mode 0) or
 *   2^ceil(log2(amax / 448)) (scale_mode 1); y_fp8 = e4m3(clamp(y / scale, +-448))
 *
 * Numerics: origin/model.py:191-196 (RMSNorm) and origin/kernel.py:40-125 (act_quant).
 * Stands in for qnorm_quant_kernel (kernels/wq_b_fp8_gemm.cu:139-183) and for the
 * attn_norm + FP8 tail of hc_reduce_fuse_out (kernels/hc_fused_kernel_tc.cu:319-335).
 *
 *   x_bf16   bf16 [rows, x_row_stride] (first `dim` of each row are used; 16-byte aligned)
 *   gamma    fp32 or bf16 [dim] (gamma_is_bf16), nullable
 *   y_bf16   bf16 [rows, dim], nullable;  y_fp8 e4m3 [rows, dim], nullable
 *   y_scales fp32 [rows, dim/128], required with y_fp8;  dim % 128 == 0, dim <= 24576
 */
int wuda_rmsnorm_quant_fp8(const void* x_bf16, int64_t x_row_stride, const void* gamma, int gamma_is_bf16,
                           float eps, void* y_bf16, void* y_fp8, float* y_scales, int rows, int dim,
                           int scale_mode, void* stream);

/* ------------------------------------------------------------------------------------
 * Partial RoPE + 1x128 FP8 quantisation in one pass.
 *
 * x is bf16 [tokens, heads, head_dim]; the LAST rope_dim dims of every head are rotated in
 * interleaved pairs by the angle of positions[t] (cos/sin tables fp32 [max_pos, rope_dim/2];
 * inverse != 0 rotates backwards), rounded to bf16, and the flat row of heads*head_dim
 * values is quantised per 128 consecutive elements as above.
 *
 * Numerics: origin/model.py:232-244 (apply_rotary_emb) and origin/kernel.py:40-125.
 * Stands in for the FP8 indexer-q post (include/idx_post_fp4.cuh:229-283, rope tail +
 * per-row e4m3), inv_rope_quant (kernels/mla_o_inv_rope_quant.cu:43-157, inverse = 1) and,
 * with y_fp8 == NULL, for the RoPE half of rmsnorm_rope_out (kernels/rmsnorm_prod.cu:91-158).
 * Positions outside [0, max_pos) are clamped.
 */
int wuda_rope_quant_fp8(const void* x_bf16, const int64_t* positions, const float* cos_table,
                        const float* sin_table, void* y_bf16, void* y_fp8, float* y_scales, int tokens,
                        int heads, int head_dim, int rope_dim, int max_pos, int inverse, int scale_mode,
                        void* stream);

/* ------------------------------------------------------------------------------------
 * Indexer-q post (FP8 form): every (token, index head) row of 128 bf16 values gets RoPE on its
 * last 64 dims (rounded to bf16), one scale = max(amax / 448, 1e-12), e4m3 payload, and the
 * head weight multiplied by that scale - what wuda_mqa_logits_fp8 takes as q and weights.
 *
 * Replaces idx_postprocess_fp8_standalone and the idx-post tail of wq_b_proj_gemm_merged
 * (include/idx_post_fp4.cuh:229-283, kernels/wq_b_fp8_gemm.cu:1368-1567); numerics as the
 * torch twin test/test_wq_b_fp8_gemm.py:184-196.
 *
 *   iq_bf16   bf16, row t starts at t * row_stride elements and holds heads * 128 values
 *             (so the projection's output is read in place); row_stride % 8 == 0
 *   q_pos     int32 [tokens], clamped into [0, max_pos);  tables fp32 [max_pos, 32]
 *   weights   fp32 [tokens, heads], nullable (then weights_out receives the bare scales)
 *   q_fp8     e4m3 [tokens, heads, 128];  weights_out fp32 [tokens, heads]
 */
int wuda_index_q_post_fp8(const void* iq_bf16, int64_t row_stride, const int32_t* q_pos, const float* cos_table,
                          const float* sin_table, int max_pos, const float* weights, void* q_fp8,
                          float* weights_out, int tokens, int heads, void* stream);

/* ------------------------------------------------------------------------------------
 * Indexer-q post (FP4 form): every (token, index head) row of 128 bf16 values gets RoPE on its
 * last 64 dims (rounded to bf16), a Hadamard transform of the 128 values (fp32 butterflies with
 * strides 1, 2, ... 64 in that order, times 128^-1/2, one rounding to bf16) and MXFP4
 * quantisation: per 32 values the scale 2^ceil(log2(amax / 6)) as a biased exponent byte, e2m1
 * codes rounded to nearest even - what wuda_mqa_logits_fp4 takes as q_fp4 and q_scales.  The
 * head weights are not touched in this form.
 *
 * Replaces idx_postprocess (kernels/idx_post_fp4.cu) and the FP4 idx-post tail of
 * wq_b_proj_gemm_merged (include/idx_post_fp4.cuh:79-224: same order of the butterflies, same
 * constants, so the bytes are the kernel's); torch twin test/test_wq_b_fp8_gemm.py:161-182
 * (ref_idx_chain), which multiplies by the Hadamard matrix and rounds e2m1 ties down instead.
 *
 *   iq_bf16, row_stride, q_pos, tables: as wuda_index_q_post_fp8
 *   q_fp4     uint8 [tokens, heads, 64], two codes per byte, the lower index in the low nibble
 *   q_scales  int32 [tokens, heads], byte g = exponent byte of values [32g, 32g + 32)
 */
int wuda_index_q_post_fp4(const void* iq_bf16, int64_t row_stride, const int32_t* q_pos, const float* cos_table,
                          const float* sin_table, int max_pos, void* q_fp4, void* q_scales, int tokens, int heads,
                          void* stream);

/* ------------------------------------------------------------------------------------
 * Query RMSNorm (no weight) + RoPE on the last 64 of every 512-wide head, bf16 -> bf16, in
 * one pass with one rounding.  Output head h reads input head h % input_heads.
 *
 * Replaces rmsnorm_rope_out (kernels/rmsnorm_prod.cu:91-167) and the query tail of
 * mqa_logits_fp8_decode_out (QueryRmsRopeArgs, include/mqa_logits_fp8.cuh:47-116;
 * include/query_rms_rope.cuh:20-61).
 *
 *   x_bf16    bf16, row t at t * row_stride elements, input_heads * 512 values
 *   positions int64 [tokens];  out_bf16 bf16 [tokens, output_heads, 512]
 */
int wuda_query_rms_rope(const void* x_bf16, int64_t row_stride, const int64_t* positions, const float* cos_table,
                        const float* sin_table, int max_pos, void* out_bf16, int tokens, int input_heads,
                        int output_heads, float eps, void* stream);

/* ------------------------------------------------------------------------------------
 * The cache writers of a decode step, all in one launch: the indexer compressor, the MAIN
 * compressor and the window-KV writer.  Each fills the paged pool its consumer reads and,
 * optionally, compact per-row copies of what it wrote.
 *
 * Replaces the writers the reference runs in idle warps of other kernels and their
 * stand-alone forms: idx_comp::process_row<true> and process_win_row
 * (include/idx_comp_fp4.cuh:97-201, :282-383; bundle of wq_b_proj_gemm_merged,
 * kernels/wq_b_fp8_gemm.cu:849-1365) and run_main_compressor_row / MainCompressorArgs
 * (include/mqa_logits_fp8.cuh:29-45, :133-284; mqa_compressor_fp8_standalone,
 * kernels/mqa_logits_fp8.cu:542-599).  Numerics follow their torch twins
 * (test/test_wq_b_fp8_gemm.py:550-586 with fp8=True, :646-665; test/test_mqa_logits_fp4.py:769-789):
 * IEEE division, 1/sqrt and expf where the reference kernels use the fast-math forms.
 *
 * A compressor bundle works on rows with (pos[r] + 1) % 4 == 0 and state_row[r] >= 0:
 *   state      fp32 [state_rows_total, 4*H]: entry = [kv 2H | score 2H], H = 128 (indexer) or
 *              512 (MAIN); state_row[r] = block * ring_entries + (pos % ring_entries)
 *   the 8 entries ending at state_row (walking back inside the block, modulo ring_entries) are
 *   combined per column by softmax(score) * kv - entries 0..3 use columns [0,H), 4..7 use [H,2H) -
 *   -> bf16 -> RMSNorm(H, norm_w fp32 [H]) -> bf16 -> RoPE on the last 64 at position pos - 3 -> bf16
 *   indexer: scale = max(amax / 448, 1e-12); 128 e4m3 bytes at page + off*128 and the fp32
 *            scale at page + entries_per_block*128 + off*4 (the kv_pages format of
 *            wuda_mqa_logits_fp8); compact q8 [rows,128], s8 fp32 [rows]
 *   MAIN:    a MODEL1 record: columns [0,448) e4m3 with one power-of-two scale per 64
 *            (2^ceil(log2(max(amax/448, 1e-4)))), columns [448,512) bf16; body at
 *            page + off*576, 7 biased-exponent bytes at page + entries_per_block*576 + off*8;
 *            compact q8 [rows,448], s8 fp32 [rows,7], rope bf16 [rows,64]
 * The window bundle works on every row: y fp32 [rows,512] -> RMSNorm from the raw row ->
 * [0,448) rounded to bf16 and quantised as above, [448,512) rotated in fp32 at pos[r] -> bf16,
 * written as a MODEL1 record like MAIN.
 * dst[r] = page * entries_per_block + off; dst[r] < 0 writes no record (compact outputs are
 * still written).  A bundle with state (or y) == NULL is skipped; pool, q8, s8, rope are each
 * optional.  Rows that do not compress leave their compact outputs untouched.  Out-of-range
 * destinations or state rows are skipped and reported in status_word (nullable).
 */
typedef struct wuda_compressor_bundle {
    const float* state;
    const int64_t* state_row;
    const float* norm_w;
    int64_t state_rows_total;
    int ring_entries;
    int entries_per_block;
    int num_blocks;
    int reserved;
    int64_t block_stride_bytes;
    uint8_t* pool;
    const int64_t* dst;
    uint8_t* q8;
    float* s8;
    void* rope; /* MAIN only */
} wuda_compressor_bundle;

typedef struct wuda_window_bundle {
    const float* y;
    const float* norm_w;
    int entries_per_block;
    int num_blocks;
    int64_t block_stride_bytes;
    uint8_t* pool;
    const int64_t* dst;
    uint8_t* q8;
    float* s8;
    void* rope;
} wuda_window_bundle;

typedef struct wuda_cache_writers {
    const int64_t* pos;     /* [rows] token positions                               */
    const float* cos_table; /* fp32 [max_pos, 32]                                    */
    const float* sin_table;
    int max_pos;            /* rotation positions are clamped into [0, max_pos)      */
    float eps;
    wuda_compressor_bundle indexer;
    wuda_compressor_bundle main;
    wuda_window_bundle window;
} wuda_cache_writers;

int wuda_cache_writers_fp8(const wuda_cache_writers* args, int rows, int32_t* status_word, void* stream);

/* The same launch with the indexer compressor in its FP4 form (idx_comp::process_row<false>,
 * include/idx_comp_fp4.cuh:203-274; torch twin ref_comp_step with fp8=False,
 * test/test_wq_b_fp8_gemm.py:550-586): behind the rotation a Hadamard transform of the 128 values
 * (fp32 butterflies, strides 1, 2, ... 64, times 128^-1/2, one rounding to bf16) and per 32 values
 * the scale 2^ceil(log2(amax / 6)) with e2m1 codes (nearest even).  The indexer record is 64 code
 * bytes at page + off*64 and 4 exponent bytes at page + entries_per_block*64 + off*4 (the kv_pages
 * format of wuda_mqa_logits_fp4); the indexer bundle's compact outputs are q8 = codes uint8
 * [rows, 64] and s8 = exponent bytes uint8 [rows, 4] (the pointer is taken as bytes).  MAIN and
 * window writers are unchanged. */
int wuda_cache_writers_fp4(const wuda_cache_writers* args, int rows, int32_t* status_word, void* stream);

/* ------------------------------------------------------------------------------------
 * Layer launch of the indexer half of one decode step: q RMSNorm + quantisation, the merged
 * q projection, query RMSNorm + RoPE of the main heads, indexer-q post, the three cache
 * writers, paged MQA logits and top-k - seven launches enqueued on `stream`, nothing
 * allocated, no host synchronisation, so the call can be captured into a CUDA graph.
 *
 * Replaces the part of decode_step (test/test_e2e_decode.py:475-800) between the front GEMM
 * and the sparse attention: qnorm_quant + wq_b_proj_gemm_merged, mqa_logits_fp8_decode_out
 * with its compressor and query bundles, and topk_v2.  Its inputs are what the front GEMM
 * publishes (q_raw, w64, win_y2, the fresh state-ring rows), its outputs what the sparse
 * attention consumes (top-k page indices, normalised and rotated queries, the three caches).
 *
 * The merged weight holds the index heads first: rows [0, index_heads*128) then
 * [.., + main_heads*512), K = q_lora, with fp32 128x128 block scales.  All pointers are
 * device pointers; row arrays (pos, rows, dst) have m entries and the meaning they have in
 * wuda_cache_writers_fp8.  n_compressed[r] is the number of indexer entries of request r
 * INCLUDING the one written this step; block_table maps its logical indexer pages.
 * 1 <= m <= 128.  status_word collects the device status of every kernel of the step.
 */
typedef struct wuda_csa_weights {
    const void* wq_b;          /* e4m3 [index_heads*128 + main_heads*512, q_lora]            */
    const float* wq_b_scales;  /* fp32 [ceil(rows/128), q_lora/128]                           */
    const float* q_norm;       /* fp32 [q_lora]                                               */
    const float* idx_norm;     /* fp32 [128]                                                  */
    const float* main_norm;    /* fp32 [512]                                                  */
    const float* win_norm;     /* fp32 [512]                                                  */
    const float* cos_table;    /* fp32 [max_pos, 32]                                          */
    const float* sin_table;
    int max_pos;
    int q_lora;
    int index_heads;
    int main_heads;            /* heads of 512 in the weight                                  */
    int out_heads;             /* heads of q_main_out (a multiple of main_heads)              */
    float eps;
    int scales_pow2;           /* non-zero: every wq_b scale is a power of two (the reference's UE8M0 scales) and the
                                  projection takes wuda_gemm_fp8_blockscaled_pow2                                  */
} wuda_csa_weights;

typedef struct wuda_csa_caches {
    float* idx_state;          /* fp32 [state_rows_total, 512]; NULL skips the writer          */
    float* main_state;         /* fp32 [state_rows_total, 2048]; NULL skips the writer         */
    int64_t state_rows_total;
    int ring_entries;
    int idx_entries_per_block, cmp_entries_per_block, swa_entries_per_block;
    int idx_num_blocks, cmp_num_blocks, swa_num_blocks;
    int idx_fp4;               /* non-zero: the indexer pool holds MXFP4 records (68 bytes per entry) and the step takes
                                  the FP4 forms: wuda_index_q_post_fp4, wuda_cache_writers_fp4, wuda_mqa_logits_fp4
                                  (index_heads must be 64; workspace.iq_fp8 receives the codes, workspace.w_folded the
                                  query's scale words, and the logits take step.w64 as head weights)              */
    int64_t idx_block_stride_bytes, cmp_block_stride_bytes, swa_block_stride_bytes;
    uint8_t* idx_pool;
    uint8_t* cmp_pool;
    uint8_t* swa_pool;
} wuda_csa_caches;

typedef struct wuda_csa_step {
    const void* q_raw;         /* bf16, row r at r * q_raw_stride elements, q_lora values      */
    int64_t q_raw_stride;
    const float* w64;          /* fp32 [m, index_heads] head weights                           */
    const float* win_y2;       /* fp32 [m, 512]; NULL skips the window writer                  */
    const int64_t* pos;
    const int32_t* q_pos;
    const int64_t* main_state_row;
    const int64_t* idx_state_row;
    const int64_t* idx_dst;
    const int64_t* cmp_dst;
    const int64_t* swa_dst;
    const int32_t* idx_block_table; /* int32 [m, block_table_stride]: pages of the indexer pool */
    const int32_t* cmp_block_table; /* int32 [m, block_table_stride]: pages the top-k positions are
                                       translated with (the compressed-KV pool the attention reads,
                                       test/test_e2e_decode.py:655-657); NULL = idx_block_table  */
    const int32_t* n_compressed;    /* int32 [m]                                               */
    int block_table_stride;
    int topk;
    int64_t logits_stride;
    float* logits;             /* fp32 [m, logits_stride], caller pre-fills -inf if it reads it */
    int32_t* topk_indices;     /* int32 [m, topk] page-transformed                             */
    int32_t* topk_raw;         /* int32 [m, topk] or NULL                                      */
    void* q_main_out;          /* bf16 [m, out_heads, 512] or NULL                             */
} wuda_csa_step;

typedef struct wuda_csa_workspace {
    void* q_fp8;               /* e4m3 [m, q_lora]                                             */
    float* q_scales;           /* fp32 [m, q_lora/128]                                         */
    void* y;                   /* bf16 [m, index_heads*128 + main_heads*512]                   */
    void* iq_fp8;              /* e4m3 [m, index_heads, 128]                                   */
    float* w_folded;           /* fp32 [m, index_heads]                                        */
    void* gemm_scratch;        /* wuda_gemm_fp8_scratch_bytes(m, rows of wq_b), zeroed once    */
    int64_t gemm_scratch_bytes;
    int32_t* status_word;
} wuda_csa_workspace;

int wuda_csa_decode_step(const wuda_csa_weights* weights, const wuda_csa_caches* caches, const wuda_csa_step* step,
                         const wuda_csa_workspace* workspace, int m, void* stream);

/* ------------------------------------------------------------------------------------
 * Paged MQA logits on MXFP4 operands (the FP4 form of the indexer):
 *   logits[b, t] = sum_h weights[b, h] * relu(q[b, h, :] . k[t, :]),  t < context_lens[b]
 * q_fp4 uint8 [batch, 64, 64]: 128 e2m1 values per head, two per byte, low nibble first;
 * q_scales int32 [batch, 64]: four ue8m0 bytes per head, byte g scales values [32g, 32g+32);
 * kv_pages uint8 [num_blocks, page_stride_bytes]: entries_per_block rows of 64 key bytes, then
 * entries_per_block scale words of the same form (68 bytes per token); weights fp32 [batch, 64];
 * context_lens int32 [batch]; block_table int32 [batch, block_table_stride]; logits fp32
 * [batch, logits_stride], only t < context is written (a -inf pre-fill by the caller persists).
 * The block scales are applied inside the tensor core (block-scaled MMA); sums in fp32.
 *
 * Replaces mqa_logits_fp4_decode_out (kernels/mqa_logits_fp4.cu:474-650); formats as
 * test/test_mqa_logits_fp4.py:100-115 and :228-256, arithmetic as its twin (:207-218) over the
 * dequantised values.  A block_table entry outside [0, num_blocks) reads page 0 and is reported
 * as WUDA_DEV_BAD_PAGE_INDEX; a context length beyond logits_stride (or, with pages of 32, 64, 128
 * or 256 entries, beyond block_table_stride * entries_per_block) is cut to that and reported as
 * WUDA_DEV_BAD_CONTEXT_LEN.  Pages of 32, 64, 128 or 256 entries are brought in whole by tensor
 * copies (the fast kernel); any other entries_per_block >= 1 takes a slower gather kernel.
 */
int wuda_mqa_logits_fp4(const void* q_fp4, const void* q_scales, const void* kv_pages, const float* weights,
                        const int32_t* context_lens, const int32_t* block_table, float* logits, int batch,
                        int max_context, int num_blocks, int entries_per_block, int64_t page_stride_bytes,
                        int block_table_stride, int64_t logits_stride, int32_t* status_word, void* stream);

/* ------------------------------------------------------------------------------------
 * Sparse MLA decode attention over gathered FP8 cache records: per request one query token
 * with `heads` heads of 512 dims attends to swa_lengths[b] sliding-window entries and then
 * cmp_lengths[b] top-k compressed entries, each named by a pool entry index
 * (page * entries_per_block + offset; a negative index is skipped).  A pool page holds
 * entries_per_block records of 576 bytes (448 e4m3, then 64 bf16), then entries_per_block
 * groups of 8 scale bytes (7 power-of-two exponents + 1 pad): the record format
 * wuda_cache_writers_fp8 writes.  The value vector of a key is the key itself.
 *   logit[h, t] = softmax_scale * q[h, :] . k[t, :]
 *   out[h, :]   = sum_t exp(logit[h, t]) k[t, :] / (sum_t exp(logit[h, t]) + exp(attn_sink[h]))
 * A request without a valid key gives a zero row.  fp32 logits and sums.  The tensor cores run on
 * fp16 operands: key values e4m3 * 2^E are exact for scale exponents E in [-15, 7] (the cache writers
 * produce E >= -13; E > 7 would mean activations beyond 57344), a scale byte outside that range is
 * clamped into it and reported as WUDA_DEV_MLA_SCALE_RANGE; query and rotary bf16 values are exact
 * in fp16 between 6.1e-5 and 65504 in magnitude; the probabilities are rounded to fp16 before
 * they meet the values.
 *
 * Replaces the third-party call at test/test_e2e_decode.py:719-728 (flash_mla_with_kvcache
 * with indices / extra_indices_in_kvcache / attn_sink); arithmetic as the torch twin
 * ref_flash_attn (test/test_e2e_decode.py:377-392) over deq_model1_row (:346-356) and as
 * origin/kernel.py:276-352.
 *
 * An index at or beyond pages * entries_per_block is skipped and reported as
 * WUDA_DEV_BAD_PAGE_INDEX.  Either pool may be absent (capacity 0).
 */
typedef struct wuda_sparse_mla_args {
    const void* q;               /* bf16 [batch, heads, 512], after RMSNorm and RoPE        */
    const void* swa_pool;        /* uint8 [swa_pages, swa_stride]                           */
    int64_t swa_stride;
    const int32_t* swa_indices;  /* int32 [batch, swa_capacity]                             */
    const int32_t* swa_lengths;  /* int32 [batch], clamped to [0, swa_capacity]             */
    const void* cmp_pool;        /* uint8 [cmp_pages, cmp_stride]                           */
    int64_t cmp_stride;
    const int32_t* cmp_indices;  /* int32 [batch, cmp_capacity]                             */
    const int32_t* cmp_lengths;  /* int32 [batch]                                           */
    const float* attn_sink;      /* fp32 [heads] or NULL                                    */
    void* out;                   /* bf16 [batch, heads, 512]                                */
    void* workspace;             /* wuda_sparse_mla_workspace_bytes(...) bytes, or NULL      */
    int64_t workspace_bytes;
    int32_t swa_pages, swa_entries_per_block, swa_capacity;
    int32_t cmp_pages, cmp_entries_per_block, cmp_capacity;
    int32_t batch, heads;
    float softmax_scale;
} wuda_sparse_mla_args;

/* With a workspace, a small batch is spread over the whole device: several CTAs take runs of a
 * request's keys and a second launch merges their partial sums (same arithmetic, another order of
 * the fp32 additions).  Bytes needed for key_capacity = swa_capacity + cmp_capacity; 0 when the batch
 * fills the device by itself; -1 on bad arguments.  Without a workspace (NULL) requests are never split. */
int64_t wuda_sparse_mla_workspace_bytes(int batch, int heads, int key_capacity);
int wuda_sparse_mla_decode(const wuda_sparse_mla_args* args, int32_t* status_word, void* stream);

/* ------------------------------------------------------------------------------------
 * mHC pre, the head of a half-layer: from the 4 residual streams of each token
 *   r = 1/sqrt(mean(x^2) + rms_eps) over the 4*hidden values;  mix = (x . weight^T) * r   [24]
 *   pre  = sigmoid(mix[0:4] * scale[0] + base[0:4]) + hc_eps
 *   post = 2 * sigmoid(mix[4:8] * scale[1] + base[4:8])
 *   comb = 20 Sinkhorn iterations on softmax_rows(mix[8:24] * scale[2] + base[8:24]) + hc_eps
 *   collapsed = bf16(sum_h pre[h] * x[h, :])
 *   normed    = bf16((collapsed * 1/sqrt(mean collapsed^2 + norm_eps)) * gamma)
 *   x_fp8, x_scales = power-of-two 1x128 quantisation of normed (amax / 448 clamped at 1e-4)
 *
 * Replaces the reference's pair tf32_hc_prenorm_gemm (third party) + hc_reduce_fuse_out
 * (kernels/hc_fused_kernel_tc.cu:420-540) with its Sinkhorn tail (include/front_mixed_gemm.cuh:
 * 438-489); numerics as the torch twin test/test_hc_fused_tc.py:115-136 and origin/model.py:673-681,
 * with fp32 products where the reference's GEMM rounds its operands to TF32.
 *
 *   hidden_states bf16 [m, 4, hidden];  weight fp32 [24, 4*hidden];  base fp32 [24];  scale fp32 [3]
 *   attn_norm_gamma bf16 [hidden], required with normed / x_fp8
 *   pre, post fp32 [m, 4];  comb fp32 [m, 4, 4] ([row][column]);  each nullable
 *   collapsed_bf16, normed_bf16 bf16 [m, hidden];  x_fp8 e4m3 [m, hidden] with x_scales fp32
 *   [m, hidden/128];  each nullable
 *   workspace: wuda_mhc_pre_workspace_bytes(m, hidden) bytes, contents irrelevant
 * hidden % 128 == 0, hidden <= 8192.
 */
int64_t wuda_mhc_pre_workspace_bytes(int m, int hidden);
int wuda_mhc_pre(const void* hidden_states, const float* weight, const float* base, const float* scale,
                 const void* attn_norm_gamma, float hc_eps, float rms_eps, float norm_eps, float* pre, float* post,
                 float* comb, void* collapsed_bf16, void* normed_bf16, void* x_fp8, float* x_scales,
                 void* workspace, int64_t workspace_bytes, int m, int hidden, void* stream);
/* The same operation in the pieces the reference calls one by one (test/test_e2e_decode.py:441-470):
 * wuda_mhc_pre_mix = the split-K mix projection alone (the role of the third-party tf32_hc_prenorm_gemm):
 *   partial sums fp32 [splits][m][25] (24 dot products and the sum of squares) into `workspace`,
 *   splits = ceil(4 * hidden / 512);
 * wuda_mhc_pre_finish = everything behind it (hc_reduce_fuse_out, kernels/hc_fused_kernel_tc.cu:420-520) on
 *   partial sums of ANY split count in that layout, plus mix_out fp32 [m, 24] = the mixes times r (nullable),
 *   which is what the reference's front projection computes post and comb from in its tail;
 * wuda_mhc_tail = that tail alone (include/front_mixed_gemm.cuh:438-489): post fp32 [m, 4] and comb
 *   fp32 [m, 16] from mix_out. */
int wuda_mhc_pre_mix(const void* hidden_states, const float* weight, void* workspace, int64_t workspace_bytes, int m,
                     int hidden, void* stream);
int wuda_mhc_pre_finish(const void* hidden_states, const float* partials, int splits, const float* base,
                        const float* scale, const void* attn_norm_gamma, float hc_eps, float rms_eps, float norm_eps,
                        float* pre, float* post, float* comb, float* mix_out, void* collapsed_bf16, void* normed_bf16,
                        void* x_fp8, float* x_scales, int m, int hidden, void* stream);
int wuda_mhc_tail(const float* mix, const float* base, const float* scale, float hc_eps, float* post, float* comb, int m,
                  void* stream);
/* The origin's hc_split_sinkhorn (origin/kernel.py:355-436) with hc_mult = 4 and 20 iterations: from mixes fp32
 * [tokens, 24] (pre 0..3 | post 4..7 | comb 8..23), scale fp32 [3] and base fp32 [24]:
 *   pre = sigmoid(mix * scale[0] + base) + eps;  post = 2 sigmoid(mix * scale[1] + base);
 *   comb = softmax over each row of (mix * scale[2] + base) + eps, columns normalised, then 19 x (rows, columns),
 *   every division by (sum + eps).  pre, post fp32 [tokens, 4]; comb fp32 [tokens, 4, 4]. */
int wuda_hc_split_sinkhorn(const float* mixes, const float* scale, const float* base, float hc_eps, float* pre, float* post,
                           float* comb, int64_t tokens, void* stream);

/* ------------------------------------------------------------------------------------
 * MoE router: expert logits -> top-k experts and routing weights.
 *   score = softmax (0) | sigmoid (1) | sqrt(softplus) (2) of the logits; the k largest of
 *   score + bias are selected (ties to the lower expert, listed in descending order);
 *   weights = score[selected], divided by their sum unless softmax, times route_scale.
 *
 * Replaces Gate.forward of the origin (origin/model.py:563-584) behind its projection, which is
 * wuda_gemm_bf16 with fp32 output (x bf16 [tokens, dim] x gate weight bf16 [experts, dim]).  The
 * hash-routed form of the first layers (a table lookup by token id) needs no kernel.
 *
 *   logits fp32 [tokens, experts];  bias fp32 [experts], nullable
 *   weights fp32 [tokens, k];  indices int32 [tokens, k];  experts <= 512, k <= 32
 */
int wuda_moe_route(const float* logits, const float* bias, float* weights, int32_t* indices, int tokens, int experts,
                   int k, int score_func, float route_scale, void* stream);

/* ------------------------------------------------------------------------------------
 * Routed experts of the MoE block (origin/model.py:587-644, MoE.forward / Expert.forward), as five
 * calls that never synchronise with the host: the number of row groups stays on the device.
 *
 *   wuda_moe_dispatch            (token, expert) pairs -> rows sorted by expert, each expert's rows
 *                                padded to groups of 16 (a GEMM row tile), stable in token order
 *   wuda_moe_gather_quant_nvfp4  row pair_row[t, j] <- activation of token t, quantised to NVFP4
 *   wuda_gemm_nvfp4_grouped      c[group rows] = a[group rows] . w[expert of the group]^T; with row_token given
 *                                the rows without a token are not stored (their inputs were never written);
 *                                with row_token NULL every row is stored and padding rows hold whatever
 *                                their unwritten inputs give
 *   wuda_moe_swiglu_quant_nvfp4  silu(min(gate, L)) * clamp(up, +-L) * routing weight -> bf16 -> NVFP4
 *   wuda_moe_combine             y[t] = bf16(sum_j out[pair_row[t, j]] (+ shared[t])), slot order
 * The reference has no kernel for this block (its MoE runs through the origin's TileLang GEMMs,
 * which are W4A8 with e8m0 scales); NVFP4 (e2m1, one ue4m3 scale per 16 values, one fp32 scale per
 * tensor) on both operands is the form the benchmark configuration names.
 *
 * Arrays (all device memory): max_groups >= wuda_moe_max_groups(tokens, k, experts);
 *   group_expert int32 [max_groups] (-1 = unused);  num_groups int32 [1]
 *   row_token int32 [max_groups*16] (-1 = padding);  row_weight fp32 [max_groups*16]
 *   pair_row int32 [tokens, k] (row of each pair; -1 for an invalid expert index)
 *   a_fp4 uint8 [max_groups*16, K/2] (two e2m1 per byte, low nibble first); padding rows (row_token < 0)
 *       are never written, neither values nor scales: 16-row groups of a decode batch are mostly padding
 *   a_sf_packed uint8 [max_groups, K/256, 2048]: scale of row r, values [16j, 16j+16) of K block kb at
 *       ((g*K/256 + kb)*2048) + ((j/4)%4)*512 + (r%16)*16 + j%4, g = r/16; ZERO before the first call
 *       (only rows 0..15 of each 128-row image are ever written)
 *   expert weights: w uint8 [experts*n, K/2]; w_sf_packed per expert in the layout of wuda_gemm_nvfp4,
 *       experts concatenated; w_global_scales fp32 [experts]
 * NVFP4 quantisation of 16 values with tensor scale gs: sf = e4m3(min(amax/6/gs, 448)),
 * q = e2m1(x / (sf*gs)) to the nearest code, ties to the smaller magnitude.
 */
int wuda_moe_max_groups(int tokens, int k, int experts);
int wuda_moe_dispatch(const int32_t* indices, const float* weights, int32_t* group_expert, int32_t* num_groups,
                      int32_t* row_token, float* row_weight, int32_t* pair_row, int tokens, int k, int experts,
                      int max_groups, int32_t* status_word, void* stream);
/* Expert parallelism: this rank holds experts [expert_first, expert_first + experts) of experts_total.
 * Pairs routed to another rank's expert are skipped (pair_row -1) without a report; an index outside
 * [0, experts_total) is reported as WUDA_DEV_BAD_EXPERT.  group_expert holds LOCAL expert numbers. */
int wuda_moe_dispatch_range(const int32_t* indices, const float* weights, int32_t* group_expert, int32_t* num_groups,
                            int32_t* row_token, float* row_weight, int32_t* pair_row, int tokens, int k, int experts,
                            int expert_first, int experts_total, int max_groups, int32_t* status_word, void* stream);
int wuda_moe_gather_quant_nvfp4(const void* x_bf16, const int32_t* pair_row, void* a_fp4, void* a_sf_packed,
                                float global_scale, int tokens, int topk, int k, void* stream);
int wuda_gemm_nvfp4_grouped(const void* a, const void* a_sf_packed, float a_global_scale, const void* w,
                            const void* w_sf_packed, const float* w_global_scales, const int32_t* group_expert,
                            const int32_t* num_groups, const int32_t* row_token, void* c_bf16, int max_groups,
                            int experts, int n, int k, void* scratch, int64_t scratch_bytes, int32_t* status_word,
                            void* stream);
/* pair_weight fp32 [tokens, topk]: the routing weights the dispatch was given. */
int wuda_moe_swiglu_quant_nvfp4(const void* h_bf16, const int32_t* pair_row, const float* pair_weight, void* a_fp4,
                                void* a_sf_packed, float global_scale, float swiglu_limit, int tokens, int topk,
                                int inter, void* stream);
int wuda_moe_combine(const void* expert_out_bf16, const int32_t* pair_row, const void* shared_bf16, void* y_bf16,
                     int tokens, int k, int dim, void* stream);
/* The combine step of two expert-parallel ranks (each holds half of the experts, the all-reduce site of
 * origin/model.py:641-642): every rank sums its own experts' rows per token in fp32, pushes the partial
 * row into the peer GPU's inbox over NVLink peer memory, awaits the peer's row and adds it; y is
 * bit-identical on both ranks.  Inboxes: wuda_moe_ep2_inbox_bytes(tokens_max, dim) bytes (tokens_max <= 512,
 * dim <= 8192) from wuda_tp2_alloc, the peer's mapped with wuda_tp2_open; zero-initialised.  `epoch` counts the
 * calls of the pair from 1 and must advance by one on both ranks; a rank may be one call ahead of its peer.
 * epoch = 0 lets the link number its calls itself (a counter in the inbox that the kernel advances), so that the
 * same launch can be replayed from a CUDA graph; a link uses one of the two forms for its whole life.
 * shared_bf16 is added by the rank that passes it (one of the two).  A peer that does not answer within
 * peer_wait_ms leaves WUDA_DEV_TIMEOUT_PEER_FLAG in status_word and the local sum in y. */
int64_t wuda_moe_ep2_inbox_bytes(int tokens_max, int dim);
int wuda_moe_combine_ep2(const void* expert_out_bf16, const int32_t* pair_row, const void* shared_bf16, void* y_bf16,
                         int tokens, int k, int dim, void* my_inbox, void* peer_inbox, int tokens_max, int epoch,
                         int peer_wait_ms, int32_t* status_word, void* stream);

/* ------------------------------------------------------------------------------------
 * mHC post mix, the last op of an attention half-layer:
 *   output[t, j, d] = post[t, j] * attention_out[t, d] + sum_i comb[t, i, j] * residual[t, i, d]
 *
 * Replaces mhc_post_out / mhc_post_run (kernels/mhc_post.cu:41-99 kernel, :102-137 validate
 * and run; include/mhc_post.cuh:16-33 argument block).  fp32 arithmetic in the reference
 * kernel's order: one rounded product, then fused multiply-adds over i = 0..3, then bf16
 * round-to-nearest-even - results are bit-identical to that kernel.
 *
 *   attention_out bf16 [m, hidden];  residual bf16 [m, 4, hidden];  post fp32 [m, 4]
 *   comb fp32 [m, 4, 4] indexed [input stream i][output stream j];  output bf16 [m, 4, hidden]
 * m >= 1, hidden % 8 == 0 (7168 in the model), every buffer 16-byte aligned, output must not
 * overlap any input (checked, as the reference checks it).  The reference also refuses
 * m > 128, its decode batch limit; this entry takes any m.
 */
int wuda_mhc_post(const void* attention_out, const void* residual, const float* post, const float* comb,
                  void* output, int m, int hidden, void* stream);

/* ------------------------------------------------------------------------------------
 * SwiGLU of a dense (shared) expert + 1x128 FP8 quantisation in one pass:
 *   y = bf16(silu(min(gate, L)) * clamp(up, -L, L)),  h = [gate | up] bf16 [rows, 2*inter];  L = 0: no clamp
 * Expert.forward of the origin (origin/model.py:596-606) between its w1|w3 and w2 projections,
 * which are wuda_gemm_fp8_blockscaled calls.  Outputs as wuda_rmsnorm_quant_fp8; inter % 128 == 0.
 */
int wuda_swiglu_quant_fp8(const void* h_bf16, void* y_bf16, void* y_fp8, float* y_scales, int rows, int inter,
                          float swiglu_limit, int scale_mode, void* stream);

/* ------------------------------------------------------------------------------------
 * Block-scaled FP8 GEMM for decode-sized M:
 *
 *   c[m, n] = bf16( sum_kb a_s[m, kb] * w_s[n / 128, kb] * sum_{k in block kb} a[m, k] * w[n, k] )
 *
 * Each 128-wide K block is accumulated in fp32 and promoted with its scales into a second
 * fp32 accumulator, as the origin's fp8_gemm does (origin/kernel.py:203-273; Python
 * signature fp8_gemm(a, a_s, b, b_s) at :257).  It is the generic form of the reference's
 * fixed-shape wq_b / wo_b projections (kernels/wq_b_fp8_gemm.cu:849-1365,
 * test/o_proj_csa.py:454-480).
 *
 *   a         e4m3 [m, k], 16-byte aligned;   a_scales fp32 [m, k/128]
 *   w         e4m3 [n, k], 16-byte aligned;   w_scales fp32 [ceil(n/128), k/128]
 *   c_bf16    bf16 [m, n];   1 <= m <= 256, k % 128 == 0
 *   scratch   device memory of at least wuda_gemm_fp8_scratch_bytes(m, n) bytes, 256-byte
 *             aligned, ZERO before the first call; the kernel leaves it zero again, so the
 *             same scratch can serve call after call (calls that share it must not overlap
 *             on the GPU).  It holds the fp32 partial tiles of weight tiles whose K range is
 *             split across SMs.
 */
/* The GEMM launches the CALLING THREAD makes from now on (FP8, BF16, NVFP4) cover at most max_sms SMs; 0 gives
 * them the whole device again.  Returns the previous setting.  For callers that run two launches side by side on
 * two streams: a GEMM of a few dozen MB is bound by its fixed latencies rather than by bandwidth, so two of them
 * on disjoint halves of the device finish sooner than one after the other (a GEMM launched on every SM leaves no
 * room for anything beside it).  The number of CTAs decides how a weight tile's K range is cut and therefore the
 * order of the fp32 additions: results are reproducible for a given setting, not across settings. */
int wuda_gemm_sm_limit(int max_sms);
int64_t wuda_gemm_fp8_scratch_bytes(int m, int n);
int wuda_gemm_fp8_blockscaled(const void* a, const float* a_scales, const void* w, const float* w_scales,
                              void* c_bf16, int m, int n, int k, void* scratch, int64_t scratch_bytes,
                              int32_t* status_word, void* stream);

/* ------------------------------------------------------------------------------------
 * Grouped block-scaled FP8 GEMM: `groups` independent projections in one launch,
 *   c[m, g * n_per_group + j] = sum_k a[m, g * k + kk] * w[g * n_per_group + j, kk]   (scaled as above)
 * i.e. group g multiplies its own k columns of the activation row by its own n_per_group weight
 * rows - the low-rank output projection wo_a of the reference ([groups, 1024, 4096] applied to the
 * attention output viewed as [M, groups, 4096]; test/o_proj_csa.py:319-494, origin/model.py:520-540).
 *
 *   a e4m3 [m, groups * k];  a_scales fp32 [m, groups * k / 128]
 *   w e4m3 [groups * n_per_group, k];  w_scales fp32 [groups * n_per_group / 128, k / 128]
 *   c_bf16 bf16 [m, groups * n_per_group];  n_per_group % 128 == 0;  scratch as for
 *   wuda_gemm_fp8_blockscaled with n = groups * n_per_group.
 */
int wuda_gemm_fp8_grouped(const void* a, const float* a_scales, const void* w, const float* w_scales, void* c_bf16,
                          int m, int n_per_group, int k, int groups, void* scratch, int64_t scratch_bytes,
                          int32_t* status_word, void* stream);

/* ------------------------------------------------------------------------------------
 * The same two GEMMs for scales that are exact powers of two (what the reference's checkpoints and its
 * quantisers hold: UE8M0 scales, kernels/wq_b_fp8_gemm.cu:139-183, include/cluster_mma_fp8.cuh:144-301).
 * The scales are then applied inside the tensor core (tcgen05.mma kind::mxf8f6f4.block_scale, exponent
 * bytes in tensor memory), a weight tile accumulates over its whole K range there, and the per-block
 * promotion on CUDA cores that bounds the general entry points from 64 rows up is gone.  Arguments,
 * layouts, scratch (wuda_gemm_fp8_scratch_bytes) and results as for wuda_gemm_fp8_blockscaled /
 * wuda_gemm_fp8_grouped, with the products added in fp32 inside the tensor core instead of block by block.
 * A scale that is not a power of two is truncated to the one below and reported as
 * WUDA_DEV_SCALE_NOT_POW2; a zero scale reads as 2^-127.
 */
int wuda_gemm_fp8_blockscaled_pow2(const void* a, const float* a_scales, const void* w, const float* w_scales,
                                   void* c_bf16, int m, int n, int k, void* scratch, int64_t scratch_bytes,
                                   int32_t* status_word, void* stream);
int wuda_gemm_fp8_grouped_pow2(const void* a, const float* a_scales, const void* w, const float* w_scales, void* c_bf16,
                               int m, int n_per_group, int k, int groups, void* scratch, int64_t scratch_bytes,
                               int32_t* status_word, void* stream);

/* ------------------------------------------------------------------------------------
 * FP8 activations x 4-bit weights, C = A . W^T (origin/kernel.py:441-536, fp4_gemm: the format of the origin's
 * routed experts, origin/model.py:108-135,623).
 *
 *   a        e4m3 [m, k], a_scales fp32 [m, k/128]: one POWER-OF-TWO scale per row and 128 K-elements
 *            (act_quant with scale_fmt "ue8m0"; a float8_e8m0fnu tensor converts exactly)
 *   w_packed e2m1 [n, k/2] bytes, the element of the lower K index in the low nibble (torch.float4_e2m1fn_x2);
 *            32-byte aligned
 *   w_sf     [n, k/32] exponent bytes (torch.float8_e8m0fnu): weight (row, j) = code * 2^(w_sf[row, j/32] - 127)
 *   c_bf16   bf16 [m, n];  0 <= m <= 256 (above 128 rows: two passes), k % 128 == 0
 *   scratch  as for wuda_gemm_fp8_blockscaled (wuda_gemm_fp8_scratch_bytes(m, n))
 *
 * The kernel of wuda_gemm_fp8_blockscaled_pow2 with the weight operand read as e2m1 (the tile is 8 KB of global
 * memory, expanded by the copy engine to the padded form the tensor core wants) and one exponent byte per weight
 * row and 32 K-elements in tensor memory.  The products are added in fp32 inside the tensor core; the origin adds
 * them 32-block by 32-block on CUDA cores: same value up to fp32 summation order.
 */
int wuda_gemm_fp8_fp4_pow2(const void* a, const float* a_scales, const void* w_packed, const void* w_sf, void* c_bf16,
                           int m, int n, int k, void* scratch, int64_t scratch_bytes, int32_t* status_word,
                           void* stream);

/* ------------------------------------------------------------------------------------
 * Block-wise FP4 quantisation of bf16 rows (origin/kernel.py:126-200, fp4_act_quant): per 32 values
 * amax = max(max|x|, 6 * 2^-126), scale = 2^ceil(log2(amax / 6)), code = e2m1(x / scale) rounded to nearest even.
 *
 *   x_bf16  bf16 [rows, cols] with row_stride elements between rows (row_stride % 8 == 0), cols % 32 == 0
 *   inplace == 0:  codes u8 [rows, cols/2] (lower index in the low nibble), scales u8 [rows, cols/32] (exponent
 *                  bytes, float8_e8m0fnu)
 *   inplace != 0:  x is overwritten with code * scale as bf16 (the quantise-dequantise of origin/model.py:370,416);
 *                  codes and scales may be NULL
 */
int wuda_fp4_act_quant(const void* x_bf16, int64_t row_stride, void* codes, void* scales, int inplace, int64_t rows,
                       int cols, void* stream);

/* Sum of squares of every 512-value head of bf16 rows (head_ssq_standalone, kernels/wq_b_fp8_gemm.cu:101-123,
 * 1548-1566): y bf16 [rows, heads * 512] with row_stride elements between rows -> ssq fp32 [rows, heads].  Lane l of
 * a warp chains fused multiply-adds over values [16 l, 16 l + 16) of a head; a butterfly over lane distances
 * 16, 8, 4, 2, 1 adds the lanes: the reference kernel's order, so the sums are identical bit for bit. */
int wuda_head_ssq(const void* y_bf16, int64_t row_stride, float* ssq, int64_t rows, int heads, void* stream);

/* ------------------------------------------------------------------------------------
 * BF16 GEMM for decode-sized M:  c[m, n] = sum_k a[m, k] * w[n, k], fp32 accumulation, written
 * as bf16 or (c_is_fp32 != 0) as fp32.
 *
 * Carries the projections the reference keeps in BF16: the BF16 segment of the front mixed GEMM
 * (kernels/front_mixed_gemm_csa_swapab.cu:10-258), whose outputs feed fp32 state, and the
 * origin's `linear` on bf16 weights (origin/model.py:108-120).
 *
 *   a_bf16 bf16 [m, k];  w_bf16 bf16 [n, k];  c bf16 or fp32 [m, n];  1 <= m <= 128, k % 64 == 0
 *   scratch: wuda_gemm_bf16_scratch_bytes(m, n) bytes, 256-byte aligned, zero before the first
 *   call (left zero again), not shared by calls that overlap on the GPU.
 */
int64_t wuda_gemm_bf16_scratch_bytes(int m, int n);
int wuda_gemm_bf16(const void* a_bf16, const void* w_bf16, void* c, int c_is_fp32, int m, int n, int k,
                   void* scratch, int64_t scratch_bytes, int32_t* status_word, void* stream);

/* ------------------------------------------------------------------------------------
 * FRONT-EMIT: scatters the front projection's outputs of a decode step.  The front GEMM yields
 * per token [q 1536 | win 512] (FP8 segment, bf16 out) and [main 2048 | idx 512 | w64 64] (BF16
 * segment, fp32 out of wuda_gemm_bf16):
 *   win_y2[t]  = fp32 of y8[t, 1536:2048]
 *   main_state[main_state_row[t]] = y16[t, 0:2048],    + ape[pos % 4] on its second half
 *   idx_state[idx_state_row[t]]   = y16[t, 2048:2560], + idx_ape[pos % 4] on its second half
 *   w64[t]     = fp32(bf16(y16[t, 2560:2624]))
 *
 * Replaces the side-channel epilogue of front_mixed_gemm_csa_swapab (FrontEmitArgs,
 * include/front_mixed_gemm.cuh:390-425; its test stand-in publish_fresh,
 * test/test_wq_b_fp8_gemm.py:539-547).  Rows < 0 are skipped, rows >= state_rows_total are
 * skipped and reported in status_word.  Each output group is optional (NULL).
 *
 *   y8_bf16 bf16 [m, 2048];  y16_f32 fp32 [m, 2624];  pos int64 [m]
 *   main_state fp32 [state_rows_total, 2048], ape fp32 [4, 1024];  idx_state fp32
 *   [state_rows_total, 512], idx_ape fp32 [4, 256];  win_y2 fp32 [m, 512];  w64 fp32 [m, 64]
 */
int wuda_front_emit(const void* y8_bf16, const float* y16_f32, const int64_t* pos, float* main_state,
                    const float* ape, const int64_t* main_state_row, float* idx_state, const float* idx_ape,
                    const int64_t* idx_state_row, float* win_y2, float* w64, int64_t state_rows_total, int m,
                    int32_t* status_word, void* stream);

/* ------------------------------------------------------------------------------------
 * NVFP4 block-scaled GEMM for decode-sized M:
 *
 *   c[m, n] = bf16( a_global_scale * w_global_scale *
 *                   sum_k (e2m1 a[m,k] * ue4m3 a_sf[m,k/16]) * (e2m1 w[n,k] * ue4m3 w_sf[n,k/16]) )
 *
 * Operands are packed e2m1 (two per byte, low nibble = even k; value table and rounding as the
 * reference's FP4 helpers, origin/convert.py:11-14, test/test_mqa_logits_fp4.py:69-115).  The
 * reference has no NVFP4 GEMM: its fp4_gemm (origin/kernel.py:441-536) is FP8-activation x
 * FP4-weight with 1x32 e8m0 scales; this entry is the 16-element-ue4m3 + per-tensor-fp32 form.
 *
 *   a  uint8 [m, k/2];  w  uint8 [n, k/2];  1 <= m <= 256 (above 128 rows: two passes over the weights), k % 256 == 0; 16-byte aligned
 *   a_sf_packed, w_sf_packed: the ue4m3 scale bytes in tensor-core order: per 128 rows x 256 K one
 *      2048-byte block [K/64 step (4)][row % 32 (32)][row / 32 (4)][scale of the step (4)],
 *      blocks ordered [row tile][k / 256]; rows beyond m / n are zero-padded to a multiple of 128
 *   scratch: wuda_gemm_nvfp4_scratch_bytes(m, n) bytes, 256-byte aligned, zero before the first
 *      call; left zero by the kernel
 */
int64_t wuda_gemm_nvfp4_scratch_bytes(int m, int n);
int wuda_gemm_nvfp4(const void* a, const void* a_sf_packed, float a_global_scale, const void* w,
                    const void* w_sf_packed, float w_global_scale, void* c_bf16, int m, int n, int k,
                    void* scratch, int64_t scratch_bytes, int32_t* status_word, void* stream);

/* ------------------------------------------------------------------------------------
 * Two-rank tensor-parallel FP8 GEMM with the all-reduce fused into its epilogue.
 *
 * The K dimension is split across two GPUs (a row-parallel linear, origin/model.py:166-180:
 * per-rank partial products summed in fp32, then cast).  Each rank calls this function with
 * its K slice; finished fp32 tiles are stored directly into the peer GPU's inbox over NVLink
 * and the peer's tiles are added from the local inbox, so both ranks end with the same bf16
 * c = bf16(partial_0 + partial_1).  No NCCL call is involved.  The reference's megakernel has
 * no such collective (it fabricates the sum, test/test_e2e_decode.py:186-194).
 *
 * An inbox is device memory of wuda_tp2_inbox_bytes(m, n) bytes created by wuda_tp2_alloc,
 * which also returns a 64-byte CUDA IPC handle; the peer process maps it with wuda_tp2_open
 * (the handles travel by any host-side channel).  `epoch` is the call's sequence number: it
 * must start at 1 and grow by one per call, identically on both ranks; epoch = 0 lets the link
 * number its calls itself (a counter in the inbox that the kernel advances), so that the same
 * launch can be replayed from a CUDA graph - a link uses one of the two forms for its whole
 * life.  m <= 128 (larger batches: several calls).  A wait for the peer
 * that exceeds peer_wait_ms ends the kernel with WUDA_DEV_TIMEOUT_PEER_FLAG in status_word
 * (c is then not fully written); nothing traps or hangs.
 */
int64_t wuda_tp2_inbox_bytes(int m, int n);
int wuda_tp2_alloc(int64_t bytes, void** local_base, unsigned char* ipc_handle_64);
int wuda_tp2_open(const unsigned char* ipc_handle_64, void** peer_base);
int wuda_tp2_close(void* peer_base);
int wuda_tp2_free(void* local_base);
int wuda_gemm_fp8_blockscaled_tp2(const void* a, const float* a_scales, const void* w,
                                  const float* w_scales, void* c_bf16, int m, int n, int k_local,
                                  void* scratch, int64_t scratch_bytes, void* my_inbox, void* peer_inbox,
                                  int epoch, int peer_wait_ms, int32_t* status_word, void* stream);

/* The same GEMM for callers that cannot provide scratch memory and must not trigger a device
 * allocation (a process that has handed all device memory to its own pool, a loop in which
 * cudaMalloc would stall the device).  No counterpart in the reference.  The scratch is a fixed
 * 6,292,480-byte array inside the library's device image, present on every GPU that loads the
 * library until the process exits; the entry point allocates nothing and frees nothing.
 * Limits and rules: m <= 64 (larger m is refused with WUDA_ERR_UNSUPPORTED); calls on one
 * device share the array, so they must not overlap on the GPU (issue them on one stream, or
 * order the streams); the first call on each device looks the array's address up and should
 * therefore be made once before any stream capture begins.  Results are identical to
 * wuda_gemm_fp8_blockscaled.
 */
int wuda_gemm_fp8_blockscaled_noalloc(const void* a, const float* a_scales, const void* w,
                                      const float* w_scales, void* c_bf16, int m, int n, int k,
                                      int32_t* status_word, void* stream);

/* ------------------------------------------------------------------------------------
 * The whole decode layer as one call: the origin's Block.forward (origin/model.py:688-700) for one token
 * per request.  The attention half is the reference's decode_step (test/test_e2e_decode.py:475-800: mHC
 * pre, front projection with its scatter into the state rings, the indexer half-step of
 * wuda_csa_decode_step, sparse MLA attention, the output projection chain of test/o_proj_csa.py:319-494,
 * mHC post); the feed-forward half (mHC pre with the ffn weights, ffn RMSNorm, router, shared expert, routed
 * NVFP4 experts, mHC post; origin/model.py:546-644) has no counterpart in the reference's megakernel.
 * Every stage is one of the entry points above, enqueued in order on `stream`: no allocation, no host
 * synchronisation, capturable into a CUDA graph (one call outside a capture first: kernel attributes are
 * set on first use).
 *
 * Tensor-parallel pair: give every rank its share - csa.wq_b with its main heads only, wo_a with its
 * groups, wo_b with its K columns, attn_sink of its heads, its routed experts (expert_first,
 * experts_local), its half of the shared expert's intermediate columns - and the two exchange buffers
 * (wuda_tp2_inbox_bytes(m_max, hidden) and wuda_moe_ep2_inbox_bytes(m_max, hidden) bytes from wuda_tp2_alloc,
 * the peer's opened with wuda_tp2_open).  wo_b then sums over the pair inside its epilogue and the combine
 * step exchanges the partial rows, both over NVLink peer memory with the call numbering kept on the device
 * (epoch 0 of those entry points); both ranks must make the same calls.  NULL inboxes: one GPU.
 *
 * workspace: wuda_layer_workspace_bytes(weights, m_max, topk, logits_stride, window) bytes, 256-byte
 * aligned, zeroed once before the first call (it holds the GEMMs' stream-K flags); its layout depends on
 * m_max only.  wuda_layer_workspace_offset names where the stages' results lie in it ("logits",
 * "topk_indices", "topk_raw", "q_main", "mla_out", "attn_out", "gate_logits", "route_indices",
 * "route_weights", "moe_out", "front_out", "q_proj", "iq_fp8", "w_folded", "win_y2", "w64"), for callers that
 * read them.
 */
typedef struct wuda_layer_weights {
    wuda_csa_weights csa;           /* q projection, norm weights, rotary tables                            */
    const float* attn_hc_weight;    /* fp32 [24, 4 * hidden]                                                */
    const float* attn_hc_base;      /* fp32 [24]                                                            */
    const float* attn_hc_scale;     /* fp32 [3]                                                             */
    const void* attn_norm;          /* bf16 [hidden]                                                        */
    const void* front_w8;           /* e4m3 [2048, hidden], fp32 128x128 scales                             */
    const float* front_w8_scales;
    const void* front_w16;          /* bf16 [2624, hidden]                                                  */
    const float* ape;               /* fp32 [4, 1024]                                                       */
    const float* idx_ape;           /* fp32 [4, 256]                                                        */
    const void* wo_a;               /* e4m3 [o_groups, 1024, heads / o_groups * 512]                        */
    const float* wo_a_scales;
    const void* wo_b;               /* e4m3 [hidden, o_groups * 1024]                                       */
    const float* wo_b_scales;
    const float* attn_sink;         /* fp32 [csa.out_heads]                                                 */
    const float* ffn_hc_weight;     /* as the attention-side three                                          */
    const float* ffn_hc_base;
    const float* ffn_hc_scale;
    const void* ffn_norm;           /* bf16 [hidden]                                                        */
    const void* gate_weight;        /* bf16 [experts_total, hidden]                                         */
    const float* gate_bias;         /* fp32 [experts_total] or NULL                                         */
    const void* w13;                /* packed e2m1 [experts_local, 2 * inter, hidden / 2]  (w1 rows, then w3) */
    const void* w13_sf;             /* their ue4m3 scales in tensor-core order, per expert                  */
    const float* w13_gs;            /* fp32 [experts_local] tensor scales                                   */
    const void* w2;                 /* packed e2m1 [experts_local, hidden, inter / 2]                       */
    const void* w2_sf;
    const float* w2_gs;
    const void* shared_w13;         /* e4m3 [2 * shared_inter, hidden] or NULL: no shared expert            */
    const float* shared_w13_scales;
    const void* shared_w2;          /* e4m3 [hidden, shared_inter]                                          */
    const float* shared_w2_scales;
    int hidden;
    int o_groups;
    int experts_total, expert_first, experts_local;
    int moe_topk;
    int score_func;                 /* 0 softmax, 1 sigmoid, 2 sqrt(softplus)                               */
    int inter;
    int shared_inter;
    float route_scale;
    float swiglu_limit;
    float act_scale_in, act_scale_mid;  /* tensor scales of the NVFP4 activations                           */
    float softmax_scale;
    float hc_eps, rms_eps, norm_eps;
    int fp8_scales_pow2;            /* non-zero: the FP8 weights' scales are powers of two; projections whose shape gains
                                       from it (wo_a) take the *_pow2 GEMMs                                        */
} wuda_layer_weights;

typedef struct wuda_layer_state {
    wuda_csa_caches caches;
    void* workspace;
    int64_t workspace_bytes;
    void* tp_my_inbox;              /* wo_b exchange of a tensor-parallel pair, or NULL                     */
    void* tp_peer_inbox;
    void* ep_my_inbox;              /* combine exchange of the pair, or NULL                                */
    void* ep_peer_inbox;
    int ep_tokens_max;              /* the row count the combine inboxes were sized for                     */
    int peer_wait_ms;               /* limit of one wait for the peer, [1, 10000]                           */
    int m_max;                      /* rows the workspace was laid out for, <= 128                          */
    int reserved;
    int32_t* status_word;
} wuda_layer_state;

typedef struct wuda_layer_step {
    const void* hidden_in;          /* bf16 [m, 4, hidden] residual streams                                 */
    void* hidden_out;               /* bf16 [m, 4, hidden]                                                  */
    const int64_t* pos;             /* per-request arrays as in wuda_csa_step                               */
    const int32_t* q_pos;
    const int64_t* main_state_row;
    const int64_t* idx_state_row;
    const int64_t* idx_dst;
    const int64_t* cmp_dst;
    const int64_t* swa_dst;
    const int32_t* idx_block_table;
    const int32_t* cmp_block_table;
    const int32_t* n_compressed;
    const int32_t* swa_indices;     /* int32 [m, window] entries of the window pool                         */
    const int32_t* swa_lengths;     /* int32 [m]                                                            */
    const int32_t* cmp_lengths;     /* int32 [m]: min(n_compressed, topk)                                   */
    int block_table_stride;
    int topk;
    int window;
    int reserved;
    int64_t logits_stride;
} wuda_layer_step;

int64_t wuda_layer_workspace_bytes(const wuda_layer_weights* weights, int m_max, int topk, int64_t logits_stride,
                                   int window);
int64_t wuda_layer_workspace_offset(const wuda_layer_weights* weights, int m_max, int topk, int64_t logits_stride,
                                    int window, const char* name);
int wuda_layer_decode(const wuda_layer_weights* weights, const wuda_layer_state* state, const wuda_layer_step* step,
                      int m, void* stream);

/* ------------------------------------------------------------------------------------
 * Host-buffer form of the indexer step: paged MQA logits, then top-k with the request's
 * block table as the page table (page_size = entries_per_block).
 *
 * The reference has no host-buffer call; this is the form a host program uses when its
 * tensors live in host memory (the reference's decode_step keeps them on the device,
 * test/test_e2e_decode.py:537-660).  A plan owns device staging buffers sized for
 * max_batch requests; wuda_indexer_topk_host copies the *_host inputs to the device on
 * `stream`, runs both kernels, copies page_indices [batch*next_n, k] (and the logits
 * [batch*next_n, logits_stride] when logits_host != NULL) back, and synchronises the
 * stream - on every path, also after a refused launch, so the host buffers are free when
 * the call returns.  Host buffers should be page-locked for full copy bandwidth.
 * kv_pages_host == NULL skips the upload of the key pool: the pages of the previous call
 * on this plan stay in place (a decode server changes a few pages per step, not the pool).
 * The plan belongs to the device that was current when it was created; a call with another
 * device current is refused.  A non-zero device status is returned as WUDA_ERR_DEVICE_STATUS.
 */
typedef struct wuda_indexer_plan wuda_indexer_plan;
int wuda_indexer_plan_create(wuda_indexer_plan** plan, int max_batch, int next_n, int num_blocks,
                             int entries_per_block, int64_t page_stride_bytes,
                             int block_table_stride, int64_t logits_stride, int k);
int wuda_indexer_plan_destroy(wuda_indexer_plan* plan);
int wuda_indexer_topk_host(wuda_indexer_plan* plan, const void* q_host, const void* kv_pages_host,
                           const float* weights_host, const int32_t* context_lens_host,
                           const int32_t* block_table_host, int32_t* page_indices_host,
                           float* logits_host, int batch, void* stream);
/* The same call for a pool that lives on the device between steps: only the pages listed in dirty_pages_host
 * (n_dirty page numbers; runs of consecutive numbers travel as one copy) are taken from kv_pages_host, the rest of
 * the pool is what earlier calls on this plan left there.  A decode step appends a token or two per request, i.e.
 * touches one page per request.  With a list (even an empty one) nothing else of the pool is uploaded; with
 * dirty_pages_host == NULL the call is wuda_indexer_topk_host. */
int wuda_indexer_topk_host_pages(wuda_indexer_plan* plan, const void* q_host, const void* kv_pages_host,
                                 const int32_t* dirty_pages_host, int n_dirty, const float* weights_host,
                                 const int32_t* context_lens_host, const int32_t* block_table_host,
                                 int32_t* page_indices_host, float* logits_host, int batch, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* WUDA_B200_H_ */
