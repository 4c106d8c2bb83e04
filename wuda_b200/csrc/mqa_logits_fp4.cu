// Paged MQA logits on MXFP4 keys and queries (the FP4 form of the indexer):
//   logits[b, t] = sum_h w[b, h] * relu( sum_d q[b, h, d] * k[t, d] ),   t < context_lens[b]
// q and k are packed e2m1 (two values per byte, low nibble first) with one ue8m0 scale byte per 32
// values (four per 128-dim row, packed little-endian in an int32); a key page holds
// entries_per_block rows of 64 key bytes, then entries_per_block scale words (68 B per token).
// Replaces mqa_logits_fp4_decode_out (dsv4_megakernel/megakernel/kernels/mqa_logits_fp4.cu:474-650);
// formats as dsv4_megakernel/megakernel/test/test_mqa_logits_fp4.py:100-115 (per_token_cast_to_fp4) and
// :228-256 (build_paged_cache), arithmetic as its twin ref_fp8_mqa_logits (:207-218) over the
// dequantised values.
//
// A CTA of 128 threads serves one request and walks its tiles of 128 tokens with the grid's stride; four
// CTAs share an SM (each holds 128 tensor-memory columns) and overlap one another.  The request's 64
// query rows, their scale words and the head weights are loaded once.  A thread owns one token row of a
// tile: it keeps the rows of the CTA's next two tiles in registers (plain 16-byte loads; per-thread
// cp.async copies were tried and throttled in the load/store queue), stores the current row into the
// unswizzled K-major operand layout, and after the MMAs reduces its row of the accumulator.  Per tile
// the scale words go to tensor memory (tcgen05.cp) and two block-scaled MMAs (kind::mxf4nvf4,
// scale_vec::2X, ue8m0) apply them inside the tensor core; the epilogue is relu, head weight, sum over
// the 64 head columns.
#include <climits>

#include "host.h"
#include "ptx.cuh"

namespace wuda {
namespace mqa4 {

constexpr int kHeads = 64;
constexpr int kDim = 128;
constexpr int kRowBytes = kDim / 2;    // 64
constexpr int kTile = 128;             // tokens per CTA (UMMA M)
constexpr int kThreads = 128;
constexpr uint32_t kTmemCols = 128;    // 64 accumulator columns, 4 + 4 scale columns
constexpr uint32_t kColSfa = 64, kColSfb = 68;
constexpr int kPadBytes = 40 * 1024;     // unused dynamic shared memory: 14 + 40 KB per CTA, four CTAs per SM
constexpr int kStages = 1;             // one key tile in shared memory; the next two wait in registers

// shared memory (static): operands as [16-byte K chunk][row][16 B], scale images of 512 B
struct Smem {
    alignas(128) uint8_t keys[kStages][4 * kTile * 16];   // 8 KB
    alignas(128) uint8_t query[4 * kHeads * 16];          // 4 KB
    alignas(128) uint32_t key_scales[kStages][128];       // [row % 32][row / 32]
    alignas(128) uint32_t query_scales[128];
    alignas(16) float weights[kHeads];
    alignas(8) uint64_t mma_done;
    uint32_t tmem_slot;
    int abort_flag;
};

struct Params {
    const uint8_t* q;            // [batch, 64, 64]
    const uint32_t* q_scales;    // [batch, 64]
    const uint8_t* kv_pages;     // [num_blocks, page_stride]
    const float* weights;        // [batch, 64]
    const int32_t* context_lens; // [batch]
    const int32_t* block_table;  // [batch, bt_stride]
    float* logits;               // [batch, logits_stride]
    int32_t* status;
    int64_t page_stride, logits_stride;
    int num_blocks, epb, bt_stride;
    int epb_shift;               // log2(epb) when epb is a power of two, else -1
};

__device__ __forceinline__ void umma_mxf4_2x(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                             uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::2X "
        "[%0], %1, %2, %3, [%5], [%6], p;\n\t"
        "}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
        : "memory");
}

constexpr int kNoToken = INT_MIN;   // fetch_page's answer for a token at or beyond the context

// The block-table entry of token t of request b, unchecked (kNoToken beyond the context).  Requested one
// tile before the copies that depend on it are started and looked at only then, so nothing waits for it.
__device__ __forceinline__ int fetch_page(const Params& p, int b, int t, int ctx) {
    if (t >= ctx) return kNoToken;
    const int slot = p.epb_shift >= 0 ? t >> p.epb_shift : t / p.epb;
    return slot < p.bt_stride ? __ldg(p.block_table + static_cast<int64_t>(b) * p.bt_stride + slot) : -1;
}

struct KeyRow {
    uint4 k[4];
    uint32_t scale;
};

// Loads token row `t` (block-table entry `phys`, unchecked) into registers; zeros beyond the context.
__device__ __forceinline__ KeyRow load_row(const Params& p, int t, int phys) {
    KeyRow r;
#pragma unroll
    for (int c = 0; c < 4; ++c) r.k[c] = make_uint4(0, 0, 0, 0);
    r.scale = 0;
    if (phys == kNoToken) return r;
    if (phys < 0 || phys >= p.num_blocks) {   // a bad entry reads page 0 and is reported
        if (p.status) atomicCAS(p.status, 0, static_cast<int>(kDevBadPageIndex));
        phys = 0;
    }
    const int off = p.epb_shift >= 0 ? t & (p.epb - 1) : t % p.epb;
    const uint8_t* page = p.kv_pages + static_cast<int64_t>(phys) * p.page_stride;
    const uint4* row = reinterpret_cast<const uint4*>(page + static_cast<int64_t>(off) * kRowBytes);
#pragma unroll
    for (int c = 0; c < 4; ++c) r.k[c] = __ldcg(row + c);   // pool pages may have been written by a kernel of the same chain
    r.scale = __ldcg(reinterpret_cast<const uint32_t*>(page + static_cast<int64_t>(p.epb) * kRowBytes) + off);
    return r;
}

__global__ void __launch_bounds__(kThreads) mqa_logits_fp4_kernel(const Params p) {
    __shared__ Smem sm;
    const int b = blockIdx.y;
    const int tid = threadIdx.x, warp = tid >> 5;
    pdl_launch_dependents();
    pdl_wait();   // nothing of global memory is touched before the kernel ahead has finished
    const int ctx = __ldg(p.context_lens + b);
    const int tiles = (ctx + kTile - 1) / kTile;
    if (static_cast<int>(blockIdx.x) >= tiles) return;   // whole CTA: no tile of this request is left for it

    if (tid == 0) {
        sm.abort_flag = 0;
        mbar_init(smem_u32(&sm.mma_done), 1);
        fence_mbar_init();
    }
    if (warp == 0) {
        tmem_alloc(smem_u32(&sm.tmem_slot), kTmemCols);
        tmem_relinquish();
    }
    // the request's query rows, scale words and head weights, once per CTA
    {
        uint32_t qs = 0x7f7f7f7fu;
        if (tid < kHeads) {
            const uint4* row = reinterpret_cast<const uint4*>(p.q + (static_cast<int64_t>(b) * kHeads + tid) * kRowBytes);
#pragma unroll
            for (int c = 0; c < 4; ++c) *reinterpret_cast<uint4*>(sm.query + (c * kHeads + tid) * 16) = __ldcg(row + c);
            qs = __ldcg(p.q_scales + static_cast<int64_t>(b) * kHeads + tid);
            sm.weights[tid] = __ldcg(p.weights + static_cast<int64_t>(b) * kHeads + tid);
        }
        sm.query_scales[(tid & 31) * 4 + (tid >> 5)] = qs;
    }
    const int stride_tokens = gridDim.x * kTile;
    const int t0 = blockIdx.x * kTile + tid;
    KeyRow r0 = load_row(p, t0, fetch_page(p, b, t0, ctx));                                   // this CTA's first tile
    KeyRow r1 = load_row(p, t0 + stride_tokens, fetch_page(p, b, t0 + stride_tokens, ctx));   // and its second
    int page_ahead = fetch_page(p, b, t0 + 2 * stride_tokens, ctx);
    fence_proxy_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = sm.tmem_slot;
    if (warp == 0 && lane_id() == 0)
        tmem_cp_32x128b_warpx4(tmem_base + kColSfb, umma_smem_desc_noswz(smem_u32(sm.query_scales), 16, 128));

    // A CTA walks the request's tiles with the grid's stride; the rows of its next two tiles are in flight
    // (in registers) while one tile is multiplied and reduced.
    bool alive = true;
    int it = 0;
    for (int tile = blockIdx.x; tile < tiles && alive; tile += gridDim.x, ++it) {
        const int s = 0;
        // the tile's rows go from registers to the operand layout (every thread has awaited the MMAs of the tile before)
#pragma unroll
        for (int c = 0; c < 4; ++c) *reinterpret_cast<uint4*>(sm.keys[0] + (c * kTile + tid) * 16) = r0.k[c];
        sm.key_scales[0][(tid & 31) * 4 + (tid >> 5)] = r0.scale;
        fence_proxy_async_smem();
        tc_fence_before();      // the previous tile's accumulator reads are done
        __syncthreads();
        if (warp == 0 && lane_id() == 0) {
            tc_fence_after();
            tmem_cp_32x128b_warpx4(tmem_base + kColSfa, umma_smem_desc_noswz(smem_u32(sm.key_scales[s]), 16, 128));
            const uint32_t a_addr = smem_u32(sm.keys[s]), b_addr = smem_u32(sm.query);
#pragma unroll
            for (int k = 0; k < 2; ++k) {   // 64 dims each: two 16-byte K chunks, scale bytes 2k and 2k+1 of a row's word
                const uint32_t idesc = umma_idesc_block_scaled(kTile, kHeads, 1, 1, 1, 2 * k, 2 * k);
                umma_mxf4_2x(tmem_base, umma_smem_desc_noswz(a_addr + k * 2 * kTile * 16, kTile * 16, 128),
                             umma_smem_desc_noswz(b_addr + k * 2 * kHeads * 16, kHeads * 16, 128), idesc,
                             tmem_base + kColSfa, tmem_base + kColSfb, k);
            }
            umma_commit(smem_u32(&sm.mma_done));
        }
        __syncwarp();

        {   // rows two tiles ahead are requested now; the block-table entry for them was requested a tile ago
            const int t_ahead = (tile + 2 * static_cast<int>(gridDim.x)) * kTile + tid;
            r0 = r1;
            r1 = load_row(p, t_ahead, page_ahead);
            page_ahead = fetch_page(p, b, t_ahead + stride_tokens, ctx);
        }
        // ---- epilogue: thread = token row = tensor-memory lane
        alive = mbar_wait_warp(smem_u32(&sm.mma_done), it & 1u, &sm.abort_flag, p.status, kDevTimeoutFullTmem);
        if (alive) {
            tc_fence_after();
            const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
            float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
            for (int c = 0; c < kHeads; c += 32) {
                uint32_t v[32];
                tmem_ld_32x32(lane_addr + c, v);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; i += 4) {
                    const float4 w4 = *reinterpret_cast<const float4*>(sm.weights + c + i);
                    acc0 = fmaf(fmaxf(__uint_as_float(v[i]), 0.f), w4.x, acc0);
                    acc1 = fmaf(fmaxf(__uint_as_float(v[i + 1]), 0.f), w4.y, acc1);
                    acc0 = fmaf(fmaxf(__uint_as_float(v[i + 2]), 0.f), w4.z, acc0);
                    acc1 = fmaf(fmaxf(__uint_as_float(v[i + 3]), 0.f), w4.w, acc1);
                }
            }
            const int t = tile * kTile + tid;
            if (t < ctx) p.logits[static_cast<int64_t>(b) * p.logits_stride + t] = acc0 + acc1;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (sm.abort_flag) abort_drain_sleep();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

}  // namespace mqa4
}  // namespace wuda

extern "C" int wuda_mqa_logits_fp4(const void* q_fp4, const void* q_scales, const void* kv_pages, const float* weights,
                                   const int32_t* context_lens, const int32_t* block_table, float* logits, int batch,
                                   int max_context, int num_blocks, int entries_per_block, int64_t page_stride_bytes,
                                   int block_table_stride, int64_t logits_stride, int32_t* status_word, void* stream) {
    using namespace wuda;
    using namespace wuda::mqa4;
    clear_error();
    WUDA_REQUIRE(batch >= 0 && max_context >= 0, "batch and max_context must be >= 0");
    if (batch == 0 || max_context == 0) return WUDA_OK;
    WUDA_REQUIRE(batch <= 65535, "batch must be <= 65535 (got %d)", batch);
    WUDA_REQUIRE(q_fp4 && q_scales && kv_pages && weights && context_lens && block_table && logits,
                 "no array may be NULL");
    WUDA_REQUIRE(num_blocks >= 1 && entries_per_block >= 1, "num_blocks and entries_per_block must be >= 1");
    WUDA_REQUIRE(page_stride_bytes >= static_cast<int64_t>(entries_per_block) * (kRowBytes + 4) && page_stride_bytes % 16 == 0,
                 "page_stride_bytes must be a multiple of 16 and hold %d entries of 68 bytes", entries_per_block);
    WUDA_REQUIRE(aligned16(q_fp4) && aligned16(kv_pages), "q and kv_pages must be 16-byte aligned");
    WUDA_REQUIRE(block_table_stride >= 1 && logits_stride >= max_context, "block_table_stride >= 1 and logits_stride >= max_context");
    Params p;
    p.q = static_cast<const uint8_t*>(q_fp4);
    p.q_scales = static_cast<const uint32_t*>(q_scales);
    p.kv_pages = static_cast<const uint8_t*>(kv_pages);
    p.weights = weights;
    p.context_lens = context_lens;
    p.block_table = block_table;
    p.logits = logits;
    p.status = status_word;
    p.page_stride = page_stride_bytes;
    p.logits_stride = logits_stride;
    p.num_blocks = num_blocks;
    p.epb = entries_per_block;
    p.bt_stride = block_table_stride;
    p.epb_shift = -1;
    for (int sft = 0; sft < 20; ++sft)
        if ((1 << sft) == entries_per_block) p.epb_shift = sft;
    // enough CTAs to give every SM four (tensor memory allows four of them per SM), each walking its
    // request's tiles with the grid's stride
    DeviceInfo dev;
    const int st = current_device_info(&dev);
    if (st != WUDA_OK) return st;
    const int tiles = (max_context + kTile - 1) / kTile;
    int per_request = 4 * dev.num_sms / batch;      // rounded down: a CTA beyond the resident ones would run as a second wave
    if (per_request < 1) per_request = 1;
    if (per_request > tiles) per_request = tiles;
    // Tensor memory holds four of these CTAs per SM, but the block scheduler only counts shared memory and
    // registers and would place a fifth, which then waits in its allocation while other SMs stay empty: an
    // unused dynamic allocation makes shared memory the limit at four.
    WUDA_CUDA(cudaFuncSetAttribute(mqa_logits_fp4_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPadBytes));
    WUDA_CUDA(launch_pdl(mqa_logits_fp4_kernel, dim3(per_request, batch), dim3(kThreads), kPadBytes,
                         static_cast<cudaStream_t>(stream), p));
    return WUDA_OK;
}
