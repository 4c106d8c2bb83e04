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
// First form of this kernel: one CTA per (request, tile of 128 tokens), no pipeline inside a CTA -
// several CTAs per SM overlap each other's loads.  A CTA gathers its 128 key rows and the request's
// 64 query rows with plain loads into the unswizzled K-major operand layout, copies the scale words
// to tensor memory (tcgen05.cp), issues two block-scaled MMAs (kind::mxf4nvf4, scale_vec::2X, ue8m0:
// the scales are applied inside the tensor core) and reduces the 64 head columns of each token row
// with relu and the head weights.
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

// shared memory (static): operands as [16-byte K chunk][row][16 B], scale images of 512 B
struct Smem {
    alignas(128) uint8_t keys[4 * kTile * 16];     // 8 KB
    alignas(128) uint8_t query[4 * kHeads * 16];   // 4 KB
    alignas(128) uint32_t key_scales[128];         // [row % 32][row / 32]
    alignas(128) uint32_t query_scales[128];
    float weights[kHeads];
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

__global__ void __launch_bounds__(kThreads) mqa_logits_fp4_kernel(const Params p) {
    __shared__ Smem sm;
    const int b = blockIdx.y, tile = blockIdx.x;
    const int tid = threadIdx.x, warp = tid >> 5;
    pdl_launch_dependents();
    pdl_wait();   // nothing of global memory is touched before the kernel ahead has finished
    const int ctx = __ldg(p.context_lens + b);
    if (tile * kTile >= ctx) return;   // whole CTA: nothing of this tile is valid

    if (tid == 0) {
        sm.abort_flag = 0;
        mbar_init(smem_u32(&sm.mma_done), 1);
        fence_mbar_init();
    }
    if (warp == 0) {
        tmem_alloc(smem_u32(&sm.tmem_slot), kTmemCols);
        tmem_relinquish();
    }

    // ---- gather: thread = token row of the tile; threads 0..63 also take one query row
    {
        const int t = tile * kTile + tid;
        uint4 k4[4] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)};
        uint32_t ks = 0x7f7f7f7fu;   // scale 1.0: a row of zeros stays zero
        if (t < ctx) {
            const int slot = t / p.epb, off = t - slot * p.epb;
            int phys = slot < p.bt_stride ? __ldg(p.block_table + static_cast<int64_t>(b) * p.bt_stride + slot) : -1;
            if (phys < 0 || phys >= p.num_blocks) {
                if (p.status) atomicCAS(p.status, 0, static_cast<int>(kDevBadPageIndex));
                phys = 0;
            }
            const uint8_t* page = p.kv_pages + static_cast<int64_t>(phys) * p.page_stride;
            const uint4* row = reinterpret_cast<const uint4*>(page + static_cast<int64_t>(off) * kRowBytes);
#pragma unroll
            for (int c = 0; c < 4; ++c) k4[c] = __ldg(row + c);
            ks = __ldg(reinterpret_cast<const uint32_t*>(page + static_cast<int64_t>(p.epb) * kRowBytes) + off);
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) *reinterpret_cast<uint4*>(sm.keys + (c * kTile + tid) * 16) = k4[c];
        sm.key_scales[(tid & 31) * 4 + (tid >> 5)] = ks;
        uint32_t qs = 0x7f7f7f7fu;
        if (tid < kHeads) {
            const uint4* row = reinterpret_cast<const uint4*>(p.q + (static_cast<int64_t>(b) * kHeads + tid) * kRowBytes);
#pragma unroll
            for (int c = 0; c < 4; ++c) *reinterpret_cast<uint4*>(sm.query + (c * kHeads + tid) * 16) = __ldg(row + c);
            qs = __ldg(p.q_scales + static_cast<int64_t>(b) * kHeads + tid);
            sm.weights[tid] = __ldg(p.weights + static_cast<int64_t>(b) * kHeads + tid);
        }
        sm.query_scales[(tid & 31) * 4 + (tid >> 5)] = qs;
    }
    fence_proxy_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = sm.tmem_slot;

    if (warp == 0 && lane_id() == 0) {
        tmem_cp_32x128b_warpx4(tmem_base + kColSfa, umma_smem_desc_noswz(smem_u32(sm.key_scales), 16, 128));
        tmem_cp_32x128b_warpx4(tmem_base + kColSfb, umma_smem_desc_noswz(smem_u32(sm.query_scales), 16, 128));
        const uint32_t a_addr = smem_u32(sm.keys), b_addr = smem_u32(sm.query);
#pragma unroll
        for (int k = 0; k < 2; ++k) {   // 64 dims each: two 16-byte K chunks, scale bytes 2k and 2k+1 of a row's word
            const uint32_t idesc = umma_idesc_block_scaled(kTile, kHeads, 1, 1, 1, 2 * k, 2 * k);
            umma_mxf4_2x(tmem_base, umma_smem_desc_noswz(a_addr + k * 2 * kTile * 16, kTile * 16, 128),
                         umma_smem_desc_noswz(b_addr + k * 2 * kHeads * 16, kHeads * 16, 128), idesc, tmem_base + kColSfa,
                         tmem_base + kColSfb, k);
        }
        umma_commit(smem_u32(&sm.mma_done));
    }
    __syncwarp();

    // ---- epilogue: thread = token row = tensor-memory lane
    const bool alive = mbar_wait_warp(smem_u32(&sm.mma_done), 0u, &sm.abort_flag, p.status, kDevTimeoutFullTmem);
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
            for (int i = 0; i < 32; i += 2) {
                acc0 = fmaf(fmaxf(__uint_as_float(v[i]), 0.f), sm.weights[c + i], acc0);
                acc1 = fmaf(fmaxf(__uint_as_float(v[i + 1]), 0.f), sm.weights[c + i + 1], acc1);
            }
        }
        const int t = tile * kTile + tid;
        if (t < ctx) p.logits[static_cast<int64_t>(b) * p.logits_stride + t] = acc0 + acc1;
        tc_fence_before();
    }
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
    const int tiles = (max_context + kTile - 1) / kTile;
    WUDA_CUDA(launch_pdl(mqa_logits_fp4_kernel, dim3(tiles, batch), dim3(kThreads), 0, static_cast<cudaStream_t>(stream), p));
    return WUDA_OK;
}
