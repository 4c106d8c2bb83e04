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
// Two kernels.  Pages of 32, 64, 128 or 256 entries take mqa_logits_fp4_paged_kernel: a persistent grid of one
// CTA per SM whose producer warps bring whole pages into shared memory with tiled tensor copies (the 64-byte key
// rows land in the 64-byte swizzle, which is the K-major operand layout as it stands), two scale warps turn the
// pages' scale words into the 512-byte images tcgen05.cp wants, two issuer threads run the block-scaled MMAs of
// an item of 256 tokens (two accumulators of 128 tokens x 64 heads) and four math warpgroups reduce them.
// Any other page size takes the gather kernel below it:
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
#include <cuda.h>

#include "host.h"
#include "ptx.cuh"
#include "tile_cursor.cuh"

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
    int max_ctx;                 // logits_stride as an int
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
    const int raw_ctx = __ldg(p.context_lens + b);
    const int ctx = min(max(raw_ctx, 0), p.max_ctx);   // no more tokens than a row of the logits holds
    if (raw_ctx > p.max_ctx && p.status && threadIdx.x == 0 && blockIdx.x == 0)
        atomicCAS(p.status, 0, static_cast<int>(kDevBadContextLen));
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


// ---------------------------------------------------------------------------------------------------------------
// The paged form: whole pages by tensor copies, roles in separate warps.
//
// Work item = 256 tokens of one request = two UMMA A tiles of 128 tokens (64-byte rows, SWIZZLE_64B: a row is one
// swizzle span, 8-row groups 512 bytes apart) against the request's 64 query rows (B, same layout).  Per half two
// MMAs of K = 64 (kind::mxf4nvf4, scale_vec::2X, ue8m0); the half's 128 scale words reach tensor memory as one
// 512-byte image [row % 32][row / 32].  A page's scale words are contiguous in the pool, so a tensor copy cannot
// write that image: the words are copied as they lie and a scale warp transposes them in shared memory.
// Tensor memory: two item stages of 128 accumulator columns (an item stage always belongs to the same issuer and
// to the same pair of math warpgroups - one per half), 2 x 4 key-scale columns per item stage, 4 query-scale
// columns per issuer and query stage.
namespace paged {

using namespace tiles;

constexpr int kItem = 2 * kTile;              // tokens per work item
constexpr int kQStages = 2;
constexpr int kItemStages = 2;                // accumulator stages in tensor memory
constexpr int kMaxKvStages = 12;
constexpr int kProducers = 4;                 // warps 0..3
constexpr int kIssuers = 2;                   // warps 4, 5
constexpr int kScaleWarps = 2;                // warps 6, 7
constexpr int kFirstScaleWarp = kProducers + kIssuers;
constexpr int kFirstMathWarp = 8;             // a multiple of 4: tensor-memory lane quarter = warp % 4
constexpr int kMathGroups = 4;                // group g reduces half g % 2 of the items n with n % 2 == g / 2
constexpr int kMathWarps = 4 * kMathGroups;
constexpr int kPagedThreads = 32 * (kFirstMathWarp + kMathWarps);
constexpr int kStageQuantum = 4;              // lcm of the role counts: a key stage always meets the same agents
static_assert(kMaxKvStages % kStageQuantum == 0 && kStageQuantum % kProducers == 0 && kStageQuantum % kIssuers == 0 &&
                  kStageQuantum % kScaleWarps == 0 && kItemStages == kIssuers && kMathGroups == 2 * kItemStages,
              "every stage must belong to one producer, one scale warp, one issuer and one pair of math groups");
constexpr int kKvBytes = kItem * kRowBytes;   // 16 KB of key rows per item
constexpr int kLinBytes = kItem * 4;          // its scale words as they lie in the pages
constexpr int kImgBytes = 2 * 512;            // and as the two images
constexpr int kQBytes = kHeads * kRowBytes;   // 4 KB
constexpr int kQImgBytes = 512;
constexpr int kWBytes = kHeads * 4;
constexpr uint32_t kTmemAlloc = 512;
constexpr uint32_t kColSfaBase = kItemStages * 2 * kHeads;                 // 256
constexpr uint32_t kColSfbBase = kColSfaBase + kItemStages * 8;            // 272
static_assert(kColSfbBase + kIssuers * kQStages * 4 <= kTmemAlloc, "tensor-memory columns");

// byte offsets from the 1024-aligned base
struct Layout {
    static constexpr int q_off = 0;
    static constexpr int kv_off = q_off + kQStages * kQBytes;
    static __host__ __device__ constexpr int lin_off(int stages) { return kv_off + stages * kKvBytes; }
    static __host__ __device__ constexpr int img_off(int stages) { return lin_off(stages) + stages * kLinBytes; }
    static __host__ __device__ constexpr int qimg_off(int stages) { return img_off(stages) + stages * kImgBytes; }
    static __host__ __device__ constexpr int w_off(int stages) { return qimg_off(stages) + kQStages * kQImgBytes; }
    static __host__ __device__ constexpr int bar_off(int stages) { return w_off(stages) + kQStages * kWBytes; }
    // barriers: full_q[2] empty_q[2] full_kv[12] img_ready[12] empty_kv[12] full_tm[2] empty_tm[2] = 44 x 8 B
    static __host__ __device__ constexpr int misc_off(int stages) { return bar_off(stages) + 44 * 8; }
    static __host__ __device__ constexpr int total(int stages) { return misc_off(stages) + 16 + 1024; }
};

struct PagedParams {
    const uint32_t* q_scales;    // [batch, 64]
    const float* weights;        // [batch, 64]
    const int32_t* context_lens; // [batch]
    const int32_t* block_table;  // [batch, bt_stride]
    float* logits;               // [batch, logits_stride]
    int32_t* status;
    int64_t logits_stride;
    int batch, num_blocks, epb, bt_stride, kv_stages;
    int max_ctx;                 // min(logits_stride, bt_stride * epb)
};

// K-major operand whose rows are exactly one 64-byte swizzle span (TMA SWIZZLE_64B): 8-row groups 512 bytes
// apart; the tile base is 512-byte aligned and K advances by adding bytes to the address.
__device__ __forceinline__ uint64_t umma_smem_desc_sw64(uint32_t addr) {
    return (static_cast<uint64_t>((addr & 0x3FFFFu) >> 4)) | (static_cast<uint64_t>(512 >> 4) << 32) |
           (static_cast<uint64_t>(1) << 46) | (static_cast<uint64_t>(4) << 61);
}

__global__ void __launch_bounds__(kPagedThreads, 1)
mqa_logits_fp4_paged_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap kv_map,
                            const __grid_constant__ CUtensorMap sf_map, const PagedParams p) {
    using L = Layout;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t base = (raw_addr + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (base - raw_addr);
    const int S = p.kv_stages;

    const uint32_t q_smem = base + L::q_off;
    const uint32_t kv_smem = base + L::kv_off;
    const uint32_t lin_smem = base + L::lin_off(S);
    const uint32_t img_smem = base + L::img_off(S);
    const uint32_t qimg_smem = base + L::qimg_off(S);
    const uint32_t w_smem = base + L::w_off(S);
    const uint32_t bars = base + L::bar_off(S);
    const uint32_t full_q = bars, empty_q = bars + 16;
    const uint32_t full_kv = bars + 32, img_ready = full_kv + kMaxKvStages * 8, empty_kv = img_ready + kMaxKvStages * 8;
    const uint32_t full_tm = empty_kv + kMaxKvStages * 8, empty_tm = full_tm + kItemStages * 8;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(base_ptr + L::misc_off(S));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(base_ptr + L::misc_off(S) + 4);
    const float* w_ptr = reinterpret_cast<const float*>(base_ptr + L::w_off(S));

    const int warp = threadIdx.x >> 5;
    const uint32_t lane = lane_id();

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int i = 0; i < kQStages; ++i) {
            mbar_init(full_q + i * 8, 2);                        // the copies' announcer and the scale-image builder
            mbar_init(empty_q + i * 8, kIssuers + kMathWarps);   // every issuer and math warp
        }
        for (int i = 0; i < S; ++i) {
            mbar_init(full_kv + i * 8, 1);
            mbar_init(img_ready + i * 8, 1);
            mbar_init(empty_kv + i * 8, 1);                      // the issuer's commit behind the item's MMAs
        }
        for (int i = 0; i < kItemStages; ++i) {
            mbar_init(full_tm + i * 8, 1);
            mbar_init(empty_tm + i * 8, 8);                      // the eight math warps of the stage's two groups
        }
        fence_mbar_init();
    }
    if (warp == kProducers) {
        tmem_alloc(smem_u32(tmem_slot), kTmemAlloc);
        tmem_relinquish();
    }
    if (warp == 0 && lane == 0) {
        prefetch_tmap(&q_map);
        prefetch_tmap(&kv_map);
        prefetch_tmap(&sf_map);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // the prologue above ran while the kernel ahead was still finishing; global memory from here on
    pdl_launch_dependents();
    pdl_wait();

    TileCursor cur = make_cursor<1, kItem>(p.context_lens, p.batch, p.max_ctx);
    const int nitems = cur.count;

    // Every role walks its own items n = r, r + R, ... of the CTA's range with a cursor that jumps R items at a
    // time; entering a request runs the role's part of the query-stage protocol, and after its last item a role
    // walks on to the end of the range so that it enters (and thereby releases) every request in it.
    if (warp < kProducers) {
        // ------------------------------------------------------------ producers
        // All copies of an item (key rows and scale words of every page) go out as ONE tensor-copy instruction
        // with one lane per copy.
        const int me = warp;
        const uint64_t stream_policy = policy_evict_first();
        const int ppi = kItem / p.epb;                   // pages per item: 8, 4, 2 or 1
        const int ppi_shift = ppi == 8 ? 3 : (ppi == 4 ? 2 : (ppi == 2 ? 1 : 0));
        const uint32_t page_bytes = p.epb * kRowBytes;
        const uint32_t page_scale_bytes = p.epb * 4;
        const int pg = static_cast<int>(lane) & (ppi - 1);   // this lane's page inside the item
        const bool is_scale = static_cast<int>(lane) >= ppi;
        const bool copier = static_cast<int>(lane) < 2 * ppi;
        const void* my_map = is_scale ? static_cast<const void*>(&sf_map) : static_cast<const void*>(&kv_map);
        const uint32_t my_dst = (is_scale ? lin_smem + pg * page_scale_bytes : kv_smem + pg * page_bytes);
        const uint32_t my_stage_bytes = is_scale ? kLinBytes : kKvBytes;
        int qc = 0, pages_b = 0;
        int64_t bt_row = 0;
        // block-table window: 32 entries in use, the next 32 already requested
        int win_base = 0, win_val = -1, nxt_val = -1;
        bool win_cold = true;
        bool alive = true;
        auto on_enter = [&](const TileCursor& c) {
            if (me == 0 && alive) {
                const int qs = qc & 1;
                alive = mbar_wait_lane0(empty_q + qs * 8, ((qc >> 1) & 1) ^ 1, abort_flag, p.status, kDevTimeoutEmptyQ);
                if (alive && lane == 0) {
                    mbar_arrive_expect_tx(full_q + qs * 8, kQBytes + kWBytes);
                    tma_load_2d(q_smem + qs * kQBytes, &q_map, full_q + qs * 8, 0, c.b * kHeads);
                    bulk_load(w_smem + qs * kWBytes, p.weights + static_cast<int64_t>(c.b) * kHeads, kWBytes,
                              full_q + qs * 8);
                }
            }
            ++qc;
            pages_b = (c.ctx_b + p.epb - 1) / p.epb;
            bt_row = static_cast<int64_t>(c.b) * p.bt_stride;
            win_cold = true;
        };
        Ring ring;
        int at = 0;
        if (nitems > 0) on_enter(cur);
        ring.step(me, S);       // the host guarantees S >= kProducers
        for (int n = me; n < nitems && alive; n += kProducers) {
            advance_by<1, kItem>(cur, n - at, p.context_lens, p.batch, p.max_ctx, on_enter);
            at = n;
            if (!alive) break;
            const int first_page = cur.j << ppi_shift;
            const int valid = min(ppi, pages_b - first_page);
            if (win_cold || first_page < win_base || first_page >= win_base + 64) {
                win_cold = false;
                win_base = first_page;
                const int e0 = win_base + lane, e1 = e0 + 32;
                win_val = (e0 < pages_b && e0 < p.bt_stride) ? __ldg(p.block_table + bt_row + e0) : -1;
                nxt_val = (e1 < pages_b && e1 < p.bt_stride) ? __ldg(p.block_table + bt_row + e1) : -1;
            } else if (first_page >= win_base + 32) {    // slide: the prefetched half becomes current
                win_base += 32;
                win_val = nxt_val;
                const int e1 = win_base + 32 + lane;
                nxt_val = (e1 < pages_b && e1 < p.bt_stride) ? __ldg(p.block_table + bt_row + e1) : -1;
            }
            int phys = __shfl_sync(0xffffffffu, win_val, (first_page + pg - win_base) & 31);
            const bool mine = copier && pg < valid;
            if (mine && (phys < 0 || phys >= p.num_blocks)) {
                if (p.status) atomicCAS(p.status, 0, kDevBadPageIndex);
                phys = 0;
            }
            const int s = ring.idx;
            alive = mbar_wait_lane0(empty_kv + s * 8, ring.phase ^ 1u, abort_flag, p.status, kDevTimeoutEmptyKv);
            if (!alive) break;
            if (lane == 0) mbar_arrive_expect_tx(full_kv + s * 8, valid * (page_bytes + page_scale_bytes));
            __syncwarp();
            if (mine)
                tma_load_3d_hint(my_dst + s * my_stage_bytes, my_map, full_kv + s * 8, 0, 0, phys, stream_policy);
            ring.step(kProducers, S);
        }
        if (alive && nitems > 0 && at < nitems - 1)
            advance_by<1, kItem>(cur, nitems - 1 - at, p.context_lens, p.batch, p.max_ctx, on_enter);
    } else if (warp < kFirstScaleWarp) {
        // ------------------------------------------------------------ issuers
        // One thread per warp runs the whole loop; issuer e owns the items n with n % 2 == e and item stage e.
        if (lane == 0) {
            const int me = warp - kProducers;
            const uint32_t acc = tmem_base + me * 2 * kHeads;
            const uint32_t sfa = tmem_base + kColSfaBase + me * 8;
            int qc = 0, qs = 0;
            uint32_t sfb = 0;
            bool alive = true;
            auto on_enter = [&](const TileCursor&) {
                if (qc > 0) umma_commit(empty_q + qs * 8);   // this issuer's MMAs and scale copy on the old q stage retired
                qs = qc & 1;
                if (alive) alive = mbar_wait(full_q + qs * 8, (qc >> 1) & 1, abort_flag, p.status, kDevTimeoutFullQ);
                ++qc;
                if (alive) {
                    tc_fence_after();
                    sfb = tmem_base + kColSfbBase + (me * kQStages + qs) * 4;
                    tmem_cp_32x128b_warpx4(sfb, umma_smem_desc_noswz(qimg_smem + qs * kQImgBytes, 16, 128));
                }
            };
            Ring ring;
            uint32_t tphase = 0;
            int at = 0;
            if (nitems > 0) on_enter(cur);
            ring.step(me, S);
            for (int n = me; n < nitems && alive; n += kIssuers) {
                advance_by<1, kItem>(cur, n - at, p.context_lens, p.batch, p.max_ctx, on_enter);
                at = n;
                if (!alive) break;
                const int s = ring.idx;
                if (!mbar_wait(img_ready + s * 8, ring.phase, abort_flag, p.status, kDevTimeoutFullKv)) break;
                if (!mbar_wait(full_kv + s * 8, ring.phase, abort_flag, p.status, kDevTimeoutFullKv)) break;
                if (!mbar_wait(empty_tm + me * 8, tphase ^ 1u, abort_flag, p.status, kDevTimeoutEmptyTmem)) break;
                tc_fence_after();
                const uint32_t a_addr = kv_smem + s * kKvBytes;
                const uint32_t b_addr = q_smem + qs * kQBytes;
                const uint32_t i_addr = img_smem + s * kImgBytes;
#pragma unroll
                for (int h = 0; h < 2; ++h)
                    tmem_cp_32x128b_warpx4(sfa + h * 4, umma_smem_desc_noswz(i_addr + h * 512, 16, 128));
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int k = 0; k < 2; ++k) {   // 64 dims each; scale bytes 2k and 2k+1 of a row's word
                        const uint32_t idesc = umma_idesc_block_scaled(kTile, kHeads, 1, 1, 1, 2 * k, 2 * k);
                        umma_mxf4_2x(acc + h * kHeads, umma_smem_desc_sw64(a_addr + h * (kKvBytes / 2) + k * 32),
                                     umma_smem_desc_sw64(b_addr + k * 32), idesc, sfa + h * 4, sfb, k);
                    }
                umma_commit(full_tm + me * 8);
                umma_commit(empty_kv + s * 8);     // nothing reads the key stage after these MMAs
                ring.step(kIssuers, S);
                tphase ^= 1u;
            }
            if (alive && nitems > 0 && at < nitems - 1)
                advance_by<1, kItem>(cur, nitems - 1 - at, p.context_lens, p.batch, p.max_ctx, on_enter);
        }
    } else if (warp < kFirstMathWarp) {
        // ------------------------------------------------------------ scale warps
        // Scale warp e turns the scale words of the items n with n % 2 == e into the two images; warp 0 also
        // builds the query's image when a request is entered.
        const int me = warp - kFirstScaleWarp;
        int qc = 0;
        bool alive = true;
        auto on_enter = [&](const TileCursor& c) {
            if (me == 0 && alive) {
                const int qs = qc & 1;
                alive = mbar_wait_lane0(empty_q + qs * 8, ((qc >> 1) & 1) ^ 1, abort_flag, p.status, kDevTimeoutEmptyQ);
                if (alive) {
                    const uint32_t* src = p.q_scales + static_cast<int64_t>(c.b) * kHeads;
                    // lane = head % 32: the words of heads lane and lane + 32; rows 64..127 do not exist (scale 1)
                    const uint4 v = make_uint4(__ldcg(src + lane), __ldcg(src + 32 + lane), 0x7f7f7f7fu, 0x7f7f7f7fu);
                    *reinterpret_cast<uint4*>(base_ptr + L::qimg_off(S) + qs * kQImgBytes + lane * 16) = v;
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(full_q + qs * 8);
                }
            }
            ++qc;
        };
        Ring ring;
        int at = 0;
        if (nitems > 0) on_enter(cur);
        ring.step(me, S);
        for (int n = me; n < nitems && alive; n += kScaleWarps) {
            advance_by<1, kItem>(cur, n - at, p.context_lens, p.batch, p.max_ctx, on_enter);
            at = n;
            if (!alive) break;
            const int s = ring.idx;
            alive = mbar_wait_warp(full_kv + s * 8, ring.phase, abort_flag, p.status, kDevTimeoutFullKv);
            if (!alive) break;
            const uint32_t* lin = reinterpret_cast<const uint32_t*>(base_ptr + L::lin_off(S) + s * kLinBytes);
            uint8_t* img = base_ptr + L::img_off(S) + s * kImgBytes;
#pragma unroll
            for (int h = 0; h < 2; ++h) {   // image word [lane][j] = scale word of row j * 32 + lane of the half
                const uint4 v = make_uint4(lin[h * kTile + lane], lin[h * kTile + 32 + lane], lin[h * kTile + 64 + lane],
                                           lin[h * kTile + 96 + lane]);
                *reinterpret_cast<uint4*>(img + h * 512 + lane * 16) = v;
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(img_ready + s * 8);
            ring.step(kScaleWarps, S);
        }
        if (alive && nitems > 0 && at < nitems - 1)
            advance_by<1, kItem>(cur, nitems - 1 - at, p.context_lens, p.batch, p.max_ctx, on_enter);
    } else {
        // ------------------------------------------------------------ math warps
        // Group g reduces half g % 2 of the items n with n % 2 == g / 2 (item stage g / 2).  A thread is one key
        // token: relu, head weight, sum over its 64 accumulator columns (the block scales were applied by the MMA).
        const int g = (warp - kFirstMathWarp) >> 2;
        const int half = g & 1, ts = g >> 1;
        const int row_in_item = half * kTile + (warp & 3) * 32 + static_cast<int>(lane);
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16) + ts * 2 * kHeads + half * kHeads;
        int qc = 0, qs = 0;
        int ctx_row = 0;
        bool alive = true;
        auto on_enter = [&](const TileCursor& c) {
            if (qc > 0) {
                __syncwarp();
                if (lane == 0) mbar_arrive(empty_q + qs * 8);
            }
            qs = qc & 1;
            if (alive)
                alive = mbar_wait_warp_fast(full_q + qs * 8, (qc >> 1) & 1, abort_flag, p.status, kDevTimeoutFullQ);
            ++qc;
            const int raw = __ldg(p.context_lens + c.b);
            ctx_row = clamp_ctx(raw, p.max_ctx);
            if (raw > p.max_ctx && p.status) atomicCAS(p.status, 0, kDevBadContextLen);
        };
        uint32_t tphase = 0;
        int at = 0;
        if (nitems > 0) on_enter(cur);
        for (int n = ts; n < nitems && alive; n += kItemStages) {
            advance_by<1, kItem>(cur, n - at, p.context_lens, p.batch, p.max_ctx, on_enter);
            at = n;
            if (!alive) break;
            alive = mbar_wait_warp_fast(full_tm + ts * 8, tphase, abort_flag, p.status, kDevTimeoutFullTmem);
            if (!alive) break;
            tc_fence_after();
            uint32_t v[2][32];
            tmem_ld_32x32(taddr, v[0]);
            const int t = cur.j * kItem + row_in_item;
            float2 acc0 = make_float2(0.f, 0.f), acc1 = make_float2(0.f, 0.f);
            float2 acc2 = make_float2(0.f, 0.f), acc3 = make_float2(0.f, 0.f);
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                tmem_ld_wait();
                if (c == 0) tmem_ld_32x32(taddr + 32, v[1]);
                if (c == 1) {   // every accumulator column of this warp's rows is in registers
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(empty_tm + ts * 8);
                }
                const float4* w4 = reinterpret_cast<const float4*>(w_ptr + qs * kHeads + c * 32);
                const uint32_t* x = v[c];
#pragma unroll
                for (int e = 0; e < 32; e += 8) {
                    const float4 wa = w4[e >> 2], wb = w4[(e >> 2) + 1];
                    acc0 = __ffma2_rn(make_float2(fmaxf(__uint_as_float(x[e + 0]), 0.f), fmaxf(__uint_as_float(x[e + 1]), 0.f)),
                                      make_float2(wa.x, wa.y), acc0);
                    acc1 = __ffma2_rn(make_float2(fmaxf(__uint_as_float(x[e + 2]), 0.f), fmaxf(__uint_as_float(x[e + 3]), 0.f)),
                                      make_float2(wa.z, wa.w), acc1);
                    acc2 = __ffma2_rn(make_float2(fmaxf(__uint_as_float(x[e + 4]), 0.f), fmaxf(__uint_as_float(x[e + 5]), 0.f)),
                                      make_float2(wb.x, wb.y), acc2);
                    acc3 = __ffma2_rn(make_float2(fmaxf(__uint_as_float(x[e + 6]), 0.f), fmaxf(__uint_as_float(x[e + 7]), 0.f)),
                                      make_float2(wb.z, wb.w), acc3);
                }
            }
            const float2 sum = __fadd2_rn(__fadd2_rn(acc0, acc1), __fadd2_rn(acc2, acc3));
            if (t < ctx_row) p.logits[static_cast<int64_t>(cur.b) * p.logits_stride + t] = sum.x + sum.y;
            tphase ^= 1u;
        }
        if (alive && nitems > 0 && at < nitems - 1)
            advance_by<1, kItem>(cur, nitems - 1 - at, p.context_lens, p.batch, p.max_ctx, on_enter);
    }

    __syncthreads();
    if (*abort_flag) abort_drain_sleep();
    __syncthreads();
    if (warp == kProducers) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemAlloc);
    }
}

}  // namespace paged

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
    DeviceInfo dev;
    const int st = current_device_info(&dev);
    if (st != WUDA_OK) return st;
    if (entries_per_block == 32 || entries_per_block == 64 || entries_per_block == 128 || entries_per_block == 256) {
        // ---- whole pages by tensor copies (the usual page sizes)
        using namespace wuda::mqa4::paged;
        WUDA_REQUIRE(static_cast<int64_t>(batch) * kHeads < (1ll << 31), "batch too large");
        CUtensorMap q_map, kv_map, sf_map;
        int e;
        {
            const uint64_t dims[2] = {static_cast<uint64_t>(kRowBytes), static_cast<uint64_t>(batch) * kHeads};
            const uint64_t strides[1] = {static_cast<uint64_t>(kRowBytes)};
            const uint32_t box[2] = {static_cast<uint32_t>(kRowBytes), static_cast<uint32_t>(kHeads)};
            e = encode_tensor_map(&q_map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, q_fp4, dims, strides, box,
                                  CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B);
            if (e != WUDA_OK) return e;
        }
        {
            const uint64_t dims[3] = {static_cast<uint64_t>(kRowBytes), static_cast<uint64_t>(entries_per_block),
                                      static_cast<uint64_t>(num_blocks)};
            const uint64_t strides[2] = {static_cast<uint64_t>(kRowBytes), static_cast<uint64_t>(page_stride_bytes)};
            const uint32_t box[3] = {static_cast<uint32_t>(kRowBytes), static_cast<uint32_t>(entries_per_block), 1u};
            e = encode_tensor_map(&kv_map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, kv_pages, dims, strides, box,
                                  CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
            if (e != WUDA_OK) return e;
        }
        {   // the scale words: entries_per_block of them after the key rows of each page
            const uint64_t dims[3] = {static_cast<uint64_t>(entries_per_block), 1ull, static_cast<uint64_t>(num_blocks)};
            const uint64_t strides[2] = {static_cast<uint64_t>(page_stride_bytes), static_cast<uint64_t>(page_stride_bytes)};
            const uint32_t box[3] = {static_cast<uint32_t>(entries_per_block), 1u, 1u};
            e = encode_tensor_map(&sf_map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3,
                                  static_cast<const uint8_t*>(kv_pages) + static_cast<int64_t>(entries_per_block) * kRowBytes,
                                  dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE);
            if (e != WUDA_OK) return e;
        }
        PagedParams pp;
        pp.q_scales = static_cast<const uint32_t*>(q_scales);
        pp.weights = weights;
        pp.context_lens = context_lens;
        pp.block_table = block_table;
        pp.logits = logits;
        pp.status = status_word;
        pp.logits_stride = logits_stride;
        pp.batch = batch;
        pp.num_blocks = num_blocks;
        pp.epb = entries_per_block;
        pp.bt_stride = block_table_stride;
        {
            const int64_t by_table = static_cast<int64_t>(block_table_stride) * entries_per_block;
            const int64_t cap = logits_stride < by_table ? logits_stride : by_table;
            pp.max_ctx = static_cast<int>(cap < 0x7fffff00 ? cap : 0x7fffff00);
        }
        int stages = kMaxKvStages;   // as many key stages as shared memory allows, in multiples of the role counts
        while (stages > kStageQuantum && Layout::total(stages) > dev.smem_optin) stages -= kStageQuantum;
        if (Layout::total(stages) > dev.smem_optin)
            return fail(WUDA_ERR_UNSUPPORTED, "device offers %d bytes of shared memory per block; the kernel needs more",
                        dev.smem_optin);
        pp.kv_stages = stages;
        const int smem = Layout::total(stages);
        WUDA_CUDA(cudaFuncSetAttribute(mqa_logits_fp4_paged_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        WUDA_CUDA(launch_pdl(mqa_logits_fp4_paged_kernel, dim3(dev.num_sms), dim3(kPagedThreads), smem,
                             static_cast<cudaStream_t>(stream), q_map, kv_map, sf_map, pp));
        return WUDA_OK;
    }
    // ---- any other page size: the gather kernel
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
    p.max_ctx = static_cast<int>(logits_stride < 0x7fffff00 ? logits_stride : 0x7fffff00);
    p.epb_shift = -1;
    for (int sft = 0; sft < 20; ++sft)
        if ((1 << sft) == entries_per_block) p.epb_shift = sft;
    // enough CTAs to give every SM four (tensor memory allows four of them per SM), each walking its
    // request's tiles with the grid's stride
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
