// Paged FP8 MQA logits for sm_100a.
//
//   logits[r, t] = scale[t] * sum_h w[r, h] * relu( q[r, h, :] . k[t, :] )
//
// Formula and page layout follow the reference's test oracle
// (dsv4_megakernel/megakernel/test/test_mqa_logits_fp4.py:207-218 and :443-474); the
// order "dot -> relu -> weighted head sum -> times token scale" follows the reference
// kernel (include/mqa_logits_fp8.cuh:685-734).  The design is this library's own:
//
//  * persistent grid, one CTA per SM; the flat list of (request, 128-token tile) work
//    items is cut into equal contiguous chunks inside the kernel (no host schedule);
//  * a 128-token tile of keys is the UMMA A operand (M = 128 tokens, K = 128 dims,
//    each token row is exactly one 128-byte swizzle span, so a page lands in shared
//    memory with one tiled TMA copy per page and needs no repacking);
//  * the request's next_n x 64 query heads are the B operand (N = 64 * next_n), loaded
//    once per request, so the keys of a request are read from HBM once for all its rows;
//  * tcgen05.mma kind::f8f6f4 accumulates into TMEM (4 accumulator stages); four math
//    warpgroups, one per stage, take tiles in turn: tcgen05.ld, relu, weighted head sum, token scale,
//    coalesced fp32 stores;
//  * every mbarrier wait is bounded and reports through the status word.
#include <cuda.h>
#include <cuda_runtime.h>

#include "host.h"
#include "ptx.cuh"
#include "tile_cursor.cuh"

namespace wuda {
namespace mqa {

constexpr int kHeads = 64;
constexpr int kDim = 128;
constexpr int kTile = 128;          // tokens per work item (UMMA M)
constexpr int kQStages = 2;
constexpr int kTmemStages = 4;

constexpr int kMaxKvStages = 12;
// Math warpgroups; group g owns tiles n with n % kMathGroups == g.  The TMEM stage count
// must be a multiple of both this and the number of UMMA issuers, so that every stage is
// always produced by the same issuer and consumed by the same group: a parity wait may
// not run more than one phase ahead of its barrier.
constexpr int kMathGroups = 4;
constexpr int kMathWarps = 4 * kMathGroups;
static_assert(kTmemStages % kMathGroups == 0, "TMEM stages must be a multiple of the math group count");
static_assert(kMaxKvStages % 4 == 0, "key stages come in multiples of the role counts");
// Warp roles.  A single thread runs a dependent instruction chain at a few cycles per
// instruction, so the bookkeeping of one tile costs a role several hundred cycles; the
// roles are therefore replicated and take tiles round-robin: four producer warps, two
// UMMA issuers, four math warpgroups (a tile's reduction is a chain of tcgen05.ld latencies of about
// 2000 cycles against a tile period of about 700 at HBM speed, so it takes three or more groups in
// flight to keep up; 768 threads leave each 80 registers, which the reduction fits without spills).
constexpr int kProducers = 4;       // warps 0..3, producer p takes tiles n with n % 4 == p
constexpr int kIssuers = 2;         // warps 4, 5
constexpr int kMmaWarp0 = kProducers;
constexpr int kStageQuantum = 4;    // lcm(kProducers, kIssuers, kMathGroups)
static_assert(kStageQuantum % kProducers == 0 && kStageQuantum % kIssuers == 0 && kStageQuantum % kMathGroups == 0,
              "every stage must belong to one producer, one issuer and one math group");
static_assert(kTmemStages % kIssuers == 0, "TMEM stages must be a multiple of the UMMA issuer count");
constexpr int kFirstMathWarp = 8;   // a multiple of 4: TMEM lane quarter = warp % 4 (warps 6, 7 idle)
constexpr int kThreads = 32 * (kFirstMathWarp + kMathWarps);
constexpr int kKvTileBytes = kTile * kDim;      // 16 KB
constexpr int kScaleTileBytes = kTile * 4;      // 512 B

struct Params {
    const uint8_t* kv_pages;
    const float* weights;
    const int32_t* context_lens;
    const int32_t* block_table;
    float* logits;
    int32_t* status;
    int64_t page_stride;
    int64_t logits_stride;
    int batch;
    int num_blocks;
    int epb;
    int bt_stride;
    int kv_stages;
    int max_ctx;      // min(logits_stride, bt_stride * epb): no row may claim more tokens than its row of the
                      // logits and of the block table holds
};

template <int NEXT_N>
struct Smem {
    static constexpr int kN = NEXT_N * kHeads;
    static constexpr int kQBytes = kN * kDim;
    static constexpr int kWBytes = kN * 4;
    // byte offsets from the 1024-aligned base
    static constexpr int q_off = 0;
    static constexpr int kv_off = q_off + kQStages * kQBytes;
    static __host__ __device__ constexpr int scale_off(int stages) { return kv_off + stages * kKvTileBytes; }
    static __host__ __device__ constexpr int w_off(int stages) { return scale_off(stages) + stages * kScaleTileBytes; }
    static __host__ __device__ constexpr int bar_off(int stages) { return w_off(stages) + kQStages * kWBytes; }
    // barriers: full_q[2] empty_q[2] full_kv[12] empty_kv[12] full_tmem[4] empty_tmem[4] = 36 x 8 B
    static __host__ __device__ constexpr int misc_off(int stages) { return bar_off(stages) + 36 * 8; }
    static __host__ __device__ constexpr int total(int stages) { return misc_off(stages) + 16 + 1024; }
};

using namespace tiles;

template <int NEXT_N>
__global__ void __launch_bounds__(kThreads, 1)
mqa_logits_fp8_kernel(const __grid_constant__ CUtensorMap q_map,
                      const __grid_constant__ CUtensorMap kv_map,
                      const __grid_constant__ CUtensorMap sf_map, const Params p) {
    using L = Smem<NEXT_N>;
    constexpr int kN = L::kN;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t base = (raw_addr + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (base - raw_addr);
    const int S = p.kv_stages;

    const uint32_t q_smem = base + L::q_off;
    const uint32_t kv_smem = base + L::kv_off;
    const uint32_t scale_smem = base + L::scale_off(S);
    const uint32_t w_smem = base + L::w_off(S);
    const uint32_t bars = base + L::bar_off(S);
    const uint32_t full_q = bars, empty_q = bars + 16;
    const uint32_t full_kv = bars + 32, empty_kv = full_kv + kMaxKvStages * 8;
    const uint32_t full_tm = empty_kv + kMaxKvStages * 8, empty_tm = full_tm + kTmemStages * 8;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(base_ptr + L::misc_off(S));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(base_ptr + L::misc_off(S) + 4);
    const float* scale_ptr = reinterpret_cast<const float*>(base_ptr + L::scale_off(S));
    const float* w_ptr = reinterpret_cast<const float*>(base_ptr + L::w_off(S));

    const int warp = threadIdx.x >> 5;
    const uint32_t lane = lane_id();

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int i = 0; i < kQStages; ++i) {
            mbar_init(full_q + i * 8, 1);
            mbar_init(empty_q + i * 8, kIssuers + kMathWarps);   // every UMMA issuer and math warp
        }
        for (int i = 0; i < S; ++i) {
            mbar_init(full_kv + i * 8, 1);
            mbar_init(empty_kv + i * 8, 4);   // the four math warps that consume the stage
        }
        for (int i = 0; i < kTmemStages; ++i) {
            mbar_init(full_tm + i * 8, 1);
            mbar_init(empty_tm + i * 8, 4);
        }
        fence_mbar_init();
    }
    if (warp == kMmaWarp0) {
        tmem_alloc(smem_u32(tmem_slot), kTmemStages * kN);
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

    TileCursor cur = make_cursor<NEXT_N, kTile>(p.context_lens, p.batch, p.max_ctx);
    const int ntiles = cur.count;

    // Every role walks its own tiles n = r, r + R, ... of the CTA's range with a cursor
    // that jumps R tiles at a time; entering a request runs the role's part of the
    // query-stage protocol, and after its last tile a role walks on to the end of the
    // range so that it enters (and thereby releases) every request in it.
    if (warp < kProducers) {
        // ------------------------------------------------------------ TMA producers
        // All copies of a tile (key bytes and scales of every page) go out as ONE
        // tensor-copy instruction with one lane per copy.
        const int me = warp;
        const uint64_t stream_policy = policy_evict_first();
        const int ppt = kTile / p.epb;                   // pages per tile: 4, 2 or 1
        const int ppt_shift = ppt == 4 ? 2 : (ppt == 2 ? 1 : 0);
        const uint32_t page_bytes = p.epb * kDim;
        const uint32_t page_scale_bytes = p.epb * 4;
        const int pg = static_cast<int>(lane) & (ppt - 1);   // this lane's page inside the tile
        const bool is_scale = static_cast<int>(lane) >= ppt;
        const bool copier = static_cast<int>(lane) < 2 * ppt;
        const void* my_map = is_scale ? static_cast<const void*>(&sf_map) : static_cast<const void*>(&kv_map);
        const uint32_t my_dst = (is_scale ? scale_smem + pg * page_scale_bytes : kv_smem + pg * page_bytes);
        const uint32_t my_stage_bytes = is_scale ? kScaleTileBytes : kKvTileBytes;
        int qc = 0, pages_b = 0;
        int64_t bt_row = 0;
        // block-table window: 32 entries in use, the next 32 already requested
        int win_base = 0, win_val = -1, nxt_val = -1;
        bool win_cold = true;
        bool alive = true;
        auto on_enter = [&](const TileCursor& c) {
            if (me == 0 && alive) {
                const int qs = qc & 1;
                alive = mbar_wait_lane0(empty_q + qs * 8, ((qc >> 1) & 1) ^ 1, abort_flag, p.status,
                                                         kDevTimeoutEmptyQ);
                if (alive && lane == 0) {
                    mbar_arrive_expect_tx(full_q + qs * 8, L::kQBytes + L::kWBytes);
                    tma_load_2d(q_smem + qs * L::kQBytes, &q_map, full_q + qs * 8, 0, c.b * kN);
                    bulk_load(w_smem + qs * L::kWBytes, p.weights + static_cast<int64_t>(c.b) * kN, L::kWBytes,
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
        if (ntiles > 0) on_enter(cur);
        ring.step(me, S);       // the host guarantees S >= kProducers
        for (int n = me; n < ntiles && alive; n += kProducers) {
            advance_by<NEXT_N, kTile>(cur, n - at, p.context_lens, p.batch, p.max_ctx, on_enter);
            at = n;
            if (!alive) break;
            const int first_page = cur.j << ppt_shift;
            const int valid = min(ppt, pages_b - first_page);
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
            alive = mbar_wait_lane0(empty_kv + s * 8, ring.phase ^ 1u, abort_flag, p.status,
                                                     kDevTimeoutEmptyKv);
            if (!alive) break;
            if (lane == 0) mbar_arrive_expect_tx(full_kv + s * 8, valid * (page_bytes + page_scale_bytes));
            __syncwarp();
            if (mine)
                tma_load_3d_hint(my_dst + s * my_stage_bytes, my_map, full_kv + s * 8, 0, 0, phys, stream_policy);
            ring.step(kProducers, S);
        }
        if (alive && ntiles > 0 && at < ntiles - 1)
            advance_by<NEXT_N, kTile>(cur, ntiles - 1 - at, p.context_lens, p.batch, p.max_ctx, on_enter);
    } else if (warp < kMmaWarp0 + kIssuers) {
        // ------------------------------------------------------------ UMMA issuers
        // One thread per warp runs the whole loop (the other lanes go straight to the
        // final barrier, so no warp-level synchronisation sits between UMMAs).
        if (lane == 0) {
            const int me = warp - kMmaWarp0;
            constexpr uint32_t idesc = umma_idesc(kTile, kN, 0, 0);
            int qc = 0, qs = 0;
            bool alive = true;
            auto on_enter = [&](const TileCursor&) {
                if (qc > 0) umma_commit(empty_q + qs * 8);   // this issuer's UMMAs on the old q stage retired
                qs = qc & 1;
                if (alive)
                    alive = mbar_wait(full_q + qs * 8, (qc >> 1) & 1, abort_flag, p.status,
                                                      kDevTimeoutFullQ);
                ++qc;
            };
            Ring ring, tring;
            int at = 0;
            if (ntiles > 0) on_enter(cur);
            ring.step(me, S);
            tring.step(me, kTmemStages);
            for (int n = me; n < ntiles && alive; n += kIssuers) {
                advance_by<NEXT_N, kTile>(cur, n - at, p.context_lens, p.batch, p.max_ctx, on_enter);
                at = n;
                if (!alive) break;
                const int s = ring.idx, ts = tring.idx;
                if (!mbar_wait(full_kv + s * 8, ring.phase, abort_flag, p.status, kDevTimeoutFullKv))
                    break;
                if (!mbar_wait(empty_tm + ts * 8, tring.phase ^ 1u, abort_flag, p.status,
                                               kDevTimeoutEmptyTmem))
                    break;
                tc_fence_after();
                const uint32_t a_addr = kv_smem + s * kKvTileBytes;
                const uint32_t b_addr = q_smem + qs * L::kQBytes;
                const uint32_t d_addr = tmem_base + ts * kN;
#pragma unroll
                for (int k = 0; k < kDim / 32; ++k) {
                    umma_f8f6f4(d_addr, umma_smem_desc_sw128(a_addr + k * 32),
                                umma_smem_desc_sw128(b_addr + k * 32), idesc, k > 0 ? 1u : 0u);
                }
                umma_commit(full_tm + ts * 8);
                ring.step(kIssuers, S);
                tring.step(kIssuers, kTmemStages);
            }
            if (alive && ntiles > 0 && at < ntiles - 1)
                advance_by<NEXT_N, kTile>(cur, ntiles - 1 - at, p.context_lens, p.batch, p.max_ctx, on_enter);
        }
    } else if (warp >= kFirstMathWarp) {
        // ------------------------------------------------------------ math warps
        // Warpgroup g owns tiles n with n % kMathGroups == g.  A thread is one key token: it reads
        // its accumulator row from TMEM in 32-column chunks (the next chunk is in
        // flight while the current one is reduced), applies relu, the per-head weight
        // (packed fp32x2 FMAs) and the token scale, and stores one logit per query row.
        const int wg = (warp - kFirstMathWarp) >> 2;
        const int row_in_tile = (warp & 3) * 32 + lane;
        const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
        constexpr int kChunks = kN / 32;              // 32-column chunks per tile
        int qc = 0, qs = 0;
        int ctx_row[NEXT_N];
        bool alive = true;
        auto on_enter = [&](const TileCursor& c) {
            if (qc > 0) {
                __syncwarp();
                if (lane == 0) mbar_arrive(empty_q + qs * 8);
            }
            qs = qc & 1;
            if (alive)
                alive = mbar_wait_warp_fast(full_q + qs * 8, (qc >> 1) & 1, abort_flag, p.status,
                                                             kDevTimeoutFullQ);
            ++qc;
#pragma unroll
            for (int i = 0; i < NEXT_N; ++i) {
                const int raw = __ldg(p.context_lens + c.b * NEXT_N + i);
                ctx_row[i] = clamp_ctx(raw, p.max_ctx);
                if (raw > p.max_ctx && p.status) atomicCAS(p.status, 0, kDevBadContextLen);
            }
        };
        Ring ring, tring;
        int at = 0;
        if (ntiles > 0) on_enter(cur);
        ring.step(wg, S);
        tring.step(wg, kTmemStages);
        for (int n = wg; n < ntiles && alive; n += kMathGroups) {
            advance_by<NEXT_N, kTile>(cur, n - at, p.context_lens, p.batch, p.max_ctx, on_enter);
            at = n;
            if (!alive) break;
            const int s = ring.idx, ts = tring.idx;
            // full_tm completes after the UMMAs that read key stage s retired, and those
            // were issued after the stage's copies had landed: one wait covers the
            // accumulator and the stage's scales.
            alive = mbar_wait_warp_fast(full_tm + ts * 8, tring.phase, abort_flag, p.status,
                                                         kDevTimeoutFullTmem);
            if (!alive) break;
            tc_fence_after();
            const uint32_t taddr = tmem_base + lane_base + ts * kN;
            uint32_t v[2][32];
            tmem_ld_32x32(taddr, v[0]);
            const float scale = scale_ptr[s * kTile + row_in_tile];
            const int t = cur.j * kTile + row_in_tile;
            float2 acc0 = make_float2(0.f, 0.f), acc1 = make_float2(0.f, 0.f);
            float2 acc2 = make_float2(0.f, 0.f), acc3 = make_float2(0.f, 0.f);
#pragma unroll
            for (int c = 0; c < kChunks; ++c) {
                tmem_ld_wait();
                if (c + 1 < kChunks) tmem_ld_32x32(taddr + (c + 1) * 32, v[(c + 1) & 1]);
                if (c + 1 == kChunks) {
                    // every accumulator column is in registers, the scale too
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) {
                        mbar_arrive(empty_tm + ts * 8);
                        mbar_arrive(empty_kv + s * 8);
                    }
                }
                const float4* w4 = reinterpret_cast<const float4*>(w_ptr + qs * kN + c * 32);
                const uint32_t* x = v[c & 1];
#pragma unroll
                for (int e = 0; e < 32; e += 8) {
                    const float4 wa = w4[e >> 2], wb = w4[(e >> 2) + 1];
                    acc0 = __ffma2_rn(make_float2(fmaxf(__uint_as_float(x[e + 0]), 0.f),
                                                  fmaxf(__uint_as_float(x[e + 1]), 0.f)),
                                      make_float2(wa.x, wa.y), acc0);
                    acc1 = __ffma2_rn(make_float2(fmaxf(__uint_as_float(x[e + 2]), 0.f),
                                                  fmaxf(__uint_as_float(x[e + 3]), 0.f)),
                                      make_float2(wa.z, wa.w), acc1);
                    acc2 = __ffma2_rn(make_float2(fmaxf(__uint_as_float(x[e + 4]), 0.f),
                                                  fmaxf(__uint_as_float(x[e + 5]), 0.f)),
                                      make_float2(wb.x, wb.y), acc2);
                    acc3 = __ffma2_rn(make_float2(fmaxf(__uint_as_float(x[e + 6]), 0.f),
                                                  fmaxf(__uint_as_float(x[e + 7]), 0.f)),
                                      make_float2(wb.z, wb.w), acc3);
                }
                if ((c & 1) == 1) {   // a query row (64 heads = two chunks) is complete
                    const int i = c >> 1;
                    const float2 sum = __fadd2_rn(__fadd2_rn(acc0, acc1), __fadd2_rn(acc2, acc3));
                    const float r = (sum.x + sum.y) * scale;
                    if (t < ctx_row[i])
                        p.logits[static_cast<int64_t>(cur.b * NEXT_N + i) * p.logits_stride + t] = r;
                    acc0 = acc1 = acc2 = acc3 = make_float2(0.f, 0.f);
                }
            }
            ring.step(kMathGroups, S);
            tring.step(kMathGroups, kTmemStages);
        }
        if (alive && ntiles > 0 && at < ntiles - 1)
            advance_by<NEXT_N, kTile>(cur, ntiles - 1 - at, p.context_lens, p.batch, p.max_ctx, on_enter);
    }

    __syncthreads();
    if (*abort_flag) abort_drain_sleep();
    __syncthreads();
    if (warp == kMmaWarp0) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemStages * kN);
    }
}

template <int NEXT_N>
static int launch(const CUtensorMap& q_map, const CUtensorMap& kv_map, const CUtensorMap& sf_map, const Params& p, int grid,
                  cudaStream_t stream) {
    const int smem = Smem<NEXT_N>::total(p.kv_stages);
    auto kernel = mqa_logits_fp8_kernel<NEXT_N>;
    WUDA_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    WUDA_CUDA(launch_pdl(kernel, dim3(grid), dim3(kThreads), smem, stream, q_map, kv_map, sf_map, p));
    return WUDA_OK;
}

}  // namespace mqa
}  // namespace wuda

extern "C" int wuda_mqa_logits_fp8(const void* q, const void* kv_pages, const float* weights,
                                   const int32_t* context_lens, const int32_t* block_table,
                                   float* logits, int batch, int next_n, int num_blocks,
                                   int entries_per_block, int64_t page_stride_bytes,
                                   int block_table_stride, int64_t logits_stride,
                                   int32_t* status_word, void* stream) {
    using namespace wuda;
    using namespace wuda::mqa;
    clear_error();
    WUDA_REQUIRE(batch >= 0, "batch must be >= 0 (got %d)", batch);
    if (next_n != 1 && next_n != 2)
        return fail(WUDA_ERR_UNSUPPORTED, "next_n must be 1 or 2 (got %d)", next_n);
    WUDA_REQUIRE(entries_per_block == 32 || entries_per_block == 64 || entries_per_block == 128,
                 "entries_per_block must be 32, 64 or 128 (got %d)", entries_per_block);
    WUDA_REQUIRE(page_stride_bytes >= static_cast<int64_t>(entries_per_block) * (kDim + 4) &&
                     page_stride_bytes % 16 == 0,
                 "page_stride_bytes must be a multiple of 16 and >= entries_per_block * 132 (got %lld)",
                 static_cast<long long>(page_stride_bytes));
    WUDA_REQUIRE(num_blocks >= 1, "num_blocks must be >= 1 (got %d)", num_blocks);
    WUDA_REQUIRE(block_table_stride >= 1, "block_table_stride must be >= 1 (got %d)", block_table_stride);
    WUDA_REQUIRE(logits_stride >= 1, "logits_stride must be >= 1");
    if (batch == 0) return WUDA_OK;
    WUDA_REQUIRE(q && kv_pages && weights && context_lens && block_table && logits,
                 "q, kv_pages, weights, context_lens, block_table and logits must not be NULL");
    WUDA_REQUIRE(aligned16(q) && aligned16(kv_pages) && aligned16(weights),
                 "q, kv_pages and weights must be 16-byte aligned");
    WUDA_REQUIRE(static_cast<int64_t>(batch) * next_n * kHeads < (1ll << 31), "batch too large");

    DeviceInfo dev;
    int st = current_device_info(&dev);
    if (st != WUDA_OK) return st;

    const int kN = next_n * kHeads;
    CUtensorMap q_map, kv_map, sf_map;
    {
        const uint64_t dims[2] = {static_cast<uint64_t>(kDim), static_cast<uint64_t>(batch) * kN};
        const uint64_t strides[1] = {static_cast<uint64_t>(kDim)};
        const uint32_t box[2] = {static_cast<uint32_t>(kDim), static_cast<uint32_t>(kN)};
        st = encode_tensor_map(&q_map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, q, dims, strides, box,
                               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B);
        if (st != WUDA_OK) return st;
    }
    {
        const uint64_t dims[3] = {static_cast<uint64_t>(kDim), static_cast<uint64_t>(entries_per_block),
                                  static_cast<uint64_t>(num_blocks)};
        const uint64_t strides[2] = {static_cast<uint64_t>(kDim), static_cast<uint64_t>(page_stride_bytes)};
        const uint32_t box[3] = {static_cast<uint32_t>(kDim), static_cast<uint32_t>(entries_per_block), 1u};
        st = encode_tensor_map(&kv_map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, kv_pages, dims, strides, box,
                               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
        if (st != WUDA_OK) return st;
    }

    {   // per-token scales: entries_per_block fp32 after the key bytes of each page
        const uint64_t dims[3] = {static_cast<uint64_t>(entries_per_block), 1ull, static_cast<uint64_t>(num_blocks)};
        const uint64_t strides[2] = {static_cast<uint64_t>(page_stride_bytes), static_cast<uint64_t>(page_stride_bytes)};
        const uint32_t box[3] = {static_cast<uint32_t>(entries_per_block), 1u, 1u};
        st = encode_tensor_map(&sf_map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3,
                               static_cast<const uint8_t*>(kv_pages) + static_cast<int64_t>(entries_per_block) * kDim,
                               dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE);
        if (st != WUDA_OK) return st;
    }

    Params p;
    p.kv_pages = static_cast<const uint8_t*>(kv_pages);
    p.weights = weights;
    p.context_lens = context_lens;
    p.block_table = block_table;
    p.logits = logits;
    p.status = status_word;
    p.page_stride = page_stride_bytes;
    p.logits_stride = logits_stride;
    p.batch = batch;
    p.num_blocks = num_blocks;
    p.epb = entries_per_block;
    p.bt_stride = block_table_stride;
    {
        const int64_t by_table = static_cast<int64_t>(block_table_stride) * entries_per_block;
        const int64_t cap = logits_stride < by_table ? logits_stride : by_table;
        p.max_ctx = static_cast<int>(cap < 0x7fffff00 ? cap : 0x7fffff00);
    }
    // As many key stages as shared memory allows (a stage = 128 tokens = 16.5 KB), in
    // multiples of kStageQuantum: a stage must always be filled by the same producer,
    // read by the same issuer and released by the same math group, because a parity
    // wait is only sound while its waiter is at most one phase ahead of the barrier,
    // and only an agent's own earlier use of the stage guarantees that.
    int stages = kMaxKvStages;
    while (stages > kStageQuantum &&
           (next_n == 1 ? Smem<1>::total(stages) : Smem<2>::total(stages)) > dev.smem_optin)
        stages -= kStageQuantum;
    if ((next_n == 1 ? Smem<1>::total(stages) : Smem<2>::total(stages)) > dev.smem_optin)
        return fail(WUDA_ERR_UNSUPPORTED, "device offers %d bytes of shared memory per block; the kernel needs more",
                    dev.smem_optin);
    p.kv_stages = stages;

    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (next_n == 1) return launch<1>(q_map, kv_map, sf_map, p, dev.num_sms, s);
    return launch<2>(q_map, kv_map, sf_map, p, dev.num_sms, s);
}
