// NVFP4 block-scaled GEMM for decode-sized M on sm_100a:
//
//   C[M, N] (bf16) = gs_a * gs_w * sum_k (e2m1 a[m,k] * ue4m3 a_sf[m, k/16]) * (e2m1 w[n,k] * ue4m3 w_sf[n, k/16])
//
// Operands are packed 4-bit e2m1 (two per byte, low nibble first; value table and rounding as in
// dsv4_megakernel/origin/convert.py:11-14 and megakernel/test/test_mqa_logits_fp4.py:69-115), with one
// ue4m3 scale per 16 elements along K and one fp32 scale per tensor.  The reference has no NVFP4
// GEMM (its FP4 path, origin/kernel.py:441-536, is W4A8 with 1x32 e8m0 scales); this is the form the
// benchmark configuration names.
//
// The block scales ride the tensor core: tcgen05.mma kind::mxf4nvf4.block_scale.scale_vec::4X reads
// them from TMEM, where tcgen05.cp puts them from shared memory, so a tile accumulates over its whole
// K range in TMEM and the epilogue runs once per tile (times gs_a * gs_w, to bf16).  Everything else
// follows the FP8 GEMM of this library: swap-AB (UMMA M = 128 weight rows, UMMA N = padded M),
// stream-K over the flat (weight tile, 256-wide K block) list, one TMA instruction per unit (weights,
// activations and both scale blocks, one lane each), partial tiles through per-CTA scratch slots
// added in CTA order, bounded waits.
//
// Scale layout in global memory ("packed"): per 128 rows x 256 K one 2 KB block
// [4 K/64 steps][32 = row % 32][4 = row / 32][4 scales of the step], blocks ordered [row tile][K/256].
// It is the image tcgen05.cp.32x128b.warpx4 expects, so a unit's scales are one contiguous copy.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstring>

#include "host.h"
#include "ptx.cuh"

namespace wuda {
namespace gemm4 {

constexpr int kTileN = 128;          // weight rows per tile (UMMA M)
constexpr int kBlockK = 256;         // K elements per unit = 128 bytes per row
constexpr int kRowBytes = 128;
constexpr int kProducers = 4;        // warps 0..3: a warp needs ~1000 cycles to start a unit's four copies, a unit lasts ~800
constexpr int kIssuers = 2;          // warps 2, 3: each accumulates its own units into its own TMEM tile
constexpr int kFirstEpiWarp = 8;     // warps 8..11 (6 and 7 idle: the TMEM lane quarter of a warp is warp % 4)
constexpr int kEpiWarps = 4;
constexpr int kThreads = 32 * (kFirstEpiWarp + kEpiWarps);
// Role layout by tile width.  Up to 64 activation rows: four producers (warps 0..3), two issuers (4, 5), epilogue
// warps 8..11.  128 rows: the epilogue holds 128 accumulators per thread and needs the registers of a 256-thread
// CTA, and the wide stages leave room for few of them: two producers (0, 1), issuers 2, 3, epilogue 4..7.
__host__ __device__ constexpr int producers_for(int m_pad) { return m_pad >= 128 ? 2 : kProducers; }
__host__ __device__ constexpr int first_epi_warp_for(int m_pad) { return (producers_for(m_pad) + kIssuers + 3) / 4 * 4; }
__host__ __device__ constexpr int threads_for(int m_pad) { return 32 * (first_epi_warp_for(m_pad) + kEpiWarps); }
constexpr int kWBytes = kTileN * kRowBytes;   // 16 KB
constexpr int kSfBytes = 2048;                // one packed scale block
constexpr int kMaxGrid = 192;
constexpr int64_t kFlagBytes = 1024;   // the flags lead the scratch: calls of any row count find them in the same place

struct Params {
    __nv_bfloat16* c;
    float* scratch;            // [grid][M_PAD][128] fp32 partial-tile slots
    int32_t* flags;            // [grid]
    int32_t* status;
    float out_scale;           // gs_a * gs_w
    int M, N, kb;              // kb = K / 256
    int n_tiles;
    int stages;
    // grouped form (routed experts): row group g (16 activation rows) belongs to expert
    // group_expert[g]; flat tile T = g * n_tiles + tile of the expert's N rows.  The number of groups
    // is read on the device, so nothing is synchronised with the host between routing and the GEMM.
    const int32_t* group_expert = nullptr;   // [num_groups]
    const int32_t* row_token = nullptr;      // [num_groups * 16] or nullptr: rows without a token (< 0) are not stored
    const int32_t* num_groups = nullptr;     // [1]
    const float* expert_scale = nullptr;     // [experts] per-expert weight tensor scale (times out_scale)
};

template <int M_PAD>
struct Smem {
    static constexpr int kABytes = M_PAD * kRowBytes;
    static constexpr int kStageBytes = kWBytes + kABytes + 2 * kSfBytes;
    // TMEM columns: one accumulator tile per issuer, then per issuer 16 + 16 scale columns
    static constexpr int kAccCols = kIssuers * M_PAD;
    static constexpr int kUsedCols = kAccCols + kIssuers * 32;
    static constexpr int kTmemCols = kUsedCols <= 64 ? 64 : (kUsedCols <= 128 ? 128 : (kUsedCols <= 256 ? 256 : 512));
    static __host__ __device__ constexpr int bar_off(int stages) { return stages * kStageBytes; }
    // barriers: full[16] empty[16] full_tm empty_tm
    static __host__ __device__ constexpr int misc_off(int stages) { return bar_off(stages) + 34 * 8; }
    static __host__ __device__ constexpr int total(int stages) { return misc_off(stages) + 32 + 1024; }
};

struct Ring {
    int idx = 0;
    uint32_t phase = 0;
    __device__ __forceinline__ void step(int n, int size) {
        idx += n;
        if (idx >= size) {
            idx -= size;
            phase ^= 1u;
        }
    }
};

__device__ __forceinline__ void epi_bar_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
__device__ __forceinline__ void st_release_gpu(int32_t* p, int v) {
    asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_gpu(const int32_t* p) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ long long range_begin(long long units, int c, int grid) { return units * c / grid; }
__device__ __forceinline__ int cta_of(long long units, long long u, int grid) {
    int c = static_cast<int>(u * grid / units);
    while (c + 1 < grid && range_begin(units, c + 1, grid) <= u) ++c;
    while (c > 0 && range_begin(units, c, grid) > u) --c;
    return c;
}

template <int M_PAD>
__global__ void __launch_bounds__(threads_for(M_PAD), 1)
gemm_nvfp4_kernel(const __grid_constant__ CUtensorMap w_map, const __grid_constant__ CUtensorMap a_map,
                  const __grid_constant__ CUtensorMap wsf_map, const __grid_constant__ CUtensorMap asf_map,
                  const Params p) {
    using L = Smem<M_PAD>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t base = (raw_addr + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (base - raw_addr);
    const int S = p.stages;
    const uint32_t bars = base + L::bar_off(S);
    const uint32_t full = bars, empty = bars + 16 * 8, full_tm = bars + 32 * 8, empty_tm = bars + 33 * 8;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(base_ptr + L::misc_off(S));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(base_ptr + L::misc_off(S) + 4);

    const int warp = threadIdx.x >> 5;
    const uint32_t lane = lane_id();

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int i = 0; i < S; ++i) {
            mbar_init(full + i * 8, 1);
            mbar_init(empty + i * 8, 1);
        }
        mbar_init(full_tm, kIssuers);      // both issuers' accumulators of a segment are complete
        mbar_init(empty_tm, kEpiWarps);    // the epilogue has read them
        fence_mbar_init();
    }
    if (warp == producers_for(M_PAD)) {
        tmem_alloc(smem_u32(tmem_slot), L::kTmemCols);
        tmem_relinquish();
    }
    if (warp == 0 && lane == 0) {
        prefetch_tmap(&w_map);
        prefetch_tmap(&a_map);
        prefetch_tmap(&wsf_map);
        prefetch_tmap(&asf_map);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // the prologue above ran while the kernel ahead was still finishing; global memory from here on
    pdl_launch_dependents();
    pdl_wait();

    const bool grouped = p.group_expert != nullptr;
    const int groups = grouped ? *p.num_groups : 1;
    const long long units = static_cast<long long>(groups) * p.n_tiles * p.kb;
    // Only the first min(grid, units) CTAs take part (the grouped form is launched with one CTA per SM
    // before the number of groups is known): every participating CTA then owns at least one unit, which
    // the fix-up relies on when it waits for the CTAs that share a tile.
    const int grid = units < static_cast<long long>(gridDim.x) ? static_cast<int>(units) : static_cast<int>(gridDim.x);
    const bool taking_part = static_cast<int>(blockIdx.x) < grid;
    const long long u0 = taking_part ? range_begin(units, blockIdx.x, grid) : 0;
    const long long u1 = taking_part ? range_begin(units, blockIdx.x + 1, grid) : 0;
    const int count = static_cast<int>(u1 - u0);

    // wide activation tiles leave room for few stages; they keep two producers so that the stage count can be
    // any even number (a stage always belongs to one producer and one issuer)
    constexpr int kProd = producers_for(M_PAD);
    constexpr int kIssuer0 = kProd;                       // first issuer warp (it owns the TMEM allocation)
    constexpr int kEpi0 = first_epi_warp_for(M_PAD);
    if (warp < kProd) {
        // ------------------------------------------------------------ TMA producers
        const int me = warp;
        const uint64_t stream_policy = policy_evict_first();
        const uint64_t keep_policy = policy_evict_last();
        Ring ring;
        ring.step(me, S);
        int tile = static_cast<int>((u0 + me) / p.kb), kb = static_cast<int>((u0 + me) % p.kb);
        int seen_tile = -1, grp = grouped ? -1 : 0, expert = 0, wtile = 0;
        bool alive = true;
        for (int n = me; n < count && alive; n += kProd) {
            const int s = ring.idx;
            alive = mbar_wait_lane0(empty + s * 8, ring.phase ^ 1u, abort_flag, p.status, kDevTimeoutGemmEmpty);
            if (!alive) break;
            if (lane == 0) mbar_arrive_expect_tx(full + s * 8, L::kStageBytes);
            __syncwarp();
            // one instruction, four lanes: weights, activations, weight scales, activation scales
            const uint32_t stage = base + s * L::kStageBytes;
            uint32_t dst = stage;
            const void* map = &w_map;
            // grouped: `tile` is the flat index; the weight tile is the expert's, the activations the group's
            // (the group's expert is looked up only when the group changes: a dependent global load per
            // unit would sit in the producer's critical path)
            if (grouped && tile != seen_tile) {
                seen_tile = tile;
                const int g_now = tile / p.n_tiles;
                if (g_now != grp) {
                    grp = g_now;
                    expert = __ldcg(p.group_expert + grp);   // written by the dispatch kernel of the same chain
                }
                wtile = expert * p.n_tiles + (tile - grp * p.n_tiles);
            } else if (!grouped) {
                wtile = tile;
            }
            int c0 = kb * kRowBytes, c1 = wtile * kTileN;
            uint64_t policy = stream_policy;
            if (lane == 1) {
                dst = stage + kWBytes;
                map = &a_map;
                c1 = grp * M_PAD;
                policy = keep_policy;
            } else if (lane == 2) {
                dst = stage + kWBytes + L::kABytes;
                map = &wsf_map;
                c0 = 0;
                c1 = (wtile * p.kb + kb) * 4;
            } else if (lane == 3) {
                dst = stage + kWBytes + L::kABytes + kSfBytes;
                map = &asf_map;
                c0 = 0;
                c1 = (grp * p.kb + kb) * 4;
                policy = keep_policy;
            }
            if (lane < 4) tma_load_2d_hint(dst, map, full + s * 8, c0, c1, policy);
            ring.step(kProd, S);
            kb += kProd;
            while (kb >= p.kb) {
                kb -= p.kb;
                ++tile;
            }
        }
    } else if (warp >= kIssuer0 && warp < kIssuer0 + kIssuers) {
        // ------------------------------------------------------------ UMMA issuers (one thread each)
        // Issuer i takes units n with n % 2 == i and accumulates them into its own TMEM tile; the
        // epilogue adds the two tiles.  (Two threads must not chain accumulations into one tile:
        // only operations of one thread are ordered.)
        if (lane == 0) {
            const int me = warp - kIssuer0;
            // kind::mxf4nvf4: formats e2m1 (1), scale format ue4m3 (0), both operands K-major
            constexpr uint32_t idesc = umma_idesc_block_scaled(kTileN, M_PAD, 1, 1, 0, 0, 0);
            const uint32_t d_addr = tmem_base + me * M_PAD;
            const uint32_t sfw_t = tmem_base + L::kAccCols + me * 32;
            const uint32_t sfa_t = sfw_t + 16;
            Ring ring;
            ring.step(me, S);
            int kb = static_cast<int>(u0 % p.kb);
            uint32_t seg = 0;
            bool alive = true;
            // Both issuers walk every segment (a maximal run of units inside one weight tile), even
            // one in which they own no unit, so that both barriers advance once per segment for
            // everybody.
            for (int n = 0; n < count && alive;) {
                const int seg_len = min(p.kb - kb, count - n);
                if (seg > 0) {   // the epilogue must have drained the previous segment's accumulators
                    if (!mbar_wait(empty_tm, (seg - 1) & 1u, abort_flag, p.status, kDevTimeoutGemmTmemEmpty)) break;
                    tc_fence_after();
                }
                uint32_t accumulate = 0;
                for (int u = n + ((me ^ n) & 1); u < n + seg_len; u += kIssuers) {
                    const int s = ring.idx;
                    if (!mbar_wait(full + s * 8, ring.phase, abort_flag, p.status, kDevTimeoutGemmFull)) {
                        alive = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t stage = base + s * L::kStageBytes;
                    const uint32_t w_addr = stage, a_addr = stage + kWBytes;
                    const uint32_t wsf_addr = stage + kWBytes + L::kABytes, asf_addr = wsf_addr + kSfBytes;
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        // 32 rows x 16 bytes per K/64 step; 8-row groups 128 bytes apart
                        tmem_cp_32x128b_warpx4(sfw_t + k * 4, umma_smem_desc_noswz(wsf_addr + k * 512, 16, 128));
                        tmem_cp_32x128b_warpx4(sfa_t + k * 4, umma_smem_desc_noswz(asf_addr + k * 512, 16, 128));
                    }
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        umma_nvf4(d_addr, umma_smem_desc_sw128(w_addr + k * 32), umma_smem_desc_sw128(a_addr + k * 32),
                                  idesc, sfw_t + k * 4, sfa_t + k * 4, accumulate);
                        accumulate = 1;
                    }
                    umma_commit(empty + s * 8);     // the stage's bytes are consumed once these retire
                    ring.step(kIssuers, S);
                }
                if (!alive) break;
                umma_commit(full_tm);               // this issuer's part of the segment is complete
                n += seg_len;
                kb += seg_len;
                if (kb == p.kb) kb = 0;
                ++seg;
            }
        }
    } else if (warp >= kEpi0) {
        // ------------------------------------------------------------ epilogue warps
        const int et = (warp - kEpi0) * 32 + lane;       // 0..127 = weight row inside the tile
        const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
        bool alive = true;
        int tile = static_cast<int>(u0 / p.kb), kb = static_cast<int>(u0 % p.kb);
        uint32_t tm_phase = 0;
        int n = 0;
        while (n < count) {
            // the segment [kb, kb_end) of `tile`
            const int seg_len = min(p.kb - kb, count - n);
            const bool from_zero = (kb == 0), to_end = (kb + seg_len == p.kb);
            // Issuer i owns the units with n % 2 == i; a one-unit segment has only its first issuer's tile.
            const bool both = seg_len >= 2;
            const int first_issuer = n & 1;
            if (alive) alive = mbar_wait_warp_fast(full_tm, tm_phase, abort_flag, p.status, kDevTimeoutGemmTmemFull);
            tm_phase ^= 1u;
            float acc[M_PAD];
            if (alive) {
                tc_fence_after();
#pragma unroll
                for (int c = 0; c < M_PAD; c += 16) {
                    uint32_t v0[16], v1[16];
                    tmem_ld_32x16(tmem_base + lane_base + first_issuer * M_PAD + c, v0);
                    if (both) tmem_ld_32x16(tmem_base + lane_base + (first_issuer ^ 1) * M_PAD + c, v1);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 16; ++i)
                        acc[c + i] = __uint_as_float(v0[i]) + (both ? __uint_as_float(v1[i]) : 0.f);
                }
                tc_fence_before();
            } else {
#pragma unroll
                for (int i = 0; i < M_PAD; ++i) acc[i] = 0.f;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty_tm);

            const int grp = grouped ? tile / p.n_tiles : 0;
            const int nrow = (tile - grp * p.n_tiles) * kTileN + et;
            if (!from_zero) {
                float* slot = p.scratch + static_cast<int64_t>(blockIdx.x) * (M_PAD * kTileN) + et;
                if (alive) {
#pragma unroll
                    for (int i = 0; i < M_PAD; ++i) __stcg(slot + i * kTileN, acc[i]);
                }
                __threadfence();
                epi_bar_sync();
                if (et == 0 && alive) st_release_gpu(p.flags + blockIdx.x, 1);
            } else {
                if (!to_end) {
                    const long long t_end = static_cast<long long>(tile + 1) * p.kb - 1;
                    const int last = cta_of(units, t_end, grid);
                    // every contributor's flag is awaited by a thread of its own, then the partials are added in
                    // CTA order (the loads of different partials overlap)
                    for (int c = blockIdx.x + 1 + et; c <= last && alive; c += 32 * kEpiWarps) {
                        const unsigned long long start = globaltimer_ns();
                        uint32_t spins = 0;
                        while (ld_acquire_gpu(p.flags + c) == 0) {
                            if ((++spins & 255u) == 0u && (*abort_flag || globaltimer_ns() - start > kWaitLimitNs)) {
                                *abort_flag = 1;
                                if (p.status) atomicCAS(p.status, 0, kDevTimeoutPeerFlag);
                                break;
                            }
                            __nanosleep(64);
                        }
                    }
                    epi_bar_sync();
                    alive = alive && !*abort_flag;
                    if (alive) {
                        for (int c = blockIdx.x + 1; c <= last; ++c) {
                            const float* peer = p.scratch + static_cast<int64_t>(c) * (M_PAD * kTileN) + et;
#pragma unroll
                            for (int i = 0; i < M_PAD; ++i) acc[i] += __ldcg(peer + i * kTileN);
                        }
                    }
                    epi_bar_sync();
                    if (alive)
                        for (int c = blockIdx.x + 1 + et; c <= last; c += 32 * kEpiWarps) p.flags[c] = 0;
                }
                if (alive && nrow < p.N) {
                    const float scale = grouped ? p.out_scale * __ldg(p.expert_scale + __ldcg(p.group_expert + grp)) : p.out_scale;
                    __nv_bfloat16* c = p.c + static_cast<int64_t>(grp) * M_PAD * p.N;
                    uint32_t stored = 0xffffffffu;   // grouped rows without a token are padding: nobody reads them
                    if (M_PAD <= 32 && grouped && p.row_token) {
                        const int tok = lane < M_PAD ? __ldcg(p.row_token + grp * M_PAD + lane) : -1;
                        stored = __ballot_sync(0xffffffffu, tok >= 0);
                    }
#pragma unroll
                    for (int i = 0; i < M_PAD; ++i)
                        if (i < p.M && (M_PAD > 32 || ((stored >> i) & 1u)))
                            c[static_cast<int64_t>(i) * p.N + nrow] = __float2bfloat16_rn(acc[i] * scale);
                }
            }
            n += seg_len;
            kb += seg_len;
            if (kb == p.kb) {
                kb = 0;
                ++tile;
            }
        }
    }

    __syncthreads();
    if (*abort_flag) abort_drain_sleep();
    __syncthreads();
    if (warp == producers_for(M_PAD)) {
        tc_fence_after();
        tmem_dealloc(tmem_base, L::kTmemCols);
    }
}

template <int M_PAD>
static int launch(const CUtensorMap& w_map, const CUtensorMap& a_map, const CUtensorMap& wsf_map,
                  const CUtensorMap& asf_map, Params& p, const DeviceInfo& dev, cudaStream_t stream) {
    using L = Smem<M_PAD>;
    // stage counts are multiples of the producer and issuer counts (a stage always belongs to the same
    // producer and the same issuer)
    int stages = 16;
    constexpr int kStep = M_PAD >= 128 ? 2 : 4;   // lcm of the producer and issuer counts
    while (stages > kStep && L::total(stages) > dev.smem_optin) stages -= kStep;
    if (L::total(stages) > dev.smem_optin)
        return fail(WUDA_ERR_UNSUPPORTED, "device offers %d bytes of shared memory per block; the kernel needs more",
                    dev.smem_optin);
    p.stages = stages;
    auto kernel = gemm_nvfp4_kernel<M_PAD>;
    WUDA_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::total(stages)));
    const long long units = static_cast<long long>(p.n_tiles) * p.kb;
    // (grouped: the number of groups is only known on the device; one CTA per SM, idle ones return at once)
    // CTAs that may share one weight tile: the owner adds their partials serially, which costs about as much
    // per partial as streaming M_PAD / 64 units
    constexpr int kMaxSplit = M_PAD <= 16 ? 16 : (M_PAD == 32 ? 12 : (M_PAD == 64 ? 8 : 6));
    const int sms = gemm_sms(dev);
    int grid = (!p.group_expert && units < sms) ? static_cast<int>(units) : sms;
    if (!p.group_expert && static_cast<long long>(p.n_tiles) * kMaxSplit < grid) grid = p.n_tiles * kMaxSplit;
    WUDA_CUDA(launch_pdl(kernel, dim3(grid), dim3(threads_for(M_PAD)), L::total(stages), stream, w_map, a_map, wsf_map, asf_map, p));
    return WUDA_OK;
}

}  // namespace gemm4
}  // namespace wuda

extern "C" int64_t wuda_gemm_nvfp4_scratch_bytes(int m, int n) {
    if (m < 1 || n < 1 || m > 256) return -1;
    int m_pad = 16;
    while (m_pad < m && m_pad < 128) m_pad *= 2;      // above 128 rows: passes of <= 128 rows
    return wuda::gemm4::kFlagBytes + static_cast<int64_t>(wuda::gemm4::kMaxGrid) * m_pad * 128 * 4;
}

extern "C" int wuda_gemm_nvfp4(const void* a, const void* a_sf_packed, float a_global_scale, const void* w,
                               const void* w_sf_packed, float w_global_scale, void* c_bf16, int m, int n, int k,
                               void* scratch, int64_t scratch_bytes, int32_t* status_word, void* stream) {
    using namespace wuda;
    using namespace wuda::gemm4;
    clear_error();
    WUDA_REQUIRE(m >= 0 && m <= 256, "m must be in [0, 256] (got %d)", m);
    WUDA_REQUIRE(n >= 1, "n must be >= 1 (got %d)", n);
    WUDA_REQUIRE(k >= 256 && k % 256 == 0, "k must be a positive multiple of 256 (got %d)", k);
    if (m == 0) return WUDA_OK;
    WUDA_REQUIRE(a && a_sf_packed && w && w_sf_packed && c_bf16 && scratch,
                 "a, a_sf_packed, w, w_sf_packed, c and scratch must not be NULL");
    if (m > 128) {
        // A tile holds at most 128 activation rows (the accumulator's columns): two passes over the weights,
        // one per 128-row tile of the activations and of their packed scales ([row tile][k / 256][2048 bytes]).
        int st2 = wuda_gemm_nvfp4(a, a_sf_packed, a_global_scale, w, w_sf_packed, w_global_scale, c_bf16, 128, n, k, scratch,
                                  scratch_bytes, status_word, stream);
        if (st2 != WUDA_OK) return st2;
        return wuda_gemm_nvfp4(static_cast<const uint8_t*>(a) + static_cast<int64_t>(128) * (k / 2),
                               static_cast<const uint8_t*>(a_sf_packed) + static_cast<int64_t>(k / 256) * 2048, a_global_scale,
                               w, w_sf_packed, w_global_scale,
                               static_cast<__nv_bfloat16*>(c_bf16) + static_cast<int64_t>(128) * n, m - 128, n, k, scratch,
                               scratch_bytes, status_word, stream);
    }
    WUDA_REQUIRE(aligned16(a) && aligned16(w) && aligned16(a_sf_packed) && aligned16(w_sf_packed),
                 "operands and packed scales must be 16-byte aligned");
    WUDA_REQUIRE((reinterpret_cast<uintptr_t>(scratch) & 255u) == 0, "scratch must be 256-byte aligned");
    const int64_t need = wuda_gemm_nvfp4_scratch_bytes(m, n);
    WUDA_REQUIRE(scratch_bytes >= need, "scratch holds %lld bytes; %lld are needed (wuda_gemm_nvfp4_scratch_bytes)",
                 static_cast<long long>(scratch_bytes), static_cast<long long>(need));

    DeviceInfo dev;
    int st = current_device_info(&dev);
    if (st != WUDA_OK) return st;
    WUDA_REQUIRE(dev.num_sms <= kMaxGrid, "device has %d SMs; at most %d are supported", dev.num_sms, kMaxGrid);

    int m_pad = 16;
    while (m_pad < m) m_pad *= 2;
    Params p;
    p.c = static_cast<__nv_bfloat16*>(c_bf16);
    p.status = status_word;
    p.out_scale = a_global_scale * w_global_scale;
    p.M = m;
    p.N = n;
    p.kb = k / 256;
    p.n_tiles = (n + 127) / 128;
    p.scratch = reinterpret_cast<float*>(static_cast<uint8_t*>(scratch) + kFlagBytes);
    p.flags = static_cast<int32_t*>(scratch);
    p.stages = 0;

    CUtensorMap w_map, a_map, wsf_map, asf_map;
    const uint64_t row_bytes = static_cast<uint64_t>(k) / 2;
    {
        const uint64_t dims[2] = {row_bytes, static_cast<uint64_t>(n)};
        const uint64_t strides[1] = {row_bytes};
        const uint32_t box[2] = {128u, 128u};
        st = encode_tensor_map(&w_map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, w, dims, strides, box,
                               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
        if (st != WUDA_OK) return st;
    }
    {
        const uint64_t dims[2] = {row_bytes, static_cast<uint64_t>(m)};
        const uint64_t strides[1] = {row_bytes};
        const uint32_t box[2] = {128u, static_cast<uint32_t>(m_pad)};
        st = encode_tensor_map(&a_map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, a, dims, strides, box,
                               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B);
        if (st != WUDA_OK) return st;
    }
    {   // packed scales as rows of 512 bytes (one K/64 step of 128 rows); a unit's block is 4 rows
        const uint64_t dims[2] = {128ull, static_cast<uint64_t>(p.n_tiles) * p.kb * 4};
        const uint64_t strides[1] = {512ull};
        const uint32_t box[2] = {128u, 4u};
        st = encode_tensor_map(&wsf_map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, w_sf_packed, dims, strides, box,
                               CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE);
        if (st != WUDA_OK) return st;
    }
    {
        const uint64_t dims[2] = {128ull, static_cast<uint64_t>(p.kb) * 4};
        const uint64_t strides[1] = {512ull};
        const uint32_t box[2] = {128u, 4u};
        st = encode_tensor_map(&asf_map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, a_sf_packed, dims, strides, box,
                               CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE);
        if (st != WUDA_OK) return st;
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (m_pad) {
        case 16: return launch<16>(w_map, a_map, wsf_map, asf_map, p, dev, s);
        case 32: return launch<32>(w_map, a_map, wsf_map, asf_map, p, dev, s);
        case 64: return launch<64>(w_map, a_map, wsf_map, asf_map, p, dev, s);
        default: return launch<128>(w_map, a_map, wsf_map, asf_map, p, dev, s);
    }
}

// Grouped form for the routed experts: activations [max_groups * 16, k] quantised per group (see
// moe.cu), expert weights stacked [experts * n, k / 2] with their packed scales stacked per expert.
extern "C" int wuda_gemm_nvfp4_grouped(const void* a, const void* a_sf_packed, float a_global_scale, const void* w,
                                       const void* w_sf_packed, const float* w_global_scales,
                                       const int32_t* group_expert, const int32_t* num_groups, const int32_t* row_token,
                                       void* c_bf16, int max_groups, int experts, int n, int k, void* scratch, int64_t scratch_bytes,
                                       int32_t* status_word, void* stream) {
    using namespace wuda;
    using namespace wuda::gemm4;
    clear_error();
    WUDA_REQUIRE(max_groups >= 1 && experts >= 1, "max_groups and experts must be >= 1");
    WUDA_REQUIRE(n >= 128 && n % 128 == 0, "n (rows per expert) must be a positive multiple of 128 (got %d)", n);
    WUDA_REQUIRE(k >= 256 && k % 256 == 0, "k must be a positive multiple of 256 (got %d)", k);
    WUDA_REQUIRE(a && a_sf_packed && w && w_sf_packed && w_global_scales && group_expert && num_groups && c_bf16 && scratch,
                 "no array may be NULL");
    WUDA_REQUIRE(aligned16(a) && aligned16(w) && aligned16(a_sf_packed) && aligned16(w_sf_packed),
                 "operands and packed scales must be 16-byte aligned");
    WUDA_REQUIRE((reinterpret_cast<uintptr_t>(scratch) & 255u) == 0, "scratch must be 256-byte aligned");
    const int64_t need = wuda_gemm_nvfp4_scratch_bytes(16, n);
    WUDA_REQUIRE(scratch_bytes >= need, "scratch holds %lld bytes; %lld are needed (wuda_gemm_nvfp4_scratch_bytes(16, n))",
                 static_cast<long long>(scratch_bytes), static_cast<long long>(need));
    DeviceInfo dev;
    int st = current_device_info(&dev);
    if (st != WUDA_OK) return st;
    WUDA_REQUIRE(dev.num_sms <= kMaxGrid, "device has %d SMs; at most %d are supported", dev.num_sms, kMaxGrid);

    constexpr int m_pad = 16;
    Params p;
    p.c = static_cast<__nv_bfloat16*>(c_bf16);
    p.status = status_word;
    p.out_scale = a_global_scale;
    p.M = m_pad;
    p.N = n;
    p.kb = k / 256;
    p.n_tiles = n / 128;
    p.scratch = reinterpret_cast<float*>(static_cast<uint8_t*>(scratch) + kFlagBytes);
    p.flags = static_cast<int32_t*>(scratch);
    p.stages = 0;
    p.group_expert = group_expert;
    p.num_groups = num_groups;
    p.row_token = row_token;
    p.expert_scale = w_global_scales;

    CUtensorMap w_map, a_map, wsf_map, asf_map;
    const uint64_t row_bytes = static_cast<uint64_t>(k) / 2;
    {
        const uint64_t dims[2] = {row_bytes, static_cast<uint64_t>(experts) * n};
        const uint64_t strides[1] = {row_bytes};
        const uint32_t box[2] = {128u, 128u};
        st = encode_tensor_map(&w_map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, w, dims, strides, box,
                               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
        if (st != WUDA_OK) return st;
    }
    {
        const uint64_t dims[2] = {row_bytes, static_cast<uint64_t>(max_groups) * m_pad};
        const uint64_t strides[1] = {row_bytes};
        const uint32_t box[2] = {128u, static_cast<uint32_t>(m_pad)};
        st = encode_tensor_map(&a_map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, a, dims, strides, box,
                               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B);
        if (st != WUDA_OK) return st;
    }
    {
        const uint64_t dims[2] = {128ull, static_cast<uint64_t>(experts) * p.n_tiles * p.kb * 4};
        const uint64_t strides[1] = {512ull};
        const uint32_t box[2] = {128u, 4u};
        st = encode_tensor_map(&wsf_map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, w_sf_packed, dims, strides, box,
                               CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE);
        if (st != WUDA_OK) return st;
    }
    {
        const uint64_t dims[2] = {128ull, static_cast<uint64_t>(max_groups) * p.kb * 4};
        const uint64_t strides[1] = {512ull};
        const uint32_t box[2] = {128u, 4u};
        st = encode_tensor_map(&asf_map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, a_sf_packed, dims, strides, box,
                               CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE);
        if (st != WUDA_OK) return st;
    }
    return launch<16>(w_map, a_map, wsf_map, asf_map, p, dev, static_cast<cudaStream_t>(stream));
}
