// Block-scaled FP8 GEMM whose scales are powers of two, with the scales applied INSIDE the tensor core:
//
//   C[M, N] (bf16) = sum over 128-wide K blocks of (a[m, kb] * a_scale[m, kb]) . (w[n, kb] * w_scale[n/128, kb])
//
// Same operands and layouts as wuda_gemm_fp8_blockscaled (e4m3, fp32 scales: 1x128 for the activations,
// 128x128 for the weights; origin/kernel.py:203-273), restricted to scales that are exact powers of two -
// which is what the reference's checkpoints and quantisers produce (UE8M0 scales:
// dsv4_megakernel/megakernel/kernels/wq_b_fp8_gemm.cu:139-183 writes them, include/cluster_mma_fp8.cuh:144-301
// consumes them through block-scaled MMAs).  Then tcgen05.mma kind::mxf8f6f4.block_scale (one UE8M0 scale per
// 32 K-elements and operand row, read from tensor memory) multiplies by 2^(e_a - 127) * 2^(e_w - 127) on the way
// into the accumulator, a weight tile accumulates over its whole K range in TMEM, and the CUDA-core promotion of
// every K block - what bounds the general kernel from 64 rows up - is gone.  The epilogue runs once per tile
// segment.
//
// Skeleton as in the other GEMMs of this library: swap-AB (UMMA M = 128 weight rows, UMMA N = padded M), stream-K
// over the flat (weight tile, K block) list, one TMA instruction per unit, two issuer warps that take units
// alternately into their own TMEM tiles, partial tiles through per-CTA scratch slots added in CTA order, bounded
// waits.  New here:
//   * The scale images.  A unit (128 x 128 bytes) is four MMAs of K = 32; their scale bytes are the four bytes
//     of one 32-bit TMEM column per row, chosen by the instruction descriptor's scale ids.  The producer warp
//     that fetches a unit also builds its two 512-byte images in the stage ([row % 32][row / 32] words, the
//     layout tcgen05.cp.32x128b.warpx4 copies) while the copies are in flight: the weight image is one
//     exponent byte repeated, the activation image one byte per row, both read from the fp32 scales a unit
//     ahead.  The issuer thread only copies the images to TMEM and issues.
//   * Up to 64 rows the accumulators are double-buffered over segments, so the issuers start a tile's MMAs
//     while the epilogue still drains the previous one (at K = 1536 a tile is only 12 units long).
// A scale that is not a power of two is truncated to one and reported (WUDA_DEV_SCALE_NOT_POW2); a zero scale
// reads as 2^-127.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstring>

#include "host.h"
#include "ptx.cuh"

namespace wuda {
namespace gemm8mx {

constexpr int kTileN = 128;          // weight rows per tile (UMMA M)
constexpr int kRowBytes = 128;       // K elements (bytes) per unit
constexpr int kProducers = 4;
constexpr int kIssuers = 2;
constexpr int kEpiWarps = 4;
// RES ("resident"): the whole activation matrix [M_PAD, K] stays in shared memory for the kernel's lifetime (short K:
// the q projection's 1536), so a unit's copy is the weight tile alone - at 64 rows a third less for the SM to take
// in - and two producers are enough (which also lets the stage count be any even number).
__host__ __device__ constexpr int producers_for(int m_pad, bool res = false) { return (m_pad >= 128 || res) ? 2 : kProducers; }
__host__ __device__ constexpr int first_epi_warp_for(int m_pad, bool res = false) { return (producers_for(m_pad, res) + kIssuers + 3) / 4 * 4; }
__host__ __device__ constexpr int threads_for(int m_pad, bool res = false) { return 32 * (first_epi_warp_for(m_pad, res) + kEpiWarps); }
__host__ __device__ constexpr int acc_buffers_for(int m_pad) { return m_pad <= 64 ? 2 : 1; }
constexpr int kWBytes = kTileN * kRowBytes;   // 16 KB
constexpr int kSfBytes = 512;                 // one scale image: 32 rows x 16 bytes
constexpr int kSfDepth = 4;                   // W4: units a producer requests its weight scales ahead
constexpr int kMaxGrid = 192;
constexpr int64_t kFlagBytes = 1024;          // as in gemm_fp8.cu: the two kernels share a scratch

struct Params {
    __nv_bfloat16* c;
    const float* a_scales;     // [M, scale_cols]
    const float* w_scales;     // [tiles, kb] = flat unit order (FP8 weights)
    const uint8_t* w_sf;       // W4: [N, K/32] exponent bytes, one per weight row and 32 K-elements
    int sf_stride;             // W4: bytes between the rows of w_sf
    float* scratch;            // [grid][M_PAD][128] fp32 partial-tile slots
    int32_t* flags;            // [grid]
    int32_t* status;
    int M, N, kb;              // N = all output columns, kb = K blocks per tile
    int n_tiles;               // all weight tiles (of all groups)
    int tiles_per_group;       // grouped form: tile t belongs to group t / tiles_per_group, whose activations start at
                               // K block group * kb; plain form: tiles_per_group = n_tiles (one group)
    int scale_cols;            // K blocks of an activation row (all groups)
    int stages;
};

template <int M_PAD, bool RES = false>
struct Smem {
    static constexpr int kABytes = M_PAD * kRowBytes;
    static constexpr int kStageBytes = kWBytes + (RES ? 0 : kABytes) + 2 * kSfBytes;   // W | [A] | two scale images
    static constexpr int kSfOff = kWBytes + (RES ? 0 : kABytes);
    static constexpr int kBuffers = acc_buffers_for(M_PAD);
    // TMEM columns: per buffer one accumulator tile per issuer, then per issuer 4 + 4 scale columns (16 reserved)
    static constexpr int kAccCols = kBuffers * kIssuers * M_PAD;
    static constexpr int kUsedCols = kAccCols + kIssuers * 16;
    static constexpr int kTmemCols = kUsedCols <= 64 ? 64 : (kUsedCols <= 128 ? 128 : (kUsedCols <= 256 ? 256 : 512));
    // behind the stages: the resident activations, kb tiles of kABytes (RES only)
    static __host__ __device__ constexpr int res_off(int stages) { return stages * kStageBytes; }
    static __host__ __device__ constexpr int bar_off(int stages, int kb) { return res_off(stages) + (RES ? kb * kABytes : 0); }
    // barriers: full[16] empty[16] full_tm[2] empty_tm[2] a_full
    static __host__ __device__ constexpr int misc_off(int stages, int kb) { return bar_off(stages, kb) + 38 * 8; }
    // W4: behind the 32 bytes of odds and ends, per producer warp a ring of kSfDepth weight-scale images (512 B each)
    // that cp.async fills kSfDepth units ahead
    static __host__ __device__ constexpr int sf_ring_off(int stages, int kb) { return misc_off(stages, kb) + 32; }
    static __host__ __device__ constexpr int total(int stages, int kb, bool w4 = false) {
        return sf_ring_off(stages, kb) + (w4 ? kProducers * kSfDepth * kSfBytes : 0) + 1024;
    }
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

__device__ __forceinline__ void umma_mxf8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t sfa_tmem,
                                          uint32_t sfb_tmem, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale.scale_vec::1X "
        "[%0], %1, %2, %3, [%5], [%6], p;\n\t"
        "}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
        : "memory");
}

// 4 bytes global -> shared without a register in between (src_bytes = 0: zeros); groups are counted per thread
__device__ __forceinline__ void cp_async_4(uint32_t dst, const void* src, uint32_t src_bytes) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Exponent byte of a power-of-two fp32 scale; anything else is reported and truncated to the power of two below.
__device__ __forceinline__ uint32_t exponent_byte(float scale, int32_t* status) {
    const uint32_t bits = __float_as_uint(scale);
    if (((bits & 0x807fffffu) != 0u || (bits >> 23) == 0xffu) && scale != 0.f && status)
        atomicCAS(status, 0, static_cast<int>(kDevScaleNotPow2));
    const uint32_t e = (bits >> 23) & 0xffu;
    return e == 0xffu ? 0xfeu : e;
}

// W4: the weights are e2m1, two to a byte ([N, K/2], low nibble first), with one exponent byte per row and 32 K-elements
// (origin/kernel.py:441-536, fp4_gemm).  The tensor core reads 4-bit operands of this kind from shared memory in the
// padded form - 16 values in 8 bytes, then 8 bytes of nothing - which is what a tensor map of type 16U4_ALIGN16B makes
// of the packed rows: a unit's weight tile still fills 16 KB of the stage but is 8 KB of global memory, and the
// barrier counts those 8 KB.  Its scale image is no longer one byte repeated: word (row) = the row's four exponent
// bytes of this K block, read straight from w_sf a unit ahead.
template <int M_PAD, bool RES, bool W4>
__global__ void __launch_bounds__(threads_for(M_PAD, RES), 1)
gemm_fp8_mx_kernel(const __grid_constant__ CUtensorMap w_map, const __grid_constant__ CUtensorMap a_map, const Params p) {
    using L = Smem<M_PAD, RES>;
    constexpr int kBuffers = L::kBuffers;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t base = (raw_addr + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (base - raw_addr);
    const int S = p.stages;
    const uint32_t bars = base + L::bar_off(S, p.kb);
    const uint32_t full = bars, empty = bars + 16 * 8, full_tm = bars + 32 * 8, empty_tm = bars + 34 * 8, a_full = bars + 36 * 8;
    const uint32_t a_res = base + L::res_off(S);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(base_ptr + L::misc_off(S, p.kb));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(base_ptr + L::misc_off(S, p.kb) + 4);

    const int warp = threadIdx.x >> 5;
    const uint32_t lane = lane_id();
    constexpr int kProd = producers_for(M_PAD, RES);
    constexpr int kIssuer0 = kProd;
    constexpr int kEpi0 = first_epi_warp_for(M_PAD, RES);

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int i = 0; i < S; ++i) {
            mbar_init(full + i * 8, 2);     // the copies have landed and the scale images are written
            mbar_init(empty + i * 8, 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(full_tm + b * 8, kIssuers);      // both issuers' accumulators of a segment are complete
            mbar_init(empty_tm + b * 8, kEpiWarps);    // the epilogue has read them
        }
        mbar_init(a_full, 1);
        fence_mbar_init();
    }
    if (warp == kIssuer0) {
        tmem_alloc(smem_u32(tmem_slot), L::kTmemCols);
        tmem_relinquish();
    }
    if (warp == 0 && lane == 0) {
        prefetch_tmap(&w_map);
        prefetch_tmap(&a_map);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // the prologue above ran while the kernel ahead was still finishing; global memory from here on
    pdl_launch_dependents();
    pdl_wait();

    const long long units = static_cast<long long>(p.n_tiles) * p.kb;
    const long long u0 = range_begin(units, blockIdx.x, gridDim.x);
    const long long u1 = range_begin(units, blockIdx.x + 1, gridDim.x);
    const int count = static_cast<int>(u1 - u0);

    if (warp < kProd) {
        // ------------------------------------------------------------ producers: a unit's copies, then its scale images
        const int me = warp;
        const uint64_t stream_policy = policy_evict_first();
        const uint64_t keep_policy = policy_evict_last();
        Ring ring;
        ring.step(me, S);
        int tile = static_cast<int>((u0 + me) / p.kb), kb = static_cast<int>((u0 + me) % p.kb);
        bool alive = true;
        // weight scales of this producer's next 32 units: lane j holds the one of unit n = first + kProd * j
        int batch_first = me;
        auto load_batch = [&](int first) {
            const long long u = u0 + first + kProd * static_cast<int>(lane);
            return u < u1 ? __ldg(p.w_scales + u) : 1.0f;
        };
        float w_now = 1.0f, w_next = 1.0f;
        if constexpr (!W4) {
            w_now = load_batch(batch_first);
            w_next = load_batch(batch_first + 32 * kProd);
        }
        // W4: lane l fetches the exponent words of weight rows l, l + 32, l + 64, l + 96 of a unit - its 16 bytes of the
        // unit's image - into this warp's ring, kSfDepth of the warp's units ahead: a register prefetch would let one
        // request per iteration be in flight, and the words come from DRAM (every row's sector, every eighth K block).
        // Rows beyond N read as zeros (2^-127 times an operand row of zeros).
        const uint32_t sf_ring = base + L::sf_ring_off(S, p.kb) + me * (kSfDepth * kSfBytes) + lane * 16;
        auto request_wsf = [&](int slot, long long u) {
            if (u < u1) {
                const int t = static_cast<int>(u / p.kb), k = static_cast<int>(u - static_cast<long long>(t) * p.kb);
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const int row = t * kTileN + q * 32 + static_cast<int>(lane);
                    const int safe = row < p.N ? row : 0;
                    cp_async_4(sf_ring + slot * kSfBytes + q * 4, p.w_sf + static_cast<int64_t>(safe) * p.sf_stride + k * 4,
                               row < p.N ? 4u : 0u);
                }
            }
            cp_async_commit();
        };
        int sf_slot = 0;
        if constexpr (W4) {
#pragma unroll
            for (int d = 0; d < kSfDepth; ++d) request_wsf(d, u0 + me + d * kProd);
        }
        // activation scales of a unit: lane l holds those of rows l, l + 32, .. (rows beyond M: 2^0, their operand rows
        // are zeros); the next unit's are requested before this unit's copies are started
        constexpr int kRowsPerLane = (M_PAD + 31) / 32;
        auto load_scales = [&](int t, int k, float (&v)[kRowsPerLane]) {
            const int colx = (t / p.tiles_per_group) * p.kb + k;
#pragma unroll
            for (int q = 0; q < kRowsPerLane; ++q) {
                const int row = q * 32 + static_cast<int>(lane);
                v[q] = (row < p.M && t < p.n_tiles) ? __ldcg(p.a_scales + static_cast<int64_t>(row) * p.scale_cols + colx) : 1.0f;
            }
        };
        float a_now[kRowsPerLane], a_next[kRowsPerLane];
        load_scales(tile, kb, a_now);
        if (RES && me == 0 && count > 0) {   // the whole activation matrix, once (plain form: one group)
            if (lane == 0) mbar_arrive_expect_tx(a_full, p.kb * L::kABytes);
            __syncwarp();
            for (int k = static_cast<int>(lane); k < p.kb; k += 32)
                tma_load_2d_hint(a_res + k * L::kABytes, &a_map, a_full, k * kRowBytes, 0, keep_policy);
        }
        for (int n = me; n < count && alive; n += kProd) {
            const int s = ring.idx;
            int tile_next = tile, kb_next = kb + kProd;
            while (kb_next >= p.kb) {
                kb_next -= p.kb;
                ++tile_next;
            }
            load_scales(tile_next, kb_next, a_next);
            alive = mbar_wait_lane0(empty + s * 8, ring.phase ^ 1u, abort_flag, p.status, kDevTimeoutGemmEmpty);
            if (!alive) break;
            if (lane == 0) mbar_arrive_expect_tx(full + s * 8, (W4 ? kWBytes / 2 : kWBytes) + (RES ? 0 : L::kABytes));
            __syncwarp();
            // one instruction, two lanes: lane 0 fetches the weight tile, lane 1 the activations of the tile's group
            const uint32_t stage = base + s * L::kStageBytes;
            uint8_t* stage_ptr = base_ptr + s * L::kStageBytes;
            const int group = tile / p.tiles_per_group;
            const uint32_t dst = stage + (lane == 1 ? kWBytes : 0);
            const void* map = lane == 1 ? static_cast<const void*>(&a_map) : static_cast<const void*>(&w_map);
            if (lane < (RES ? 1u : 2u))
                tma_load_2d_hint(dst, map, full + s * 8, (lane == 1 ? group * p.kb + kb : kb) * kRowBytes, lane == 1 ? 0 : tile * kTileN,
                                 lane == 1 ? keep_policy : stream_policy);
            // scale images: lane l writes row l of each (16 bytes: the words of rows l, l + 32, l + 64, l + 96)
            if constexpr (W4) {
                cp_async_wait<kSfDepth - 1>();      // this unit's words have landed (a lane reads only what it fetched)
                uint4 words;
                asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                             : "=r"(words.x), "=r"(words.y), "=r"(words.z), "=r"(words.w)
                             : "r"(sf_ring + sf_slot * kSfBytes));
                *reinterpret_cast<uint4*>(stage_ptr + L::kSfOff + lane * 16) = words;
                request_wsf(sf_slot, u0 + n + static_cast<long long>(kSfDepth) * kProd);   // the slot is read: refill it
                sf_slot = sf_slot + 1 == kSfDepth ? 0 : sf_slot + 1;
            } else {
                if (n >= batch_first + 32 * kProd) {
                    batch_first += 32 * kProd;
                    w_now = w_next;
                    w_next = load_batch(batch_first + 32 * kProd);
                }
                const float w_scale = __shfl_sync(0xffffffffu, w_now, (n - batch_first) / kProd);
                const uint32_t ew = exponent_byte(w_scale, p.status) * 0x01010101u;
                *reinterpret_cast<uint4*>(stage_ptr + L::kSfOff + lane * 16) = make_uint4(ew, ew, ew, ew);
            }
            uint32_t aw[4] = {0u, 0u, 0u, 0u};
#pragma unroll
            for (int q = 0; q < kRowsPerLane; ++q) aw[q] = exponent_byte(a_now[q], p.status) * 0x01010101u;
            *reinterpret_cast<uint4*>(stage_ptr + L::kSfOff + kSfBytes + lane * 16) = make_uint4(aw[0], aw[1], aw[2], aw[3]);
            fence_proxy_async_smem();       // the images are read by tcgen05.cp
            __syncwarp();
            if (lane == 0) mbar_arrive(full + s * 8);
            ring.step(kProd, S);
            tile = tile_next, kb = kb_next;
#pragma unroll
            for (int q = 0; q < kRowsPerLane; ++q) a_now[q] = a_next[q];
        }
    } else if (warp < kIssuer0 + kIssuers) {
        // ------------------------------------------------------------ UMMA issuers (one thread each)
        // Issuer i takes units n with n % 2 == i and accumulates them into its own TMEM tile; the epilogue adds the
        // two tiles.  (Two threads must not chain accumulations into one tile: only operations of one thread are
        // ordered.)
        if (lane == 0) {
            const int me = warp - kIssuer0;
            const uint32_t sfw_t = tmem_base + L::kAccCols + me * 16;
            const uint32_t sfa_t = sfw_t + 8;
            Ring ring;
            ring.step(me, S);
            int kb = static_cast<int>(u0 % p.kb);
            uint32_t seg = 0;
            bool alive = true;
            if (RES && count > 0) alive = mbar_wait(a_full, 0, abort_flag, p.status, kDevTimeoutGemmFull);
            for (int n = 0; n < count && alive;) {
                const int seg_len = min(p.kb - kb, count - n);
                const uint32_t buf = kBuffers == 2 ? (seg & 1u) : 0u;
                if (seg >= static_cast<uint32_t>(kBuffers)) {   // the epilogue must have drained this buffer's previous segment
                    const uint32_t use = seg / kBuffers - 1u;
                    if (!mbar_wait(empty_tm + buf * 8, use & 1u, abort_flag, p.status, kDevTimeoutGemmTmemEmpty)) break;
                    tc_fence_after();
                }
                const uint32_t d_addr = tmem_base + (buf * kIssuers + me) * M_PAD;
                uint32_t accumulate = 0;
                for (int u = n + ((me ^ n) & 1); u < n + seg_len; u += kIssuers) {
                    const int s = ring.idx;
                    if (!mbar_wait(full + s * 8, ring.phase, abort_flag, p.status, kDevTimeoutGemmFull)) {
                        alive = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t stage = base + s * L::kStageBytes;
                    const uint32_t w_addr = stage, a_addr = RES ? a_res + (kb + (u - n)) * L::kABytes : stage + kWBytes;
                    const uint32_t wsf_addr = stage + L::kSfOff, asf_addr = wsf_addr + kSfBytes;
                    // 32 rows x 16 bytes; 8-row groups 128 bytes apart
                    tmem_cp_32x128b_warpx4(sfw_t, umma_smem_desc_noswz(wsf_addr, 16, 128));
                    tmem_cp_32x128b_warpx4(sfa_t, umma_smem_desc_noswz(asf_addr, 16, 128));
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        // weights e4m3 (format 0) or e2m1 (5) x e4m3, ue8m0 scales (1), the k-th scale byte of both operands
                        const uint32_t idesc = umma_idesc_block_scaled(kTileN, M_PAD, W4 ? 5 : 0, 0, 1, k, k);
                        umma_mxf8(d_addr, umma_smem_desc_sw128(w_addr + k * 32), umma_smem_desc_sw128(a_addr + k * 32), idesc, sfw_t,
                                  sfa_t, accumulate);
                        accumulate = 1;
                    }
                    umma_commit(empty + s * 8);     // the stage's bytes are consumed once these retire
                    ring.step(kIssuers, S);
                }
                if (!alive) break;
                umma_commit(full_tm + buf * 8);     // this issuer's part of the segment is complete
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
        uint32_t seg = 0;
        int n = 0;
        while (n < count) {
            // the segment [kb, kb_end) of `tile`
            const int seg_len = min(p.kb - kb, count - n);
            const bool from_zero = (kb == 0), to_end = (kb + seg_len == p.kb);
            // Issuer i owns the units with n % 2 == i; a one-unit segment has only its first issuer's tile.
            const bool both = seg_len >= 2;
            const int first_issuer = n & 1;
            const uint32_t buf = kBuffers == 2 ? (seg & 1u) : 0u;
            if (alive) alive = mbar_wait_warp_fast(full_tm + buf * 8, (seg / kBuffers) & 1u, abort_flag, p.status, kDevTimeoutGemmTmemFull);
            float acc[M_PAD];
            if (alive) {
                tc_fence_after();
                const uint32_t t0 = tmem_base + lane_base + buf * kIssuers * M_PAD;
#pragma unroll
                for (int c = 0; c < M_PAD; c += 16) {
                    uint32_t v0[16], v1[16];
                    tmem_ld_32x16(t0 + first_issuer * M_PAD + c, v0);
                    if (both) tmem_ld_32x16(t0 + (first_issuer ^ 1) * M_PAD + c, v1);
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
            if (lane == 0) mbar_arrive(empty_tm + buf * 8);

            const int nrow = tile * kTileN + et;
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
                    const int last = cta_of(units, t_end, gridDim.x);
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
#pragma unroll
                    for (int i = 0; i < M_PAD; ++i)
                        if (i < p.M) p.c[static_cast<int64_t>(i) * p.N + nrow] = __float2bfloat16_rn(acc[i]);
                }
            }
            n += seg_len;
            kb += seg_len;
            if (kb == p.kb) {
                kb = 0;
                ++tile;
            }
            ++seg;
        }
    }

    __syncthreads();
    if (*abort_flag) abort_drain_sleep();
    __syncthreads();
    if (warp == kIssuer0) {
        tc_fence_after();
        tmem_dealloc(tmem_base, L::kTmemCols);
    }
}

template <int M_PAD, bool RES, bool W4>
static int launch_as(const CUtensorMap& w_map, const CUtensorMap& a_map, Params& p, const DeviceInfo& dev, int stages,
                     cudaStream_t stream) {
    using L = Smem<M_PAD, RES>;
    p.stages = stages;
    auto kernel = gemm_fp8_mx_kernel<M_PAD, RES, W4>;
    WUDA_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::total(stages, p.kb, W4)));
    const long long units = static_cast<long long>(p.n_tiles) * p.kb;
    // CTAs that may share one weight tile: the owner adds their partials one after the other
    constexpr int kMaxSplit = M_PAD <= 16 ? 16 : (M_PAD == 32 ? 12 : (M_PAD == 64 ? 8 : 6));
    const int sms = gemm_sms(dev);
    int grid = units < sms ? static_cast<int>(units) : sms;
    if (static_cast<long long>(p.n_tiles) * kMaxSplit < grid) grid = p.n_tiles * kMaxSplit;
    WUDA_CUDA(launch_pdl(kernel, dim3(grid), dim3(threads_for(M_PAD, RES)), L::total(stages, p.kb, W4), stream, w_map, a_map, p));
    return WUDA_OK;
}

template <int M_PAD, bool W4>
static int launch(const CUtensorMap& w_map, const CUtensorMap& a_map, Params& p, const DeviceInfo& dev, cudaStream_t stream) {
    // Short K, one group, 32 or 64 rows: the activations stay resident if at least six weight stages fit beside them.
    if (M_PAD >= 32 && M_PAD <= 64 && p.tiles_per_group == p.n_tiles && p.kb * Smem<M_PAD>::kABytes <= 96 * 1024) {
        using R = Smem<M_PAD, true>;
        int stages = 16;
        while (stages > 2 && R::total(stages, p.kb, W4) > dev.smem_optin) stages -= 2;
        if (stages >= 6 && R::total(stages, p.kb, W4) <= dev.smem_optin) return launch_as<M_PAD, true, W4>(w_map, a_map, p, dev, stages, stream);
    }
    using L = Smem<M_PAD, false>;
    int stages = 16;
    constexpr int kStep = M_PAD >= 128 ? 2 : 4;   // lcm of the producer and issuer counts
    while (stages > kStep && L::total(stages, p.kb, W4) > dev.smem_optin) stages -= kStep;
    if (L::total(stages, p.kb, W4) > dev.smem_optin)
        return fail(WUDA_ERR_UNSUPPORTED, "device offers %d bytes of shared memory per block; the kernel needs more",
                    dev.smem_optin);
    return launch_as<M_PAD, false, W4>(w_map, a_map, p, dev, stages, stream);
}

// One pass of at most 128 rows.  groups = 1 is the plain GEMM.  w_sf != NULL: 4-bit weights (plain form only).
static int run(const void* a, const float* a_scales, const void* w, const float* w_scales, const uint8_t* w_sf, void* c_bf16, int m,
               int n_per_group, int k, int groups, void* scratch, int64_t scratch_bytes, int32_t* status_word, void* stream) {
    const int n = n_per_group * groups;
    const bool w4 = w_sf != nullptr;
    WUDA_REQUIRE(aligned16(a) && aligned16(w), "a and w must be 16-byte aligned");
    WUDA_REQUIRE(!w4 || ((reinterpret_cast<uintptr_t>(w) & 31u) == 0 && (reinterpret_cast<uintptr_t>(w_sf) & 3u) == 0),
                 "packed 4-bit weights must be 32-byte aligned and their scale bytes 4-byte aligned");
    WUDA_REQUIRE((reinterpret_cast<uintptr_t>(scratch) & 255u) == 0, "scratch must be 256-byte aligned");
    const int64_t need = wuda_gemm_fp8_scratch_bytes(m, n);
    WUDA_REQUIRE(scratch_bytes >= need, "scratch holds %lld bytes; %lld are needed (wuda_gemm_fp8_scratch_bytes)",
                 static_cast<long long>(scratch_bytes), static_cast<long long>(need));
    DeviceInfo dev;
    int st = current_device_info(&dev);
    if (st != WUDA_OK) return st;
    WUDA_REQUIRE(dev.num_sms <= kMaxGrid, "device has %d SMs; at most %d are supported", dev.num_sms, kMaxGrid);
    int m_pad = 16;
    while (m_pad < m) m_pad *= 2;
    Params p;
    p.c = static_cast<__nv_bfloat16*>(c_bf16);
    p.a_scales = a_scales;
    p.w_scales = w_scales;
    p.w_sf = w_sf;
    p.sf_stride = k / 32;
    p.status = status_word;
    p.M = m;
    p.N = n;
    p.kb = k / 128;
    p.n_tiles = (n + 127) / 128;
    p.tiles_per_group = groups > 1 ? n_per_group / 128 : p.n_tiles;
    p.scale_cols = groups * p.kb;
    p.scratch = reinterpret_cast<float*>(static_cast<uint8_t*>(scratch) + kFlagBytes);
    p.flags = static_cast<int32_t*>(scratch);
    p.stages = 0;

    CUtensorMap w_map, a_map;
    {
        // 4-bit weights: dimensions and box in elements, the row stride in bytes; shared memory gets the padded form
        const uint64_t dims[2] = {static_cast<uint64_t>(k), static_cast<uint64_t>(n)};
        const uint64_t strides[1] = {static_cast<uint64_t>(w4 ? k / 2 : k)};
        const uint32_t box[2] = {128u, 128u};
        st = encode_tensor_map(&w_map, w4 ? CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B : CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, w, dims, strides,
                               box, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
        if (st != WUDA_OK) return st;
    }
    {
        const uint64_t row = static_cast<uint64_t>(k) * groups;
        const uint64_t dims[2] = {row, static_cast<uint64_t>(m)};
        const uint64_t strides[1] = {row};
        const uint32_t box[2] = {128u, static_cast<uint32_t>(m_pad)};
        st = encode_tensor_map(&a_map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, a, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B,
                               CU_TENSOR_MAP_L2_PROMOTION_L2_128B);
        if (st != WUDA_OK) return st;
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (w4) {
        switch (m_pad) {
            case 16: return launch<16, true>(w_map, a_map, p, dev, s);
            case 32: return launch<32, true>(w_map, a_map, p, dev, s);
            case 64: return launch<64, true>(w_map, a_map, p, dev, s);
            default: return launch<128, true>(w_map, a_map, p, dev, s);
        }
    }
    switch (m_pad) {
        case 16: return launch<16, false>(w_map, a_map, p, dev, s);
        case 32: return launch<32, false>(w_map, a_map, p, dev, s);
        case 64: return launch<64, false>(w_map, a_map, p, dev, s);
        default: return launch<128, false>(w_map, a_map, p, dev, s);
    }
}

}  // namespace gemm8mx
}  // namespace wuda

extern "C" int wuda_gemm_fp8_grouped_pow2(const void* a, const float* a_scales, const void* w, const float* w_scales, void* c_bf16,
                                          int m, int n_per_group, int k, int groups, void* scratch, int64_t scratch_bytes,
                                          int32_t* status_word, void* stream) {
    using namespace wuda;
    clear_error();
    WUDA_REQUIRE(m >= 0 && m <= 256, "m must be in [0, 256] (got %d)", m);
    WUDA_REQUIRE(groups >= 1 && n_per_group >= 1, "groups and n_per_group must be >= 1");
    WUDA_REQUIRE(groups == 1 || n_per_group % 128 == 0, "n_per_group must be a multiple of 128 when there are several groups (got %d)",
                 n_per_group);
    WUDA_REQUIRE(k >= 128 && k % 128 == 0, "k must be a positive multiple of 128 (got %d)", k);
    if (m == 0) return WUDA_OK;
    WUDA_REQUIRE(a && a_scales && w && w_scales && c_bf16 && scratch, "a, a_scales, w, w_scales, c and scratch must not be NULL");
    const int64_t n = static_cast<int64_t>(n_per_group) * groups;
    const int64_t row = static_cast<int64_t>(k) * groups;
    for (int m0 = 0; m0 < m; m0 += 128) {   // a tile holds at most 128 activation rows: passes over the weights
        const int rows = m - m0 < 128 ? m - m0 : 128;
        const int st = gemm8mx::run(static_cast<const uint8_t*>(a) + m0 * row, a_scales + m0 * (row / 128), w, w_scales, nullptr,
                                    static_cast<__nv_bfloat16*>(c_bf16) + m0 * n, rows, n_per_group, k, groups, scratch, scratch_bytes,
                                    status_word, stream);
        if (st != WUDA_OK) return st;
    }
    return WUDA_OK;
}

extern "C" int wuda_gemm_fp8_blockscaled_pow2(const void* a, const float* a_scales, const void* w, const float* w_scales, void* c_bf16,
                                              int m, int n, int k, void* scratch, int64_t scratch_bytes, int32_t* status_word,
                                              void* stream) {
    return wuda_gemm_fp8_grouped_pow2(a, a_scales, w, w_scales, c_bf16, m, n, k, 1, scratch, scratch_bytes, status_word, stream);
}

// FP8 activations x 4-bit weights (origin/kernel.py:441-536, fp4_gemm): a e4m3 [m, k] with one power-of-two fp32 scale per
// row and 128 K-elements; w e2m1 [n, k/2] bytes, the element of the lower K index in the low nibble (torch.float4_e2m1fn_x2),
// with one exponent byte (float8_e8m0fnu) per row and 32 K-elements, [n, k/32]; c bf16 [m, n].
extern "C" int wuda_gemm_fp8_fp4_pow2(const void* a, const float* a_scales, const void* w_packed, const void* w_sf, void* c_bf16,
                                      int m, int n, int k, void* scratch, int64_t scratch_bytes, int32_t* status_word,
                                      void* stream) {
    using namespace wuda;
    clear_error();
    WUDA_REQUIRE(m >= 0 && m <= 256, "m must be in [0, 256] (got %d)", m);
    WUDA_REQUIRE(n >= 1, "n must be >= 1 (got %d)", n);
    WUDA_REQUIRE(k >= 128 && k % 128 == 0, "k must be a positive multiple of 128 (got %d)", k);
    if (m == 0) return WUDA_OK;
    WUDA_REQUIRE(a && a_scales && w_packed && w_sf && c_bf16 && scratch, "a, a_scales, w_packed, w_sf, c and scratch must not be NULL");
    for (int m0 = 0; m0 < m; m0 += 128) {   // a tile holds at most 128 activation rows: passes over the weights
        const int rows = m - m0 < 128 ? m - m0 : 128;
        const int st = gemm8mx::run(static_cast<const uint8_t*>(a) + static_cast<int64_t>(m0) * k, a_scales + static_cast<int64_t>(m0) * (k / 128),
                                    w_packed, nullptr, static_cast<const uint8_t*>(w_sf),
                                    static_cast<__nv_bfloat16*>(c_bf16) + static_cast<int64_t>(m0) * n, rows, n, k, 1, scratch,
                                    scratch_bytes, status_word, stream);
        if (st != WUDA_OK) return st;
    }
    return WUDA_OK;
}
