// BF16 GEMM for decode-sized M on sm_100a:
//
//   C[M, N] (bf16 or fp32) = A[M, K] (bf16) x W[N, K]^T (bf16), fp32 accumulation
//
// It carries the projections the reference keeps in BF16 because their outputs feed fp32 state:
// the BF16 segment of the front mixed GEMM (dsv4_megakernel/megakernel/kernels/
// front_mixed_gemm_csa_swapab.cu:10-258, segment layout include/front_mixed_gemm.cuh:390-425) and
// the origin's plain `linear` (origin/model.py:108-120).
//
// Same skeleton as the FP8 and NVFP4 GEMMs of this library: swap-AB (UMMA M = 128 weight rows,
// UMMA N = padded M), stream-K over the flat (weight tile, 64-wide K block) list, one TMA
// instruction per unit (weight tile and activation tile, one lane each), four
// tcgen05.mma kind::f16 (K = 16) per unit.  Nothing is rescaled between K blocks, so a tile
// accumulates over its whole K range in TMEM and the epilogue runs once per segment; two issuer
// threads take units alternately into two TMEM tiles that the epilogue adds.  Partial tiles go
// through per-CTA scratch slots added in CTA order; every wait is bounded.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstring>

#include "host.h"
#include "ptx.cuh"

namespace wuda {
namespace gemm16 {

constexpr int kTileN = 128;          // weight rows per tile (UMMA M)
constexpr int kBlockK = 64;          // K elements per unit = 128 bytes per row
constexpr int kRowBytes = 128;
constexpr int kProducers = 4;        // warps 0..3: starting a unit's copies costs a warp several hundred cycles
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
constexpr int kMaxGrid = 192;
constexpr int64_t kFlagBytes = 1024;   // the flags lead the scratch: calls of any row count find them in the same place

struct Params {
    void* c;                   // bf16 or fp32 [M, N]
    int c_is_fp32;
    float* scratch;            // [grid][M_PAD][128] fp32 partial-tile slots
    int32_t* flags;            // [grid]
    int32_t* status;
    int M, N, kb;              // kb = K / 64
    int n_tiles;
    int stages;
};

template <int M_PAD>
struct Smem {
    static constexpr int kABytes = M_PAD * kRowBytes;
    static constexpr int kStageBytes = kWBytes + kABytes;
    // TMEM columns: one accumulator tile per issuer
    static constexpr int kAccCols = kIssuers * M_PAD;
    static constexpr int kUsedCols = kAccCols;
    static constexpr int kTmemCols = kUsedCols <= 32 ? 32 : kUsedCols <= 64 ? 64 : (kUsedCols <= 128 ? 128 : (kUsedCols <= 256 ? 256 : 512));
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
gemm_bf16_kernel(const __grid_constant__ CUtensorMap w_map, const __grid_constant__ CUtensorMap a_map,
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
        bool alive = true;
        for (int n = me; n < count && alive; n += kProd) {
            const int s = ring.idx;
            alive = mbar_wait_lane0(empty + s * 8, ring.phase ^ 1u, abort_flag, p.status, kDevTimeoutGemmEmpty);
            if (!alive) break;
            if (lane == 0) mbar_arrive_expect_tx(full + s * 8, L::kStageBytes);
            __syncwarp();
            // one instruction, two lanes: lane 0 fetches the weight tile, lane 1 the activations
            const uint32_t stage = base + s * L::kStageBytes;
            const uint32_t dst = stage + (lane == 1 ? kWBytes : 0);
            const void* map = lane == 1 ? static_cast<const void*>(&a_map) : static_cast<const void*>(&w_map);
            if (lane < 2)
                tma_load_2d_hint(dst, map, full + s * 8, kb * kBlockK, lane == 1 ? 0 : tile * kTileN,
                                 lane == 1 ? keep_policy : stream_policy);
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
            // kind::f16 with BF16 operands (format 1), fp32 accumulator, both operands K-major
            constexpr uint32_t idesc = umma_idesc(kTileN, M_PAD, 1, 1);
            const uint32_t d_addr = tmem_base + me * M_PAD;
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
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        umma_f16(d_addr, umma_smem_desc_sw128(w_addr + k * 32), umma_smem_desc_sw128(a_addr + k * 32), idesc,
                                 accumulate);
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
                    if (p.c_is_fp32) {
                        float* c = static_cast<float*>(p.c);
#pragma unroll
                        for (int i = 0; i < M_PAD; ++i)
                            if (i < p.M) c[static_cast<int64_t>(i) * p.N + nrow] = acc[i];
                    } else {
                        __nv_bfloat16* c = static_cast<__nv_bfloat16*>(p.c);
#pragma unroll
                        for (int i = 0; i < M_PAD; ++i)
                            if (i < p.M) c[static_cast<int64_t>(i) * p.N + nrow] = __float2bfloat16_rn(acc[i]);
                    }
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
static int launch(const CUtensorMap& w_map, const CUtensorMap& a_map, Params& p, const DeviceInfo& dev,
                  cudaStream_t stream) {
    using L = Smem<M_PAD>;
    int stages = 16;
    constexpr int kStep = M_PAD >= 128 ? 2 : 4;   // lcm of the producer and issuer counts
    while (stages > kStep && L::total(stages) > dev.smem_optin) stages -= kStep;
    if (L::total(stages) > dev.smem_optin)
        return fail(WUDA_ERR_UNSUPPORTED, "device offers %d bytes of shared memory per block; the kernel needs more",
                    dev.smem_optin);
    p.stages = stages;
    auto kernel = gemm_bf16_kernel<M_PAD>;
    WUDA_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::total(stages)));
    const long long units = static_cast<long long>(p.n_tiles) * p.kb;
    // at most kMaxSplit CTAs share one weight tile: the tile's owner adds the others' partials one after
    // the other, which costs more than it saves when a few tiles are cut into a hundred pieces
    // (adding one partial costs the owner about as much as streaming M_PAD / 64 units, so wide tiles split less)
    constexpr int kMaxSplit = M_PAD <= 16 ? 16 : (M_PAD == 32 ? 12 : (M_PAD == 64 ? 8 : 6));
    const int sms = gemm_sms(dev);
    int grid = units < sms ? static_cast<int>(units) : sms;
    if (static_cast<long long>(p.n_tiles) * kMaxSplit < grid) grid = p.n_tiles * kMaxSplit;
    WUDA_CUDA(launch_pdl(kernel, dim3(grid), dim3(threads_for(M_PAD)), L::total(stages), stream, w_map, a_map, p));
    return WUDA_OK;
}

}  // namespace gemm16
}  // namespace wuda

extern "C" int64_t wuda_gemm_bf16_scratch_bytes(int m, int n) {
    if (m < 1 || n < 1 || m > 128) return -1;
    int m_pad = 16;
    while (m_pad < m) m_pad *= 2;
    return wuda::gemm16::kFlagBytes + static_cast<int64_t>(wuda::gemm16::kMaxGrid) * m_pad * 128 * 4;
}

extern "C" int wuda_gemm_bf16(const void* a_bf16, const void* w_bf16, void* c, int c_is_fp32, int m, int n, int k,
                              void* scratch, int64_t scratch_bytes, int32_t* status_word, void* stream) {
    using namespace wuda;
    using namespace wuda::gemm16;
    clear_error();
    WUDA_REQUIRE(m >= 0 && m <= 128, "m must be in [0, 128] (got %d)", m);
    WUDA_REQUIRE(n >= 1, "n must be >= 1 (got %d)", n);
    WUDA_REQUIRE(k >= 64 && k % 64 == 0, "k must be a positive multiple of 64 (got %d)", k);
    if (m == 0) return WUDA_OK;
    WUDA_REQUIRE(a_bf16 && w_bf16 && c && scratch, "a, w, c and scratch must not be NULL");
    WUDA_REQUIRE(aligned16(a_bf16) && aligned16(w_bf16), "a and w must be 16-byte aligned");
    WUDA_REQUIRE((reinterpret_cast<uintptr_t>(scratch) & 255u) == 0, "scratch must be 256-byte aligned");
    const int64_t need = wuda_gemm_bf16_scratch_bytes(m, n);
    WUDA_REQUIRE(scratch_bytes >= need, "scratch holds %lld bytes; %lld are needed (wuda_gemm_bf16_scratch_bytes)",
                 static_cast<long long>(scratch_bytes), static_cast<long long>(need));

    DeviceInfo dev;
    int st = current_device_info(&dev);
    if (st != WUDA_OK) return st;
    WUDA_REQUIRE(dev.num_sms <= kMaxGrid, "device has %d SMs; at most %d are supported", dev.num_sms, kMaxGrid);

    int m_pad = 16;
    while (m_pad < m) m_pad *= 2;
    Params p;
    p.c = c;
    p.c_is_fp32 = c_is_fp32 != 0;
    p.status = status_word;
    p.M = m;
    p.N = n;
    p.kb = k / kBlockK;
    p.n_tiles = (n + 127) / 128;
    p.scratch = reinterpret_cast<float*>(static_cast<uint8_t*>(scratch) + kFlagBytes);
    p.flags = static_cast<int32_t*>(scratch);
    p.stages = 0;

    CUtensorMap w_map, a_map;
    {
        const uint64_t dims[2] = {static_cast<uint64_t>(k), static_cast<uint64_t>(n)};
        const uint64_t strides[1] = {static_cast<uint64_t>(k) * 2};
        const uint32_t box[2] = {64u, 128u};
        st = encode_tensor_map(&w_map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, w_bf16, dims, strides, box,
                               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
        if (st != WUDA_OK) return st;
    }
    {
        const uint64_t dims[2] = {static_cast<uint64_t>(k), static_cast<uint64_t>(m)};
        const uint64_t strides[1] = {static_cast<uint64_t>(k) * 2};
        const uint32_t box[2] = {64u, static_cast<uint32_t>(m_pad)};
        st = encode_tensor_map(&a_map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a_bf16, dims, strides, box,
                               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B);
        if (st != WUDA_OK) return st;
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (m_pad) {
        case 16: return launch<16>(w_map, a_map, p, dev, s);
        case 32: return launch<32>(w_map, a_map, p, dev, s);
        case 64: return launch<64>(w_map, a_map, p, dev, s);
        default: return launch<128>(w_map, a_map, p, dev, s);
    }
}
