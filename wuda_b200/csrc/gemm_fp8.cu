// Block-scaled FP8 GEMM for decode-sized M on sm_100a:
//
//   C[M, N] (bf16) = A[M, K] (e4m3, fp32 scale per 1x128) x W[N, K]^T (e4m3, fp32 scale per 128x128)
//
// Numerics contract (dsv4_megakernel/origin/kernel.py:203-273, fp8_gemm_kernel): every
// 128-wide K block is accumulated in fp32 on its own and then added, multiplied by
// a_s[m, kb] * w_s[n / 128, kb], to a second fp32 accumulator (lines 246-250).  This is
// the generic form of the reference's wq_b / wo_b projections
// (dsv4_megakernel/megakernel/kernels/wq_b_fp8_gemm.cu:189-780, test/o_proj_csa.py:454-480),
// which use power-of-two UE8M0 scales; fp32 scales cannot ride the tensor core's
// block-scale path, so the promotion happens in registers.
//
// Design: decode GEMMs are bound by the weight stream (N*K bytes once from HBM), so
//  * swap-AB: the UMMA M dimension (128) is a tile of weight rows, the UMMA N dimension
//    is the padded activation count (16..256); the activations (a few MB at most) are
//    re-read from L2 for every weight tile;
//  * stream-K: the flat list of (weight tile, K block) units is cut into one equal
//    contiguous range per SM, so every SM streams the same number of bytes whatever N is;
//    a range that does not start a tile's K range writes its fp32 partial to the CTA's own
//    scratch slot in global memory and raises a flag; the CTA holding the start of the
//    range adds the partials in CTA order (deterministic) and writes the bf16 tile;
//  * per unit: one TMA instruction fetches the weight tile (128 x 128 B) and the
//    activation tile (M_PAD x 128 B), four tcgen05.mma kind::f8f6f4 fill a fresh TMEM
//    stage, and an epilogue warpgroup adds the stage, times the unit's scales, to its register
//    accumulators.  One unit's epilogue is a chain of waits (scales, TMEM stage, tcgen05.ld), so
//    the two epilogue warpgroups take units alternately and their chains overlap; the two
//    accumulator sets are added when a tile's segment ends.  (Above 64 activation rows a thread
//    cannot hold all columns; the groups then split the columns and both take every unit.);
//  * roles are replicated (2 producers, 2 issuers) and take units round-robin; stage
//    counts are multiples of the role counts; every wait is bounded and reports through
//    the status word.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstring>
#include <mutex>

#include "host.h"
#include "ptx.cuh"

namespace wuda {
namespace gemm8 {

constexpr int kTileN = 128;          // weight rows per tile (UMMA M)
constexpr int kBlockK = 128;         // K per unit
constexpr int kProducers = 2;        // warps 0, 1
constexpr int kIssuers = 2;          // warps 2, 3
constexpr int kFirstEpiWarp = 4;     // warps 4..11: two warpgroups, half the columns each
constexpr int kEpiWarps = 8;
constexpr int kThreads = 32 * (kFirstEpiWarp + kEpiWarps);
constexpr int kWBytes = kTileN * kBlockK;   // 16 KB
constexpr int kScaleSlots = 8;       // scale ring depth
constexpr int kScaleAhead = 6;       // units of look-ahead of the scale fetch (< kScaleSlots - 1)

struct Params {
    const float* a_scales;     // [M, K/128]
    const float* w_scales;     // [ceil(N/128), K/128]
    __nv_bfloat16* c;          // [M, N]
    float* scratch;            // [grid][M_PAD][128] fp32: one partial-tile slot per CTA
    int32_t* flags;            // [grid]: slot c is published; zero between calls
    int32_t* status;
    int M, N, K, kb;           // kb = K / 128
    int n_tiles;
    int stages;
    int a_resident = 0;        // the whole activation matrix stays in shared memory (see Smem)
    // grouped form: weight tile t belongs to group t / group_tiles and reads the activations'
    // columns [group * K, (group + 1) * K); a_kb_total = K blocks in an activation row (0: kb)
    int group_tiles = 0;
    int a_kb_total = 0;
    // two-rank tensor parallelism (K split across two GPUs): peer exchange of fp32 tiles
    float* tp_my_inbox = nullptr;      // [2 sets][n_tiles][M_PAD][128] fp32 in THIS GPU's memory
    float* tp_peer_inbox = nullptr;    // the same buffer of the peer, mapped into this process
    int32_t* tp_my_flags = nullptr;    // [2 sets][n_tiles]: sequence number of the last tile received
    int32_t* tp_peer_flags = nullptr;
    int32_t* tp_ctrl = nullptr;        // this rank's control words: [0] last finished call, [1] CTAs done
    int tp_epoch = 0;                  // sequence number of this call (> 0, same on both ranks); 0: tp_ctrl[0] + 1
    unsigned long long tp_wait_ns = 0; // limit of one wait for the peer
};

template <int M_PAD>
struct Smem {
    static constexpr int kABytes = M_PAD * kBlockK;
    static constexpr int kStageBytes = kWBytes + kABytes;
    static constexpr int kTmemStages = M_PAD <= 128 ? 4 : 2;
    static constexpr int kTmemCols = kTmemStages * M_PAD < 32 ? 32 : kTmemStages * M_PAD;
    // Two layouts.  Streaming: every stage holds a weight tile and the matching activation tile.
    // Resident: when the padded activation matrix (kb tiles of kABytes) fits beside at least six
    // weight stages it is loaded once per CTA and the stages hold weight tiles only - a CTA then
    // ingests 16 KB per unit instead of 16 KB + kABytes, which is what bounds decode shapes with
    // many rows and a short K.
    static __host__ __device__ constexpr int stage_bytes(bool resident) { return resident ? kWBytes : kStageBytes; }
    static __host__ __device__ constexpr int scale_off(int stages, int resident_kb = 0) {
        return stages * stage_bytes(resident_kb > 0) + resident_kb * kABytes;
    }
    // Up to M_PAD = 64 the two epilogue warpgroups take units alternately (all columns each) and add
    // their accumulators through a [M_PAD][128] fp32 buffer when a tile's segment ends; above that a
    // thread cannot hold M_PAD accumulators and the groups split the columns instead.
    static constexpr bool kAlternate = M_PAD <= 64;
    static constexpr int kCombineBytes = kAlternate ? M_PAD * kTileN * 4 : 0;
    // scale rings, one set per epilogue group: kScaleSlots x (M_PAD activation scales) + kScaleSlots
    // weight scales
    static constexpr int kRingFloats = kScaleSlots * M_PAD + kScaleSlots;
    static __host__ __device__ constexpr int comb_off(int stages, int resident_kb = 0) {
        return scale_off(stages, resident_kb) + 2 * kRingFloats * 4;
    }
    static __host__ __device__ constexpr int bar_off(int stages, int resident_kb = 0) {
        return comb_off(stages, resident_kb) + kCombineBytes;
    }
    // barriers: full[16] empty[16] full_tm[4] empty_tm[4] a_full[1]
    static __host__ __device__ constexpr int misc_off(int stages, int resident_kb = 0) {
        return bar_off(stages, resident_kb) + 48 * 8;
    }
    static __host__ __device__ constexpr int total(int stages, int resident_kb = 0) {
        return misc_off(stages, resident_kb) + 32 + 1024;
    }
};

struct Ring {
    int idx = 0;
    uint32_t phase = 0;
    __device__ __forceinline__ void step(int n, int size) {   // n <= size
        idx += n;
        if (idx >= size) {
            idx -= size;
            phase ^= 1u;
        }
    }
};

__device__ __forceinline__ void epi_bar_sync() { asm volatile("bar.sync 1, 256;" ::: "memory"); }
__device__ __forceinline__ void cp_async4(uint32_t dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void st_release_gpu(int32_t* p, int v) {
    asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_release_sys(int32_t* p, int v) {
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int32_t* p) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ float ld_volatile_f32(const float* p) {   // written by the peer GPU: bypass L1
    float v;
    asm volatile("ld.volatile.global.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ int ld_acquire_gpu(const int32_t* p) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Range boundary of CTA c in the flat unit list.
__device__ __forceinline__ long long range_begin(long long units, int c, int grid) { return units * c / grid; }
// The CTA whose range holds unit u.
__device__ __forceinline__ int cta_of(long long units, long long u, int grid) {
    int c = static_cast<int>(u * grid / units);
    while (c + 1 < grid && range_begin(units, c + 1, grid) <= u) ++c;
    while (c > 0 && range_begin(units, c, grid) > u) --c;
    return c;
}

template <int M_PAD>
__global__ void __launch_bounds__(kThreads, 1)
gemm_fp8_kernel(const __grid_constant__ CUtensorMap w_map, const __grid_constant__ CUtensorMap a_map,
                const Params p) {
    using L = Smem<M_PAD>;
    constexpr int kTS = L::kTmemStages;
    constexpr int kHalf = M_PAD / 2;                 // columns per epilogue warpgroup
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t base = (raw_addr + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (base - raw_addr);
    const int S = p.stages;
    const bool resident = p.a_resident != 0;
    const int rkb = resident ? p.kb : 0;
    const int stage_bytes = L::stage_bytes(resident);
    const uint32_t a_res = base + S * stage_bytes;      // resident activations: kb tiles of kABytes
    const uint32_t bars = base + L::bar_off(S, rkb);
    const uint32_t full = bars, empty = bars + 16 * 8, full_tm = bars + 32 * 8, empty_tm = bars + 36 * 8;
    const uint32_t a_full = bars + 40 * 8;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(base_ptr + L::misc_off(S, rkb));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(base_ptr + L::misc_off(S, rkb) + 4);
    float* rings = reinterpret_cast<float*>(base_ptr + L::scale_off(S, rkb));
    float* comb = reinterpret_cast<float*>(base_ptr + L::comb_off(S, rkb));
    constexpr bool kAlt = L::kAlternate;
    constexpr bool kPreScale = M_PAD >= 64;   // multiply activation and weight scales once per column, not per thread

    const int warp = threadIdx.x >> 5;
    const uint32_t lane = lane_id();

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int i = 0; i < S; ++i) {
            mbar_init(full + i * 8, 1);
            mbar_init(empty + i * 8, 1);          // released by the UMMA commit
        }
        for (int i = 0; i < kTS; ++i) {
            mbar_init(full_tm + i * 8, 1);
            mbar_init(empty_tm + i * 8, kAlt ? kEpiWarps / 2 : kEpiWarps);   // the warps that read a stage
        }
        mbar_init(a_full, kProducers);
        fence_mbar_init();
    }
    if (warp == kProducers) {   // first issuer warp owns the TMEM allocation
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

    // two-rank form with the link's own numbering: this call's number is one more than the last
    // finished call's (the word is rewritten only after every CTA of this call has read it)
    const int tp_epoch = (p.tp_peer_inbox && p.tp_epoch == 0) ? ld_acquire_gpu(p.tp_ctrl) + 1 : p.tp_epoch;

    const long long units = static_cast<long long>(p.n_tiles) * p.kb;
    const long long u0 = range_begin(units, blockIdx.x, gridDim.x);
    const long long u1 = range_begin(units, blockIdx.x + 1, gridDim.x);
    const int count = static_cast<int>(u1 - u0);

    if (warp < kProducers) {
        // ------------------------------------------------------------ TMA producers
        const int me = warp;
        const uint64_t stream_policy = policy_evict_first();
        const uint64_t keep_policy = policy_evict_last();
        Ring ring;
        ring.step(me, S);
        int tile = static_cast<int>((u0 + me) / p.kb), kb = static_cast<int>((u0 + me) % p.kb);
        bool alive = true;
        if (resident && count > 0) {
            // this producer's share of the activation tiles (K blocks me, me + kProducers, ..), one lane
            // per tile in a single instruction
            const int mine = me < p.kb ? (p.kb - me + kProducers - 1) / kProducers : 0;
            if (lane == 0) {
                if (mine > 0) mbar_arrive_expect_tx(a_full, static_cast<uint32_t>(mine) * L::kABytes);
                else mbar_arrive(a_full);
            }
            __syncwarp();
            for (int j0 = 0; j0 < mine; j0 += 32) {
                const int j = j0 + static_cast<int>(lane);
                const int kbj = me + j * kProducers;
                if (j < mine) tma_load_2d_hint(a_res + kbj * L::kABytes, &a_map, a_full, kbj * kBlockK, 0, keep_policy);
            }
        }
        const uint32_t lanes_loading = resident ? 1u : 2u;
        for (int n = me; n < count && alive; n += kProducers) {
            const int s = ring.idx;
            alive = mbar_wait_lane0(empty + s * 8, ring.phase ^ 1u, abort_flag, p.status, kDevTimeoutGemmEmpty);
            if (!alive) break;
            if (lane == 0) mbar_arrive_expect_tx(full + s * 8, stage_bytes);
            __syncwarp();
            // one instruction, two lanes: lane 0 fetches the weight tile, lane 1 the activations
            const uint32_t dst = base + s * stage_bytes + (lane == 1 ? kWBytes : 0);
            const void* map = lane == 1 ? static_cast<const void*>(&a_map) : static_cast<const void*>(&w_map);
            const int a_x = kb * kBlockK + (p.group_tiles ? (tile / p.group_tiles) * p.K : 0);
            if (lane < lanes_loading)
                tma_load_2d_hint(dst, map, full + s * 8, lane == 1 ? a_x : kb * kBlockK, lane == 1 ? 0 : tile * kTileN,
                                 lane == 1 ? keep_policy : stream_policy);
            ring.step(kProducers, S);
            kb += kProducers;
            while (kb >= p.kb) {
                kb -= p.kb;
                ++tile;
            }
        }
    } else if (warp < kProducers + kIssuers) {
        // ------------------------------------------------------------ UMMA issuers (one thread each)
        if (lane == 0) {
            const int me = warp - kProducers;
            constexpr uint32_t idesc = umma_idesc(kTileN, M_PAD, 0, 0);
            Ring ring, tring;
            ring.step(me, S);
            tring.step(me, kTS);
            int kbi = static_cast<int>((u0 + me) % p.kb);   // K block of this issuer's next unit
            bool a_ready = !resident || count <= me ||
                           mbar_wait(a_full, 0u, abort_flag, p.status, kDevTimeoutGemmFull);
            for (int n = me; n < count && a_ready; n += kIssuers) {
                const int s = ring.idx, ts = tring.idx;
                if (!mbar_wait(full + s * 8, ring.phase, abort_flag, p.status, kDevTimeoutGemmFull)) break;
                if (!mbar_wait(empty_tm + ts * 8, tring.phase ^ 1u, abort_flag, p.status, kDevTimeoutGemmTmemEmpty)) break;
                tc_fence_after();
                const uint32_t w_addr = base + s * stage_bytes;
                const uint32_t a_addr = resident ? a_res + kbi * L::kABytes : w_addr + kWBytes;
                kbi += kIssuers;
                while (kbi >= p.kb) kbi -= p.kb;
                const uint32_t d_addr = tmem_base + ts * M_PAD;
#pragma unroll
                for (int k = 0; k < kBlockK / 32; ++k)
                    umma_f8f6f4(d_addr, umma_smem_desc_sw128(w_addr + k * 32), umma_smem_desc_sw128(a_addr + k * 32),
                                idesc, k > 0 ? 1u : 0u);
                umma_commit(full_tm + ts * 8);
                umma_commit(empty + s * 8);      // the stage's bytes are consumed once the UMMAs retire
                ring.step(kIssuers, S);
                tring.step(kIssuers, kTS);
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue warps
        // Thread = one weight row (TMEM lane) x half of the activation columns.
        const int ew = warp - kFirstEpiWarp;            // 0..7
        const int grp = ew >> 2;                        // epilogue warpgroup
        const int half = grp;                           // the half of the columns this group finishes
        const int et = (ew * 32 + lane);                // 0..255 among epilogue threads
        const int gt = et & 127;                        // 0..127 inside the group
        const int row_in_tile = (warp & 3) * 32 + lane;
        const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
        // kAlt: this group takes the units with (n & 1) == grp and accumulates every column;
        // otherwise both groups take every unit and half of the columns each.
        constexpr int kCols = kAlt ? M_PAD : kHalf;
        const int col0 = kAlt ? 0 : half * kHalf;
        constexpr int kStep = kAlt ? 2 : 1;
        const int first = kAlt ? grp : 0;               // this group's first unit
        __align__(8) float acc[kCols];
#pragma unroll
        for (int i = 0; i < kCols; ++i) acc[i] = 0.f;
        Ring tring;
        tring.step(first, kTS);
        bool alive = true;
        int tile = static_cast<int>(u0 / p.kb), kb = static_cast<int>(u0 % p.kb);
        int seg_kb0 = kb;                               // first K block of the running segment

        // Scales of a unit (activation scales a_s[:, kb], weight scale w_s[tile, kb]) are fetched
        // kScaleAhead of the group's units early with 4-byte asynchronous copies into the group's rings
        // of kScaleSlots slots, so their L2 latency never sits between two units.
        float* a_ring = rings + (kAlt ? grp * L::kRingFloats : 0);   // one ring per group, or one shared
        float* w_ring = a_ring + kScaleSlots * M_PAD;
        const int fetcher = kAlt ? gt : et;             // thread index among those that share the rings
        const int fetchers = kAlt ? 128 : 256;
        int ftile = static_cast<int>((u0 + first) / p.kb), fkb = static_cast<int>((u0 + first) % p.kb);
        auto fetch_scales = [&](int j) {                // j-th unit of this group
            if (first + j * kStep < count) {
                const int slot = j & (kScaleSlots - 1);
                const int a_stride = p.a_kb_total ? p.a_kb_total : p.kb;
                const int a_col = fkb + (p.group_tiles ? (ftile / p.group_tiles) * p.kb : 0);
                for (int r = fetcher; r < p.M; r += fetchers)
                    cp_async4(smem_u32(a_ring + slot * M_PAD + r), p.a_scales + static_cast<int64_t>(r) * a_stride + a_col);
                if (fetcher == fetchers - 1)
                    cp_async4(smem_u32(w_ring + slot), p.w_scales + static_cast<int64_t>(ftile) * p.kb + fkb);
                fkb += kStep;
                while (fkb >= p.kb) {
                    fkb -= p.kb;
                    ++ftile;
                }
            }
            cp_async_commit();                           // one group per unit, empty or not
        };
        for (int j = 0; j < kScaleAhead; ++j) fetch_scales(j);
        auto ring_sync = [&]() {                         // the threads that share this group's rings
            if constexpr (kAlt) {
                if (grp == 0) asm volatile("bar.sync 2, 128;" ::: "memory");
                else asm volatile("bar.sync 3, 128;" ::: "memory");
            } else {
                epi_bar_sync();
            }
        };

        // An aborting CTA keeps walking the loop (every wait then fails at once) so that all
        // 256 epilogue threads reach every named barrier; it only skips the arithmetic.
        int j = 0;                                       // units this group has taken
        for (int n = 0; n < count; ++n) {
            if (!kAlt || (n & 1) == grp) {
            fetch_scales(j + kScaleAhead);
            cp_async_wait<kScaleAhead>();                // this thread's copies for the unit have landed
            ring_sync();                                 // ... and so have everybody else's
            if constexpr (kPreScale) {   // the unit's scale products a_s[c] * w_s, once per column
                const int slot = j & (kScaleSlots - 1);
                if (fetcher < M_PAD) a_ring[slot * M_PAD + fetcher] = __fmul_rn(a_ring[slot * M_PAD + fetcher], w_ring[slot]);
                ring_sync();
            }
            const int ts = tring.idx;
            if (alive)
                alive = mbar_wait_warp_fast(full_tm + ts * 8, tring.phase, abort_flag, p.status, kDevTimeoutGemmTmemFull);
            if (alive) {
                tc_fence_after();
                const int slot = j & (kScaleSlots - 1);
                const float wsc = kPreScale ? 1.0f : w_ring[slot];   // wide tiles hold a_s[c] * w_s already
                const float* sc = a_ring + slot * M_PAD + col0;
                const uint32_t taddr = tmem_base + lane_base + ts * M_PAD + col0;
                // acc[c] += v[c] * (a_s[c] * w_s): the products come as 16-byte shared-memory loads, the
                // sums as packed fp32x2 operations (one instruction per two columns)
                float2* acc2 = reinterpret_cast<float2*>(acc);
                const float2 w2 = make_float2(wsc, wsc);
                if constexpr (kCols >= 32) {
                    uint32_t v[2][32];
                    tmem_ld_32x32(taddr, v[0]);
#pragma unroll
                    for (int c = 0; c < kCols; c += 32) {
                        tmem_ld_wait();
                        if (c + 32 < kCols) tmem_ld_32x32(taddr + c + 32, v[((c >> 5) + 1) & 1]);
                        const uint32_t* x = v[(c >> 5) & 1];
                        const float4* s4 = reinterpret_cast<const float4*>(sc + c);
#pragma unroll
                        for (int i = 0; i < 32; i += 4) {
                            const float4 sv = s4[i >> 2];
                            const float2 s01 = kPreScale ? make_float2(sv.x, sv.y) : __fmul2_rn(make_float2(sv.x, sv.y), w2);
                            const float2 s23 = kPreScale ? make_float2(sv.z, sv.w) : __fmul2_rn(make_float2(sv.z, sv.w), w2);
                            acc2[(c + i) >> 1] = __ffma2_rn(make_float2(__uint_as_float(x[i]), __uint_as_float(x[i + 1])),
                                                            s01, acc2[(c + i) >> 1]);
                            acc2[((c + i) >> 1) + 1] = __ffma2_rn(
                                make_float2(__uint_as_float(x[i + 2]), __uint_as_float(x[i + 3])), s23,
                                acc2[((c + i) >> 1) + 1]);
                        }
                    }
                } else if constexpr (kCols == 16) {
                    uint32_t v[16];
                    tmem_ld_32x16(taddr, v);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 16; ++i) acc[i] = fmaf(__uint_as_float(v[i]), sc[i] * wsc, acc[i]);
                } else {
                    uint32_t v[8];
                    tmem_ld_32x8(taddr, v);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 8; ++i) acc[i] = fmaf(__uint_as_float(v[i]), sc[i] * wsc, acc[i]);
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(empty_tm + ts * 8);
            }
            tring.step(kStep, kTS);
            ++j;
            }

            // ---- end of a segment: the tile's K range ended, or this CTA's range did
            const bool seg_end = (kb + 1 == p.kb) || (n + 1 == count);
            if (seg_end) {
                if constexpr (kAlt) {
                    // Each group hands the other the columns that one finishes and adds what it gets
                    // to its own half; the sums land in acc[0, kHalf).  x + y == y + x, so the result
                    // does not depend on which group held which units.
                    // (constant register indices in both branches: the accumulators stay in registers)
                    if (half == 0) {
#pragma unroll
                        for (int i = 0; i < kHalf; ++i) comb[(kHalf + i) * kTileN + row_in_tile] = acc[kHalf + i];
                    } else {
#pragma unroll
                        for (int i = 0; i < kHalf; ++i) comb[i * kTileN + row_in_tile] = acc[i];
                    }
                    epi_bar_sync();
                    if (half == 0) {
#pragma unroll
                        for (int i = 0; i < kHalf; ++i) acc[i] = acc[i] + comb[i * kTileN + row_in_tile];
                    } else {
#pragma unroll
                        for (int i = 0; i < kHalf; ++i) acc[i] = acc[kHalf + i] + comb[(kHalf + i) * kTileN + row_in_tile];
                    }
                    epi_bar_sync();                      // the buffer is free for the next segment
                }
                const int nrow = tile * kTileN + row_in_tile;
                const bool from_zero = (seg_kb0 == 0), to_end = (kb + 1 == p.kb);
                if (!from_zero) {
                    // A partial that does not start the tile's K range goes to this CTA's slot;
                    // the CTA that holds the start of the range collects it.  Layout
                    // [column][row]: a warp's 32 rows are contiguous.
                    float* slot = p.scratch + static_cast<int64_t>(blockIdx.x) * (M_PAD * kTileN) + row_in_tile;
                    if (alive) {
#pragma unroll
                        for (int i = 0; i < kHalf; ++i) __stcg(slot + (half * kHalf + i) * kTileN, acc[i]);
                    }
                    __threadfence();
                    epi_bar_sync();
                    if (et == 0 && alive) st_release_gpu(p.flags + blockIdx.x, 1);
                } else {
                    if (!to_end) {
                        // This CTA holds the start of the tile's K range and the range continues in
                        // the following CTAs (all resident: the grid is one CTA per SM).  Add their
                        // partials in CTA order, so the sum does not depend on timing.
                        const long long t_end = static_cast<long long>(tile + 1) * p.kb - 1;
                        const int last = cta_of(units, t_end, gridDim.x);
                        // every contributor's flag is awaited by a thread of its own, then the partials are
                        // added in CTA order (the loads of different partials overlap)
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
                                const float* peer = p.scratch + static_cast<int64_t>(c) * (M_PAD * kTileN) + row_in_tile;
#pragma unroll
                                for (int i = 0; i < kHalf; ++i) acc[i] += __ldcg(peer + (half * kHalf + i) * kTileN);
                            }
                        }
                        epi_bar_sync();
                        if (alive)
                            for (int c = blockIdx.x + 1 + et; c <= last; c += 32 * kEpiWarps) p.flags[c] = 0;   // free again
                    }
                    if (p.tp_peer_inbox) {
                        // Two-rank all-reduce fused into the epilogue: the finished fp32 tile goes
                        // straight into the peer GPU's inbox over NVLink (plain stores through the
                        // peer mapping, then a system-scope release of the tile's flag), and the
                        // peer's tile is awaited in this GPU's own inbox and added.  a + b == b + a
                        // in fp32, so both ranks hold bit-identical sums.  Inbox sets alternate
                        // with the call's sequence number: a rank can be one call ahead of its
                        // peer's reads, never two.
                        const int64_t set = static_cast<int64_t>(tp_epoch & 1) * p.n_tiles;
                        const int64_t tile_off = (set + tile) * (M_PAD * kTileN) + row_in_tile;
                        if (alive) {
#pragma unroll
                            for (int i = 0; i < kHalf; ++i)
                                p.tp_peer_inbox[tile_off + (half * kHalf + i) * kTileN] = acc[i];
                        }
                        __threadfence_system();
                        epi_bar_sync();
                        if (et == 0 && alive) {
                            st_release_sys(p.tp_peer_flags + set + tile, tp_epoch);
                            const unsigned long long start = globaltimer_ns();
                            uint32_t spins = 0;
                            while (ld_acquire_sys(p.tp_my_flags + set + tile) != tp_epoch) {
                                if ((++spins & 63u) == 0u && (*abort_flag || globaltimer_ns() - start > p.tp_wait_ns)) {
                                    *abort_flag = 1;
                                    if (p.status) atomicCAS(p.status, 0, kDevTimeoutPeerFlag);
                                    break;
                                }
                                __nanosleep(100);
                            }
                        }
                        epi_bar_sync();
                        alive = alive && !*abort_flag;
                        if (alive) {
#pragma unroll
                            for (int i = 0; i < kHalf; ++i)
                                acc[i] += ld_volatile_f32(p.tp_my_inbox + tile_off + (half * kHalf + i) * kTileN);
                        }
                    }
                    if (alive && nrow < p.N) {
#pragma unroll
                        for (int i = 0; i < kHalf; ++i) {
                            const int m = half * kHalf + i;
                            if (m < p.M) p.c[static_cast<int64_t>(m) * p.N + nrow] = __float2bfloat16_rn(acc[i]);
                        }
                    }
                }
#pragma unroll
                for (int i = 0; i < kCols; ++i) acc[i] = 0.f;
                seg_kb0 = 0;
            }
            if (++kb == p.kb) {
                kb = 0;
                ++tile;
            }
        }
        cp_async_wait<0>();
    }

    __syncthreads();
    if (*abort_flag) abort_drain_sleep();
    __syncthreads();
    if (warp == kProducers) {
        tc_fence_after();
        tmem_dealloc(tmem_base, L::kTmemCols);
    }
    if (p.tp_peer_inbox && p.tp_epoch == 0 && threadIdx.x == 0) {
        // the last CTA to get here has seen every other CTA finish, hence read the old number
        __threadfence();
        if (atomicAdd(p.tp_ctrl + 1, 1) == static_cast<int>(gridDim.x) - 1) {
            p.tp_ctrl[1] = 0;
            st_release_gpu(p.tp_ctrl, tp_epoch);
        }
    }
}

template <int M_PAD>
static int launch(const CUtensorMap& w_map, const CUtensorMap& a_map, Params& p, const DeviceInfo& dev,
                  cudaStream_t stream) {
    using L = Smem<M_PAD>;
    // resident activations if they leave room for six or more weight stages (96 KB in flight)
    int stages = 16, rkb = p.kb;
    while (stages > 6 && L::total(stages, rkb) > dev.smem_optin) stages -= 2;
    if (p.group_tiles || L::total(stages, rkb) > dev.smem_optin) {   // groups read different activation columns
        rkb = 0;
        stages = 16;
        while (stages > 2 && L::total(stages) > dev.smem_optin) stages -= 2;
    }
    const int smem = L::total(stages, rkb);
    if (smem > dev.smem_optin)
        return fail(WUDA_ERR_UNSUPPORTED, "device offers %d bytes of shared memory per block; the kernel needs more",
                    dev.smem_optin);
    p.stages = stages;
    p.a_resident = rkb > 0;
    auto kernel = gemm_fp8_kernel<M_PAD>;
    WUDA_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, dev.smem_optin));
    const long long units = static_cast<long long>(p.n_tiles) * p.kb;
    // at most kMaxSplit CTAs share one weight tile: the tile's owner adds the others' partials one after
    // the other, which costs more than it saves when a few tiles are cut into a hundred pieces
    // (adding one partial costs the owner about as much as streaming M_PAD / 64 units, so wide tiles split less)
    constexpr int kMaxSplit = M_PAD <= 16 ? 16 : (M_PAD == 32 ? 12 : (M_PAD == 64 ? 8 : 6));
    const int sms = gemm_sms(dev);
    int grid = units < sms ? static_cast<int>(units) : sms;
    if (static_cast<long long>(p.n_tiles) * kMaxSplit < grid) grid = p.n_tiles * kMaxSplit;
    WUDA_CUDA(launch_pdl(kernel, dim3(grid), dim3(kThreads), smem, stream, w_map, a_map, p));
    return WUDA_OK;
}

}  // namespace gemm8
}  // namespace wuda

// Scratch = one flag per CTA (the first kFlagBytes bytes), then one fp32 partial tile [M_PAD][128] per CTA.
// The grid never exceeds kMaxGrid CTAs (one per SM).  The flags come first so that calls with different row
// counts, which size their slots differently, find them in the same place: one scratch buffer can then serve
// every GEMM of a stream without a slot of one call ever covering the flags of another.
constexpr int kMaxGrid = 192;
constexpr int64_t kFlagBytes = 1024;

extern "C" int64_t wuda_gemm_fp8_scratch_bytes(int m, int n) {
    if (m < 1 || n < 1 || m > 256) return -1;
    int m_pad = 16;
    while (m_pad < m) m_pad *= 2;
    return kFlagBytes + static_cast<int64_t>(kMaxGrid) * m_pad * 128 * 4;
}

namespace {

// What every entry point of this file hands to the one set-up routine below.
struct GemmCall {
    const void* a = nullptr;
    const float* a_scales = nullptr;
    const void* w = nullptr;
    const float* w_scales = nullptr;
    void* c = nullptr;
    int m = 0, n = 0, k = 0;          // n = rows per group
    int groups = 1;
    float* slots = nullptr;           // [kMaxGrid][m_pad][128] fp32 partial tiles
    int32_t* flags = nullptr;         // [kMaxGrid], zero between calls
    int32_t* status = nullptr;
    cudaStream_t stream = nullptr;
    // two-rank form (inboxes == nullptr: none)
    void* my_inbox = nullptr;
    void* peer_inbox = nullptr;
    int epoch = 0;
    int peer_wait_ms = 0;
};

constexpr int64_t kTpFlagBytes = 4096;      // 2 sets x n_tiles tile flags, then the control words
constexpr int64_t kTpCtrlBytes = 64;        // last bytes of the flag block: {call sequence, CTAs done}

int64_t tp_bytes(int m, int n) {
    if (m < 1 || m > 256 || n < 1) return -1;
    int m_pad = 16;
    while (m_pad < m) m_pad *= 2;
    const int64_t n_tiles = (n + 127) / 128;
    if (2 * n_tiles * 4 > kTpFlagBytes - kTpCtrlBytes) return -1;
    return kTpFlagBytes + 2 * n_tiles * m_pad * 128 * 4;
}

// Parameter block, the two tensor maps and the launch for 1 <= m <= 128 (checked by the callers).
int gemm_fp8_setup_and_launch(const GemmCall& g) {
    using namespace wuda;
    using namespace wuda::gemm8;
    DeviceInfo dev;
    int st = current_device_info(&dev);
    if (st != WUDA_OK) return st;
    WUDA_REQUIRE(dev.num_sms <= kMaxGrid, "device has %d SMs; at most %d are supported", dev.num_sms, kMaxGrid);
    const int n_all = g.n * g.groups;
    int m_pad = 16;
    while (m_pad < g.m) m_pad *= 2;
    Params p;
    p.a_scales = g.a_scales;
    p.w_scales = g.w_scales;
    p.c = static_cast<__nv_bfloat16*>(g.c);
    p.status = g.status;
    p.M = g.m;
    p.N = n_all;
    p.K = g.k;
    p.kb = g.k / 128;
    p.n_tiles = (n_all + 127) / 128;
    p.group_tiles = g.groups > 1 ? g.n / 128 : 0;
    p.a_kb_total = g.groups * (g.k / 128);
    p.scratch = g.slots;
    p.flags = g.flags;
    p.stages = 0;
    if (g.peer_inbox) {
        p.tp_my_flags = static_cast<int32_t*>(g.my_inbox);
        p.tp_peer_flags = static_cast<int32_t*>(g.peer_inbox);
        p.tp_my_inbox = reinterpret_cast<float*>(static_cast<uint8_t*>(g.my_inbox) + kTpFlagBytes);
        p.tp_peer_inbox = reinterpret_cast<float*>(static_cast<uint8_t*>(g.peer_inbox) + kTpFlagBytes);
        p.tp_ctrl = reinterpret_cast<int32_t*>(static_cast<uint8_t*>(g.my_inbox) + kTpFlagBytes - kTpCtrlBytes);
        p.tp_epoch = g.epoch;
        p.tp_wait_ns = static_cast<unsigned long long>(g.peer_wait_ms) * 1000ull * 1000ull;
    }

    CUtensorMap w_map, a_map;
    {
        const uint64_t dims[2] = {static_cast<uint64_t>(g.k), static_cast<uint64_t>(n_all)};
        const uint64_t strides[1] = {static_cast<uint64_t>(g.k)};
        const uint32_t box[2] = {128u, 128u};
        st = encode_tensor_map(&w_map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, g.w, dims, strides, box,
                               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
        if (st != WUDA_OK) return st;
    }
    {
        const uint64_t dims[2] = {static_cast<uint64_t>(g.k) * g.groups, static_cast<uint64_t>(g.m)};
        const uint64_t strides[1] = {static_cast<uint64_t>(g.k) * g.groups};
        const uint32_t box[2] = {128u, static_cast<uint32_t>(m_pad)};
        st = encode_tensor_map(&a_map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, g.a, dims, strides, box,
                               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B);
        if (st != WUDA_OK) return st;
    }
    switch (m_pad) {
        case 16: return launch<16>(w_map, a_map, p, dev, g.stream);
        case 32: return launch<32>(w_map, a_map, p, dev, g.stream);
        case 64: return launch<64>(w_map, a_map, p, dev, g.stream);
        default: return launch<128>(w_map, a_map, p, dev, g.stream);
    }
}

// groups == 1: the plain GEMM.  groups > 1: `n` rows per group, group g multiplies the activations'
// columns [g * k, (g + 1) * k) by the weight rows [g * n, (g + 1) * n).
int gemm_fp8_entry(const void* a, const float* a_scales, const void* w, const float* w_scales, void* c_bf16,
                   int m, int n, int k, int groups, void* scratch, int64_t scratch_bytes,
                   int32_t* status_word, void* stream) {
    using namespace wuda;
    clear_error();
    WUDA_REQUIRE(groups >= 1, "groups must be >= 1 (got %d)", groups);
    WUDA_REQUIRE(groups == 1 || n % 128 == 0, "with groups the rows per group must be a multiple of 128 (got %d)", n);
    const int n_all = n * groups;
    WUDA_REQUIRE(m >= 0 && m <= 256, "m must be in [0, 256] (got %d)", m);
    WUDA_REQUIRE(n >= 1, "n must be >= 1 (got %d)", n);
    WUDA_REQUIRE(k >= 128 && k % 128 == 0, "k must be a positive multiple of 128 (got %d)", k);
    if (m == 0) return WUDA_OK;
    WUDA_REQUIRE(a && a_scales && w && w_scales && c_bf16 && scratch,
                 "a, a_scales, w, w_scales, c and scratch must not be NULL");
    WUDA_REQUIRE(aligned16(a) && aligned16(w), "a and w must be 16-byte aligned");
    WUDA_REQUIRE((reinterpret_cast<uintptr_t>(scratch) & 255u) == 0, "scratch must be 256-byte aligned");
    const int64_t need = wuda_gemm_fp8_scratch_bytes(m, n_all);
    WUDA_REQUIRE(scratch_bytes >= need, "scratch holds %lld bytes; %lld are needed (wuda_gemm_fp8_scratch_bytes)",
                 static_cast<long long>(scratch_bytes), static_cast<long long>(need));
    if (m > 128) {
        // Above 128 rows a warpgroup's 128 accumulator columns no longer fit the register file;
        // two passes of <= 128 rows (the weights stream twice) are faster than one that spills.
        int st2 = gemm_fp8_entry(a, a_scales, w, w_scales, c_bf16, 128, n, k, groups, scratch, scratch_bytes, status_word,
                                 stream);
        if (st2 != WUDA_OK) return st2;
        return gemm_fp8_entry(static_cast<const uint8_t*>(a) + static_cast<int64_t>(128) * k * groups,
                              a_scales + static_cast<int64_t>(128) * (k / 128) * groups, w, w_scales,
                              static_cast<__nv_bfloat16*>(c_bf16) + static_cast<int64_t>(128) * n_all, m - 128, n, k,
                              groups, scratch, scratch_bytes, status_word, stream);
    }
    GemmCall g;
    g.a = a, g.a_scales = a_scales, g.w = w, g.w_scales = w_scales, g.c = c_bf16;
    g.m = m, g.n = n, g.k = k, g.groups = groups;
    g.flags = static_cast<int32_t*>(scratch);
    g.slots = reinterpret_cast<float*>(static_cast<uint8_t*>(scratch) + kFlagBytes);
    g.status = status_word;
    g.stream = static_cast<cudaStream_t>(stream);
    return gemm_fp8_setup_and_launch(g);
}

}  // namespace

extern "C" int wuda_gemm_fp8_blockscaled(const void* a, const float* a_scales, const void* w, const float* w_scales,
                                         void* c_bf16, int m, int n, int k, void* scratch, int64_t scratch_bytes,
                                         int32_t* status_word, void* stream) {
    return gemm_fp8_entry(a, a_scales, w, w_scales, c_bf16, m, n, k, 1, scratch, scratch_bytes, status_word, stream);
}

extern "C" int wuda_gemm_fp8_grouped(const void* a, const float* a_scales, const void* w, const float* w_scales,
                                     void* c_bf16, int m, int n_per_group, int k, int groups, void* scratch,
                                     int64_t scratch_bytes, int32_t* status_word, void* stream) {
    return gemm_fp8_entry(a, a_scales, w, w_scales, c_bf16, m, n_per_group, k, groups, scratch, scratch_bytes,
                          status_word, stream);
}

// ---------------------------------------------------------------------------------------------
// Allocation-free entry point.
//
// Some hosts must never see a device allocation from a library they call: a serving process
// that carved up all device memory at start-up and hands it out through its own pool (a stray
// cudaMalloc can fail there, or fragment what is left), and latency-critical loops in which
// cudaMalloc / cudaFree would synchronise the whole device and stall every other stream.  The
// regular entry point leaves the scratch to the caller; this one needs no scratch argument at
// all: the partial-tile slots and flags of the stream-K fix-up live in a fixed array inside the
// library's device image.  The price is a limit on m (kNoAllocMaxM) and kNoAllocScratchBytes of
// device memory held by every GPU that loads the library, until the process exits.
//
// The array is shared by every call on a device and keeps what the last call left in it.  The
// partial tiles are always written before they are read, so only the flags have to start at
// zero; the kernel resets each flag after use, and the entry point clears all of them again
// before every launch in case an earlier call ended abnormally.  Two calls that overlap on the
// GPU (different streams) would race on the slots: calls through this entry point must be
// ordered one after another on the device.  The flags sit at the start of the array, so calls with
// different m (different slot sizes) share it without moving them.
constexpr int kNoAllocMaxM = 64;
constexpr int64_t kNoAllocSlotBytes = static_cast<int64_t>(kMaxGrid) * kNoAllocMaxM * 128 * 4;
constexpr int64_t kNoAllocScratchBytes = kFlagBytes + kNoAllocSlotBytes;   // 6,292,480 bytes

static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

// The array's name is only a handle in host code; the device address comes from
// cudaGetSymbolAddress, asked once per device with that device current.
static int noalloc_scratch_address(int device, void** out) {
    static std::mutex mu;
    static void* cached[64] = {};
    if (device < 0 || device >= 64) return wuda::fail(WUDA_ERR_UNSUPPORTED, "device ordinal %d out of range", device);
    std::lock_guard<std::mutex> lock(mu);
    if (!cached[device]) {
        void* ptr = nullptr;
        cudaError_t err = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
        if (err != cudaSuccess || !ptr) {
            cudaGetLastError();
            return wuda::fail(WUDA_ERR_CUDA, "cudaGetSymbolAddress(no-alloc scratch) failed: %s", cudaGetErrorString(err));
        }
        cached[device] = ptr;
    }
    *out = cached[device];
    return WUDA_OK;
}

extern "C" int wuda_gemm_fp8_blockscaled_noalloc(const void* a, const float* a_scales, const void* w,
                                                 const float* w_scales, void* c_bf16, int m, int n, int k,
                                                 int32_t* status_word, void* stream) {
    using namespace wuda;
    clear_error();
    WUDA_REQUIRE(m >= 0, "m must be >= 0 (got %d)", m);
    if (m > kNoAllocMaxM)
        return fail(WUDA_ERR_UNSUPPORTED,
                    "the allocation-free entry point handles m <= %d (got %d): its built-in scratch is %lld bytes; "
                    "use wuda_gemm_fp8_blockscaled with caller-provided scratch for larger m",
                    kNoAllocMaxM, m, static_cast<long long>(kNoAllocScratchBytes));
    WUDA_REQUIRE(n >= 1, "n must be >= 1 (got %d)", n);
    WUDA_REQUIRE(k >= 128 && k % 128 == 0, "k must be a positive multiple of 128 (got %d)", k);
    if (m == 0) return WUDA_OK;
    WUDA_REQUIRE(a && a_scales && w && w_scales && c_bf16, "a, a_scales, w, w_scales and c must not be NULL");
    WUDA_REQUIRE(aligned16(a) && aligned16(w), "a and w must be 16-byte aligned");

    DeviceInfo dev;
    int st = current_device_info(&dev);
    if (st != WUDA_OK) return st;
    void* scratch = nullptr;
    st = noalloc_scratch_address(dev.device, &scratch);   // first call on a device: symbol lookup
    if (st != WUDA_OK) return st;

    GemmCall g;
    g.a = a, g.a_scales = a_scales, g.w = w, g.w_scales = w_scales, g.c = c_bf16;
    g.m = m, g.n = n, g.k = k;
    g.flags = static_cast<int32_t*>(scratch);
    g.slots = reinterpret_cast<float*>(static_cast<uint8_t*>(scratch) + kFlagBytes);
    g.status = status_word;
    g.stream = static_cast<cudaStream_t>(stream);
    // the flags must start at zero whatever the previous call left behind
    WUDA_CUDA(cudaMemsetAsync(g.flags, 0, kMaxGrid * sizeof(int32_t), g.stream));
    return gemm_fp8_setup_and_launch(g);
}

// ---------------------------------------------------------------------------------------------
// Two-rank tensor-parallel form: the K dimension is split across two GPUs (row-parallel
// linear, dsv4_megakernel/origin/model.py:166-180: y = x_r W_r^T summed over ranks in fp32,
// then cast; the reference's megakernel only fabricates this sum,
// dsv4_megakernel/megakernel/test/test_e2e_decode.py:186-194).  Each rank runs the same GEMM on
// its K slice; the all-reduce happens tile by tile inside the epilogue through peer memory.
//
// The exchange buffer of a rank ("inbox") is ordinary device memory made visible to the peer
// process with CUDA IPC.  Layout: a 4 KB flag block (2 sets x n_tiles int32 tile flags; its last
// 64 bytes hold the link's own call sequence number and a count of finished CTAs), then
// 2 sets x n_tiles x [M_PAD][128] fp32 tiles.
//
// Call sequence numbers.  A tile's flag carries the number of the call that delivered it, so both
// ranks must number their calls alike.  epoch >= 1: the host numbers them (1, 2, 3, .. on both
// ranks).  epoch == 0: the link numbers them itself - every CTA reads the last finished number from
// the control words and the last CTA to finish stores the new one - so the same launch can be
// replayed from a CUDA graph.  A link uses one of the two forms for its whole life.
extern "C" int64_t wuda_tp2_inbox_bytes(int m, int n) { return tp_bytes(m, n); }

extern "C" int wuda_tp2_alloc(int64_t bytes, void** local_base, unsigned char* ipc_handle_64) {
    using namespace wuda;
    clear_error();
    WUDA_REQUIRE(bytes > 0 && local_base && ipc_handle_64, "bytes must be > 0 and the outputs must not be NULL");
    void* ptr = nullptr;
    WUDA_CUDA(cudaMalloc(&ptr, static_cast<size_t>(bytes)));
    cudaError_t err = cudaMemset(ptr, 0, static_cast<size_t>(bytes));
    cudaIpcMemHandle_t h;
    if (err == cudaSuccess) err = cudaIpcGetMemHandle(&h, ptr);
    if (err != cudaSuccess) {
        cudaFree(ptr);
        cudaGetLastError();
        return fail(WUDA_ERR_CUDA, "preparing the exchange buffer failed: %s", cudaGetErrorString(err));
    }
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle is 64 bytes");
    memcpy(ipc_handle_64, &h, 64);
    *local_base = ptr;
    return WUDA_OK;
}

extern "C" int wuda_tp2_open(const unsigned char* ipc_handle_64, void** peer_base) {
    using namespace wuda;
    clear_error();
    WUDA_REQUIRE(ipc_handle_64 && peer_base, "handle and output must not be NULL");
    cudaIpcMemHandle_t h;
    memcpy(&h, ipc_handle_64, 64);
    WUDA_CUDA(cudaIpcOpenMemHandle(peer_base, h, cudaIpcMemLazyEnablePeerAccess));
    return WUDA_OK;
}

extern "C" int wuda_tp2_close(void* peer_base) {
    using namespace wuda;
    clear_error();
    if (peer_base) WUDA_CUDA(cudaIpcCloseMemHandle(peer_base));
    return WUDA_OK;
}

extern "C" int wuda_tp2_free(void* local_base) {
    using namespace wuda;
    clear_error();
    if (local_base) WUDA_CUDA(cudaFree(local_base));
    return WUDA_OK;
}

extern "C" int wuda_gemm_fp8_blockscaled_tp2(const void* a, const float* a_scales, const void* w,
                                             const float* w_scales, void* c_bf16, int m, int n, int k_local,
                                             void* scratch, int64_t scratch_bytes, void* my_inbox, void* peer_inbox,
                                             int epoch, int peer_wait_ms, int32_t* status_word, void* stream) {
    using namespace wuda;
    clear_error();
    // one pass only: a second pass of rows would need a second exchange under its own sequence number
    WUDA_REQUIRE(m >= 1 && m <= 128, "m must be in [1, 128] (got %d); split larger batches into calls of <= 128 rows", m);
    WUDA_REQUIRE(n >= 1, "n must be >= 1 (got %d)", n);
    WUDA_REQUIRE(k_local >= 128 && k_local % 128 == 0, "k_local must be a positive multiple of 128 (got %d)", k_local);
    WUDA_REQUIRE(a && a_scales && w && w_scales && c_bf16 && scratch && my_inbox && peer_inbox,
                 "a, a_scales, w, w_scales, c, scratch and both inboxes must not be NULL");
    WUDA_REQUIRE(epoch >= 0, "epoch must be >= 1 and grow by one per call on both ranks, or 0 for the link's own "
                 "numbering (got %d)", epoch);
    WUDA_REQUIRE(peer_wait_ms >= 1 && peer_wait_ms <= 10000, "peer_wait_ms must be in [1, 10000] (got %d)", peer_wait_ms);
    WUDA_REQUIRE(aligned16(a) && aligned16(w), "a and w must be 16-byte aligned");
    WUDA_REQUIRE((reinterpret_cast<uintptr_t>(scratch) & 255u) == 0, "scratch must be 256-byte aligned");
    const int64_t need = wuda_gemm_fp8_scratch_bytes(m, n);
    WUDA_REQUIRE(scratch_bytes >= need, "scratch holds %lld bytes; %lld are needed (wuda_gemm_fp8_scratch_bytes)",
                 static_cast<long long>(scratch_bytes), static_cast<long long>(need));
    WUDA_REQUIRE(tp_bytes(m, n) > 0, "n is too large for the exchange buffer's flag block");
    GemmCall g;
    g.a = a, g.a_scales = a_scales, g.w = w, g.w_scales = w_scales, g.c = c_bf16;
    g.m = m, g.n = n, g.k = k_local;
    g.flags = static_cast<int32_t*>(scratch);
    g.slots = reinterpret_cast<float*>(static_cast<uint8_t*>(scratch) + kFlagBytes);
    g.status = status_word;
    g.stream = static_cast<cudaStream_t>(stream);
    g.my_inbox = my_inbox, g.peer_inbox = peer_inbox, g.epoch = epoch, g.peer_wait_ms = peer_wait_ms;
    return gemm_fp8_setup_and_launch(g);
}
