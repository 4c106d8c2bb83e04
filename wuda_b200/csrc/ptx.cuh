// Thin inline-PTX layer for sm_100a: mbarrier (with bounded waits), TMA (bulk and
// tiled tensor copies, never cluster-broadcast forms), tcgen05 (TMEM allocation, UMMA
// issue/commit, TMEM loads) and the shared-memory / instruction descriptors UMMA needs.
//
// Every wait in this file is bounded.  A wait that runs out of time records a code in
// the kernel's status word, raises a CTA-wide abort flag and returns false; callers
// leave their loops, the CTA drains and exits normally, and the host reports the code.
// Nothing here traps, asserts or spins without a limit.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace wuda {

// ---------------------------------------------------------------- status codes
// Written (first writer wins) to the int32 status word a kernel is given.
enum DeviceStatus : int {
    kDevOk = 0,
    kDevTimeoutFullQ = 101,
    kDevTimeoutEmptyQ = 102,
    kDevTimeoutFullKv = 103,
    kDevTimeoutEmptyKv = 104,
    kDevTimeoutFullTmem = 105,
    kDevTimeoutEmptyTmem = 106,
    kDevBadPageIndex = 110,
    kDevBadContextLen = 111,        // a context length beyond the logits row / block-table row was cut to fit
    kDevTimeoutGemmFull = 121,
    kDevTimeoutGemmEmpty = 122,
    kDevTimeoutGemmTmemFull = 123,
    kDevTimeoutGemmTmemEmpty = 124,
    kDevScaleNotPow2 = 125,         // a scale given to the power-of-two GEMM was not one: the power of two below it was used
    kDevTimeoutPeerFlag = 131,
    kDevTimeoutMlaKeys = 151,       // sparse attention: a key block never arrived
    kDevTimeoutMlaScores = 152,     // ... its scores never completed
    kDevTimeoutMlaScoresRead = 153, // ... the softmax never released a score buffer
    kDevTimeoutMlaProbs = 154,      // ... its probabilities never arrived
    kDevTimeoutMlaOutput = 155,     // ... its weighted sum never completed
    kDevMlaScaleRange = 156,        // a key's scale exponent outside [-15, 7] was clamped into that range
};

// Wall-clock limit of one device-side wait.  Generous next to any real pipeline
// latency (microseconds), small next to a watchdog.
constexpr unsigned long long kWaitLimitNs = 2000ull * 1000ull * 1000ull;  // 2 s

__device__ __forceinline__ unsigned long long globaltimer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint32_t lane_id() {
    uint32_t l;
    asm volatile("mov.u32 %0, %%laneid;" : "=r"(l));
    return l;
}

__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "elect.sync _|p, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}\n"
        : "=r"(pred));
    return pred != 0;
}

// ---------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// Bounded wait.  `abort_flag` lives in shared memory and is shared by the whole CTA.
// Returns true when the phase completed, false when the CTA is aborting (either this
// wait ran out of time or another one did).  The fast path is a bare try_wait loop
// (the instruction itself suspends the thread for a while); the clock and the abort
// flag are consulted only after many failed polls, because reading %globaltimer on
// every wait adds its latency to each producer/consumer hand-off.
static __device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                            int* status_word, int code) {
    const unsigned long long t0 = globaltimer_ns();
    uint32_t spins = 0;
    while (!mbar_try_wait(bar, parity)) {
        if ((++spins & 63u) == 0u) {
            if (*abort_flag) return false;
            if (globaltimer_ns() - t0 > kWaitLimitNs) {
                *abort_flag = 1;
                if (status_word) atomicCAS(status_word, 0, code);
                return false;
            }
        }
    }
    return true;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          int* status_word, int code) {
#pragma unroll 1
    for (uint32_t spins = 0; spins < 4096u; ++spins)
        if (mbar_try_wait(bar, parity)) return true;
    return mbar_wait_slow(bar, parity, abort_flag, status_word, code);
}

// Warp-uniform forms, so that all 32 lanes take the same branch afterwards (callers use
// full-mask shuffles and __syncwarp).  `_warp`: every lane polls (each lane that later
// reads data written by the async proxy must observe the barrier itself), then votes.
// `_lane0`: only lane 0 polls and the result is broadcast.
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity,
                                               volatile int* abort_flag, int* status_word,
                                               int code) {
    const bool ok = mbar_wait(bar, parity, abort_flag, status_word, code);
    return __all_sync(0xffffffffu, ok);
}
__device__ __forceinline__ bool mbar_wait_lane0(uint32_t bar, uint32_t parity,
                                                volatile int* abort_flag, int* status_word,
                                                int code) {
    int ok = 1;
    if (lane_id() == 0) ok = mbar_wait(bar, parity, abort_flag, status_word, code) ? 1 : 0;
    return __shfl_sync(0xffffffffu, ok, 0) != 0;
}

// Sleep used on the abort path so that copies and MMAs already in flight land before
// the CTA gives its shared memory and TMEM back.
__device__ __forceinline__ void abort_drain_sleep() {
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 1000ull * 1000ull) __nanosleep(2000);
}

// ---------------------------------------------------------------- TMA
// Tiled tensor copies global -> this CTA's shared memory, completion on an mbarrier.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void* tmap, uint32_t bar, int c0,
                                            int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(tmap), "r"(bar), "r"(c0), "r"(c1)
        : "memory");
}
__device__ __forceinline__ void tma_load_2d_hint(uint32_t dst, const void* tmap, uint32_t bar,
                                                 int c0, int c1, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
        ".L2::cache_hint [%0], [%1, {%3, %4}], [%2], %5;"
        ::"r"(dst), "l"(tmap), "r"(bar), "r"(c0), "r"(c1), "l"(policy)
        : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const void* tmap, uint32_t bar, int c0,
                                            int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(tmap), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}
__device__ __forceinline__ void tma_load_3d_hint(uint32_t dst, const void* tmap, uint32_t bar,
                                                 int c0, int c1, int c2, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
        ".L2::cache_hint [%0], [%1, {%3, %4, %5}], [%2], %6;"
        ::"r"(dst), "l"(tmap), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "l"(policy)
        : "memory");
}
// Untiled bulk copy; both addresses 16-byte aligned, size a multiple of 16.
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes,
                                          uint32_t bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
        : "memory");
}
__device__ __forceinline__ void prefetch_tmap(const void* tmap) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}
__device__ __forceinline__ uint64_t policy_evict_first() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ uint64_t policy_evict_last() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
    return p;
}

// ---------------------------------------------------------------- tcgen05 / TMEM
// One warp allocates `cols` (power of two, >= 32) TMEM columns; the base address is
// written to shared memory at `dst_smem`.
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem),
                 "r"(cols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols)
                 : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// Arrive (count 1) on an mbarrier once every UMMA issued so far by this thread is done.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                     bar)
                 : "memory");
}
// D[tmem] (+)= A[smem] * B[smem], 8-bit float operands (format in the descriptor).
__device__ __forceinline__ void umma_f8f6f4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                            uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t"
        "}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// D[tmem] (+)= A[smem] * B[smem], bf16/fp16 operands.
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                         uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Block-scaled 4-bit float MMA: 16-element ue4m3 scale vectors read from TMEM.
// The same with operand A in tensor memory: row i of A in lane i, two 16-bit K elements per
// 32-bit column starting at `a_tmem` (8 columns per K step of 16).
__device__ __forceinline__ void umma_f16_ta(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
        "}\n"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ void umma_nvf4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                          uint32_t idesc, uint32_t sfa_tmem, uint32_t sfb_tmem,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X "
        "[%0], %1, %2, %3, [%5], [%6], p;\n\t"
        "}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem),
        "r"(sfb_tmem)
        : "memory");
}
// Shared memory -> TMEM copy of scale factors: 32 lanes x 128 bits, replicated to the
// four lane quarters.
__device__ __forceinline__ void tmem_cp_32x128b_warpx4(uint32_t taddr, uint64_t s_desc) {
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(s_desc)
                 : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns: thread i of the warp receives lane
// (warp%4)*32+i, columns [col, col+32).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
          "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
          "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_32x8(uint32_t taddr, uint32_t (&r)[8]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
        : "r"(taddr)
        : "memory");
}

// Warp-wide wait whose common case (phase already complete) costs one poll and one
// vote: all lanes test the barrier together; only when that fails does lane 0 take the
// polling loop and broadcast the outcome.
__device__ __forceinline__ bool mbar_wait_warp_fast(uint32_t bar, uint32_t parity,
                                                    volatile int* abort_flag, int* status_word,
                                                    int code) {
    if (__all_sync(0xffffffffu, mbar_try_wait(bar, parity))) return true;
    return mbar_wait_lane0(bar, parity, abort_flag, status_word, code);
}

__device__ __forceinline__ void tmem_ld_wait() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// The store twin of tmem_ld_32x32: thread i of the warp writes lane (warp%4)*32+i,
// columns [col, col+32).
__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() {
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// ---------------------------------------------------------------- descriptors
// Shared-memory matrix descriptor for a K-major operand whose rows are exactly one
// 128-byte swizzle span (TMA SWIZZLE_128B layout): 8-row groups 1024 bytes apart.
// `addr` is a shared-memory byte address; the tile base must be 1024-byte aligned, and
// stepping K by 32 bytes inside the span is done by adding to `addr`.
__host__ __device__ constexpr uint64_t umma_smem_desc_sw128(uint32_t addr) {
    return (static_cast<uint64_t>((addr & 0x3FFFFu) >> 4))        // start address
           | (static_cast<uint64_t>(0) << 16)                      // leading byte offset (unused)
           | (static_cast<uint64_t>(1024 >> 4) << 32)              // stride byte offset
           | (static_cast<uint64_t>(1) << 46)                      // descriptor version (sm_100)
           | (static_cast<uint64_t>(2) << 61);                     // SWIZZLE_128B
}

// Unswizzled K-major descriptor: 8x16-byte core matrices; `lbo` = byte distance between
// core matrices adjacent in K, `sbo` = between core matrices adjacent in M/N.
__host__ __device__ constexpr uint64_t umma_smem_desc_noswz(uint32_t addr, uint32_t lbo,
                                                            uint32_t sbo) {
    return (static_cast<uint64_t>((addr & 0x3FFFFu) >> 4)) |
           (static_cast<uint64_t>(lbo >> 4) << 16) | (static_cast<uint64_t>(sbo >> 4) << 32) |
           (static_cast<uint64_t>(1) << 46);
}

// MN-major operand in the 128-byte swizzle: 64 consecutive M/N elements of 16 bits form one
// 128-byte row, 8 rows (8 steps of K) form a 1024-byte group.  `lbo` = byte distance between
// blocks of 64 M/N elements, the groups of 8 K steps are 1024 bytes apart.  The bytes are
// arranged exactly as in the K-major form with the roles of the two dimensions exchanged.
__host__ __device__ constexpr uint64_t umma_smem_desc_mn_sw128(uint32_t addr, uint32_t lbo) {
    return (static_cast<uint64_t>((addr & 0x3FFFFu) >> 4)) | (static_cast<uint64_t>(lbo >> 4) << 16) |
           (static_cast<uint64_t>(1024 >> 4) << 32) | (static_cast<uint64_t>(1) << 46) |
           (static_cast<uint64_t>(2) << 61);
}

// Instruction descriptor, dense, fp32 accumulate, both operands K-major.
// fmt: kind::f8f6f4 -> 0 e4m3, 1 e5m2, 5 e2m1; kind::f16 -> 0 f16, 1 bf16.
__host__ __device__ constexpr uint32_t umma_idesc(uint32_t m, uint32_t n, uint32_t a_fmt,
                                                  uint32_t b_fmt) {
    return (1u << 4) | (a_fmt << 7) | (b_fmt << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}
// The same with operand B MN-major (its N dimension contiguous in shared memory).
__host__ __device__ constexpr uint32_t umma_idesc_b_mn(uint32_t m, uint32_t n, uint32_t a_fmt, uint32_t b_fmt) {
    return umma_idesc(m, n, a_fmt, b_fmt) | (1u << 16);
}
// Block-scaled variant (kind::mxf4nvf4): scale format bit 23 (0 ue4m3, 1 ue8m0), scale
// ids select which byte column of the TMEM scale words is used.
__host__ __device__ constexpr uint32_t umma_idesc_block_scaled(uint32_t m, uint32_t n,
                                                               uint32_t a_fmt, uint32_t b_fmt,
                                                               uint32_t scale_fmt, uint32_t a_sf_id,
                                                               uint32_t b_sf_id) {
    return (b_sf_id << 4) | (a_fmt << 7) | (b_fmt << 10) | ((n >> 3) << 17) | (scale_fmt << 23) |
           ((m >> 4) << 24) | (a_sf_id << 29);
}

}  // namespace wuda
