// Exact per-row top-k index selection over fp32 scores, followed by the page-table
// transform, for sm_100a.
//
// Contract (dsv4_megakernel/megakernel/kernels/topk_v2.cu:329-439 and
// test/test_topk_v2.py:86-135): for each row r the indices of the k largest values of
// scores[r, 0:seq_len[r]], in no particular order; rows with seq_len <= k give
// [0..n) followed by -1; page_indices = (page_table[r, i >> bits] << bits) | (i & mask).
// Equal values are resolved towards the LOWER index, so the selected set is exactly
// torch.argsort(-scores, stable=True)[:k] - stricter than the reference, which leaves the
// choice among exact duplicates unspecified.  The order of a row's output is a function of
// the row alone (no atomics decide a position), so a rerun writes the same bytes.
//
// A row is the work of one CTA of 512 threads, or of a cluster of two (rows beyond 16 K
// scores while the device has room: two CTAs fit an SM, so 128 rows keep all 148 SMs busy
// and the longest row's scan is halved).
//
// Fast path (n >= 4k): 2048 evenly spaced samples give a 12-bit key digit that bounds the
// k-th value from below with a 5-sigma margin.  ONE pass over the row then parks every
// element at or above it - a few hundred more than k - as (key, index) pairs in the lead
// CTA's shared memory: every warp owns a segment of the candidate list and compacts into
// it with one ballot per 32 elements, no atomics and no scans; the second CTA of a cluster
// writes its segments through distributed shared memory.  Among the candidates one
// 4096-bin histogram of (key - key_lo) >> 12 resolves 20 key bits; the handful of
// candidates in the threshold bin are then ranked exactly by (key, lower index first), which
// also settles ties: the first of them take the last output positions, the candidates above the bin the
// positions before, from per-segment prefix sums.  The row's page-table entries wait in shared memory.
//
// Exact path (short rows, a sample that misled, duplicates by the thousand): a three-level
// radix select (12 + 12 + 8 key bits) with one pass over the row per level and an ordered
// emit pass, by the lead CTA alone.
//
// No global scratch memory is used and nothing is allocated.
#include <cooperative_groups.h>
#include <cuda_runtime.h>

#include "host.h"

namespace wuda {
namespace topk {

constexpr int kThreads = 512;
constexpr int kWarps = kThreads / 32;
constexpr int kBins = 4096;
constexpr int kCandCap = 8192;
constexpr int kSamples = 2048;
constexpr int kTieCap = 2048;       // candidates of the threshold bin that are ranked exactly in shared memory
constexpr int kPairwiseMax = 128;   // up to this many they are ranked by counting (quadratic); more are sorted
constexpr int kMaxCluster = 2;
constexpr int kMaxSeg = kMaxCluster * kWarps;
constexpr int kLoadBatch = 4;       // 16-byte loads in flight per thread in the scan (more only queue up in the L2)
constexpr int kPageCache = 1024;    // page-table entries of a row kept in shared memory (64 K scores at 64 per page)

struct Params {
    const float* scores;
    const int32_t* seq_lens;
    const int32_t* page_table;
    int32_t* page_indices;
    int32_t* raw;
    int64_t score_stride;
    int64_t pt_stride;
    int rows;
    int k;
    int page_bits;
    int rows_per_table_row;
};

__device__ __forceinline__ uint32_t key_of(float x) {
    uint32_t u = __float_as_uint(x);
    if (u == 0x80000000u) u = 0u;  // -0 and +0 compare equal
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ __forceinline__ float float_of_key(uint32_t key) {   // inverse of key_of
    return __uint_as_float((key & 0x80000000u) ? (key & 0x7FFFFFFFu) : ~key);
}

// Bin i of the histogram lives at word i + (i >> 5): a thread's run of 8 consecutive bins and the runs of the
// 31 other lanes then fall into 32 different banks (unpadded, every fourth lane would collide).
__device__ __forceinline__ int hslot(uint32_t bin) { return static_cast<int>(bin + (bin >> 5)); }

struct Shared {
    uint32_t hist[kBins + kBins / 32];
    uint2 cand[kCandCap];            // (key, index)
    unsigned long long tie[kTieCap];   // (key << 32) | ~index: larger = larger key, then lower index; all distinct
    int32_t pages[kPageCache];       // the row's page-table entries
    uint32_t seg_cnt[kMaxSeg];
    uint32_t seg_off[kMaxSeg];
    uint32_t warp_tot[kWarps];
    uint32_t warp_excl[kWarps];
    uint32_t sel_digit, sel_above, sel_count;
    uint32_t tie_count;
    uint32_t total;
    int pages_cached;
};

__device__ __forceinline__ void zero_hist(Shared& s, int nbins) {
    for (int i = threadIdx.x; i < nbins + nbins / 32; i += kThreads) s.hist[i] = 0;
}

// Finds the digit T with  count(digit > T) < need <= count(digit >= T)  and leaves T in
// s.sel_digit, count(digit > T) in s.sel_above and count(digit == T) in s.sel_count.
// Needs 1 <= need <= total and nbins a multiple of 32 * kWarps or at most 256.  Two barriers: every
// warp sums its run of bins (thread = a few consecutive bins), all warps then read the 16 warp totals,
// and the one warp whose run holds the threshold locates it with a shuffle scan.  The histogram must be
// complete on entry (caller's barrier) and is unchanged on exit.
__device__ __forceinline__ void find_threshold(Shared& s, int nbins, uint32_t need) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int per = nbins >= kThreads ? nbins / kThreads : 1;     // bins per thread
    const int lo = threadIdx.x * per;
    uint32_t h[kBins / kThreads];
    uint32_t local = 0;
#pragma unroll
    for (int b = 0; b < kBins / kThreads; ++b) {
        h[b] = (b < per && lo + b < nbins) ? s.hist[hslot(lo + b)] : 0u;
        local += h[b];
    }
    uint32_t v = local;   // suffix sums inside the warp: v = sum of `local` over lanes >= this one
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t t = __shfl_down_sync(0xffffffffu, v, o);
        if (lane + o < 32) v += t;
    }
    if (lane == 0) s.warp_tot[warp] = v;
    __syncthreads();
    uint32_t above = 0;   // count in the bins of the warps behind this one (higher digits)
#pragma unroll
    for (int w = 0; w < kWarps; ++w) above += w > warp ? s.warp_tot[w] : 0u;
    uint32_t running = above + v - local;   // count in digits above this thread's bins
#pragma unroll
    for (int b = kBins / kThreads - 1; b >= 0; --b) {
        if (running < need && need <= running + h[b]) {      // true for exactly one (thread, b)
            s.sel_digit = lo + b;
            s.sel_above = running;
            s.sel_count = h[b];
        }
        running += h[b];
    }
    __syncthreads();
}

// Exclusive prefix sum of `count` over the CTA's threads (thread order) and the CTA total.  Three barriers.
__device__ __forceinline__ uint32_t block_exclusive_scan(Shared& s, uint32_t count, uint32_t* total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    uint32_t v = count;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t t = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += t;
    }
    __syncthreads();                                  // the arrays below may still be read from an earlier scan
    if (lane == 31) s.warp_tot[warp] = v;
    __syncthreads();
    if (warp == 0) {
        const uint32_t tot = lane < kWarps ? s.warp_tot[lane] : 0u;
        uint32_t w = tot;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t t = __shfl_up_sync(0xffffffffu, w, o);
            if (lane >= o) w += t;
        }
        if (lane < kWarps) s.warp_excl[lane] = w - tot;
        if (lane == 31) s.total = w;
    }
    __syncthreads();
    *total = s.total;
    return v - count + s.warp_excl[warp];
}

__device__ __forceinline__ int32_t page_of(const Params& p, int r, int idx) {
    if (!p.page_table) return idx;
    const int32_t page =
        __ldg(p.page_table + static_cast<int64_t>(r / p.rows_per_table_row) * p.pt_stride + (idx >> p.page_bits));
    return static_cast<int32_t>((static_cast<uint32_t>(page) << p.page_bits) |
                                static_cast<uint32_t>(idx & ((1 << p.page_bits) - 1)));
}

__device__ __forceinline__ void put(const Params& p, int r, uint32_t pos, int idx) {
    if (pos < static_cast<uint32_t>(p.k)) {
        const int64_t o = static_cast<int64_t>(r) * p.k + pos;
        if (p.raw) p.raw[o] = idx;
        p.page_indices[o] = page_of(p, r, idx);
    }
}

// f(index, value, valid) for every element of the row, every thread making the same number of calls.
template <typename F>
__device__ __forceinline__ void for_each_elem(const float* row, int n, bool vec_ok, F f) {
    if (vec_ok) {
        const int n4 = n >> 2;
        const float4* row4 = reinterpret_cast<const float4*>(row);
        for (int base = 0; base < n4; base += kThreads * 4) {
            float4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int i = base + u * kThreads + threadIdx.x;
                v[u] = i < n4 ? __ldcg(row4 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int i = base + u * kThreads + threadIdx.x;
                const bool valid = i < n4;
                f(4 * i + 0, v[u].x, valid);
                f(4 * i + 1, v[u].y, valid);
                f(4 * i + 2, v[u].z, valid);
                f(4 * i + 3, v[u].w, valid);
            }
        }
        const int i = (n4 << 2) + threadIdx.x;   // at most 3 leftover elements
        if ((n & 3) != 0) f(i, i < n ? __ldcg(row + i) : 0.f, i < n);
    } else {
        for (int base = 0; base < n; base += kThreads) {
            const int i = base + threadIdx.x;
            f(i, i < n ? __ldcg(row + i) : 0.f, i < n);
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Exact path: three histogram levels over the whole row, then one ordered pass that writes the
// values above the threshold and the lowest-indexed `need3` of those equal to it.  One CTA.
__device__ void exact_select(const Params& p, Shared& s, const float* row, int n, int r, bool vec_ok) {
    const int k = p.k;
    zero_hist(s, kBins);
    __syncthreads();
    for_each_elem(row, n, vec_ok, [&](int, float x, bool valid) {
        if (valid) atomicAdd(&s.hist[hslot(key_of(x) >> 20)], 1u);
    });
    __syncthreads();
    find_threshold(s, kBins, static_cast<uint32_t>(k));
    const uint32_t d1 = s.sel_digit;
    const uint32_t need1 = static_cast<uint32_t>(k) - s.sel_above;
    __syncthreads();
    zero_hist(s, kBins);
    __syncthreads();
    for_each_elem(row, n, vec_ok, [&](int, float x, bool valid) {
        const uint32_t key = key_of(x);
        if (valid && (key >> 20) == d1) atomicAdd(&s.hist[hslot((key >> 8) & 0xFFFu)], 1u);
    });
    __syncthreads();
    find_threshold(s, kBins, need1);
    const uint32_t prefix24 = (d1 << 12) | s.sel_digit;
    const uint32_t need2 = need1 - s.sel_above;
    __syncthreads();
    zero_hist(s, 256);
    __syncthreads();
    for_each_elem(row, n, vec_ok, [&](int, float x, bool valid) {
        const uint32_t key = key_of(x);
        if (valid && (key >> 8) == prefix24) atomicAdd(&s.hist[hslot(key & 0xFFu)], 1u);
    });
    __syncthreads();
    find_threshold(s, 256, need2);
    const uint32_t thr = (prefix24 << 8) | s.sel_digit;
    const uint32_t need3 = need2 - s.sel_above;      // values equal to thr still taken: the lowest indices
    __syncthreads();
    // ordered emit: thread t owns the contiguous chunk [beg, end)
    const int chunk = (n + kThreads - 1) / kThreads;
    const int beg = min(n, static_cast<int>(threadIdx.x) * chunk), end = min(n, beg + chunk);
    uint32_t gt = 0, eq = 0;
    for (int i = beg; i < end; ++i) {
        const uint32_t key = key_of(__ldcg(row + i));
        gt += key > thr;
        eq += key == thr;
    }
    uint32_t total_gt, total_eq;
    uint32_t at_gt = block_exclusive_scan(s, gt, &total_gt);
    uint32_t at_eq = block_exclusive_scan(s, eq, &total_eq);
    for (int i = beg; i < end; ++i) {
        const uint32_t key = key_of(__ldcg(row + i));
        if (key > thr) put(p, r, at_gt++, i);
        else if (key == thr) {
            if (at_eq < need3) put(p, r, total_gt + at_eq, i);
            ++at_eq;
        }
    }
}

// ---------------------------------------------------------------------------------------------
// One ballot per 32 elements: the lanes whose value is a candidate store (key, index) at the warp's
// running count plus their rank among the lanes below them.
__device__ __forceinline__ void park(bool pred, float x, int idx, uint2* seg, uint32_t segcap, uint32_t lane_lt,
                                     uint32_t& cnt) {
    const uint32_t b = __ballot_sync(0xffffffffu, pred);
    if (pred) {
        const uint32_t pos = cnt + __popc(b & lane_lt);
        if (pos < segcap) seg[pos] = make_uint2(key_of(x), static_cast<uint32_t>(idx));
    }
    cnt += __popc(b);
}

// Four elements per lane: the four ballots and their counts are independent of each other, so they overlap;
// only the running count links one call to the next.
__device__ __forceinline__ void park4(bool valid, const float4& v, int i4, float x_lo, uint2* seg, uint32_t segcap,
                                      uint32_t lane_lt, uint32_t& cnt) {
    const bool p0 = valid && v.x >= x_lo, p1 = valid && v.y >= x_lo, p2 = valid && v.z >= x_lo, p3 = valid && v.w >= x_lo;
    const uint32_t b0 = __ballot_sync(0xffffffffu, p0), b1 = __ballot_sync(0xffffffffu, p1);
    const uint32_t b2 = __ballot_sync(0xffffffffu, p2), b3 = __ballot_sync(0xffffffffu, p3);
    const uint32_t at0 = cnt, at1 = at0 + __popc(b0), at2 = at1 + __popc(b1), at3 = at2 + __popc(b2);
    cnt = at3 + __popc(b3);
    const uint32_t idx = 4u * static_cast<uint32_t>(i4);
    if (p0) {
        const uint32_t pos = at0 + __popc(b0 & lane_lt);
        if (pos < segcap) seg[pos] = make_uint2(key_of(v.x), idx);
    }
    if (p1) {
        const uint32_t pos = at1 + __popc(b1 & lane_lt);
        if (pos < segcap) seg[pos] = make_uint2(key_of(v.y), idx + 1);
    }
    if (p2) {
        const uint32_t pos = at2 + __popc(b2 & lane_lt);
        if (pos < segcap) seg[pos] = make_uint2(key_of(v.z), idx + 2);
    }
    if (p3) {
        const uint32_t pos = at3 + __popc(b3 & lane_lt);
        if (pos < segcap) seg[pos] = make_uint2(key_of(v.w), idx + 3);
    }
}

// Output position `pos` of row r gets index idx, translated with the row's page table: from the copy in shared
// memory when the row's pages fit it (s.pages_cached), else from global memory.
__device__ __forceinline__ void put_cached(const Params& p, const Shared& s, int r, uint32_t pos, int idx) {
    if (pos >= static_cast<uint32_t>(p.k)) return;
    const int64_t o = static_cast<int64_t>(r) * p.k + pos;
    if (p.raw) p.raw[o] = idx;
    int32_t out = idx;
    if (p.page_table) {
        const int pg = idx >> p.page_bits;
        const int32_t page = pg < s.pages_cached
                                 ? s.pages[pg]
                                 : __ldg(p.page_table + static_cast<int64_t>(r / p.rows_per_table_row) * p.pt_stride + pg);
        out = static_cast<int32_t>((static_cast<uint32_t>(page) << p.page_bits) |
                                   static_cast<uint32_t>(idx & ((1 << p.page_bits) - 1)));
    }
    p.page_indices[o] = out;
}

__global__ void __launch_bounds__(kThreads, 2) topk_kernel(const Params p) {
    extern __shared__ uint8_t smem_raw[];
    Shared& s = *reinterpret_cast<Shared*>(smem_raw);
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    const int crank = static_cast<int>(cluster.block_rank());
    const int csize = static_cast<int>(cluster.num_blocks());
    Shared& lead = *cluster.map_shared_rank(&s, 0);   // the lead CTA's shared memory
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t lane_lt = (1u << lane) - 1u;
    const int k = p.k;
    // shared memory only, so it may run while the kernel ahead is still finishing
    zero_hist(s, kBins);
    if (threadIdx.x == 0) s.tie_count = 0;
    pdl_launch_dependents();
    pdl_wait();   // nothing of global memory is touched before the kernel ahead has finished
    bool clean = true;   // the histogram and the tie counter are zero

    for (int r = blockIdx.x / csize; r < p.rows; r += gridDim.x / csize) {
        const float* row = p.scores + static_cast<int64_t>(r) * p.score_stride;
        int n = p.seq_lens[r];
        n = n < 0 ? 0 : n;
        if (static_cast<int64_t>(n) > p.score_stride) n = static_cast<int>(p.score_stride);

        if (n <= k) {  // everything is selected: [0..n) then -1
            if (crank == 0)
                for (int i = threadIdx.x; i < k; i += kThreads) {
                    const int64_t o = static_cast<int64_t>(r) * k + i;
                    const int idx = i < n ? i : -1;
                    if (p.raw) p.raw[o] = idx;
                    p.page_indices[o] = idx >= 0 ? page_of(p, r, idx) : -1;
                }
            continue;   // (no shared memory was touched: no cluster barrier needed)
        }
        const bool vec_ok = ((reinterpret_cast<uintptr_t>(row) & 15u) == 0);
        bool done = false;

        // expected sample rank of the k-th value, plus a 5-sigma margin, and the candidates that bound would let through
        const float expect = static_cast<float>(kSamples) * static_cast<float>(k) / static_cast<float>(n);
        uint32_t rank = static_cast<uint32_t>(expect + 5.f * sqrtf(expect) + 8.f);
        if (rank > static_cast<uint32_t>(kSamples)) rank = kSamples;
        const float expected_candidates = static_cast<float>(rank) * static_cast<float>(n) / static_cast<float>(kSamples);
        if (2 * k <= kCandCap && expected_candidates <= 0.75f * kCandCap) {
            // ---------------------------------------------------------------- fast path
            if (!clean) {
                zero_hist(s, kBins);
                if (threadIdx.x == 0) s.tie_count = 0;
            }
            // every CTA of the cluster takes the same samples and finds the same bound; the lead CTA also
            // fetches the row's page-table entries, which the emit at the end then finds in shared memory
            // (an aligned row is sampled in 512 evenly spaced groups of four neighbours - one 16-byte load per
            // thread; neighbours that move together only widen the margin's miss rate, and a miss is caught)
            float v[kSamples / kThreads];
            if (vec_ok) {
                const int at = static_cast<int>(static_cast<long long>(threadIdx.x) * (n >> 2) / kThreads);
                const float4 q = __ldcg(reinterpret_cast<const float4*>(row) + at);
                v[0] = q.x, v[1] = q.y, v[2] = q.z, v[3] = q.w;
            } else {
#pragma unroll
                for (int j = 0; j < kSamples / kThreads; ++j) {
                    const int t = threadIdx.x + j * kThreads;
                    v[j] = __ldcg(row + static_cast<int>(static_cast<long long>(t) * n / kSamples));
                }
            }
            if (crank == 0 && p.page_table) {
                const int pages = min(kPageCache, ((n - 1) >> p.page_bits) + 1);
                const int32_t* table = p.page_table + static_cast<int64_t>(r / p.rows_per_table_row) * p.pt_stride;
                for (int i = threadIdx.x; i < pages; i += kThreads) s.pages[i] = __ldg(table + i);
                if (threadIdx.x == 0) s.pages_cached = pages;
            }
            __syncthreads();                          // the zeroes are in place
#pragma unroll
            for (int j = 0; j < kSamples / kThreads; ++j) atomicAdd(&s.hist[hslot(key_of(v[j]) >> 20)], 1u);
            __syncthreads();
            find_threshold(s, kBins, rank);
            const uint32_t key_lo = s.sel_digit << 20;
            // digit >= d_lo  <=>  key >= key_lo  <=>  x >= the float with that key: one compare per element
            // (an unordered bound selects nothing and the row falls back to the exact path)
            const float x_lo = float_of_key(key_lo);
            zero_hist(s, kBins);                    // level A's histogram (the lead CTA's is the one used); the
                                                    // barrier at the end of the scan covers it
            // ---- the scan: this CTA's slice of the row, candidates into this warp's segment of the lead's list
            const int nseg = csize * kWarps;
            const uint32_t segcap = kCandCap / nseg;
            const int seg = crank * kWarps + warp;
            uint2* seg_ptr = lead.cand + seg * segcap;
            uint32_t cnt = 0;
            const int slice = ((n + csize - 1) / csize + 3) & ~3;
            const int lo = min(n, crank * slice), hi = min(n, lo + slice);
            if (vec_ok) {
                // two half-batches of loads are always in flight: the next is issued before the current is used
                const int hi4 = hi >> 2;             // full 16-byte groups end here (hi is a multiple of 4, or n)
                const float4* row4 = reinterpret_cast<const float4*>(row);
                constexpr int kHalf = kLoadBatch / 2;
                const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
                float4 a[kHalf], b[kHalf];
                int base = (lo >> 2) + threadIdx.x;
#pragma unroll
                for (int u = 0; u < kHalf; ++u) a[u] = base + u * kThreads < hi4 ? __ldcg(row4 + base + u * kThreads) : zero4;
                while (base - static_cast<int>(threadIdx.x) < hi4) {
                    const int next = base + kHalf * kThreads;
#pragma unroll
                    for (int u = 0; u < kHalf; ++u) b[u] = next + u * kThreads < hi4 ? __ldcg(row4 + next + u * kThreads) : zero4;
#pragma unroll
                    for (int u = 0; u < kHalf; ++u) {
                        const int i = base + u * kThreads;
                        park4(i < hi4, a[u], i, x_lo, seg_ptr, segcap, lane_lt, cnt);
                    }
                    const int next2 = next + kHalf * kThreads;
#pragma unroll
                    for (int u = 0; u < kHalf; ++u) a[u] = next2 + u * kThreads < hi4 ? __ldcg(row4 + next2 + u * kThreads) : zero4;
#pragma unroll
                    for (int u = 0; u < kHalf; ++u) {
                        const int i = next + u * kThreads;
                        park4(i < hi4, b[u], i, x_lo, seg_ptr, segcap, lane_lt, cnt);
                    }
                    base = next2;
                }
                if (hi == n && lo < hi && (n & 3) != 0 && warp == 0) {   // at most 3 leftover elements, by the last slice's warp 0
                    const int i = (hi4 << 2) + lane;
                    const float x = i < n ? __ldcg(row + i) : 0.f;
                    park(i < n && x >= x_lo, x, i, seg_ptr, segcap, lane_lt, cnt);
                }
            } else {
                for (int base = lo; base < hi; base += kThreads) {
                    const int i = base + threadIdx.x;
                    const float x = i < hi ? __ldcg(row + i) : 0.f;
                    park(i < hi && x >= x_lo, x, i, seg_ptr, segcap, lane_lt, cnt);
                }
            }
            if (lane == 0) lead.seg_cnt[seg] = cnt;
            if (csize > 1) cluster.sync();           // every slice is parked, every count is in
            else __syncthreads();
            clean = false;

            if (crank == 0) {
                // ---- the selection among the candidates, by the lead CTA
                const uint32_t mine = lane < nseg ? s.seg_cnt[lane] : 0u;     // every warp adds the counts up by itself
                uint32_t total = mine;
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
                bool ok = __all_sync(0xffffffffu, mine <= segcap) && total >= static_cast<uint32_t>(k);
                if (ok) {
                    // level A: 20 key bits at once over the candidates' window
                    for (int g = warp; g < nseg; g += kWarps) {
                        const uint32_t c = s.seg_cnt[g];
                        const uint2* cands = s.cand + g * segcap;
                        for (uint32_t j = lane; j < c; j += 32)
                            atomicAdd(&s.hist[hslot(min((cands[j].x - key_lo) >> 12, static_cast<uint32_t>(kBins - 1)))], 1u);
                    }
                    __syncthreads();
                    find_threshold(s, kBins, static_cast<uint32_t>(k));
                    // A candidate's class is (key - sub) >> shift compared with thr: the window's bin, or - when the
                    // threshold lies beyond the window - the key's upper 24 bits.
                    uint32_t sub = key_lo, shift = 12;
                    uint32_t bin_a = s.sel_digit;
                    uint32_t above_a = s.sel_above;
                    uint32_t c_a = s.sel_count;
                    if (bin_a == static_cast<uint32_t>(kBins - 1)) {
                        // The window (2^24 keys above the bound: two binades of one sign) does not reach the k-th value:
                        // the sample's bound lies several binades below it, or on the other side of zero, where keys
                        // are sparse.  Two exact levels over the candidates instead of the whole row: the key's upper 12
                        // bits (counted from the bound's), then the next 12 inside that digit.
                        const uint32_t d_lo = key_lo >> 20;
                        __syncthreads();
                        zero_hist(s, kBins);
                        __syncthreads();
                        for (int g = warp; g < nseg; g += kWarps) {
                            const uint32_t c = s.seg_cnt[g];
                            const uint2* cands = s.cand + g * segcap;
                            for (uint32_t j = lane; j < c; j += 32) atomicAdd(&s.hist[hslot((cands[j].x >> 20) - d_lo)], 1u);
                        }
                        __syncthreads();
                        find_threshold(s, kBins, static_cast<uint32_t>(k));
                        const uint32_t digit = d_lo + s.sel_digit, above_1 = s.sel_above;
                        __syncthreads();
                        zero_hist(s, kBins);
                        __syncthreads();
                        for (int g = warp; g < nseg; g += kWarps) {
                            const uint32_t c = s.seg_cnt[g];
                            const uint2* cands = s.cand + g * segcap;
                            for (uint32_t j = lane; j < c; j += 32)
                                if ((cands[j].x >> 20) == digit) atomicAdd(&s.hist[hslot((cands[j].x >> 8) & 0xFFFu)], 1u);
                        }
                        __syncthreads();
                        find_threshold(s, kBins, static_cast<uint32_t>(k) - above_1);
                        sub = 0, shift = 8;
                        bin_a = (digit << 12) | s.sel_digit;
                        above_a = above_1 + s.sel_above;
                        c_a = s.sel_count;
                    }
                    const uint32_t need_a = static_cast<uint32_t>(k) - above_a;
                    // a class with thousands of members is a row of duplicates: the exact path
                    ok = c_a <= static_cast<uint32_t>(kTieCap);
                    if (ok) {
                        // One walk over the candidates: those above the threshold bin are counted per segment,
                        // the bin's own members go to the tie list.
                        for (int g = warp; g < nseg; g += kWarps) {
                            const uint32_t c = s.seg_cnt[g];
                            uint32_t sel = 0;
                            for (uint32_t j0 = 0; j0 < c; j0 += 32) {
                                const uint32_t j = j0 + lane;
                                const uint2 cand = j < c ? s.cand[g * segcap + j] : make_uint2(key_lo, 0u);
                                const uint32_t key = cand.x;
                                const uint32_t bin = (key - sub) >> shift;
                                sel += __popc(__ballot_sync(0xffffffffu, j < c && bin > bin_a));
                                const bool in = j < c && bin == bin_a;
                                const uint32_t b = __ballot_sync(0xffffffffu, in);
                                if (b != 0) {
                                    uint32_t at = 0;
                                    if (lane == __ffs(b) - 1) at = atomicAdd(&s.tie_count, __popc(b));
                                    at = __shfl_sync(0xffffffffu, at, __ffs(b) - 1) + __popc(b & lane_lt);
                                    if (in) s.tie[at] = (static_cast<unsigned long long>(key) << 32) | (~cand.y);
                                }
                            }
                            if (lane == 0) s.seg_off[g] = sel;
                        }
                        __syncthreads();
                        // The bin's members ranked exactly - larger key first, lower index first among equals: the
                        // first need_a of them take the last output positions.  A few dozen (the usual case) are
                        // ranked by counting, each against all; a bin with hundreds of members (values crowded into
                        // a few binades, runs of equal scores) is sorted instead: counting is quadratic.
                        if (c_a <= static_cast<uint32_t>(kPairwiseMax)) {
                            for (uint32_t t = threadIdx.x; t < c_a; t += kThreads) {
                                const unsigned long long mine_t = s.tie[t];
                                uint32_t ahead = 0;
                                for (uint32_t j = 0; j < c_a; ++j) ahead += s.tie[j] > mine_t;
                                if (ahead < need_a) put_cached(p, s, r, above_a + ahead, static_cast<int>(~static_cast<uint32_t>(mine_t)));
                            }
                        } else {
                            uint32_t pow2 = 2u * kPairwiseMax;
                            while (pow2 < c_a) pow2 <<= 1;
                            for (uint32_t t = c_a + threadIdx.x; t < pow2; t += kThreads) s.tie[t] = 0ull;   // below every real entry
                            __syncthreads();
                            for (uint32_t size = 2; size <= pow2; size <<= 1)
                                for (uint32_t stride = size >> 1; stride > 0; stride >>= 1) {
                                    for (uint32_t t = threadIdx.x; t < pow2 / 2; t += kThreads) {
                                        const uint32_t a = 2u * t - (t & (stride - 1u)), b = a + stride;   // bitonic network, descending
                                        const unsigned long long va = s.tie[a], vb = s.tie[b];
                                        const bool descending = (a & size) == 0u;
                                        if ((va < vb) == descending) {
                                            s.tie[a] = vb;
                                            s.tie[b] = va;
                                        }
                                    }
                                    __syncthreads();
                                }
                            for (uint32_t t = threadIdx.x; t < need_a; t += kThreads)
                                put_cached(p, s, r, above_a + t, static_cast<int>(~static_cast<uint32_t>(s.tie[t])));
                        }
                        for (int g = warp; g < nseg; g += kWarps) {
                            uint32_t at = lane < g ? s.seg_off[lane] : 0u;       // positions taken by the segments before
#pragma unroll
                            for (int o = 16; o > 0; o >>= 1) at += __shfl_xor_sync(0xffffffffu, at, o);
                            const uint32_t c = s.seg_cnt[g];
                            for (uint32_t j0 = 0; j0 < c; j0 += 32) {
                                const uint32_t j = j0 + lane;
                                const uint2 cand = j < c ? s.cand[g * segcap + j] : make_uint2(key_lo, 0u);
                                const bool in = j < c && ((cand.x - sub) >> shift) > bin_a;
                                const uint32_t b = __ballot_sync(0xffffffffu, in);
                                if (in) put_cached(p, s, r, at + __popc(b & lane_lt), static_cast<int>(cand.y));
                                at += __popc(b);
                            }
                        }
                        done = true;
                    }
                }
                __syncthreads();
            }
        }
        if (!done && crank == 0) {
            exact_select(p, s, row, n, r, vec_ok);
            clean = false;
        }
        // the next row's candidates must not land in the lead's list while it is still being read
        if (csize > 1) cluster.sync();
        else __syncthreads();
    }
}

}  // namespace topk
}  // namespace wuda

extern "C" int wuda_topk(const float* scores, const int32_t* seq_lens, const int32_t* page_table,
                         int32_t* page_indices, int32_t* raw_indices, int rows, int64_t score_stride,
                         int64_t page_table_stride, int rows_per_table_row, int k, int page_size,
                         void* stream) {
    using namespace wuda;
    using namespace wuda::topk;
    clear_error();
    WUDA_REQUIRE(rows >= 0, "rows must be >= 0 (got %d)", rows);
    WUDA_REQUIRE(k >= 1, "k must be >= 1 (got %d)", k);
    WUDA_REQUIRE(page_size >= 1 && (page_size & (page_size - 1)) == 0, "page_size must be a power of two (got %d)",
                 page_size);
    WUDA_REQUIRE(score_stride >= 1, "score_stride must be >= 1");
    WUDA_REQUIRE(rows_per_table_row >= 1, "rows_per_table_row must be >= 1 (got %d)", rows_per_table_row);
    if (rows == 0) return WUDA_OK;
    WUDA_REQUIRE(scores && seq_lens && page_indices, "scores, seq_lens and page_indices must not be NULL");
    WUDA_REQUIRE(!page_table || page_table_stride >= 1, "page_table_stride must be >= 1");

    DeviceInfo dev;
    int st = current_device_info(&dev);
    if (st != WUDA_OK) return st;

    Params p;
    p.scores = scores;
    p.seq_lens = seq_lens;
    p.page_table = page_table;
    p.page_indices = page_indices;
    p.raw = raw_indices;
    p.score_stride = score_stride;
    p.pt_stride = page_table_stride;
    p.rows = rows;
    p.k = k;
    p.rows_per_table_row = rows_per_table_row;
    p.page_bits = 0;
    while ((1 << p.page_bits) < page_size) ++p.page_bits;

    const int smem = static_cast<int>(sizeof(Shared));
    WUDA_CUDA(cudaFuncSetAttribute(topk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    // Two CTAs fit an SM.  Rows beyond 16 K scores are scanned by a cluster of two while every cluster can be
    // resident at once; otherwise one CTA per row, and a grid-stride loop when there are more rows than places.
    const int places = 2 * dev.num_sms;
    const int csize = (score_stride > 16384 && rows * kMaxCluster <= places) ? kMaxCluster : 1;
    const int clusters = rows * csize <= places ? rows : places / csize;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(clusters * csize), 1, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = csize;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    WUDA_CUDA(cudaLaunchKernelEx(&cfg, topk_kernel, p));
    return WUDA_OK;
}
