// Exact per-row top-k index selection over fp32 scores, followed by the page-table
// transform, for sm_100a.
//
// Contract (dsv4_megakernel/megakernel/kernels/topk_v2.cu:329-439 and
// test/test_topk_v2.py:86-135): for each row r the indices of the k largest values of
// scores[r, 0:seq_len[r]], in no particular order; rows with seq_len <= k give
// [0..n) followed by -1; page_indices = (page_table[r, i >> bits] << bits) | (i & mask).
// Equal values are resolved towards the LOWER index, so the selected set is exactly
// torch.argsort(-scores, stable=True)[:k] — stricter than the reference, which leaves the
// choice among exact duplicates unspecified.
//
// One CTA of 1024 threads per row.  The selection is a most-significant-digit radix
// select on an order-preserving 32-bit key (digits of 12 + 12 + 8 bits) over a
// CANDIDATE list held in shared memory.  The candidate list is built in one of two ways:
//
//   sampled path (long rows, n >= 4k): 2048 evenly spaced samples give a 12-bit digit
//     that, with overwhelming probability, bounds the k-th value from below; ONE pass
//     over the row then parks every element at or above that digit (a few thousand
//     entries).  If the sample misled (fewer than k parked, or more than fit) the row
//     falls back to the exact path.
//   exact path: pass 1 histograms the top digit over the row, pass 2 emits everything
//     above the threshold digit and parks the threshold digit's members; when they do
//     not fit in shared memory (heavily duplicated scores) the two lower levels re-read
//     the row instead.
//
// If more values equal the final threshold than are still needed, one ordered pass over
// the row takes the lowest indices among them.  Shared-memory counters are bumped once
// per warp (ballot + popcount), not once per element.  No global scratch memory is used
// and nothing is allocated.
#include <cooperative_groups.h>
#include <cuda_runtime.h>

#include "host.h"

namespace wuda {
namespace topk {

constexpr int kThreads = 1024;
constexpr int kWarps = kThreads / 32;
constexpr int kBins = 4096;
constexpr int kCandCap = 8192;
constexpr int kSamples = 2048;
constexpr int kMaxCluster = 4;  // CTAs that may share one row's scan (thread-block cluster, distributed shared memory)

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

struct Shared {
    uint32_t hist[kBins];
    uint32_t cand_key[kCandCap];
    int32_t cand_idx[kCandCap];
    uint32_t warp_tot[kWarps];
    uint32_t warp_excl[kWarps];
    uint32_t sel_digit, sel_above;
    uint32_t out_count, cand_count;
};

// f(index, value, valid) for every element of the row.  Every thread of the CTA makes
// the same number of calls (valid = false past the end), so f may use full-warp votes.
// Loads are issued kBatch at a time before any is consumed: the row comes from L2 (the
// logits kernel has just written it) and a dependent load-use chain per 16 bytes would
// leave the pass bound by L2 latency.
constexpr int kBatch = 4;
template <typename F>
__device__ __forceinline__ void for_each_elem(const float* row, int n, bool vec_ok, F f) {
    if (vec_ok) {
        const int n4 = n >> 2;
        const float4* row4 = reinterpret_cast<const float4*>(row);
        for (int base = 0; base < n4; base += kThreads * kBatch) {
            float4 v[kBatch];
#pragma unroll
            for (int u = 0; u < kBatch; ++u) {
                const int i = base + u * kThreads + threadIdx.x;
                v[u] = i < n4 ? __ldcg(row4 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int u = 0; u < kBatch; ++u) {
                const int i = base + u * kThreads + threadIdx.x;
                const bool valid = i < n4;
                f(4 * i + 0, v[u].x, valid);
                f(4 * i + 1, v[u].y, valid);
                f(4 * i + 2, v[u].z, valid);
                f(4 * i + 3, v[u].w, valid);
            }
        }
        const int i = (n4 << 2) + threadIdx.x;   // at most 3 leftover elements
        if ((n & 3) != 0) f(i, i < n ? row[i] : 0.f, i < n);
    } else {
        for (int base = 0; base < n; base += kThreads * kBatch) {
            float v[kBatch];
#pragma unroll
            for (int u = 0; u < kBatch; ++u) {
                const int i = base + u * kThreads + threadIdx.x;
                v[u] = i < n ? row[i] : 0.f;
            }
#pragma unroll
            for (int u = 0; u < kBatch; ++u) {
                const int i = base + u * kThreads + threadIdx.x;
                f(i, v[u], i < n);
            }
        }
    }
}

// Reserves one slot per lane with `pred` set by bumping `counter` once per warp.
// Must be called by all 32 lanes of the warp.
__device__ __forceinline__ uint32_t warp_reserve(bool pred, uint32_t* counter) {
    const uint32_t mask = __ballot_sync(0xffffffffu, pred);
    if (mask == 0) return 0;
    const uint32_t lane = threadIdx.x & 31;
    uint32_t base = 0;
    if (lane == (__ffs(mask) - 1)) base = atomicAdd(counter, __popc(mask));
    base = __shfl_sync(0xffffffffu, base, __ffs(mask) - 1);
    return base + __popc(mask & ((1u << lane) - 1u));
}

__device__ __forceinline__ void zero_hist(Shared& s, int nbins) {
    for (int i = threadIdx.x; i < nbins; i += kThreads) s.hist[i] = 0;
}

// Finds the digit T with  count(digit > T) < need <= count(digit >= T)  and leaves
// T in s.sel_digit and count(digit > T) in s.sel_above.  Needs 1 <= need <= total.
__device__ __forceinline__ void find_threshold(Shared& s, int nbins, uint32_t need) {
    const int per = nbins >= kThreads ? nbins / kThreads : 1;
    const int lo = threadIdx.x * per;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    uint32_t local = 0;
    if (lo < nbins)
        for (int b = 0; b < per; ++b) local += s.hist[lo + b];
    // suffix sums: v = sum of `local` over threads >= this one
    uint32_t v = local;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t t = __shfl_down_sync(0xffffffffu, v, o);
        if (lane + o < 32) v += t;
    }
    if (lane == 0) s.warp_tot[warp] = v;
    __syncthreads();
    if (warp == 0) {
        const uint32_t mine = s.warp_tot[lane];
        uint32_t w = mine;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t t = __shfl_down_sync(0xffffffffu, w, o);
            if (lane + o < 32) w += t;
        }
        s.warp_excl[lane] = w - mine;
    }
    __syncthreads();
    uint32_t running = v - local + s.warp_excl[warp];  // count in digits above this thread's range
    if (lo < nbins) {
        for (int b = per - 1; b >= 0; --b) {
            const uint32_t h = s.hist[lo + b];
            if (running < need && need <= running + h) {
                s.sel_digit = lo + b;
                s.sel_above = running;
            }
            running += h;
        }
    }
    __syncthreads();
}

__device__ __forceinline__ int32_t page_of(const Params& p, int r, int idx) {
    if (!p.page_table) return idx;
    const int32_t page =
        __ldg(p.page_table + static_cast<int64_t>(r / p.rows_per_table_row) * p.pt_stride + (idx >> p.page_bits));
    return static_cast<int32_t>((static_cast<uint32_t>(page) << p.page_bits) |
                                static_cast<uint32_t>(idx & ((1 << p.page_bits) - 1)));
}

// Writes index `idx` to the next output slot of row r if `pred`; all 32 lanes call it.
__device__ __forceinline__ void emit(const Params& p, Shared& s, int r, int idx, bool pred) {
    const uint32_t pos = warp_reserve(pred, &s.out_count);
    if (pred && pos < static_cast<uint32_t>(p.k)) {
        const int64_t o = static_cast<int64_t>(r) * p.k + pos;
        if (p.raw) p.raw[o] = idx;
        p.page_indices[o] = page_of(p, r, idx);
    }
}

// Exclusive prefix sum of `count` over the CTA's threads (thread order) and the CTA total.
// Two barriers; uses warp_tot / warp_excl.
__device__ __forceinline__ uint32_t block_exclusive_scan(Shared& s, uint32_t count, uint32_t* total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    uint32_t v = count;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t t = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += t;
    }
    if (lane == 31) s.warp_tot[warp] = v;
    __syncthreads();
    if (warp == 0) {
        const uint32_t tot = s.warp_tot[lane];
        uint32_t w = tot;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t t = __shfl_up_sync(0xffffffffu, w, o);
            if (lane >= o) w += t;
        }
        s.warp_excl[lane] = w - tot;
        if (lane == 31) s.sel_above = w;             // the total (sel_above is free between selections)
    }
    __syncthreads();
    *total = s.sel_above;
    return v - count + s.warp_excl[warp];
}

// Writes the selected candidates (sel(key) true) to the row's output, after the `s.out_count` already
// written, without atomics: every thread counts its candidates c = tid, tid + 1024, .. (at most 8),
// one block scan hands out the positions.  All threads must call it; ends with a barrier.
template <typename Sel>
__device__ __forceinline__ void emit_candidates(const Params& p, Shared& s, int r, int ncand, Sel sel) {
    uint32_t mask = 0;
#pragma unroll
    for (int j = 0; j < kCandCap / kThreads; ++j) {
        const int c = threadIdx.x + j * kThreads;
        if (c < ncand && sel(s.cand_key[c])) mask |= 1u << j;
    }
    uint32_t total;
    const uint32_t base = s.out_count;               // stable: the caller's last barrier is behind us
    uint32_t pos = base + block_exclusive_scan(s, __popc(mask), &total);
#pragma unroll
    for (int j = 0; j < kCandCap / kThreads; ++j) {
        if ((mask >> j) & 1u) {
            if (pos < static_cast<uint32_t>(p.k)) {
                const int idx = s.cand_idx[threadIdx.x + j * kThreads];
                const int64_t o = static_cast<int64_t>(r) * p.k + pos;
                if (p.raw) p.raw[o] = idx;
                p.page_indices[o] = page_of(p, r, idx);
            }
            ++pos;
        }
    }
    __syncthreads();                                 // everybody has read out_count and sel_above
    if (threadIdx.x == 0) s.out_count = base + total;
    __syncthreads();
}

// One pass over the row that sorts every element into "emit now", "park as candidate"
// or "drop" (cls(key) = 2 / 1 / 0).  A thread classifies a whole batch of its elements
// into two bit masks first; slots in the output and in the candidate list are then
// reserved once per warp and batch (a warp scan of the per-thread counts and ONE counter
// bump), instead of a vote and a shared-memory atomic round trip per element.
constexpr int kClsBatch = 4;   // 16 elements per thread and batch: fits the 64 registers a thread of a 1024-thread CTA can have
// The pass covers elements [lo, hi) of the row (lo a multiple of 4); candidates go to
// `dst`, which may be another CTA's shared memory within the cluster; emitted indices
// are counted in `dst` as well.
template <typename Cls>
__device__ __forceinline__ void classify_pass(const float* row, int lo, int hi, bool vec_ok, const Params& p,
                                              Shared& dst, int r, Cls cls) {
    Shared& s = dst;
    const int n = hi;
    const uint32_t lane = threadIdx.x & 31;
    auto reserve = [&](uint32_t count, uint32_t* counter) -> uint32_t {   // exclusive offset for this lane
        uint32_t incl = count;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t t = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= static_cast<uint32_t>(o)) incl += t;
        }
        const uint32_t total = __shfl_sync(0xffffffffu, incl, 31);
        uint32_t base = 0;
        if (total != 0) {
            if (lane == 31) base = atomicAdd(counter, total);
            base = __shfl_sync(0xffffffffu, base, 31);
        }
        return base + incl - count;
    };
    auto put_emit = [&](uint32_t pos, int idx) {
        if (pos < static_cast<uint32_t>(p.k)) {
            const int64_t o = static_cast<int64_t>(r) * p.k + pos;
            if (p.raw) p.raw[o] = idx;
            p.page_indices[o] = page_of(p, r, idx);
        }
    };
    auto put_park = [&](uint32_t slot, int idx, uint32_t key) {
        if (slot < static_cast<uint32_t>(kCandCap)) {
            s.cand_key[slot] = key;
            s.cand_idx[slot] = idx;
        }
    };
    if (vec_ok) {
        const int n4 = n >> 2;
        const float4* row4 = reinterpret_cast<const float4*>(row);
        for (int base = lo >> 2; base < n4; base += kThreads * kClsBatch) {
            float4 v[kClsBatch];
#pragma unroll
            for (int u = 0; u < kClsBatch; ++u) {
                const int i = base + u * kThreads + threadIdx.x;
                v[u] = i < n4 ? __ldcg(row4 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
            uint32_t park = 0, emit_m = 0;
#pragma unroll
            for (int u = 0; u < kClsBatch; ++u) {
                const bool valid = base + u * kThreads + static_cast<int>(threadIdx.x) < n4;
                const float x[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const int cl = valid ? cls(x[c]) : 0;
                    park |= static_cast<uint32_t>(cl == 1) << (u * 4 + c);
                    emit_m |= static_cast<uint32_t>(cl == 2) << (u * 4 + c);
                }
            }
            uint32_t park_at = reserve(__popc(park), &s.cand_count);
            uint32_t emit_at = reserve(__popc(emit_m), &s.out_count);
            if ((park | emit_m) != 0) {
#pragma unroll
                for (int u = 0; u < kClsBatch; ++u) {
                    const int i = base + u * kThreads + threadIdx.x;
                    const float x[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        if ((park >> (u * 4 + c)) & 1u) put_park(park_at++, 4 * i + c, key_of(x[c]));
                        if ((emit_m >> (u * 4 + c)) & 1u) put_emit(emit_at++, 4 * i + c);
                    }
                }
            }
        }
        if ((n & 3) != 0) {   // at most 3 leftover elements
            const int i = (n4 << 2) + threadIdx.x;
            const float x = i < n ? row[i] : 0.f;
            const uint32_t key = key_of(x);
            const int cl = (i < n && lo < hi) ? cls(x) : 0;
            const uint32_t slot = warp_reserve(cl == 1, &s.cand_count);
            if (cl == 1) put_park(slot, i, key);
            const uint32_t pos = warp_reserve(cl == 2, &s.out_count);
            if (cl == 2) put_emit(pos, i);
        }
    } else {
        for (int base = lo; base < n; base += kThreads) {
            const int i = base + threadIdx.x;
            const float x = i < n ? row[i] : 0.f;
            const uint32_t key = key_of(x);
            const int cl = i < n ? cls(x) : 0;
            const uint32_t slot = warp_reserve(cl == 1, &s.cand_count);
            if (cl == 1) put_park(slot, i, key);
            const uint32_t pos = warp_reserve(cl == 2, &s.out_count);
            if (cl == 2) put_emit(pos, i);
        }
    }
}

__global__ void __launch_bounds__(kThreads, 1) topk_kernel(const Params p) {
    pdl_launch_dependents();
    pdl_wait();   // nothing of global memory is touched before the kernel ahead has finished
    extern __shared__ uint8_t smem_raw[];
    Shared& s = *reinterpret_cast<Shared*>(smem_raw);
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    const int crank = static_cast<int>(cluster.block_rank());
    const int csize = static_cast<int>(cluster.num_blocks());
    Shared& lead = *cluster.map_shared_rank(&s, 0);   // the cluster leader's shared memory

    // A cluster of csize CTAs (1, 2 or 4: the host uses the SMs that rows alone would leave
    // idle) takes one row at a time.  Only the scan of a long row
    // is shared (every CTA classifies its slice and parks candidates in the leader's
    // shared memory); the selection among the candidates runs in the leader alone.
    for (int r = blockIdx.x / csize; r < p.rows; r += gridDim.x / csize) {
        const float* row = p.scores + static_cast<int64_t>(r) * p.score_stride;
        int n = p.seq_lens[r];
        n = n < 0 ? 0 : n;
        if (static_cast<int64_t>(n) > p.score_stride) n = static_cast<int>(p.score_stride);
        const int k = p.k;

        // A row that fits the candidate list whole needs neither sampling nor classification.
        const bool small = n <= kCandCap;
        const bool sampled = !small && n >= 4 * k && k <= kCandCap / 2;
        if (crank != 0 && !sampled) continue;   // short rows are the leader's alone
        if (n <= k) {  // everything is selected: [0..n) then -1
            for (int i = threadIdx.x; i < k; i += kThreads) {
                const int64_t o = static_cast<int64_t>(r) * k + i;
                const int idx = i < n ? i : -1;
                if (p.raw) p.raw[o] = idx;
                p.page_indices[o] = idx >= 0 ? page_of(p, r, idx) : -1;
            }
            continue;
        }

        const bool vec_ok = ((reinterpret_cast<uintptr_t>(row) & 15u) == 0);
        zero_hist(s, kBins);
        if (threadIdx.x == 0) {
            s.out_count = 0;
            s.cand_count = 0;
        }
        __syncthreads();

        // ------------------------------------------------ sampled path: build the candidate list
        bool have_all = false;      // candidate list holds EVERY element at or above some digit
        int ncand = 0;
        uint32_t key_lo = 0;        // lower bound of the sampled scan's candidate keys
        uint32_t thr = 0, need3 = 0;   // threshold key; how many values equal to it are still taken
        bool take_all_equal = true;
        bool done = false;
        if (small) {
            // ---------------------------------------------------------- short rows: keys stay in registers
            // Thread t holds elements 4 (t + 1024 j) + c, j < 2, c < 4.  Three histogram levels
            // (12 + 12 + 8 key bits) find the threshold, one scan hands out the output positions.
            uint32_t key[8];
            uint32_t valid = 0;
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int e0 = 4 * (threadIdx.x + j * kThreads);
                if (vec_ok && e0 + 3 < n) {
                    const float4 v = __ldcg(reinterpret_cast<const float4*>(row + e0));
                    key[4 * j] = key_of(v.x), key[4 * j + 1] = key_of(v.y), key[4 * j + 2] = key_of(v.z), key[4 * j + 3] = key_of(v.w);
                    valid |= 0xFu << (4 * j);
                } else {
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const bool in = e0 + c < n;
                        key[4 * j + c] = in ? key_of(row[e0 + c]) : 0u;
                        valid |= static_cast<uint32_t>(in) << (4 * j + c);
                    }
                }
            }
#pragma unroll
            for (int e = 0; e < 8; ++e)
                if ((valid >> e) & 1u) atomicAdd(&s.hist[key[e] >> 20], 1u);
            __syncthreads();
            find_threshold(s, kBins, static_cast<uint32_t>(k));
            const uint32_t d1 = s.sel_digit;
            const uint32_t need1 = static_cast<uint32_t>(k) - s.sel_above;
            __syncthreads();
            zero_hist(s, kBins);
            __syncthreads();
#pragma unroll
            for (int e = 0; e < 8; ++e)
                if (((valid >> e) & 1u) && (key[e] >> 20) == d1) atomicAdd(&s.hist[(key[e] >> 8) & 0xFFFu], 1u);
            __syncthreads();
            find_threshold(s, kBins, need1);
            const uint32_t d2 = s.sel_digit;
            const uint32_t need2 = need1 - s.sel_above;
            __syncthreads();
            zero_hist(s, 256);
            __syncthreads();
            const uint32_t prefix24 = (d1 << 12) | d2;
#pragma unroll
            for (int e = 0; e < 8; ++e)
                if (((valid >> e) & 1u) && (key[e] >> 8) == prefix24) atomicAdd(&s.hist[key[e] & 0xFFu], 1u);
            __syncthreads();
            find_threshold(s, 256, need2);
            const uint32_t d3 = s.sel_digit;
            need3 = need2 - s.sel_above;
            thr = (prefix24 << 8) | d3;
            take_all_equal = (s.hist[d3] == need3);
            __syncthreads();
            uint32_t mask = 0;
#pragma unroll
            for (int e = 0; e < 8; ++e)
                if (((valid >> e) & 1u) && (key[e] > thr || (key[e] == thr && take_all_equal))) mask |= 1u << e;
            uint32_t total;
            uint32_t pos = block_exclusive_scan(s, __popc(mask), &total);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                if ((mask >> e) & 1u) {
                    const int idx = 4 * (threadIdx.x + (e >> 2) * kThreads) + (e & 3);
                    const int64_t o = static_cast<int64_t>(r) * k + pos;
                    if (p.raw) p.raw[o] = idx;
                    p.page_indices[o] = page_of(p, r, idx);
                    ++pos;
                }
            }
            __syncthreads();
            if (threadIdx.x == 0) s.out_count = total;
            __syncthreads();
            done = true;
        }
        if (sampled) {
            cluster.sync();   // the leader's counters are zeroed before anyone parks into them
            for (int t = threadIdx.x; t < kSamples; t += kThreads) {
                const int i = static_cast<int>(static_cast<long long>(t) * n / kSamples);
                atomicAdd(&s.hist[key_of(row[i]) >> 20], 1u);
            }
            __syncthreads();
            // expected sample rank of the k-th value, plus a 5-sigma margin
            const float expect = static_cast<float>(kSamples) * static_cast<float>(k) / static_cast<float>(n);
            uint32_t rank = static_cast<uint32_t>(expect + 5.f * sqrtf(expect) + 8.f);
            if (rank > static_cast<uint32_t>(kSamples)) rank = kSamples;
            find_threshold(s, kBins, rank);
            const uint32_t d_lo = s.sel_digit;
            __syncthreads();
            // every CTA of the cluster found the same d_lo (same samples); each scans a slice
            const int slice = ((n + csize - 1) / csize + 3) & ~3;
            const int lo = min(n, crank * slice), hi = min(n, lo + slice);
            // digit >= d_lo  <=>  key >= d_lo << 20  <=>  x >= the float with that key: one
            // compare per element (an unordered bound selects nothing and the row falls back)
            key_lo = d_lo << 20;
            const float x_lo = float_of_key(key_lo);
            classify_pass(row, lo, hi, vec_ok, p, lead, r, [&](float x) { return x >= x_lo ? 1 : 0; });
            zero_hist(s, kBins);
            cluster.sync();   // all slices are parked
            if (crank != 0) continue;
            const uint32_t total = s.cand_count;
            have_all = total >= static_cast<uint32_t>(k) && total <= static_cast<uint32_t>(kCandCap);
            ncand = have_all ? static_cast<int>(total) : 0;
            __syncthreads();
            if (!have_all && threadIdx.x == 0) s.cand_count = 0;
            __syncthreads();
        }

        const int ncand_pad = (ncand + kThreads - 1) / kThreads * kThreads;
        if (have_all && !small) {
            // ------------------------------------------------ candidates from the sampled scan
            // Their keys start at key_lo = d_lo << 20.  A 4096-bin histogram of
            // (key - key_lo) >> 12 resolves 20 key bits at once with little contention (the
            // candidates spread over many bins); one more level on the low 12 bits finishes.
            // Keys beyond the window share the last bin; if the threshold lands there
            // (never for ordinary data) the generic three-level path below takes over.
            for (int c = threadIdx.x; c < ncand; c += kThreads)
                atomicAdd(&s.hist[min((s.cand_key[c] - key_lo) >> 12, static_cast<uint32_t>(kBins - 1))], 1u);
            __syncthreads();
            find_threshold(s, kBins, static_cast<uint32_t>(k));
            const uint32_t bin_a = s.sel_digit;
            const uint32_t need_a = static_cast<uint32_t>(k) - s.sel_above;
            __syncthreads();
            zero_hist(s, kBins);
            __syncthreads();
            if (bin_a != static_cast<uint32_t>(kBins - 1)) {
                const uint32_t prefix20 = (key_lo >> 12) + bin_a;
                for (int c = threadIdx.x; c < ncand; c += kThreads) {
                    const uint32_t key = s.cand_key[c];
                    if ((key >> 12) == prefix20) atomicAdd(&s.hist[key & 0xFFFu], 1u);
                }
                __syncthreads();
                find_threshold(s, kBins, need_a);
                const uint32_t d_b = s.sel_digit;
                need3 = need_a - s.sel_above;
                take_all_equal = (s.hist[d_b] == need3);
                thr = (prefix20 << 12) | d_b;
                __syncthreads();
                {
                    const uint32_t t = thr;
                    const bool eq = take_all_equal;
                    emit_candidates(p, s, r, ncand, [&](uint32_t key) { return key > t || (key == t && eq); });
                }
                done = true;
            }
        }
        if (!done) {
        // ------------------------------------------------ level 1: the top 12 bits
        uint32_t d1, need1;
        bool parked;                // the threshold digit's members are in the candidate list
        if (have_all) {
            for (int c = threadIdx.x; c < ncand; c += kThreads) atomicAdd(&s.hist[s.cand_key[c] >> 20], 1u);
            __syncthreads();
            find_threshold(s, kBins, static_cast<uint32_t>(k));
            d1 = s.sel_digit;
            need1 = static_cast<uint32_t>(k) - s.sel_above;
            parked = true;
            __syncthreads();
            emit_candidates(p, s, r, ncand, [&](uint32_t key) { return (key >> 20) > d1; });
            zero_hist(s, kBins);
            __syncthreads();
        } else {
            for_each_elem(row, n, vec_ok, [&](int, float x, bool valid) {
                if (valid) atomicAdd(&s.hist[key_of(x) >> 20], 1u);
            });
            __syncthreads();
            find_threshold(s, kBins, static_cast<uint32_t>(k));
            d1 = s.sel_digit;
            need1 = static_cast<uint32_t>(k) - s.sel_above;   // still needed from digit d1
            parked = s.hist[d1] <= static_cast<uint32_t>(kCandCap);
            __syncthreads();
            // pass 2: emit everything above the digit, park the digit's members
            classify_pass(row, 0, n, vec_ok, p, s, r, [&](float x) {
                const uint32_t d = key_of(x) >> 20;
                return d > d1 ? 2 : ((d == d1 && parked) ? 1 : 0);
            });
            zero_hist(s, kBins);
            __syncthreads();
            ncand = parked ? static_cast<int>(min(s.cand_count, static_cast<uint32_t>(kCandCap))) : 0;
        }
        const int nmem_pad = (ncand + kThreads - 1) / kThreads * kThreads;

        // f(index, key, is_member) over the members of digit d1, with a uniform call
        // count across the CTA (is_member = false on padding calls)
        auto for_each_member = [&](auto f) {
            if (parked) {
                for (int c = threadIdx.x; c < nmem_pad; c += kThreads) {
                    const bool in = c < ncand;
                    const uint32_t key = in ? s.cand_key[c] : 0u;
                    f(in ? s.cand_idx[c] : 0, key, in && (key >> 20) == d1);
                }
            } else {
                for_each_elem(row, n, vec_ok, [&](int i, float x, bool valid) {
                    const uint32_t key = key_of(x);
                    f(i, key, valid && (key >> 20) == d1);
                });
            }
        };

        // ------------------------------------------------ level 2: the next 12 bits
        for_each_member([&](int, uint32_t key, bool in) {
            if (in) atomicAdd(&s.hist[(key >> 8) & 0xFFFu], 1u);
        });
        __syncthreads();
        find_threshold(s, kBins, need1);
        const uint32_t d2 = s.sel_digit;
        const uint32_t need2 = need1 - s.sel_above;
        __syncthreads();
        zero_hist(s, 256);
        __syncthreads();

        // ------------------------------------------------ level 3: the last 8 bits
        const uint32_t prefix24 = (d1 << 12) | d2;
        for_each_member([&](int, uint32_t key, bool in) {
            if (in && (key >> 8) == prefix24) atomicAdd(&s.hist[key & 0xFFu], 1u);
        });
        __syncthreads();
        find_threshold(s, 256, need2);
        const uint32_t d3 = s.sel_digit;
        need3 = need2 - s.sel_above;
        const uint32_t ceq = s.hist[d3];
        thr = (prefix24 << 8) | d3;
        take_all_equal = (ceq == need3);
        __syncthreads();

        for_each_member([&](int i, uint32_t key, bool in) {
            emit(p, s, r, i, in && (key > thr || (key == thr && take_all_equal)));
        });
        }

        if (!take_all_equal) {
            // More duplicates of the threshold value than needed: take the lowest indices.
            const int chunk = (n + kThreads - 1) / kThreads;
            const int beg = min(n, static_cast<int>(threadIdx.x) * chunk);
            const int end = min(n, beg + chunk);
            uint32_t mine = 0;
            for (int i = beg; i < end; ++i) mine += (key_of(row[i]) == thr);
            // exclusive prefix over threads
            const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
            uint32_t v = mine;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t t = __shfl_up_sync(0xffffffffu, v, o);
                if (lane >= o) v += t;
            }
            __syncthreads();
            if (lane == 31) s.warp_tot[warp] = v;
            __syncthreads();
            if (warp == 0) {
                const uint32_t tot = s.warp_tot[lane];
                uint32_t w = tot;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const uint32_t t = __shfl_up_sync(0xffffffffu, w, o);
                    if (lane >= o) w += t;
                }
                s.warp_excl[lane] = w - tot;
            }
            __syncthreads();
            uint32_t rank = v - mine + s.warp_excl[warp];
            for (int i = beg; i < end && rank < need3; ++i) {
                if (key_of(row[i]) == thr) {   // few and scattered: one counter bump each
                    const uint32_t pos = atomicAdd(&s.out_count, 1u);
                    if (pos < static_cast<uint32_t>(k)) {
                        const int64_t o = static_cast<int64_t>(r) * k + pos;
                        if (p.raw) p.raw[o] = i;
                        p.page_indices[o] = page_of(p, r, i);
                    }
                    ++rank;
                }
            }
        }
        __syncthreads();
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
    // One 1024-thread CTA fills an SM; when there are fewer rows than SMs the spare SMs
    // join the rows' clusters.
    // (rows of at most 16 K scores are not worth a cluster barrier: one CTA scans them in a few passes)
    int kCluster = 1;
    while (score_stride > 16384 && kCluster < kMaxCluster && rows * kCluster * 2 <= dev.num_sms) kCluster *= 2;
    const int clusters = rows * kCluster <= dev.num_sms ? rows : dev.num_sms / kCluster;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(clusters * kCluster), 1, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = kCluster;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    WUDA_CUDA(cudaLaunchKernelEx(&cfg, topk_kernel, p));
    return WUDA_OK;
}
