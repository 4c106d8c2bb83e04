// The pieces of the routed-expert block around its two grouped NVFP4 GEMMs
// (dsv4_megakernel/origin/model.py:587-644, MoE.forward and Expert.forward):
//   dispatch      (token, expert) pairs -> rows sorted by expert, every expert's rows padded to
//                 groups of 16 (one GEMM row tile), stable in token order
//   gather_quant  row r = activation of its token -> NVFP4 (e2m1 + one ue4m3 scale per 16 values +
//                 a given per-tensor scale), scales written in the layout the tensor core reads
//   swiglu_quant  h = silu(min(gate, L)) * clamp(up, +-L) * routing weight, rounded to bf16, -> NVFP4
//   combine       y[t] = bf16( sum_j out[row(t, j)] (+ shared[t]) ), pairs added in slot order
// Everything is deterministic: no floating-point atomics, fixed summation orders.
//
// NVFP4 quantisation of a block of 16 values with tensor scale gs:
//   sf  = e4m3(min(amax / 6 / gs, 448))  (round to nearest even);  d = decoded sf
//   q_i = e2m1(x_i / (d * gs)), nearest value of {0, .5, 1, 1.5, 2, 3, 4, 6}, ties to the smaller
//         magnitude, saturating at 6; an all-zero block has sf = 0 and q = 0
// Two values per byte, low nibble first.  Scale bytes of group g (16 rows), K block kb (256 values):
//   ((g * K/256 + kb) * 2048) + step * 512 + row * 16 + byte,  step = (k / 64) % 4, byte = (k / 16) % 4
// which is rows 0..15 of the 128-row image tcgen05.cp.32x128b.warpx4 copies (rows 16..127 stay zero).
#include <cuda_bf16.h>

#include "host.h"
#include "ptx.cuh"

namespace wuda {
namespace moe {

constexpr int kGroupRows = 16;

// ---------------------------------------------------------------- dispatch (one CTA)
struct DispatchParams {
    const int32_t* indices;   // [tokens, k]
    const float* weights;     // [tokens, k]
    int32_t* group_expert;    // [max_groups]
    int32_t* num_groups;      // [1]
    int32_t* row_token;       // [max_groups * 16]
    float* row_weight;        // [max_groups * 16]
    int32_t* pair_row;        // [tokens, k]
    int tokens, k, experts, max_groups;
    int first, total;         // this rank holds experts [first, first + experts) of `total`
    int32_t* status;
};

constexpr int kDispatchThreads = 1024;
constexpr int kMaxExperts = 512;
constexpr int kPairsInShared = 4096;   // up to this many pairs the ranking reads them from shared memory

__global__ void __launch_bounds__(kDispatchThreads) moe_dispatch_kernel(DispatchParams p) {
    pdl_launch_dependents();
    pdl_wait();   // nothing of global memory is touched before the kernel ahead has finished
    __shared__ int count[kMaxExperts];
    __shared__ int base[kMaxExperts];       // first group of the expert
    __shared__ int pair_expert[kPairsInShared];
    __shared__ int total_groups;
    const int pairs = p.tokens * p.k;
    const bool staged = pairs <= kPairsInShared;
    for (int e = threadIdx.x; e < p.experts; e += kDispatchThreads) count[e] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < pairs; i += kDispatchThreads) {
        const int global = __ldcg(p.indices + i), e = global - p.first;   // written by the router of the same chain
        if (staged) pair_expert[i] = global;
        if (e >= 0 && e < p.experts) atomicAdd(&count[e], 1);
        else if ((global < 0 || global >= p.total) && p.status) atomicCAS(p.status, 0, WUDA_DEV_BAD_EXPERT);
    }
    for (int r = threadIdx.x; r < p.max_groups * kGroupRows; r += kDispatchThreads) {
        p.row_token[r] = -1;
        p.row_weight[r] = 0.f;
    }
    for (int g = threadIdx.x; g < p.max_groups; g += kDispatchThreads) p.group_expert[g] = -1;
    __syncthreads();
    if (threadIdx.x < 32) {                 // exclusive scan of the experts' group counts by one warp
        const int per = (p.experts + 31) / 32, e0 = threadIdx.x * per, e1 = min(e0 + per, p.experts);
        int mine = 0;
        for (int e = e0; e < e1; ++e) mine += (count[e] + kGroupRows - 1) / kGroupRows;
        int incl = mine;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int up = __shfl_up_sync(0xffffffffu, incl, d);
            if (threadIdx.x >= d) incl += up;
        }
        int g = incl - mine;
        for (int e = e0; e < e1; ++e) {
            base[e] = g;
            g += (count[e] + kGroupRows - 1) / kGroupRows;
        }
        if (threadIdx.x == 31) {
            total_groups = incl;
            *p.num_groups = incl <= p.max_groups ? incl : 0;
            if (incl > p.max_groups && p.status) atomicCAS(p.status, 0, WUDA_DEV_BAD_DESTINATION);
        }
    }
    __syncthreads();
    if (total_groups > p.max_groups) return;
    for (int e = threadIdx.x; e < p.experts; e += kDispatchThreads) {
        const int groups = (count[e] + kGroupRows - 1) / kGroupRows;
        for (int g = 0; g < groups; ++g) p.group_expert[base[e] + g] = e;
    }
    // stable placement: the rank of a pair among the earlier pairs of the same expert
    for (int i = threadIdx.x; i < pairs; i += kDispatchThreads) {
        const int global = staged ? pair_expert[i] : __ldcg(p.indices + i), e = global - p.first;
        if (e < 0 || e >= p.experts) {   // another rank's expert, or an invalid index
            p.pair_row[i] = -1;
            continue;
        }
        int rank = 0;
        if (staged) {
#pragma unroll 8
            for (int j = 0; j < i; ++j) rank += (pair_expert[j] == global);
        } else {
            for (int j = 0; j < i; ++j) rank += (__ldcg(p.indices + j) == global);
        }
        const int row = base[e] * kGroupRows + rank;
        p.pair_row[i] = row;
        p.row_token[row] = i / p.k;
        p.row_weight[row] = __ldcg(p.weights + i);
    }
}

// ---------------------------------------------------------------- NVFP4 quantisation of 16 values
__device__ __forceinline__ uint32_t e2m1_code(float x) {
    const float a = fminf(fabsf(x), 6.0f);
    // bucket boundaries are the midpoints; a value on a boundary takes the smaller magnitude
    uint32_t idx = (a > 0.25f) + (a > 0.75f) + (a > 1.25f) + (a > 1.75f) + (a > 2.5f) + (a > 3.5f) + (a > 5.0f);
    return idx | ((x < 0.f && idx != 0) ? 8u : 0u);
}

__device__ __forceinline__ float e4m3_decode(uint32_t b) {
    const uint32_t e = (b >> 3) & 15u, m = b & 7u;
    return e == 0 ? static_cast<float>(m) * 0.001953125f : __uint_as_float(((e + 120u) << 23) | (m << 20));
}

// v: 16 values.  Returns the 8 packed bytes (as two words) and the scale byte.
__device__ __forceinline__ void quant16(const float (&v)[16], float gs, uint32_t (&packed)[2], uint32_t* sf_byte) {
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
    const float want = fminf(__fdiv_rn(__fdiv_rn(amax, 6.0f), gs), 448.0f);
    uint16_t pair;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(pair) : "f"(0.f), "f"(want));
    const uint32_t sf = pair & 0xffu;
    const float d = e4m3_decode(sf);
    const float denom = __fmul_rn(d, gs);
    packed[0] = packed[1] = 0;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const uint32_t code = d > 0.f ? e2m1_code(__fdiv_rn(v[i], denom)) : 0u;
        packed[i >> 3] |= code << (4 * (i & 7));
    }
    *sf_byte = sf;
}

__device__ __forceinline__ int64_t sf_offset(int row, int k16, int kb_per_row) {
    // k16 = index of the 16-value block along K
    const int group = row / kGroupRows, r = row % kGroupRows;
    const int kb = k16 >> 4, within = k16 & 15;
    return (static_cast<int64_t>(group) * kb_per_row + kb) * 2048 + (within >> 2) * 512 + r * 16 + (within & 3);
}

// A thread of the two quantisation kernels owns one block of 16 values of one (token, expert) pair's row; the
// four scale bytes of a 64-value step are collected by the first of its four lanes and stored as one word.
// Rows without a token are not touched at all: the grouped GEMM, given row_token, does not store their
// outputs, and nothing else reads them.
__device__ __forceinline__ void unpack_bf16x8(const uint4& raw, float* v) {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        v[2 * i] = __uint_as_float(w[i] << 16);
        v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}

__device__ __forceinline__ void store_block(uint8_t* a4, uint8_t* a_sf, int row, int b, int row_blocks, const uint32_t (&packed)[2],
                                            uint32_t sf, bool live) {
    // (every lane of the warp takes part in the shuffles; blocks of a row never straddle a group of four lanes
    // because row_blocks is a multiple of 16)
    uint32_t word = sf;
    word |= __shfl_down_sync(0xffffffffu, sf, 1) << 8;
    word |= __shfl_down_sync(0xffffffffu, sf, 2) << 16;
    word |= __shfl_down_sync(0xffffffffu, sf, 3) << 24;
    if (!live) return;
    *reinterpret_cast<uint2*>(a4 + static_cast<int64_t>(row) * (row_blocks * 8) + b * 8) = make_uint2(packed[0], packed[1]);
    if ((b & 3) == 0) *reinterpret_cast<uint32_t*>(a_sf + sf_offset(row, b, row_blocks / 16)) = word;
}

constexpr int kQuantThreads = 256;

// ---------------------------------------------------------------- gather + quantise
struct GatherParams {
    const __nv_bfloat16* x;      // [tokens, K]
    const int32_t* pair_row;     // [tokens, topk]: row of the pair, or -1
    uint8_t* a4;                 // [rows, K / 2]
    uint8_t* a_sf;               // packed scales
    float gs;
    int K, pairs, topk;
};

__global__ void __launch_bounds__(kQuantThreads) moe_gather_quant_kernel(GatherParams p) {
    pdl_launch_dependents();
    pdl_wait();   // nothing of global memory is touched before the kernel ahead has finished
    const int blocks = p.K / 16;
    const int item = blockIdx.x * kQuantThreads + threadIdx.x;
    const int pair = item / blocks, b = item - pair * blocks;
    const int row = pair < p.pairs ? __ldcg(p.pair_row + pair) : -1;
    const bool live = row >= 0;
    uint32_t packed[2] = {0u, 0u}, sf = 0u;
    if (live) {
        const uint4* src = reinterpret_cast<const uint4*>(p.x + static_cast<int64_t>(pair / p.topk) * p.K + b * 16);
        const uint4 lo = __ldcg(src), hi = __ldcg(src + 1);   // activations of a kernel of the same chain
        float v[16];
        unpack_bf16x8(lo, v);
        unpack_bf16x8(hi, v + 8);
        quant16(v, p.gs, packed, &sf);
    }
    store_block(p.a4, p.a_sf, row, b, blocks, packed, sf, live);
}

// ---------------------------------------------------------------- SwiGLU + routing weight + quantise
struct SwigluParams {
    const __nv_bfloat16* h;      // [rows, 2 * I]: gate | up
    const int32_t* pair_row;     // [tokens, topk]
    const float* pair_weight;    // [tokens, topk] routing weights
    uint8_t* a4;                 // [rows, I / 2]
    uint8_t* a_sf;
    float gs, limit;
    int I, pairs;
};

__global__ void __launch_bounds__(kQuantThreads) moe_swiglu_quant_kernel(SwigluParams p) {
    pdl_launch_dependents();
    pdl_wait();   // nothing of global memory is touched before the kernel ahead has finished
    const int blocks = p.I / 16;
    const int item = blockIdx.x * kQuantThreads + threadIdx.x;
    const int pair = item / blocks, b = item - pair * blocks;
    const int row = pair < p.pairs ? __ldcg(p.pair_row + pair) : -1;
    const bool live = row >= 0;
    uint32_t packed[2] = {0u, 0u}, sf = 0u;
    if (live) {
        const float rw = __ldcg(p.pair_weight + pair);
        const uint4* g = reinterpret_cast<const uint4*>(p.h + static_cast<int64_t>(row) * (2 * p.I) + b * 16);
        const uint4* u = reinterpret_cast<const uint4*>(p.h + static_cast<int64_t>(row) * (2 * p.I) + p.I + b * 16);
        const uint4 g0 = __ldcg(g), g1 = __ldcg(g + 1), u0 = __ldcg(u), u1 = __ldcg(u + 1);
        float gate[16], up[16], v[16];
        unpack_bf16x8(g0, gate);
        unpack_bf16x8(g1, gate + 8);
        unpack_bf16x8(u0, up);
        unpack_bf16x8(u1, up + 8);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            float gt = gate[i], uu = up[i];
            if (p.limit > 0.f) {
                uu = fminf(fmaxf(uu, -p.limit), p.limit);
                gt = fminf(gt, p.limit);
            }
            const float silu = __fdiv_rn(gt, 1.0f + expf(-gt));
            v[i] = __bfloat162float(__float2bfloat16_rn(__fmul_rn(rw, __fmul_rn(silu, uu))));
        }
        quant16(v, p.gs, packed, &sf);
    }
    store_block(p.a4, p.a_sf, row, b, blocks, packed, sf, live);
}

// ---------------------------------------------------------------- combine
struct CombineParams {
    const __nv_bfloat16* out;    // [rows, dim]
    const int32_t* pair_row;     // [tokens, k]
    const __nv_bfloat16* shared; // [tokens, dim] or nullptr
    __nv_bfloat16* y;            // [tokens, dim]
    int k, dim;
};

constexpr int kCombineSlots = 8;   // expert rows whose loads are in flight together

// The fp32 sum of a token's expert rows (in slot order) and its shared-expert row over 8 dims: all row numbers
// first, then up to eight rows' loads at once, then the additions in order.
__device__ __forceinline__ void combine_sum8(const CombineParams& p, int t, int c, float (&acc)[8]) {
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    for (int j0 = 0; j0 < p.k; j0 += kCombineSlots) {
        int row[kCombineSlots];
        uint4 raw[kCombineSlots];
#pragma unroll
        for (int j = 0; j < kCombineSlots; ++j) row[j] = j0 + j < p.k ? __ldcg(p.pair_row + t * p.k + j0 + j) : -1;
#pragma unroll
        for (int j = 0; j < kCombineSlots; ++j)
            if (row[j] >= 0) raw[j] = __ldcg(reinterpret_cast<const uint4*>(p.out + static_cast<int64_t>(row[j]) * p.dim) + c);
#pragma unroll
        for (int j = 0; j < kCombineSlots; ++j) {
            if (row[j] < 0) continue;
            float v[8];
            unpack_bf16x8(raw[j], v);
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] = __fadd_rn(acc[i], v[i]);
        }
    }
    if (p.shared) {
        float v[8];
        unpack_bf16x8(__ldcg(reinterpret_cast<const uint4*>(p.shared + static_cast<int64_t>(t) * p.dim) + c), v);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = __fadd_rn(acc[i], v[i]);
    }
}

__device__ __forceinline__ uint4 pack_bf16x8(const float (&acc)[8]) {
    uint4 o;
    uint32_t* ow = &o.x;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        __nv_bfloat162 b = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
        ow[i] = *reinterpret_cast<uint32_t*>(&b);
    }
    return o;
}

constexpr int kCombineThreads = 128;

// grid (ceil(dim / 8 / 128), tokens): one 8-dim vector per thread
__global__ void __launch_bounds__(kCombineThreads) moe_combine_kernel(CombineParams p) {
    pdl_launch_dependents();
    pdl_wait();   // nothing of global memory is touched before the kernel ahead has finished
    const int t = blockIdx.y, c = blockIdx.x * kCombineThreads + threadIdx.x;
    if (c >= p.dim / 8) return;
    float acc[8];
    combine_sum8(p, t, c, acc);
    *(reinterpret_cast<uint4*>(p.y + static_cast<int64_t>(t) * p.dim) + c) = pack_bf16x8(acc);
}

// Expert parallelism over two ranks: each rank sums the outputs of its own experts for every token, pushes
// the fp32 partial row into the peer GPU's inbox (plain stores through the peer mapping, then a system-scope
// release of the token's flag), awaits the peer's row in its own inbox and adds it: a + b == b + a in fp32, so
// both ranks hold bit-identical rows.  Inbox sets alternate with the call's sequence number.  The wait is
// bounded: a peer that does not answer leaves WUDA_DEV_TIMEOUT_PEER_FLAG and the local sum in y.
constexpr int kEpMaxTokens = 512;
constexpr int64_t kEpCtrlOffset = 2 * kEpMaxTokens * 4;   // behind the flags: {call sequence, CTAs done}
constexpr int64_t kEpFlagBytes = kEpCtrlOffset + 256;
constexpr int kEpMaxDim = 8192;         // one 8-value vector per thread of a 1024-thread CTA

struct CombineEpParams {
    CombineParams c;
    float* my_rows;      // [2 sets][tokens_max][dim] fp32 in this GPU's memory
    float* peer_rows;    // the same buffer of the peer
    int32_t* my_flags;   // [2 sets][kEpMaxTokens]
    int32_t* peer_flags;
    int32_t* ctrl;       // this rank's control words: [0] last finished call, [1] CTAs done
    int tokens_max, epoch;   // epoch 0: the call's number is ctrl[0] + 1 (replayable from a CUDA graph)
    unsigned long long wait_ns;
    int32_t* status;
};

__device__ __forceinline__ void st_release_sys(int32_t* p, int v) {
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int32_t* p) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ float4 ld_volatile_f32x4(const float* p) {   // written by the peer GPU: bypass L1
    float4 v;
    asm volatile("ld.volatile.global.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
    return v;
}

// one CTA per token, one 8-dim vector per thread (dim <= 8192)
__global__ void __launch_bounds__(1024) moe_combine_ep2_kernel(CombineEpParams q) {
    pdl_launch_dependents();
    pdl_wait();
    const CombineParams& p = q.c;
    __shared__ int peer_ok;
    const int t = blockIdx.x, c = threadIdx.x;
    const bool mine = c < p.dim / 8;
    const int epoch = q.epoch ? q.epoch : ld_acquire_sys(q.ctrl) + 1;
    const int set = epoch & 1;
    const int64_t row_off = (static_cast<int64_t>(set) * q.tokens_max + t) * p.dim;
    float acc[8];
    if (mine) {
        combine_sum8(p, t, c, acc);
        float4* dst = reinterpret_cast<float4*>(q.peer_rows + row_off + c * 8);
        dst[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
        dst[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        st_release_sys(q.peer_flags + set * kEpMaxTokens + t, epoch);
        int ok = 1;
        const unsigned long long start = globaltimer_ns();
        uint32_t spins = 0;
        while (ld_acquire_sys(q.my_flags + set * kEpMaxTokens + t) != epoch) {
            if ((++spins & 63u) == 0u && globaltimer_ns() - start > q.wait_ns) {
                if (q.status) atomicCAS(q.status, 0, static_cast<int>(kDevTimeoutPeerFlag));
                ok = 0;
                break;
            }
            __nanosleep(100);
        }
        peer_ok = ok;
    }
    __syncthreads();
    if (mine) {
        if (peer_ok != 0) {
            const float4 a = ld_volatile_f32x4(q.my_rows + row_off + c * 8), b = ld_volatile_f32x4(q.my_rows + row_off + c * 8 + 4);
            acc[0] += a.x, acc[1] += a.y, acc[2] += a.z, acc[3] += a.w;
            acc[4] += b.x, acc[5] += b.y, acc[6] += b.z, acc[7] += b.w;
        }
        *(reinterpret_cast<uint4*>(p.y + static_cast<int64_t>(t) * p.dim) + c) = pack_bf16x8(acc);
    }
    if (q.epoch == 0 && threadIdx.x == 0) {
        // the last CTA to finish has seen every other CTA read the old number; it stores the new one
        __threadfence();
        if (atomicAdd(q.ctrl + 1, 1) == static_cast<int>(gridDim.x) - 1) {
            q.ctrl[1] = 0;
            st_release_sys(q.ctrl, epoch);
        }
    }
}

}  // namespace moe
}  // namespace wuda

extern "C" int wuda_moe_max_groups(int tokens, int k, int experts) {
    if (tokens < 1 || k < 1 || experts < 1) return -1;
    // every expert can end in one partly filled group
    const long long g = (static_cast<long long>(tokens) * k + 15) / 16 + experts;
    const long long cap = static_cast<long long>(tokens) * k < experts ? static_cast<long long>(tokens) * k : g;
    return static_cast<int>(cap < g ? cap : g);
}

extern "C" int wuda_moe_dispatch(const int32_t* indices, const float* weights, int32_t* group_expert, int32_t* num_groups,
                                 int32_t* row_token, float* row_weight, int32_t* pair_row, int tokens, int k, int experts,
                                 int max_groups, int32_t* status_word, void* stream) {
    return wuda_moe_dispatch_range(indices, weights, group_expert, num_groups, row_token, row_weight, pair_row, tokens, k,
                                   experts, 0, experts, max_groups, status_word, stream);
}

extern "C" int wuda_moe_dispatch_range(const int32_t* indices, const float* weights, int32_t* group_expert,
                                       int32_t* num_groups, int32_t* row_token, float* row_weight, int32_t* pair_row,
                                       int tokens, int k, int experts, int expert_first, int experts_total, int max_groups,
                                       int32_t* status_word, void* stream) {
    using namespace wuda;
    using namespace wuda::moe;
    clear_error();
    WUDA_REQUIRE(tokens >= 1 && k >= 1, "tokens and k must be >= 1");
    WUDA_REQUIRE(expert_first >= 0 && experts_total >= 1 && expert_first + experts <= experts_total,
                 "the local experts [%d, %d + %d) must lie inside [0, %d)", expert_first, expert_first, experts, experts_total);
    WUDA_REQUIRE(experts >= 1 && experts <= kMaxExperts, "experts must be in [1, %d] (got %d)", kMaxExperts, experts);
    WUDA_REQUIRE(static_cast<long long>(tokens) * k <= 65536, "at most 65536 (token, expert) pairs per call");
    WUDA_REQUIRE(max_groups >= wuda_moe_max_groups(tokens, k, experts),
                 "max_groups must be at least wuda_moe_max_groups(tokens, k, experts) = %d (got %d)",
                 wuda_moe_max_groups(tokens, k, experts), max_groups);
    WUDA_REQUIRE(indices && weights && group_expert && num_groups && row_token && row_weight && pair_row,
                 "no array may be NULL");
    DispatchParams p;
    p.indices = indices;
    p.weights = weights;
    p.group_expert = group_expert;
    p.num_groups = num_groups;
    p.row_token = row_token;
    p.row_weight = row_weight;
    p.pair_row = pair_row;
    p.tokens = tokens;
    p.k = k;
    p.experts = experts;
    p.first = expert_first;
    p.total = experts_total;
    p.max_groups = max_groups;
    p.status = status_word;
    WUDA_CUDA(launch_pdl(moe_dispatch_kernel, dim3(1), dim3(kDispatchThreads), 0, static_cast<cudaStream_t>(stream), p));
    return WUDA_OK;
}

extern "C" int wuda_moe_gather_quant_nvfp4(const void* x_bf16, const int32_t* pair_row, void* a_fp4, void* a_sf_packed,
                                           float global_scale, int tokens, int topk, int k, void* stream) {
    using namespace wuda;
    using namespace wuda::moe;
    clear_error();
    WUDA_REQUIRE(tokens >= 1 && topk >= 1 && static_cast<long long>(tokens) * topk <= 65536, "tokens, topk >= 1 and at most 65536 pairs");
    WUDA_REQUIRE(k >= 256 && k % 256 == 0, "k must be a positive multiple of 256 (got %d)", k);
    WUDA_REQUIRE(global_scale > 0.f, "global_scale must be positive");
    WUDA_REQUIRE(x_bf16 && pair_row && a_fp4 && a_sf_packed, "no array may be NULL");
    WUDA_REQUIRE(aligned16(x_bf16) && aligned16(a_fp4) && aligned16(a_sf_packed), "x, a_fp4 and a_sf must be 16-byte aligned");
    GatherParams p;
    p.x = static_cast<const __nv_bfloat16*>(x_bf16);
    p.pair_row = pair_row;
    p.a4 = static_cast<uint8_t*>(a_fp4);
    p.a_sf = static_cast<uint8_t*>(a_sf_packed);
    p.gs = global_scale;
    p.K = k;
    p.pairs = tokens * topk;
    p.topk = topk;
    const long long items = static_cast<long long>(p.pairs) * (k / 16);
    WUDA_REQUIRE(items < (1ll << 31), "tokens * topk * k / 16 must stay below 2^31");
    WUDA_CUDA(launch_pdl(moe_gather_quant_kernel, dim3(static_cast<unsigned>((items + kQuantThreads - 1) / kQuantThreads)),
                         dim3(kQuantThreads), 0, static_cast<cudaStream_t>(stream), p));
    return WUDA_OK;
}

extern "C" int wuda_moe_swiglu_quant_nvfp4(const void* h_bf16, const int32_t* pair_row, const float* pair_weight, void* a_fp4,
                                           void* a_sf_packed, float global_scale, float swiglu_limit, int tokens, int topk,
                                           int inter, void* stream) {
    using namespace wuda;
    using namespace wuda::moe;
    clear_error();
    WUDA_REQUIRE(tokens >= 1 && topk >= 1 && static_cast<long long>(tokens) * topk <= 65536, "tokens, topk >= 1 and at most 65536 pairs");
    WUDA_REQUIRE(inter >= 256 && inter % 256 == 0, "inter must be a positive multiple of 256 (got %d)", inter);
    WUDA_REQUIRE(global_scale > 0.f, "global_scale must be positive");
    WUDA_REQUIRE(h_bf16 && pair_row && pair_weight && a_fp4 && a_sf_packed, "no array may be NULL");
    WUDA_REQUIRE(aligned16(h_bf16) && aligned16(a_fp4) && aligned16(a_sf_packed), "h, a_fp4 and a_sf must be 16-byte aligned");
    SwigluParams p;
    p.h = static_cast<const __nv_bfloat16*>(h_bf16);
    p.pair_row = pair_row;
    p.pair_weight = pair_weight;
    p.a4 = static_cast<uint8_t*>(a_fp4);
    p.a_sf = static_cast<uint8_t*>(a_sf_packed);
    p.gs = global_scale;
    p.limit = swiglu_limit;
    p.I = inter;
    p.pairs = tokens * topk;
    const long long items = static_cast<long long>(p.pairs) * (inter / 16);
    WUDA_REQUIRE(items < (1ll << 31), "tokens * topk * inter / 16 must stay below 2^31");
    WUDA_CUDA(launch_pdl(moe_swiglu_quant_kernel, dim3(static_cast<unsigned>((items + kQuantThreads - 1) / kQuantThreads)),
                         dim3(kQuantThreads), 0, static_cast<cudaStream_t>(stream), p));
    return WUDA_OK;
}

extern "C" int wuda_moe_combine(const void* expert_out_bf16, const int32_t* pair_row, const void* shared_bf16,
                                void* y_bf16, int tokens, int k, int dim, void* stream) {
    using namespace wuda;
    using namespace wuda::moe;
    clear_error();
    WUDA_REQUIRE(tokens >= 1 && tokens <= 65535 && k >= 1 && dim >= 8 && dim % 8 == 0,
                 "tokens in [1, 65535], k >= 1 and dim a positive multiple of 8");
    WUDA_REQUIRE(expert_out_bf16 && pair_row && y_bf16, "expert_out, pair_row and y must not be NULL");
    WUDA_REQUIRE(aligned16(expert_out_bf16) && aligned16(shared_bf16) && aligned16(y_bf16), "rows must be 16-byte aligned");
    CombineParams p;
    p.out = static_cast<const __nv_bfloat16*>(expert_out_bf16);
    p.pair_row = pair_row;
    p.shared = static_cast<const __nv_bfloat16*>(shared_bf16);
    p.y = static_cast<__nv_bfloat16*>(y_bf16);
    p.k = k;
    p.dim = dim;
    WUDA_CUDA(launch_pdl(moe_combine_kernel, dim3((dim / 8 + kCombineThreads - 1) / kCombineThreads, tokens), dim3(kCombineThreads), 0,
                         static_cast<cudaStream_t>(stream), p));
    return WUDA_OK;
}

extern "C" int64_t wuda_moe_ep2_inbox_bytes(int tokens_max, int dim) {
    using namespace wuda::moe;
    if (tokens_max < 1 || tokens_max > kEpMaxTokens || dim < 8 || dim % 8 != 0 || dim > kEpMaxDim) return -1;
    return kEpFlagBytes + 2ll * tokens_max * dim * 4;
}

extern "C" int wuda_moe_combine_ep2(const void* expert_out_bf16, const int32_t* pair_row, const void* shared_bf16,
                                    void* y_bf16, int tokens, int k, int dim, void* my_inbox, void* peer_inbox,
                                    int tokens_max, int epoch, int peer_wait_ms, int32_t* status_word, void* stream) {
    using namespace wuda;
    using namespace wuda::moe;
    clear_error();
    WUDA_REQUIRE(tokens >= 1 && k >= 1 && tokens <= tokens_max, "1 <= tokens <= tokens_max and k >= 1");
    WUDA_REQUIRE(wuda_moe_ep2_inbox_bytes(tokens_max, dim) > 0, "tokens_max must be in [1, %d] and dim a multiple of 8 up to %d",
                 kEpMaxTokens, kEpMaxDim);
    WUDA_REQUIRE(expert_out_bf16 && pair_row && y_bf16 && my_inbox && peer_inbox,
                 "expert_out, pair_row, y and both inboxes must not be NULL");
    WUDA_REQUIRE(aligned16(expert_out_bf16) && aligned16(shared_bf16) && aligned16(y_bf16) && aligned16(my_inbox) &&
                     aligned16(peer_inbox), "rows and inboxes must be 16-byte aligned");
    WUDA_REQUIRE(epoch >= 0, "epoch counts calls from 1, or is 0 for the link's own numbering (got %d)", epoch);
    WUDA_REQUIRE(peer_wait_ms >= 1 && peer_wait_ms <= 10000, "peer_wait_ms must be in [1, 10000] (got %d)", peer_wait_ms);
    CombineEpParams q;
    q.ctrl = reinterpret_cast<int32_t*>(static_cast<uint8_t*>(my_inbox) + kEpCtrlOffset);
    q.c.out = static_cast<const __nv_bfloat16*>(expert_out_bf16);
    q.c.pair_row = pair_row;
    q.c.shared = static_cast<const __nv_bfloat16*>(shared_bf16);
    q.c.y = static_cast<__nv_bfloat16*>(y_bf16);
    q.c.k = k;
    q.c.dim = dim;
    q.my_flags = static_cast<int32_t*>(my_inbox);
    q.peer_flags = static_cast<int32_t*>(peer_inbox);
    q.my_rows = reinterpret_cast<float*>(static_cast<uint8_t*>(my_inbox) + kEpFlagBytes);
    q.peer_rows = reinterpret_cast<float*>(static_cast<uint8_t*>(peer_inbox) + kEpFlagBytes);
    q.tokens_max = tokens_max;
    q.epoch = epoch;
    q.wait_ns = static_cast<unsigned long long>(peer_wait_ms) * 1000ull * 1000ull;
    q.status = status_word;
    WUDA_CUDA(launch_pdl(moe_combine_ep2_kernel, dim3(tokens), dim3((dim / 8 + 31) / 32 * 32), 0, static_cast<cudaStream_t>(stream), q));
    return WUDA_OK;
}
