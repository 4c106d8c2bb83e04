// The three cache writers of a decode step in ONE launch:
//   indexer compressor  state ring [kv 256 | score 256] -> 128 e4m3 + one fp32 scale in the
//                       indexer page format the MQA-logits kernel reads
//   MAIN compressor     state ring [kv 1024 | score 1024] -> a 584-byte MODEL1 record
//   window KV           fp32 row of 512 -> a 584-byte MODEL1 record
// Numerics follow the reference's torch twins (dsv4_megakernel/megakernel/test/
// test_wq_b_fp8_gemm.py:550-586 ref_comp_step with fp8=True, :646-665 ref_win_step, and the
// inline MAIN reference in test_mqa_logits_fp4.py:769-789); device-side counterparts are
// include/idx_comp_fp4.cuh:97-201 and :282-383, include/mqa_logits_fp8.cuh:133-284.
//
// A compressor row works on rows with (pos + 1) % 4 == 0 only: the 8 ring entries ending at the
// current one are combined column-wise by a softmax over their scores (the older four entries
// contribute their first half, the newer four their second half), rounded to bf16, RMS-normalised
// with a weight, rounded to bf16, rotated on the last 64 dims at position pos - 3 and quantised.
// The op is latency-bound (a few hundred KB for 64 rows): one thread owns 4 columns, so each row
// is 32 (indexer) or 128 (MAIN, window) threads that issue all their 16 loads before any math,
// and the three writers share a launch (blockIdx.y = writer).
//
// MODEL1 record of token slot `off` in a page: body at off * 576 (448 e4m3 bytes, then 64 bf16),
// scale bytes at entries_per_block * 576 + off * 8 (7 bytes, one biased power-of-two exponent per
// 64 columns; the 8th byte is not written).
#include <cuda_bf16.h>

#include "host.h"

namespace wuda {
namespace cw {

constexpr int kThreads = 128;
constexpr int kRopeDim = 64;
constexpr int kRatio = 4;
constexpr int kWindowRows = 8;
constexpr int kM1Body = 576, kM1Nope = 448, kM1ScaleBytes = 8;

struct Params {
    wuda_cache_writers a;
    int rows;
    int idx_fp4;      // the indexer entry is an MXFP4 record (64 code bytes + 4 exponent bytes) instead of 128 e4m3 + fp32
    int32_t* status;
};

__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

__device__ __forceinline__ uint32_t pack_e4m3x4(float a, float b, float c, float d) {
    uint16_t lo, hi;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(lo) : "f"(b), "f"(a));
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(hi) : "f"(d), "f"(c));
    return static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
}

// two fp32 values -> two e2m1 codes in one byte, `lo` in the low nibble; round to nearest even, saturating
__device__ __forceinline__ uint32_t pack_e2m1x2(float lo, float hi) {
    uint32_t out;
    asm("{\n\t"
        ".reg .b8 b;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 b, %2, %1;\n\t"
        "cvt.u32.u8 %0, b;\n\t"
        "}\n"
        : "=r"(out)
        : "f"(lo), "f"(hi));
    return out;
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    __nv_bfloat162 b = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&b);
}

// smallest e with 2^e >= x, for normal positive x
__device__ __forceinline__ int log2_ceil(float x) {
    const uint32_t bits = __float_as_uint(x);
    return static_cast<int>((bits >> 23) & 0xff) - 127 + ((bits & 0x7fffffu) ? 1 : 0);
}

// 1 / sqrt(x) as two correctly rounded operations, the way a CPU evaluates it
__device__ __forceinline__ float inv_sqrt(float x) { return __fdiv_rn(1.0f, __fsqrt_rn(x)); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// max over the 16 lanes that share one 64-column block (4 columns per lane)
__device__ __forceinline__ float block64_max(float v) {
#pragma unroll
    for (int o = 1; o < 16; o <<= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

__device__ __forceinline__ void report(int32_t* status, int code) {
    if (status) atomicCAS(status, 0, code);
}

// Page and slot of a flat destination; nullptr when there is nothing to write or it is out of range.
__device__ __forceinline__ uint8_t* locate(uint8_t* pool, const int64_t* dst, int row, int epb, int64_t stride,
                                           int num_blocks, int32_t* status, int* off) {
    if (!pool || !dst) return nullptr;
    const int64_t d = dst[row];
    if (d < 0) return nullptr;
    const int64_t page = d / epb;
    if (page >= num_blocks) {
        report(status, WUDA_DEV_BAD_DESTINATION);
        return nullptr;
    }
    *off = static_cast<int>(d - page * epb);
    return pool + page * stride;
}

// Rotation of the two (even, odd) pairs a thread holds; each product and each sum is rounded once.
__device__ __forceinline__ void rotate4(float (&v)[4], const float* cos_row, const float* sin_row, int first_pair,
                                        bool round_bf16) {
#pragma unroll
    for (int e = 0; e < 4; e += 2) {
        const float c = __ldg(cos_row + first_pair + e / 2), s = __ldg(sin_row + first_pair + e / 2);
        const float ev = v[e], od = v[e + 1];
        const float re = __fsub_rn(__fmul_rn(ev, c), __fmul_rn(od, s));
        const float im = __fadd_rn(__fmul_rn(ev, s), __fmul_rn(od, c));
        v[e] = round_bf16 ? bf16_round(re) : re;
        v[e + 1] = round_bf16 ? bf16_round(im) : im;
    }
}

// Writes 4 columns of a MODEL1 record (and of the compact outputs) from 4 final values.
__device__ __forceinline__ void store_model1(const float (&v)[4], int col, int lane, uint8_t* page, int off, int epb,
                                             uint8_t* q8, float* s8, __nv_bfloat16* rope, int row) {
    // every lane takes part in the shuffle (the last 16 lanes of the row only lend their lanes)
    const float amax = block64_max(fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3]))));
    if (col < kM1Nope) {
        const int e = log2_ceil(fmaxf(__fdiv_rn(amax, 448.0f), 1e-4f));
        const float inv = __uint_as_float(static_cast<uint32_t>(127 - e) << 23);   // 2^-e, exact
        const uint32_t packed = pack_e4m3x4(v[0] * inv, v[1] * inv, v[2] * inv, v[3] * inv);
        if (q8) *reinterpret_cast<uint32_t*>(q8 + static_cast<int64_t>(row) * kM1Nope + col) = packed;
        if (s8 && (lane & 15) == 0)
            s8[static_cast<int64_t>(row) * 7 + (col >> 6)] = __uint_as_float(static_cast<uint32_t>(e + 127) << 23);
        if (page) {
            *reinterpret_cast<uint32_t*>(page + off * kM1Body + col) = packed;
            if ((lane & 15) == 0)
                page[static_cast<int64_t>(epb) * kM1Body + off * kM1ScaleBytes + (col >> 6)] =
                    static_cast<uint8_t>(e + 127);
        }
    } else {
        const uint2 pk = make_uint2(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]));
        const int rc = col - kM1Nope;
        if (rope) *reinterpret_cast<uint2*>(rope + static_cast<int64_t>(row) * kRopeDim + rc) = pk;
        if (page) *reinterpret_cast<uint2*>(page + off * kM1Body + kM1Nope + rc * 2) = pk;
    }
}

// Softmax-weighted sum of the 8-entry window for the 4 columns starting at `col`.
// HALF is the width of one half of the kv (and of the score) part of a state entry.
template <int HALF>
__device__ __forceinline__ void window_sum(const float* block_base, int current, int ring, int col, float (&out)[4]) {
    constexpr int kEntry = 4 * HALF;   // [kv 2*HALF | score 2*HALF]
    int first = current - (kWindowRows - 1);
    if (first < 0) first += ring;
    float4 sc[kWindowRows], kv[kWindowRows];
#pragma unroll
    for (int r = 0; r < kWindowRows; ++r) {
        int phys = first + r;
        if (phys >= ring) phys -= ring;
        const float* entry = block_base + static_cast<int64_t>(phys) * kEntry + (r < kRatio ? col : HALF + col);
        kv[r] = *reinterpret_cast<const float4*>(entry);
        sc[r] = *reinterpret_cast<const float4*>(entry + 2 * HALF);
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        float mx = (&sc[0].x)[e];
#pragma unroll
        for (int r = 1; r < kWindowRows; ++r) mx = fmaxf(mx, (&sc[r].x)[e]);
        float den = 0.f, num = 0.f;
#pragma unroll
        for (int r = 0; r < kWindowRows; ++r) {
            const float w = expf((&sc[r].x)[e] - mx);
            den = __fadd_rn(den, w);
            num = __fadd_rn(num, __fmul_rn(w, (&kv[r].x)[e]));
        }
        out[e] = __fdiv_rn(num, den);
    }
}

__device__ __forceinline__ bool compress_row(const int64_t* pos, int row, int64_t* p) {
    *p = pos[row];
    return ((*p + 1) & (kRatio - 1)) == 0;
}

__device__ __forceinline__ int64_t clamp_pos(int64_t p, int max_pos) {
    return p < 0 ? 0 : (p >= max_pos ? max_pos - 1 : p);
}

// ---- indexer compressor: one warp per row, 4 rows per CTA
__device__ void indexer_rows(const Params& P) {
    const wuda_compressor_bundle& b = P.a.indexer;
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * 4 + (threadIdx.x >> 5);
    if (row >= P.rows) return;
    int64_t p;
    if (!compress_row(P.a.pos, row, &p)) return;
    const int64_t srow = b.state_row[row];
    if (srow < 0) return;
    if (srow >= b.state_rows_total) {
        if (lane == 0) report(P.status, WUDA_DEV_BAD_STATE_ROW);
        return;
    }
    const int current = static_cast<int>(srow % b.ring_entries);
    const int col = lane * 4;
    float v[4];
    window_sum<128>(b.state + (srow - current) * 512, current, b.ring_entries, col, v);

    float ssq = 0.f;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        v[e] = bf16_round(v[e]);
        ssq = __fadd_rn(ssq, __fmul_rn(v[e], v[e]));
    }
    ssq = warp_sum(ssq);
    const float rms = inv_sqrt(__fadd_rn(__fdiv_rn(ssq, 128.f), P.a.eps));
    const float4 nw = __ldg(reinterpret_cast<const float4*>(b.norm_w) + lane);
#pragma unroll
    for (int e = 0; e < 4; ++e) v[e] = bf16_round(__fmul_rn(__fmul_rn(v[e], rms), (&nw.x)[e]));
    if (col >= 128 - kRopeDim) {
        const int64_t rp = clamp_pos(p + 1 - kRatio, P.a.max_pos);
        rotate4(v, P.a.cos_table + rp * (kRopeDim / 2), P.a.sin_table + rp * (kRopeDim / 2), (col - 64) / 2, true);
    }
    if (P.idx_fp4) {
        // The FP4 form (include/idx_comp_fp4.cuh:239-274): Hadamard transform as fp32 butterflies with strides 1, 2
        // (inside the lane's 4 values), then 4 .. 64 (lanes l ^ 1 .. l ^ 16), times 128^-1/2, one rounding to bf16;
        // per 32 values (8 lanes) the scale 2^ceil(log2(amax / 6)) and e2m1 codes.
        const float t0 = __fadd_rn(v[0], v[1]), t1 = __fsub_rn(v[0], v[1]);
        const float t2 = __fadd_rn(v[2], v[3]), t3 = __fsub_rn(v[2], v[3]);
        v[0] = __fadd_rn(t0, t2), v[1] = __fadd_rn(t1, t3), v[2] = __fsub_rn(t0, t2), v[3] = __fsub_rn(t1, t3);
#pragma unroll
        for (int x = 1; x < 32; x <<= 1) {
            const bool upper = (lane & x) != 0;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float other = __shfl_xor_sync(0xffffffffu, v[e], x);
                v[e] = upper ? __fsub_rn(other, v[e]) : __fadd_rn(v[e], other);
            }
        }
        float amax4 = 0.f;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            v[e] = bf16_round(__fmul_rn(v[e], 0.088388347648318447f));
            amax4 = fmaxf(amax4, fabsf(v[e]));
        }
#pragma unroll
        for (int o = 4; o > 0; o >>= 1) amax4 = fmaxf(amax4, __shfl_xor_sync(0xffffffffu, amax4, o));
        amax4 = fmaxf(amax4, 6.0f * 1.1754944e-38f);
        const int se = log2_ceil(__fmul_rn(amax4, 1.0f / 6.0f));
        const float inv = __uint_as_float(static_cast<uint32_t>(127 - se) << 23);   // 2^-se, exact
        const uint16_t codes = static_cast<uint16_t>(pack_e2m1x2(v[0] * inv, v[1] * inv) |
                                                     (pack_e2m1x2(v[2] * inv, v[3] * inv) << 8));
        uint8_t* q4 = b.q8;                                   // compact outputs: [rows, 64] codes, [rows, 4] exponent bytes
        uint8_t* s4 = reinterpret_cast<uint8_t*>(b.s8);
        if (q4) *reinterpret_cast<uint16_t*>(q4 + static_cast<int64_t>(row) * 64 + lane * 2) = codes;
        if (s4 && (lane & 7) == 0) s4[static_cast<int64_t>(row) * 4 + (lane >> 3)] = static_cast<uint8_t>(se + 127);
        int off4 = 0;
        uint8_t* page4 = locate(b.pool, b.dst, row, b.entries_per_block, b.block_stride_bytes, b.num_blocks,
                                lane == 0 ? P.status : nullptr, &off4);
        if (page4) {
            *reinterpret_cast<uint16_t*>(page4 + off4 * 64 + lane * 2) = codes;
            if ((lane & 7) == 0)
                page4[static_cast<int64_t>(b.entries_per_block) * 64 + off4 * 4 + (lane >> 3)] = static_cast<uint8_t>(se + 127);
        }
        return;
    }
    float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float scale = fmaxf(__fdiv_rn(amax, 448.f), 1e-12f);
    const uint32_t packed = pack_e4m3x4(__fdiv_rn(v[0], scale), __fdiv_rn(v[1], scale), __fdiv_rn(v[2], scale),
                                        __fdiv_rn(v[3], scale));
    if (b.q8) *reinterpret_cast<uint32_t*>(b.q8 + static_cast<int64_t>(row) * 128 + col) = packed;
    if (b.s8 && lane == 0) b.s8[row] = scale;
    int off = 0;
    uint8_t* page = locate(b.pool, b.dst, row, b.entries_per_block, b.block_stride_bytes, b.num_blocks,
                           lane == 0 ? P.status : nullptr, &off);
    if (page) {
        *reinterpret_cast<uint32_t*>(page + off * 128 + col) = packed;
        if (lane == 0) *reinterpret_cast<float*>(page + static_cast<int64_t>(b.entries_per_block) * 128 + off * 4) = scale;
    }
}

// ---- MAIN compressor: one CTA (4 warps x 128 columns) per row
__device__ void main_row(const Params& P, float* warp_ssq) {
    const wuda_compressor_bundle& b = P.a.main;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int row = blockIdx.x;
    int64_t p;
    if (!compress_row(P.a.pos, row, &p)) return;       // uniform over the CTA
    const int64_t srow = b.state_row[row];
    if (srow < 0) return;
    if (srow >= b.state_rows_total) {
        if (threadIdx.x == 0) report(P.status, WUDA_DEV_BAD_STATE_ROW);
        return;
    }
    const int current = static_cast<int>(srow % b.ring_entries);
    const int col = threadIdx.x * 4;
    float v[4];
    window_sum<512>(b.state + (srow - current) * 2048, current, b.ring_entries, col, v);

    float ssq = 0.f;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        v[e] = bf16_round(v[e]);
        ssq = __fadd_rn(ssq, __fmul_rn(v[e], v[e]));
    }
    ssq = warp_sum(ssq);
    if (lane == 0) warp_ssq[warp] = ssq;
    __syncthreads();
    const float total = __fadd_rn(__fadd_rn(__fadd_rn(warp_ssq[0], warp_ssq[1]), warp_ssq[2]), warp_ssq[3]);
    const float rms = inv_sqrt(__fadd_rn(__fdiv_rn(total, 512.f), P.a.eps));
    const float4 nw = __ldg(reinterpret_cast<const float4*>(b.norm_w) + threadIdx.x);
#pragma unroll
    for (int e = 0; e < 4; ++e) v[e] = bf16_round(__fmul_rn(__fmul_rn(v[e], rms), (&nw.x)[e]));
    if (col >= kM1Nope) {
        const int64_t rp = clamp_pos(p + 1 - kRatio, P.a.max_pos);
        rotate4(v, P.a.cos_table + rp * (kRopeDim / 2), P.a.sin_table + rp * (kRopeDim / 2), (col - kM1Nope) / 2, true);
    }
    int off = 0;
    uint8_t* page = locate(b.pool, b.dst, row, b.entries_per_block, b.block_stride_bytes, b.num_blocks,
                           threadIdx.x == 0 ? P.status : nullptr, &off);
    store_model1(v, col, lane, page, off, b.entries_per_block, b.q8, b.s8, static_cast<__nv_bfloat16*>(b.rope), row);
}

// ---- window KV: every row; one CTA per row
__device__ void window_row(const Params& P, float* warp_ssq) {
    const wuda_window_bundle& b = P.a.window;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int row = blockIdx.x;
    const int col = threadIdx.x * 4;
    const float4 x = *(reinterpret_cast<const float4*>(b.y + static_cast<int64_t>(row) * 512) + threadIdx.x);
    float v[4] = {x.x, x.y, x.z, x.w};
    float ssq = 0.f;
#pragma unroll
    for (int e = 0; e < 4; ++e) ssq = __fadd_rn(ssq, __fmul_rn(v[e], v[e]));
    ssq = warp_sum(ssq);
    if (lane == 0) warp_ssq[warp] = ssq;
    __syncthreads();
    const float total = __fadd_rn(__fadd_rn(__fadd_rn(warp_ssq[0], warp_ssq[1]), warp_ssq[2]), warp_ssq[3]);
    const float rms = inv_sqrt(__fadd_rn(__fdiv_rn(total, 512.f), P.a.eps));
    const float4 nw = __ldg(reinterpret_cast<const float4*>(b.norm_w) + threadIdx.x);
#pragma unroll
    for (int e = 0; e < 4; ++e) v[e] = __fmul_rn(__fmul_rn(v[e], rms), (&nw.x)[e]);
    if (col < kM1Nope) {
#pragma unroll
        for (int e = 0; e < 4; ++e) v[e] = bf16_round(v[e]);
    } else {
        const int64_t rp = clamp_pos(P.a.pos[row], P.a.max_pos);
        rotate4(v, P.a.cos_table + rp * (kRopeDim / 2), P.a.sin_table + rp * (kRopeDim / 2), (col - kM1Nope) / 2, false);
    }
    int off = 0;
    uint8_t* page = locate(b.pool, b.dst, row, b.entries_per_block, b.block_stride_bytes, b.num_blocks,
                           threadIdx.x == 0 ? P.status : nullptr, &off);
    store_model1(v, col, lane, page, off, b.entries_per_block, b.q8, b.s8, static_cast<__nv_bfloat16*>(b.rope), row);
}

__global__ void __launch_bounds__(kThreads) cache_writers_kernel(const __grid_constant__ Params P) {
    pdl_launch_dependents();
    pdl_wait();   // nothing of global memory is touched before the kernel ahead has finished
    __shared__ float warp_ssq[4];
    if (blockIdx.y == 0) {
        if (P.a.main.state) main_row(P, warp_ssq);
    } else if (blockIdx.y == 1) {
        if (P.a.window.y) window_row(P, warp_ssq);
    } else {
        if (P.a.indexer.state && blockIdx.x * 4 < P.rows) indexer_rows(P);
    }
}

int check_pool(const char* who, const uint8_t* pool, const int64_t* dst, int epb, int64_t stride, int num_blocks,
               int record_bytes, int scale_bytes) {
    if (!pool) return WUDA_OK;
    WUDA_REQUIRE(dst, "%s: a pool needs its destination array", who);
    WUDA_REQUIRE(epb >= 1 && num_blocks >= 1, "%s: entries_per_block and num_blocks must be >= 1", who);
    WUDA_REQUIRE(stride >= static_cast<int64_t>(epb) * (record_bytes + scale_bytes),
                 "%s: block stride %lld does not cover %d entries", who, static_cast<long long>(stride), epb);
    WUDA_REQUIRE(stride % 4 == 0 && (reinterpret_cast<uintptr_t>(pool) & 15u) == 0 &&
                     (static_cast<int64_t>(epb) * record_bytes) % 4 == 0,
                 "%s: pool must be 16-byte aligned with a stride that is a multiple of 4", who);
    return WUDA_OK;
}

int check_compressor(const char* who, const wuda_compressor_bundle& b, int record_bytes, int scale_bytes) {
    if (!b.state) return WUDA_OK;
    WUDA_REQUIRE(b.state_row && b.norm_w, "%s: state_row and norm_w are required with state", who);
    WUDA_REQUIRE(b.ring_entries >= kWindowRows, "%s: the state ring must hold at least 8 entries (got %d)", who,
                 b.ring_entries);
    WUDA_REQUIRE(b.state_rows_total >= b.ring_entries && b.state_rows_total % b.ring_entries == 0,
                 "%s: state_rows_total must be a positive multiple of ring_entries", who);
    WUDA_REQUIRE(aligned16(b.state) && aligned16(b.norm_w) && aligned16(b.q8) && aligned16(b.rope),
                 "%s: state, norm_w and the compact outputs must be 16-byte aligned", who);
    return check_pool(who, b.pool, b.dst, b.entries_per_block, b.block_stride_bytes, b.num_blocks, record_bytes,
                      scale_bytes);
}

}  // namespace cw
}  // namespace wuda

namespace wuda {
namespace cw {
int launch_writers(const wuda_cache_writers* args, int rows, int idx_fp4, int32_t* status_word, void* stream);
}
}  // namespace wuda

extern "C" int wuda_cache_writers_fp8(const wuda_cache_writers* args, int rows, int32_t* status_word, void* stream) {
    wuda::clear_error();
    return wuda::cw::launch_writers(args, rows, 0, status_word, stream);
}

extern "C" int wuda_cache_writers_fp4(const wuda_cache_writers* args, int rows, int32_t* status_word, void* stream) {
    wuda::clear_error();
    return wuda::cw::launch_writers(args, rows, 1, status_word, stream);
}

int wuda::cw::launch_writers(const wuda_cache_writers* args, int rows, int idx_fp4, int32_t* status_word, void* stream) {
    using namespace wuda;
    using namespace wuda::cw;
    WUDA_REQUIRE(args, "args must not be NULL");
    WUDA_REQUIRE(rows >= 0, "rows must be >= 0 (got %d)", rows);
    if (rows == 0) return WUDA_OK;
    WUDA_REQUIRE(args->indexer.state || args->main.state || args->window.y, "no writer is enabled");
    WUDA_REQUIRE(args->pos && args->cos_table && args->sin_table && args->max_pos >= 1,
                 "pos, the cos/sin tables and max_pos >= 1 are required");
    int st = check_compressor("indexer", args->indexer, idx_fp4 ? 64 : 128, 4);
    if (st != WUDA_OK) return st;
    st = check_compressor("main", args->main, kM1Body, kM1ScaleBytes);
    if (st != WUDA_OK) return st;
    const wuda_window_bundle& w = args->window;
    if (w.y) {
        WUDA_REQUIRE(w.norm_w && aligned16(w.y) && aligned16(w.norm_w) && aligned16(w.q8) && aligned16(w.rope),
                     "window: norm_w is required; y, norm_w and the compact outputs must be 16-byte aligned");
        st = check_pool("window", w.pool, w.dst, w.entries_per_block, w.block_stride_bytes, w.num_blocks, kM1Body,
                        kM1ScaleBytes);
        if (st != WUDA_OK) return st;
    }
    Params p;
    p.a = *args;
    p.rows = rows;
    p.idx_fp4 = idx_fp4;
    p.status = status_word;
    const dim3 grid(rows, 3);
    WUDA_CUDA(launch_pdl(cache_writers_kernel, dim3(grid), dim3(kThreads), 0, static_cast<cudaStream_t>(stream), p));
    return WUDA_OK;
}
