// The two query-side tails that follow the q projection of a decode step.
//
// index_q_post: per (token, index head) row of 128 bf16 -> RoPE on the last 64 dims (rounded to
//   bf16) -> one scale per head, scale = max(amax / 448, 1e-12) -> e4m3, and the head weight folded
//   with that scale.  Torch twin: dsv4_megakernel/megakernel/test/test_wq_b_fp8_gemm.py:184-196
//   (ref_idx_fp8_chain); device counterpart include/idx_post_fp4.cuh:229-283.
// index_q_post_fp4: the FP4 form of the same tail: RoPE on the last 64 dims (rounded to bf16) -> Hadamard
//   transform of the 128 values (fp32 butterflies, strides 1, 2, ... 64 in that order; times 128^-1/2; one
//   rounding to bf16) -> per 32 values a power-of-two scale 2^ceil(log2(amax / 6)) as a biased exponent byte and
//   e2m1 codes (round to nearest even), two per byte, the four exponent bytes of a head as one word: the q / q_scales
//   operands of the MXFP4 MQA logits.  Device counterpart include/idx_post_fp4.cuh:79-224 (same order of the
//   butterflies, same constants), torch twin test/test_wq_b_fp8_gemm.py:161-182 (ref_idx_chain).
// query_rms_rope: per (token, head) row of 512 bf16 -> x * 1/sqrt(mean x^2 + eps) (no weight) ->
//   RoPE on the last 64 dims in fp32 -> one rounding to bf16.  Output head h reads input head
//   h % input_heads, which duplicates heads for a tensor-parallel consumer.  Counterpart:
//   include/query_rms_rope.cuh:20-61, kernels/rmsnorm_prod.cu:91-158.
//
// Both read rows straight out of the projection's output (a row stride is taken), so no slice
// is ever copied.  16 lanes own a 128-wide head (8 values = one 16-byte load per lane); a 512-wide
// row is one warp with two 16-byte loads per lane.
#include <cuda_bf16.h>

#include "host.h"

namespace wuda {
namespace qp {

constexpr int kThreads = 256;

__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

__device__ __forceinline__ void unpack8(const uint4& raw, float (&v)[8]) {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        v[2 * i] = __uint_as_float(w[i] << 16);
        v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    __nv_bfloat162 b = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&b);
}

__device__ __forceinline__ uint32_t pack_e4m3x4(float a, float b, float c, float d) {
    uint16_t lo, hi;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(lo) : "f"(b), "f"(a));
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(hi) : "f"(d), "f"(c));
    return static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
}

// rotates the 4 (even, odd) pairs in v; products and sums rounded separately
__device__ __forceinline__ void rotate8(float (&v)[8], const float* cos_row, const float* sin_row, int first_pair) {
    const float4 c = __ldg(reinterpret_cast<const float4*>(cos_row + first_pair));
    const float4 s = __ldg(reinterpret_cast<const float4*>(sin_row + first_pair));
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float ci = (&c.x)[i], si = (&s.x)[i];
        const float re = v[2 * i], im = v[2 * i + 1];
        v[2 * i] = __fsub_rn(__fmul_rn(re, ci), __fmul_rn(im, si));
        v[2 * i + 1] = __fadd_rn(__fmul_rn(re, si), __fmul_rn(im, ci));
    }
}

struct IndexParams {
    const __nv_bfloat16* x;
    int64_t row_stride;
    const int32_t* q_pos;
    const float* cos_t;
    const float* sin_t;
    int max_pos;
    const float* weights;
    uint8_t* q8;
    float* w_out;
    int64_t groups;   // tokens * heads
    int heads;
};

__global__ void __launch_bounds__(kThreads) index_q_post_kernel(IndexParams p) {
    pdl_launch_dependents();
    pdl_wait();   // nothing of global memory is touched before the kernel ahead has finished
    const int64_t g = (static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x) >> 4;   // (token, head)
    const int sub = threadIdx.x & 15;
    const bool live = g < p.groups;            // whole 16-lane groups are live or not
    const int64_t gg = live ? g : 0;
    const int64_t tok = gg / p.heads;
    const int head = static_cast<int>(gg - tok * p.heads);
    float v[8];
    unpack8(*reinterpret_cast<const uint4*>(p.x + tok * p.row_stride + head * 128 + sub * 8), v);
    if (sub >= 8) {
        int pos = p.q_pos[tok];
        pos = pos < 0 ? 0 : (pos >= p.max_pos ? p.max_pos - 1 : pos);
        rotate8(v, p.cos_t + static_cast<int64_t>(pos) * 32, p.sin_t + static_cast<int64_t>(pos) * 32, (sub - 8) * 4);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = bf16_round(v[i]);
    }
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
#pragma unroll
    for (int o = 1; o < 16; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if (!live) return;
    const float scale = fmaxf(__fdiv_rn(amax, 448.f), 1e-12f);
    const uint2 q = make_uint2(pack_e4m3x4(__fdiv_rn(v[0], scale), __fdiv_rn(v[1], scale), __fdiv_rn(v[2], scale),
                                            __fdiv_rn(v[3], scale)),
                               pack_e4m3x4(__fdiv_rn(v[4], scale), __fdiv_rn(v[5], scale), __fdiv_rn(v[6], scale),
                                            __fdiv_rn(v[7], scale)));
    *reinterpret_cast<uint2*>(p.q8 + g * 128 + sub * 8) = q;
    if (sub == 0) p.w_out[g] = p.weights ? __fmul_rn(p.weights[g], scale) : scale;
}

// two fp32 values (already divided by the block's power-of-two scale) -> two e2m1 codes in one byte, `lo` in the
// low nibble; round to nearest even, saturating
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

struct IndexFp4Params {
    const __nv_bfloat16* x;
    int64_t row_stride;
    const int32_t* q_pos;
    const float* cos_t;
    const float* sin_t;
    int max_pos;
    uint8_t* q4;          // [tokens, heads, 64]
    uint32_t* sf_words;   // [tokens, heads]
    int64_t groups;       // tokens * heads
    int heads;
};

// 16 lanes own a head, 8 consecutive values each: butterflies of strides 1, 2, 4 stay inside a lane, strides 8..64
// pair lanes sub ^ 1, 2, 4, 8; a block of 32 values is 4 lanes.
__global__ void __launch_bounds__(kThreads) index_q_post_fp4_kernel(IndexFp4Params p) {
    pdl_launch_dependents();
    pdl_wait();   // nothing of global memory is touched before the kernel ahead has finished
    const int64_t g = (static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x) >> 4;   // (token, head)
    const int sub = threadIdx.x & 15;
    const bool live = g < p.groups;            // whole 16-lane groups are live or not
    const int64_t gg = live ? g : 0;
    const int64_t tok = gg / p.heads;
    const int head = static_cast<int>(gg - tok * p.heads);
    float v[8];
    unpack8(*reinterpret_cast<const uint4*>(p.x + tok * p.row_stride + head * 128 + sub * 8), v);
    if (sub >= 8) {
        int pos = p.q_pos[tok];
        pos = pos < 0 ? 0 : (pos >= p.max_pos ? p.max_pos - 1 : pos);
        rotate8(v, p.cos_t + static_cast<int64_t>(pos) * 32, p.sin_t + static_cast<int64_t>(pos) * 32, (sub - 8) * 4);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = bf16_round(v[i]);
    }
#pragma unroll
    for (int s = 1; s < 8; s <<= 1)
#pragma unroll
        for (int i = 0; i < 8; ++i)
            if ((i & s) == 0) {
                const float a = v[i], b = v[i + s];
                v[i] = __fadd_rn(a, b);
                v[i + s] = __fsub_rn(a, b);
            }
#pragma unroll
    for (int x = 1; x < 16; x <<= 1) {
        const bool upper = (sub & x) != 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float other = __shfl_xor_sync(0xffffffffu, v[i], x);
            v[i] = upper ? __fsub_rn(other, v[i]) : __fadd_rn(v[i], other);
        }
    }
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        v[i] = bf16_round(__fmul_rn(v[i], 0.08838834764831845f));
        amax = fmaxf(amax, fabsf(v[i]));
    }
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    // the floor is the decimal 6 * 1.1754944e-38 of the reference kernel (one ulp above 6 * 2^-126)
    amax = fmaxf(amax, 7.052966400779935e-38f);
    const uint32_t rbits = __float_as_uint(__fmul_rn(amax, 1.0f / 6.0f));
    const int e = static_cast<int>((rbits >> 23) & 0xffu) - 127 + ((rbits & 0x7fffffu) ? 1 : 0);
    const float inv = __uint_as_float(static_cast<uint32_t>(127 - e) << 23);   // 2^-e, exact; e <= 127 - 3 for bf16 input
    uint32_t packed = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) packed |= pack_e2m1x2(v[2 * i] * inv, v[2 * i + 1] * inv) << (8 * i);
    uint32_t word = (sub & 3) == 0 ? static_cast<uint32_t>(e + 127) << (8 * (sub >> 2)) : 0u;
    word |= __shfl_xor_sync(0xffffffffu, word, 4);
    word |= __shfl_xor_sync(0xffffffffu, word, 8);
    if (!live) return;
    *reinterpret_cast<uint32_t*>(p.q4 + g * 64 + sub * 4) = packed;
    if (sub == 0) p.sf_words[g] = word;
}

struct QueryParams {
    const __nv_bfloat16* x;
    int64_t row_stride;
    const int64_t* positions;
    const float* cos_t;
    const float* sin_t;
    int max_pos;
    __nv_bfloat16* out;
    int64_t rows;   // tokens * out_heads
    int in_heads, out_heads;
    float eps;
};

__global__ void __launch_bounds__(kThreads) query_rms_rope_kernel(QueryParams p) {
    pdl_launch_dependents();
    pdl_wait();   // nothing of global memory is touched before the kernel ahead has finished
    const int64_t r = (static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x) >> 5;   // (token, out head)
    if (r >= p.rows) return;                   // whole warps
    const int lane = threadIdx.x & 31;
    const int64_t tok = r / p.out_heads;
    const int head = static_cast<int>(r - tok * p.out_heads);
    const uint4* src = reinterpret_cast<const uint4*>(p.x + tok * p.row_stride + (head % p.in_heads) * 512);
    float a[8], b[8];                          // columns [8 lane, +8) and [256 + 8 lane, +8)
    unpack8(src[lane], a);
    unpack8(src[32 + lane], b);
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) ss = __fmaf_rn(a[i], a[i], ss);
#pragma unroll
    for (int i = 0; i < 8; ++i) ss = __fmaf_rn(b[i], b[i], ss);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss = __fadd_rn(ss, __shfl_xor_sync(0xffffffffu, ss, o));
    const float scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, 512.f), p.eps)));
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        a[i] = __fmul_rn(a[i], scale);
        b[i] = __fmul_rn(b[i], scale);
    }
    if (lane >= 24) {                          // columns 448..511 sit in the second half, lanes 24..31
        int64_t pos = p.positions[tok];
        pos = pos < 0 ? 0 : (pos >= p.max_pos ? p.max_pos - 1 : pos);
        rotate8(b, p.cos_t + pos * 32, p.sin_t + pos * 32, (lane - 24) * 4);
    }
    uint4* dst = reinterpret_cast<uint4*>(p.out + r * 512);
    dst[lane] = make_uint4(pack_bf16x2(a[0], a[1]), pack_bf16x2(a[2], a[3]), pack_bf16x2(a[4], a[5]),
                           pack_bf16x2(a[6], a[7]));
    dst[32 + lane] = make_uint4(pack_bf16x2(b[0], b[1]), pack_bf16x2(b[2], b[3]), pack_bf16x2(b[4], b[5]),
                                pack_bf16x2(b[6], b[7]));
}

}  // namespace qp
}  // namespace wuda

extern "C" int wuda_index_q_post_fp8(const void* iq_bf16, int64_t row_stride, const int32_t* q_pos,
                                     const float* cos_table, const float* sin_table, int max_pos, const float* weights,
                                     void* q_fp8, float* weights_out, int tokens, int heads, void* stream) {
    using namespace wuda;
    using namespace wuda::qp;
    clear_error();
    WUDA_REQUIRE(tokens >= 0 && heads >= 1, "tokens must be >= 0 and heads >= 1");
    WUDA_REQUIRE(row_stride >= static_cast<int64_t>(heads) * 128 && row_stride % 8 == 0,
                 "row_stride must be >= heads * 128 and a multiple of 8 elements");
    WUDA_REQUIRE(max_pos >= 1, "max_pos must be >= 1");
    if (tokens == 0) return WUDA_OK;
    WUDA_REQUIRE(iq_bf16 && q_pos && cos_table && sin_table && q_fp8 && weights_out,
                 "iq, q_pos, the tables and both outputs must not be NULL");
    WUDA_REQUIRE(aligned16(iq_bf16) && aligned16(q_fp8) && aligned16(cos_table) && aligned16(sin_table),
                 "iq, q_fp8 and the tables must be 16-byte aligned");
    IndexParams p;
    p.x = static_cast<const __nv_bfloat16*>(iq_bf16);
    p.row_stride = row_stride;
    p.q_pos = q_pos;
    p.cos_t = cos_table;
    p.sin_t = sin_table;
    p.max_pos = max_pos;
    p.weights = weights;
    p.q8 = static_cast<uint8_t*>(q_fp8);
    p.w_out = weights_out;
    p.groups = static_cast<int64_t>(tokens) * heads;
    p.heads = heads;
    const int64_t blocks = (p.groups * 16 + kThreads - 1) / kThreads;
    WUDA_CUDA(launch_pdl(index_q_post_kernel, dim3(static_cast<unsigned>(blocks)), dim3(kThreads), 0, static_cast<cudaStream_t>(stream), p));
    return WUDA_OK;
}

extern "C" int wuda_index_q_post_fp4(const void* iq_bf16, int64_t row_stride, const int32_t* q_pos,
                                     const float* cos_table, const float* sin_table, int max_pos, void* q_fp4,
                                     void* q_scales, int tokens, int heads, void* stream) {
    using namespace wuda;
    using namespace wuda::qp;
    clear_error();
    WUDA_REQUIRE(tokens >= 0 && heads >= 1, "tokens must be >= 0 and heads >= 1");
    WUDA_REQUIRE(row_stride >= static_cast<int64_t>(heads) * 128 && row_stride % 8 == 0,
                 "row_stride must be >= heads * 128 and a multiple of 8 elements");
    WUDA_REQUIRE(max_pos >= 1, "max_pos must be >= 1");
    if (tokens == 0) return WUDA_OK;
    WUDA_REQUIRE(iq_bf16 && q_pos && cos_table && sin_table && q_fp4 && q_scales,
                 "iq, q_pos, the tables and both outputs must not be NULL");
    WUDA_REQUIRE(aligned16(iq_bf16) && aligned16(q_fp4) && aligned16(cos_table) && aligned16(sin_table) &&
                     (reinterpret_cast<uintptr_t>(q_scales) & 3u) == 0,
                 "iq, q_fp4 and the tables must be 16-byte aligned, q_scales 4-byte aligned");
    IndexFp4Params p;
    p.x = static_cast<const __nv_bfloat16*>(iq_bf16);
    p.row_stride = row_stride;
    p.q_pos = q_pos;
    p.cos_t = cos_table;
    p.sin_t = sin_table;
    p.max_pos = max_pos;
    p.q4 = static_cast<uint8_t*>(q_fp4);
    p.sf_words = static_cast<uint32_t*>(q_scales);
    p.groups = static_cast<int64_t>(tokens) * heads;
    p.heads = heads;
    const int64_t blocks = (p.groups * 16 + kThreads - 1) / kThreads;
    WUDA_CUDA(launch_pdl(index_q_post_fp4_kernel, dim3(static_cast<unsigned>(blocks)), dim3(kThreads), 0,
                         static_cast<cudaStream_t>(stream), p));
    return WUDA_OK;
}

namespace wuda {
namespace qp {
// Sum of squares of every 512-value head of bf16 rows, one warp per head (kernels/wq_b_fp8_gemm.cu:101-123): lane l
// chains fused multiply-adds over values [16 l, 16 l + 16), then a butterfly over lane distances 16, 8, 4, 2, 1.
__global__ void __launch_bounds__(256) head_ssq_kernel(const __nv_bfloat16* y, int64_t row_stride, float* ssq, int64_t total, int heads) {
    pdl_launch_dependents();
    pdl_wait();
    const int64_t h = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
    if (h >= total) return;
    const int lane = threadIdx.x & 31;
    const int64_t row = h / heads;
    const __nv_bfloat16* src = y + row * row_stride + (h - row * heads) * 512 + lane * 16;
    const uint4 a = *reinterpret_cast<const uint4*>(src), b = *reinterpret_cast<const uint4*>(src + 8);
    const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float lo = __uint_as_float(w[i] << 16), hi = __uint_as_float(w[i] & 0xffff0000u);
        s = __fmaf_rn(lo, lo, s);
        s = __fmaf_rn(hi, hi, s);
    }
#pragma unroll
    for (int x = 16; x >= 1; x >>= 1) s = __fadd_rn(s, __shfl_xor_sync(0xffffffffu, s, x));
    if (lane == 0) ssq[h] = s;
}
}  // namespace qp
}  // namespace wuda

extern "C" int wuda_head_ssq(const void* y_bf16, int64_t row_stride, float* ssq, int64_t rows, int heads, void* stream) {
    using namespace wuda;
    using namespace wuda::qp;
    clear_error();
    WUDA_REQUIRE(rows >= 0 && heads >= 1, "rows must be >= 0 and heads >= 1");
    WUDA_REQUIRE(row_stride >= static_cast<int64_t>(heads) * 512 && row_stride % 8 == 0,
                 "row_stride must be >= heads * 512 and a multiple of 8 elements");
    if (rows == 0) return WUDA_OK;
    WUDA_REQUIRE(y_bf16 && ssq && aligned16(y_bf16), "y (16-byte aligned) and ssq must not be NULL");
    const int64_t total = rows * heads;
    WUDA_REQUIRE((total + 7) / 8 <= 0x7fffffff, "too many heads for one launch");
    WUDA_CUDA(launch_pdl(head_ssq_kernel, dim3(static_cast<unsigned>((total + 7) / 8)), dim3(256), 0,
                         static_cast<cudaStream_t>(stream), static_cast<const __nv_bfloat16*>(y_bf16), row_stride, ssq, total, heads));
    return WUDA_OK;
}

extern "C" int wuda_query_rms_rope(const void* x_bf16, int64_t row_stride, const int64_t* positions,
                                   const float* cos_table, const float* sin_table, int max_pos, void* out_bf16,
                                   int tokens, int input_heads, int output_heads, float eps, void* stream) {
    using namespace wuda;
    using namespace wuda::qp;
    clear_error();
    WUDA_REQUIRE(tokens >= 0 && input_heads >= 1 && output_heads >= input_heads && output_heads % input_heads == 0,
                 "tokens must be >= 0 and output_heads a positive multiple of input_heads");
    WUDA_REQUIRE(row_stride >= static_cast<int64_t>(input_heads) * 512 && row_stride % 8 == 0,
                 "row_stride must be >= input_heads * 512 and a multiple of 8 elements");
    WUDA_REQUIRE(max_pos >= 1, "max_pos must be >= 1");
    if (tokens == 0) return WUDA_OK;
    WUDA_REQUIRE(x_bf16 && positions && cos_table && sin_table && out_bf16, "no argument may be NULL");
    WUDA_REQUIRE(aligned16(x_bf16) && aligned16(out_bf16) && aligned16(cos_table) && aligned16(sin_table),
                 "x, out and the tables must be 16-byte aligned");
    QueryParams p;
    p.x = static_cast<const __nv_bfloat16*>(x_bf16);
    p.row_stride = row_stride;
    p.positions = positions;
    p.cos_t = cos_table;
    p.sin_t = sin_table;
    p.max_pos = max_pos;
    p.out = static_cast<__nv_bfloat16*>(out_bf16);
    p.rows = static_cast<int64_t>(tokens) * output_heads;
    p.in_heads = input_heads;
    p.out_heads = output_heads;
    p.eps = eps;
    const int64_t blocks = (p.rows * 32 + kThreads - 1) / kThreads;
    WUDA_CUDA(launch_pdl(query_rms_rope_kernel, dim3(static_cast<unsigned>(blocks)), dim3(kThreads), 0, static_cast<cudaStream_t>(stream), p));
    return WUDA_OK;
}
