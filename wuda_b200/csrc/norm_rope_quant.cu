// Single-pass RMSNorm / partial RoPE / 1x128 FP8 quantisation kernels for sm_100a.
//
// Numerics follow the origin model (paths relative to dsv4_megakernel/origin/):
//   RMSNorm            model.py:191-196   y = bf16(gamma * (x * rsqrt(mean(x^2) + eps))), fp32 math
//   RoPE               model.py:232-244   interleaved pairs (re, im) * (cos + i sin), conjugate when
//                                         inverse, result rounded back to bf16
//   FP8 quantisation   kernel.py:40-125   per 128 elements: amax = max(|x|, 1e-4), scale = amax / 448
//                                         or 2^ceil(log2(amax / 448)); y = e4m3(clamp(x / scale))
// and stand in for the reference's fused producers: qnorm_quant_kernel
// (megakernel/kernels/wq_b_fp8_gemm.cu:139-183), the attn_norm + quant tail of
// hc_reduce_and_fuse_kernel (megakernel/kernels/hc_fused_kernel_tc.cu:319-335), the
// indexer-q post (megakernel/include/idx_post_fp4.cuh:229-283) and inv_rope_quant
// (megakernel/kernels/mla_o_inv_rope_quant.cu:43-157).
//
// Both kernels are HBM-bound and tiny at decode sizes: one CTA per row, every thread owns
// 8 consecutive elements (one 16-byte load), 16 neighbouring threads own one 128-element
// quantisation group and find its amax with shuffles; the row is read once and stays in
// registers.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "host.h"

namespace wuda {
namespace nrq {

constexpr int kMaxChunks = 3;   // 16-byte chunks per thread (rows up to 3 * 1024 * 8 = 24576 elements)

__device__ __forceinline__ uint32_t pack_e4m3x4(float a, float b, float c, float d) {
    uint16_t lo, hi;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(lo) : "f"(b), "f"(a));
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(hi) : "f"(d), "f"(c));
    return static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
}

__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

__device__ __forceinline__ float group_scale(float amax, int pow2) {
    amax = fmaxf(amax, 1e-4f);
    const float s = amax * (1.0f / 448.0f);
    if (!pow2) return s;
    const uint32_t bits = __float_as_uint(s);
    const int e = static_cast<int>((bits >> 23) & 0xFF) - 127 + ((bits & 0x7FFFFFu) != 0 ? 1 : 0);
    return __uint_as_float(static_cast<uint32_t>(e + 127) << 23);
}

// Quantises the 8 values of this thread; the 16 threads of a 128-element group share amax.
__device__ __forceinline__ void quant_store8(const float (&v)[8], int pow2, uint8_t* out8, float* scale_out,
                                             bool group_leader) {
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
    // only the 16 lanes of this group take part: the other half-warp may be past the row's end
    const uint32_t group_mask = 0xFFFFu << (threadIdx.x & 16);
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(group_mask, amax, o));
    const float s = group_scale(amax, pow2);
    float q[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) q[i] = fminf(fmaxf(__fdiv_rn(v[i], s), -448.f), 448.f);
    uint2 packed;
    packed.x = pack_e4m3x4(q[0], q[1], q[2], q[3]);
    packed.y = pack_e4m3x4(q[4], q[5], q[6], q[7]);
    *reinterpret_cast<uint2*>(out8) = packed;
    if (group_leader && scale_out) *scale_out = s;
}

__device__ __forceinline__ void unpack8(const uint4& raw, float (&v)[8]) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h[i]);
        v[2 * i] = f.x;
        v[2 * i + 1] = f.y;
    }
}
__device__ __forceinline__ uint4 pack8(const float (&v)[8]) {
    uint4 raw;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    return raw;
}

struct NormParams {
    const __nv_bfloat16* x;
    int64_t x_stride;
    const void* gamma;      // nullptr: no normalisation (plain quantisation of x)
    int gamma_is_bf16;
    float eps;
    __nv_bfloat16* y_bf16;  // nullable
    uint8_t* y_fp8;         // nullable
    float* y_scales;        // nullable
    int rows, dim, pow2;
};

__global__ void __launch_bounds__(1024, 1) rmsnorm_quant_kernel(const NormParams p) {
    pdl_launch_dependents();
    pdl_wait();   // nothing of global memory is touched before the kernel ahead has finished
    __shared__ float warp_part[32];
    __shared__ float total;
    const int row = blockIdx.x;
    const int chunks = p.dim >> 3;                     // 16-byte chunks in the row
    const __nv_bfloat16* x = p.x + static_cast<int64_t>(row) * p.x_stride;
    float v[kMaxChunks][8];
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < kMaxChunks; ++c) {
        const int ch = c * blockDim.x + threadIdx.x;
        if (ch < chunks) {
            unpack8(*reinterpret_cast<const uint4*>(x + 8 * ch), v[c]);
#pragma unroll
            for (int i = 0; i < 8; ++i) ss = fmaf(v[c][i], v[c][i], ss);
        }
    }
    float rs = 1.f;
    if (p.gamma) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if ((threadIdx.x & 31) == 0) warp_part[threadIdx.x >> 5] = ss;
        __syncthreads();
        if (threadIdx.x < 32) {
            float t = threadIdx.x < (blockDim.x >> 5) ? warp_part[threadIdx.x] : 0.f;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
            if (threadIdx.x == 0) total = t;
        }
        __syncthreads();
        rs = __fdiv_rn(1.0f, __fsqrt_rn(total / static_cast<float>(p.dim) + p.eps));
    }
#pragma unroll
    for (int c = 0; c < kMaxChunks; ++c) {
        const int ch = c * blockDim.x + threadIdx.x;
        if (ch < chunks) {   // uniform for the 16 threads of a group: dim is a multiple of 128
            if (p.gamma) {
                float g[8];
                if (p.gamma_is_bf16) {
                    unpack8(*reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(p.gamma) + 8 * ch), g);
                } else {
                    const float4* g4 = reinterpret_cast<const float4*>(static_cast<const float*>(p.gamma) + 8 * ch);
                    const float4 a = g4[0], b = g4[1];
                    g[0] = a.x; g[1] = a.y; g[2] = a.z; g[3] = a.w;
                    g[4] = b.x; g[5] = b.y; g[6] = b.z; g[7] = b.w;
                }
#pragma unroll
                for (int i = 0; i < 8; ++i) v[c][i] = bf16_round(__fmul_rn(g[i], __fmul_rn(v[c][i], rs)));
            }
            const int64_t o = static_cast<int64_t>(row) * p.dim + 8 * ch;
            if (p.y_bf16) *reinterpret_cast<uint4*>(p.y_bf16 + o) = pack8(v[c]);
            if (p.y_fp8)
                quant_store8(v[c], p.pow2, p.y_fp8 + o,
                             p.y_scales ? p.y_scales + static_cast<int64_t>(row) * (p.dim >> 7) + (ch >> 4) : nullptr,
                             (ch & 15) == 0);
        }
    }
}

struct RopeParams {
    const __nv_bfloat16* x;
    const int64_t* positions;
    const float* cos_t;
    const float* sin_t;
    __nv_bfloat16* y_bf16;  // nullable
    uint8_t* y_fp8;         // nullable
    float* y_scales;        // nullable
    int tokens, heads, head_dim, rope_dim, max_pos, inverse, pow2;
};

__global__ void __launch_bounds__(1024) rope_quant_kernel(const RopeParams p) {
    pdl_launch_dependents();
    pdl_wait();   // nothing of global memory is touched before the kernel ahead has finished
    const int t = blockIdx.x;
    const int width = p.heads * p.head_dim;
    const int chunks = width >> 3;
    const int nope = p.head_dim - p.rope_dim;
    int64_t pos = p.positions[t];
    pos = pos < 0 ? 0 : (pos >= p.max_pos ? p.max_pos - 1 : pos);   // clamp instead of reading outside the tables
    const float* cs = p.cos_t + pos * (p.rope_dim >> 1);
    const float* sn = p.sin_t + pos * (p.rope_dim >> 1);
    const __nv_bfloat16* x = p.x + static_cast<int64_t>(t) * width;
    // every thread of a 16-thread quantisation group runs the same number of iterations
    // (width is a multiple of 128), so the shuffles inside quant_store8 are convergent
    // (blockIdx.y splits a token's chunks over several CTAs when there are few tokens)
    // four 16-byte loads of a thread are in flight before the first is used: the kernel is a few MB of latency
    const int stride = blockDim.x * gridDim.y;
    for (int ch0 = blockIdx.y * blockDim.x + threadIdx.x; ch0 < chunks; ch0 += 4 * stride) {
        uint4 raw[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
            raw[u] = ch0 + u * stride < chunks ? *reinterpret_cast<const uint4*>(x + 8 * (ch0 + u * stride)) : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int ch = ch0 + u * stride;
            if (ch >= chunks) break;                 // uniform over a 16-thread group
            float v[8];
            unpack8(raw[u], v);
            const int in_head = (8 * ch) % p.head_dim;
            if (in_head >= nope) {
                const int pair0 = (in_head - nope) >> 1;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float c = cs[pair0 + i];
                    const float s = p.inverse ? -sn[pair0 + i] : sn[pair0 + i];
                    const float re = v[2 * i], im = v[2 * i + 1];
                    // unfused, as a complex multiply in fp32 (no FMA contraction)
                    v[2 * i] = bf16_round(__fsub_rn(__fmul_rn(re, c), __fmul_rn(im, s)));
                    v[2 * i + 1] = bf16_round(__fadd_rn(__fmul_rn(re, s), __fmul_rn(im, c)));
                }
            }
            const int64_t o = static_cast<int64_t>(t) * width + 8 * ch;
            if (p.y_bf16) *reinterpret_cast<uint4*>(p.y_bf16 + o) = pack8(v);
            if (p.y_fp8)
                quant_store8(v, p.pow2, p.y_fp8 + o,
                             p.y_scales ? p.y_scales + static_cast<int64_t>(t) * (width >> 7) + (ch >> 4) : nullptr,
                             (ch & 15) == 0);
        }
    }
}

struct SwigluParams {
    const __nv_bfloat16* h;   // [rows, 2 * inter]: gate | up
    __nv_bfloat16* y_bf16;    // nullable
    uint8_t* y_fp8;           // nullable
    float* y_scales;
    int rows, inter, pow2;
    float limit;
};

// SwiGLU of a dense expert: y = bf16(silu(min(gate, L)) * clamp(up, +-L)), then 1x128 FP8 quantisation
// (dsv4_megakernel/origin/model.py:596-606; L = 0 disables the clamps).
__global__ void __launch_bounds__(1024, 1) swiglu_quant_kernel(const SwigluParams p) {
    pdl_launch_dependents();
    pdl_wait();   // nothing of global memory is touched before the kernel ahead has finished
    const int r = blockIdx.x;
    const int chunks = p.inter >> 3;
    const __nv_bfloat16* g = p.h + static_cast<int64_t>(r) * (2 * p.inter);
    for (int ch = blockIdx.y * blockDim.x + threadIdx.x; ch < chunks; ch += blockDim.x * gridDim.y) {
        float gate[8], up[8], v[8];
        unpack8(*reinterpret_cast<const uint4*>(g + 8 * ch), gate);
        unpack8(*reinterpret_cast<const uint4*>(g + p.inter + 8 * ch), up);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            float a = gate[i], b = up[i];
            if (p.limit > 0.f) {
                b = fminf(fmaxf(b, -p.limit), p.limit);
                a = fminf(a, p.limit);
            }
            v[i] = bf16_round(__fmul_rn(__fdiv_rn(a, 1.0f + expf(-a)), b));
        }
        const int64_t o = static_cast<int64_t>(r) * p.inter + 8 * ch;
        if (p.y_bf16) *reinterpret_cast<uint4*>(p.y_bf16 + o) = pack8(v);
        if (p.y_fp8)
            quant_store8(v, p.pow2, p.y_fp8 + o,
                         p.y_scales ? p.y_scales + static_cast<int64_t>(r) * (p.inter >> 7) + (ch >> 4) : nullptr,
                         (ch & 15) == 0);
    }
}

}  // namespace nrq
}  // namespace wuda

extern "C" int wuda_rmsnorm_quant_fp8(const void* x_bf16, int64_t x_row_stride, const void* gamma, int gamma_is_bf16,
                                      float eps, void* y_bf16, void* y_fp8, float* y_scales, int rows, int dim,
                                      int scale_mode, void* stream) {
    using namespace wuda;
    using namespace wuda::nrq;
    clear_error();
    WUDA_REQUIRE(rows >= 0, "rows must be >= 0 (got %d)", rows);
    WUDA_REQUIRE(dim >= 128 && dim % 128 == 0 && dim <= kMaxChunks * 1024 * 8,
                 "dim must be a multiple of 128 in [128, %d] (got %d)", kMaxChunks * 1024 * 8, dim);
    WUDA_REQUIRE(x_row_stride >= dim && x_row_stride % 8 == 0, "x_row_stride must be >= dim and a multiple of 8");
    WUDA_REQUIRE(scale_mode == 0 || scale_mode == 1, "scale_mode must be 0 (amax/448) or 1 (power of two)");
    if (rows == 0) return WUDA_OK;
    WUDA_REQUIRE(x_bf16 && (y_bf16 || y_fp8), "x and at least one output must not be NULL");
    WUDA_REQUIRE(!y_fp8 || y_scales, "y_scales is required with y_fp8");
    WUDA_REQUIRE(aligned16(x_bf16) && aligned16(gamma) && aligned16(y_bf16) && aligned16(y_fp8),
                 "x, gamma and the outputs must be 16-byte aligned");
    NormParams p;
    p.x = static_cast<const __nv_bfloat16*>(x_bf16);
    p.x_stride = x_row_stride;
    p.gamma = gamma;
    p.gamma_is_bf16 = gamma_is_bf16;
    p.eps = eps;
    p.y_bf16 = static_cast<__nv_bfloat16*>(y_bf16);
    p.y_fp8 = static_cast<uint8_t*>(y_fp8);
    p.y_scales = y_scales;
    p.rows = rows;
    p.dim = dim;
    p.pow2 = scale_mode;
    const int chunks = dim / 8;
    int threads = (chunks + kMaxChunks - 1) / kMaxChunks;
    threads = (threads + 31) / 32 * 32;
    if (threads > 1024) threads = 1024;
    WUDA_CUDA(launch_pdl(rmsnorm_quant_kernel, dim3(rows), dim3(threads), 0, static_cast<cudaStream_t>(stream), p));
    return WUDA_OK;
}

extern "C" int wuda_rope_quant_fp8(const void* x_bf16, const int64_t* positions, const float* cos_table,
                                   const float* sin_table, void* y_bf16, void* y_fp8, float* y_scales, int tokens,
                                   int heads, int head_dim, int rope_dim, int max_pos, int inverse, int scale_mode,
                                   void* stream) {
    using namespace wuda;
    using namespace wuda::nrq;
    clear_error();
    WUDA_REQUIRE(tokens >= 0 && heads >= 1, "tokens must be >= 0 and heads >= 1");
    WUDA_REQUIRE(head_dim % 8 == 0 && rope_dim % 8 == 0 && rope_dim >= 0 && rope_dim <= head_dim,
                 "head_dim and rope_dim must be multiples of 8 with rope_dim <= head_dim");
    WUDA_REQUIRE((static_cast<int64_t>(heads) * head_dim) % 128 == 0, "heads * head_dim must be a multiple of 128");
    WUDA_REQUIRE(max_pos >= 1, "max_pos must be >= 1");
    WUDA_REQUIRE(scale_mode == 0 || scale_mode == 1, "scale_mode must be 0 (amax/448) or 1 (power of two)");
    if (tokens == 0) return WUDA_OK;
    WUDA_REQUIRE(x_bf16 && positions && (rope_dim == 0 || (cos_table && sin_table)) && (y_bf16 || y_fp8),
                 "x, positions, the tables and at least one output must not be NULL");
    WUDA_REQUIRE(!y_fp8 || y_scales, "y_scales is required with y_fp8");
    WUDA_REQUIRE(aligned16(x_bf16) && aligned16(y_bf16) && aligned16(y_fp8), "x and the outputs must be 16-byte aligned");
    RopeParams p;
    p.x = static_cast<const __nv_bfloat16*>(x_bf16);
    p.positions = positions;
    p.cos_t = cos_table;
    p.sin_t = sin_table;
    p.y_bf16 = static_cast<__nv_bfloat16*>(y_bf16);
    p.y_fp8 = static_cast<uint8_t*>(y_fp8);
    p.y_scales = y_scales;
    p.tokens = tokens;
    p.heads = heads;
    p.head_dim = head_dim;
    p.rope_dim = rope_dim;
    p.max_pos = max_pos;
    p.inverse = inverse;
    p.pow2 = scale_mode;
    const int chunks = heads * head_dim / 8;
    // CTAs of 256 threads, each thread four 16-byte chunks per round; a token's row is cut over as many CTAs as keep
    // the whole launch within one resident wave (a quantisation group is 16 consecutive threads, so any multiple of
    // the block size is a valid cut, and whole 16-thread groups stay in step)
    const int threads = chunks < 256 ? (chunks + 31) / 32 * 32 : 256;
    int splits = 1;
    const int rounds = (chunks + 4 * threads - 1) / (4 * threads);
    while (splits < rounds && tokens * splits * 2 <= 5 * 148) splits *= 2;
    WUDA_CUDA(launch_pdl(rope_quant_kernel, dim3(dim3(tokens, splits)), dim3(threads), 0, static_cast<cudaStream_t>(stream), p));
    return WUDA_OK;
}

extern "C" int wuda_swiglu_quant_fp8(const void* h_bf16, void* y_bf16, void* y_fp8, float* y_scales, int rows, int inter,
                                     float swiglu_limit, int scale_mode, void* stream) {
    using namespace wuda;
    using namespace wuda::nrq;
    clear_error();
    WUDA_REQUIRE(rows >= 0, "rows must be >= 0 (got %d)", rows);
    WUDA_REQUIRE(inter >= 128 && inter % 128 == 0, "inter must be a positive multiple of 128 (got %d)", inter);
    WUDA_REQUIRE(scale_mode == 0 || scale_mode == 1, "scale_mode must be 0 (amax/448) or 1 (power of two)");
    if (rows == 0) return WUDA_OK;
    WUDA_REQUIRE(h_bf16 && (y_bf16 || y_fp8), "h and at least one output must not be NULL");
    WUDA_REQUIRE(!y_fp8 || y_scales, "y_scales is required with y_fp8");
    WUDA_REQUIRE(aligned16(h_bf16) && aligned16(y_bf16) && aligned16(y_fp8), "h and the outputs must be 16-byte aligned");
    SwigluParams p;
    p.h = static_cast<const __nv_bfloat16*>(h_bf16);
    p.y_bf16 = static_cast<__nv_bfloat16*>(y_bf16);
    p.y_fp8 = static_cast<uint8_t*>(y_fp8);
    p.y_scales = y_scales;
    p.rows = rows;
    p.inter = inter;
    p.pow2 = scale_mode;
    p.limit = swiglu_limit;
    const int chunks = inter / 8;
    const int threads = chunks < 1024 ? (chunks + 31) / 32 * 32 : 1024;
    int splits = 1;
    const int passes = (chunks + threads - 1) / threads;
    while (splits < passes && rows * splits < 296) splits *= 2;
    WUDA_CUDA(launch_pdl(swiglu_quant_kernel, dim3(dim3(rows, splits)), dim3(threads), 0, static_cast<cudaStream_t>(stream), p));
    return WUDA_OK;
}
