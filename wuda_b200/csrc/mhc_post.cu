// mHC post mix, the tail of an attention half-layer:
//   output[m, j, d] = post[m, j] * attention_out[m, d] + sum_i comb[m, i, j] * residual[m, i, d]
// with 4 residual streams, bf16 in and out, fp32 arithmetic in the order the reference kernel uses
// (dsv4_megakernel/megakernel/kernels/mhc_post.cu:74-81): one rounded product, then four fused
// multiply-adds over i = 0..3, then round-to-nearest-even to bf16.
//
// The op is a pure stream: per token it reads 5 and writes 4 rows of `hidden` bf16.  One thread
// owns 8 consecutive dims (one 16-byte vector) of one token: five independent 16-byte loads, four
// 16-byte stores.  The 20 mix coefficients of a token are read through the read-only path by every
// thread of the token (they sit in L1 after the first warp).
#include <cuda_bf16.h>

#include "host.h"

namespace wuda {
namespace mhc {

constexpr int kStreams = 4;
constexpr int kThreads = 128;

struct Params {
    const uint4* x;      // [m, hidden/8]
    const uint4* res;    // [m, 4, hidden/8]
    const float* post;   // [m, 4]
    const float* comb;   // [m, 4, 4]  (input stream i, output stream j)
    uint4* out;          // [m, 4, hidden/8]
    int vectors;         // hidden / 8
    int64_t total;       // m * vectors
};

__device__ __forceinline__ float2 bf2_to_f2(uint32_t v) {
    return make_float2(__uint_as_float(v << 16), __uint_as_float(v & 0xffff0000u));
}

__device__ __forceinline__ uint32_t f2_to_bf2(float lo, float hi) {
    __nv_bfloat162 b = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&b);
}

__global__ void __launch_bounds__(kThreads) mhc_post_kernel(Params p) {
    pdl_launch_dependents();
    pdl_wait();   // nothing of global memory is touched before the kernel ahead has finished
    const int64_t t = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x;
    if (t >= p.total) return;
    const int64_t row = t / p.vectors;
    const int vec = static_cast<int>(t - row * p.vectors);

    uint4 r[kStreams];
#pragma unroll
    for (int i = 0; i < kStreams; ++i) r[i] = __ldcs(p.res + (row * kStreams + i) * p.vectors + vec);
    const uint4 xv = __ldcs(p.x + row * p.vectors + vec);

    float post[kStreams], comb[kStreams][kStreams];
    const float4 pv = __ldcg(reinterpret_cast<const float4*>(p.post) + row);   // written by a kernel of the same chain
    post[0] = pv.x, post[1] = pv.y, post[2] = pv.z, post[3] = pv.w;
#pragma unroll
    for (int i = 0; i < kStreams; ++i) {
        const float4 c = __ldcg(reinterpret_cast<const float4*>(p.comb) + row * kStreams + i);
        comb[i][0] = c.x, comb[i][1] = c.y, comb[i][2] = c.z, comb[i][3] = c.w;
    }

    const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
    for (int j = 0; j < kStreams; ++j) {
        uint32_t ow[4];
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float2 xf = bf2_to_f2(xw[w]);
            float lo = __fmul_rn(post[j], xf.x), hi = __fmul_rn(post[j], xf.y);
#pragma unroll
            for (int i = 0; i < kStreams; ++i) {
                const uint32_t rw = w == 0 ? r[i].x : w == 1 ? r[i].y : w == 2 ? r[i].z : r[i].w;
                const float2 rf = bf2_to_f2(rw);
                lo = __fmaf_rn(comb[i][j], rf.x, lo);
                hi = __fmaf_rn(comb[i][j], rf.y, hi);
            }
            ow[w] = f2_to_bf2(lo, hi);
        }
        __stcs(p.out + (row * kStreams + j) * p.vectors + vec, make_uint4(ow[0], ow[1], ow[2], ow[3]));
    }
}

bool overlaps(const void* a, size_t a_bytes, const void* b, size_t b_bytes) {
    const uintptr_t a0 = reinterpret_cast<uintptr_t>(a), b0 = reinterpret_cast<uintptr_t>(b);
    return a0 < b0 + b_bytes && b0 < a0 + a_bytes;
}

}  // namespace mhc
}  // namespace wuda

extern "C" int wuda_mhc_post(const void* attention_out, const void* residual, const float* post, const float* comb,
                             void* output, int m, int hidden, void* stream) {
    using namespace wuda;
    using namespace wuda::mhc;
    clear_error();
    WUDA_REQUIRE(m >= 1, "m must be >= 1 (got %d)", m);
    WUDA_REQUIRE(hidden >= 8 && hidden % 8 == 0, "hidden must be a positive multiple of 8 (got %d)", hidden);
    WUDA_REQUIRE(attention_out && residual && post && comb && output, "no argument may be NULL");
    WUDA_REQUIRE(aligned16(attention_out) && aligned16(residual) && aligned16(output) && aligned16(post) &&
                     aligned16(comb),
                 "all buffers must be 16-byte aligned");
    const size_t row_bytes = static_cast<size_t>(hidden) * 2, mm = static_cast<size_t>(m);
    const size_t out_bytes = mm * kStreams * row_bytes;
    WUDA_REQUIRE(!overlaps(output, out_bytes, attention_out, mm * row_bytes) &&
                     !overlaps(output, out_bytes, residual, out_bytes) &&
                     !overlaps(output, out_bytes, post, mm * kStreams * 4) &&
                     !overlaps(output, out_bytes, comb, mm * kStreams * kStreams * 4),
                 "output must not overlap an input: later streams read every input after earlier stores");
    Params p;
    p.x = static_cast<const uint4*>(attention_out);
    p.res = static_cast<const uint4*>(residual);
    p.post = post;
    p.comb = comb;
    p.out = static_cast<uint4*>(output);
    p.vectors = hidden / 8;
    p.total = static_cast<int64_t>(m) * p.vectors;
    const int64_t blocks = (p.total + kThreads - 1) / kThreads;
    WUDA_REQUIRE(blocks <= 0x7fffffffLL, "m * hidden is too large for one launch");
    WUDA_CUDA(launch_pdl(mhc_post_kernel, dim3(static_cast<unsigned>(blocks)), dim3(kThreads), 0, static_cast<cudaStream_t>(stream), p));
    return WUDA_OK;
}
