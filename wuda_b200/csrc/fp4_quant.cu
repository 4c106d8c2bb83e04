// Block-wise FP4 (e2m1) quantisation of bf16 rows with one power-of-two scale per 32 values, for sm_100a.
//
// Contract (origin/kernel.py:126-200, fp4_quant_kernel / fp4_act_quant): per block of 32 values
//   amax = max(max |x|, 6 * 2^-126);  scale = 2^ceil(log2(amax * (1/6)))  (by the exponent and mantissa bits of the fp32
//   product);  code = e2m1(clamp(x / scale, -6, 6)), round to nearest even;
// outputs the codes two to a byte (the value of the lower index in the low nibble: torch.float4_e2m1fn_x2) and the
// scale's exponent byte (torch.float8_e8m0fnu), or - `inplace` - writes code * scale back over x as bf16 (the
// quantise-dequantise the origin applies to the indexer's keys and queries, origin/model.py:370,416).
//
// Four lanes share a block (8 values = one 16-byte load each); a thread has four such loads of different blocks in
// flight.  Pure streaming: 2 bytes in, 17/32 byte out per value (or 2 in, 2 out in place).
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "host.h"
#include "ptx.cuh"

namespace wuda {
namespace fq {

constexpr int kThreads = 256;

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

// value of an e2m1 code (sign, two exponent bits, one mantissa bit)
__device__ __forceinline__ float e2m1_value(uint32_t code) {
    const uint32_t mag = code & 7u;
    const float v = mag < 2u ? 0.5f * static_cast<float>(mag)
                             : __uint_as_float((126u + (mag >> 1)) << 23) * ((mag & 1u) ? 1.5f : 1.0f);
    return (code & 8u) ? -v : v;
}

struct Params {
    const __nv_bfloat16* x;
    __nv_bfloat16* y_inplace;   // == x when dequantising in place, else NULL
    uint8_t* codes;             // [rows, cols / 2]
    uint8_t* scales;            // [rows, cols / 32]
    int64_t row_stride;         // elements between the rows of x
    int64_t blocks;             // rows * cols / 32
    int blocks_per_row;
};

// kPieces: 16-byte pieces (of kPieces different blocks) a thread has in flight: four for inputs that fill the device
// several times over, one for the small ones, where more CTAs matter more
template <int kPieces>
__global__ void __launch_bounds__(kThreads) fp4_act_quant_kernel(Params p) {
    pdl_launch_dependents();
    pdl_wait();
    // piece = 8 values = a quarter of a block; thread t of the grid takes pieces t, t + T, t + 2 T, .. (T = all
    // threads), so a warp's loads are contiguous and the four lanes of a block stay neighbours
    const int64_t threads = static_cast<int64_t>(gridDim.x) * kThreads;
    const int64_t t = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x;
    const int sub = static_cast<int>(t & 3);
    uint4 raw[kPieces];
    int64_t blk[kPieces], at[kPieces];     // block number; element offset of the thread's piece in x
    const bool dense = p.row_stride == static_cast<int64_t>(p.blocks_per_row) * 32;   // no division needed
#pragma unroll
    for (int j = 0; j < kPieces; ++j) {
        blk[j] = (t + j * threads) >> 2;
        raw[j] = make_uint4(0u, 0u, 0u, 0u);
        at[j] = 0;
        if (blk[j] < p.blocks) {
            if (dense) {
                at[j] = blk[j] * 32 + sub * 8;
            } else {
                const int64_t row = blk[j] / p.blocks_per_row;
                at[j] = row * p.row_stride + (blk[j] - row * p.blocks_per_row) * 32 + sub * 8;
            }
            raw[j] = *reinterpret_cast<const uint4*>(p.x + at[j]);
        }
    }
#pragma unroll
    for (int j = 0; j < kPieces; ++j) {
        const bool live = blk[j] < p.blocks;      // the same for the four lanes of a block
        const uint32_t w[4] = {raw[j].x, raw[j].y, raw[j].z, raw[j].w};
        float v[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            v[2 * i] = __uint_as_float(w[i] << 16);
            v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
        float amax = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
        amax = fmaxf(amax, 6.0f * 1.1754944e-38f);
        const uint32_t rbits = __float_as_uint(__fmul_rn(amax, 1.0f / 6.0f));
        const int e = static_cast<int>((rbits >> 23) & 0xffu) - 127 + ((rbits & 0x7fffffu) ? 1 : 0);
        const float inv = __uint_as_float(static_cast<uint32_t>(127 - e) << 23);   // 2^-e: e <= 126 for bf16 input
        uint32_t packed = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) packed |= pack_e2m1x2(v[2 * i] * inv, v[2 * i + 1] * inv) << (8 * i);
        if (!live) continue;
        if (p.y_inplace) {
            const float scale = __uint_as_float(static_cast<uint32_t>(e + 127) << 23);
            uint32_t o[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint32_t byte = (packed >> (8 * i)) & 0xffu;
                const __nv_bfloat162 pair = __floats2bfloat162_rn(e2m1_value(byte & 15u) * scale, e2m1_value(byte >> 4) * scale);
                o[i] = *reinterpret_cast<const uint32_t*>(&pair);
            }
            *reinterpret_cast<uint4*>(p.y_inplace + at[j]) = make_uint4(o[0], o[1], o[2], o[3]);
        } else {
            *reinterpret_cast<uint32_t*>(p.codes + blk[j] * 16 + sub * 4) = packed;
            if (sub == 0) p.scales[blk[j]] = static_cast<uint8_t>(e + 127);
        }
    }
}

}  // namespace fq
}  // namespace wuda

extern "C" int wuda_fp4_act_quant(const void* x_bf16, int64_t row_stride, void* codes, void* scales, int inplace, int64_t rows,
                                  int cols, void* stream) {
    using namespace wuda;
    using namespace wuda::fq;
    clear_error();
    WUDA_REQUIRE(rows >= 0 && cols >= 32 && cols % 32 == 0, "rows must be >= 0 and cols a positive multiple of 32 (got %d)", cols);
    WUDA_REQUIRE(row_stride >= cols && row_stride % 8 == 0, "row_stride must be >= cols and a multiple of 8 elements");
    if (rows == 0) return WUDA_OK;
    WUDA_REQUIRE(x_bf16 && aligned16(x_bf16), "x must not be NULL and must be 16-byte aligned");
    WUDA_REQUIRE(inplace || (codes && scales && (reinterpret_cast<uintptr_t>(codes) & 3u) == 0),
                 "codes (4-byte aligned) and scales must not be NULL unless the rows are dequantised in place");
    Params p;
    p.x = static_cast<const __nv_bfloat16*>(x_bf16);
    p.y_inplace = inplace ? static_cast<__nv_bfloat16*>(const_cast<void*>(x_bf16)) : nullptr;
    p.codes = static_cast<uint8_t*>(codes);
    p.scales = static_cast<uint8_t*>(scales);
    p.row_stride = row_stride;
    p.blocks_per_row = cols / 32;
    p.blocks = rows * p.blocks_per_row;
    const int pieces = p.blocks * 4 >= static_cast<int64_t>(kThreads) * 4 * 148 * 8 ? 4 : 1;
    const int64_t grid = (p.blocks * 4 + kThreads * pieces - 1) / (kThreads * pieces);
    WUDA_REQUIRE(grid <= 0x7fffffff, "too many blocks for one launch");
    if (pieces == 4)
        WUDA_CUDA(launch_pdl(fp4_act_quant_kernel<4>, dim3(static_cast<unsigned>(grid)), dim3(kThreads), 0,
                             static_cast<cudaStream_t>(stream), p));
    else
        WUDA_CUDA(launch_pdl(fp4_act_quant_kernel<1>, dim3(static_cast<unsigned>(grid)), dim3(kThreads), 0,
                             static_cast<cudaStream_t>(stream), p));
    return WUDA_OK;
}
