// mHC pre: the head of an attention (or FFN) half-layer.  From the 4 residual streams of a token,
//   x      = the 4 x hidden values as one row of K = 4 * hidden,  r = 1/sqrt(mean x^2 + eps)
//   mix    = (x . W^T) * r                    W fp32 [24, K]:  pre[0,4) | post[4,8) | comb[8,24)
//   pre    = sigmoid(mix_pre  * scale[0] + base_pre) + hc_eps
//   post   = 2 * sigmoid(mix_post * scale[1] + base_post)
//   comb   = Sinkhorn(softmax_rows(mix_comb * scale[2] + base_comb) + hc_eps), 20 iterations
//   y      = bf16(sum_h pre[h] * x[h, :])                      the collapsed stream
//   normed = bf16((y * 1/sqrt(mean y^2 + eps)) * gamma)        attention RMSNorm, bf16 gamma
//   x_fp8, x_scale = 1x128 power-of-two FP8 quantisation of normed (amax/448 clamped at 1e-4)
// Torch twin: dsv4_megakernel/megakernel/test/test_hc_fused_tc.py:115-136 (hc_reference); origin
// dsv4_megakernel/origin/model.py:673-681 (hc_pre).  Device counterparts: a TF32 tensor-core GEMM
// of a third-party library plus kernels/hc_fused_kernel_tc.cu:420-520 (hc_reduce_fuse_out, fused
// norm + quant at :300-340) and the Sinkhorn tail include/front_mixed_gemm.cuh:438-489.
//
// Two kernels.  (1) The mix, a [m, K] x [24, K]^T contraction with K = 4 * hidden, on the tensor cores with
// fp32-grade products: W is cut into three bf16 terms (hi + mid + lo carry its 24 mantissa bits, so
// x * hi, x * mid, x * lo are exact in fp32) stacked as 72 operand rows, and one tcgen05.mma kind::f16
// chain per CTA multiplies a 128-token tile of x by them; the three column groups are added in the
// epilogue.  K is cut into slices of 512: one CTA per (slice, 128-token tile) brings its x tile in with
// TMA (128-byte swizzle, rows beyond m filled with zeros), splits its 24 x 512 weights into shared memory
// in the same layout, and while the MMAs run sums the squares of its x rows from shared memory.
// Partials go to a workspace [slice][token][25] (24 dots + the sum of squares).  (2) One CTA per
// token adds the slices in order (deterministic), runs the gates and the Sinkhorn in one warp, and
// streams the 4 residual rows once for collapse + norm + quantisation.
#include <cuda.h>
#include <cuda_bf16.h>

#include "host.h"
#include "ptx.cuh"

namespace wuda {
namespace mhcpre {

constexpr int kStreams = 4;
constexpr int kMix = 24;                 // pre 4 | post 4 | comb 16
constexpr int kPart = kMix + 1;          // + sum of squares
constexpr int kSlice = 512;              // K elements per slice
constexpr int kMixThreads = 128;         // thread = token row of the tile = tensor-memory lane
constexpr int kMixTile = 128;            // tokens per CTA (UMMA M)
constexpr int kMixN = 80;                // 3 x 24 operand rows, padded to a multiple of 16 (UMMA N)
constexpr int kKBlocks = kSlice / 64;    // 128-byte K blocks per slice
constexpr int kXBlockBytes = kMixTile * 128, kWBlockBytes = kMixN * 128;
constexpr int kMixSmemBytes = kKBlocks * (kXBlockBytes + kWBlockBytes) + 64 + 1024;
constexpr int kMixTmemCols = 128;
constexpr int kFinishThreads = 256;              // the eight warps that collapse, normalise and quantise a token's row
constexpr int kFinishLaunch = kFinishThreads + 32;   // plus one warp for the post gates and the Sinkhorn iterations
constexpr int kSinkhornIters = 20;

struct Params {
    const __nv_bfloat16* x;        // [m, 4, hidden]
    const float* weight;           // [24, 4 * hidden]
    const float* base;             // [24]
    const float* scale;            // [3]
    const __nv_bfloat16* gamma;    // [hidden] or nullptr
    float* ws;                     // [slices, m, 25]
    float* pre;                    // [m, 4] or nullptr
    float* post;                   // [m, 4]
    float* comb;                   // [m, 4, 4]
    float* mix_out;                // [m, 24] or nullptr: the mixes times r (what the post / comb gates are made of)
    __nv_bfloat16* collapsed;      // [m, hidden] or nullptr
    __nv_bfloat16* normed;         // [m, hidden] or nullptr
    uint8_t* x_fp8;                // [m, hidden] or nullptr
    float* x_scales;               // [m, hidden / 128]
    int m, hidden, slices;
    float hc_eps, rms_eps, norm_eps;
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ uint32_t bf16_bits_rn(float v) {
    return static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(v)));
}

__global__ void __launch_bounds__(kMixThreads, 1) mhc_pre_mix_kernel(const __grid_constant__ CUtensorMap x_map, const Params p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t base = (raw_addr + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (base - raw_addr);
    const uint32_t x_addr = base, w_addr = base + kKBlocks * kXBlockBytes;
    uint8_t* x_ptr = base_ptr;
    uint8_t* w_ptr = base_ptr + kKBlocks * kXBlockBytes;
    const uint32_t bars = w_addr + kKBlocks * kWBlockBytes;
    const uint32_t x_full = bars, mma_done = bars + 8;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(base_ptr + kKBlocks * (kXBlockBytes + kWBlockBytes) + 16);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(base_ptr + kKBlocks * (kXBlockBytes + kWBlockBytes) + 20);
    const int warp = threadIdx.x >> 5;
    const uint32_t lane = lane_id();
    const int slice = blockIdx.x, tile = blockIdx.y;
    const int K = kStreams * p.hidden;

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        mbar_init(x_full, 1);
        mbar_init(mma_done, 1);
        fence_mbar_init();
        prefetch_tmap(&x_map);
    }
    if (warp == 0) {
        tmem_alloc(smem_u32(tmem_slot), kMixTmemCols);
        tmem_relinquish();
    }
    // the 24 x 512 weights of the slice (constants: they may be read before the kernel ahead has finished):
    // item = (row j, 8 consecutive K) -> two 16-byte loads, twelve items per thread
    constexpr int kItems = kMix * (kSlice / 8) / kMixThreads;
    float4 wraw[kItems][2];
#pragma unroll
    for (int i = 0; i < kItems; ++i) {
        const int item = threadIdx.x + i * kMixThreads, j = item / (kSlice / 8), c = item % (kSlice / 8);
        const float4* src = reinterpret_cast<const float4*>(p.weight + static_cast<int64_t>(j) * K + slice * kSlice + c * 8);
        wraw[i][0] = __ldg(src);
        wraw[i][1] = __ldg(src + 1);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_launch_dependents();
    pdl_wait();   // the residual streams come from the kernel ahead

    if (threadIdx.x == 0) {
        mbar_arrive_expect_tx(x_full, kKBlocks * kXBlockBytes);
#pragma unroll
        for (int kb = 0; kb < kKBlocks; ++kb)
            tma_load_2d(x_addr + kb * kXBlockBytes, &x_map, x_full, slice * kSlice + kb * 64, tile * kMixTile);
    }
    // w = hi + mid + lo in bf16, rows j, 24 + j, 48 + j of the operand, 128-byte swizzle (16-byte chunk c of row
    // r sits at chunk c ^ (r & 7)); rows 72..79 are zero
#pragma unroll
    for (int i = 0; i < kItems; ++i) {
        const int item = threadIdx.x + i * kMixThreads, j = item / (kSlice / 8), c = item % (kSlice / 8);
        const float w[8] = {wraw[i][0].x, wraw[i][0].y, wraw[i][0].z, wraw[i][0].w, wraw[i][1].x, wraw[i][1].y, wraw[i][1].z, wraw[i][1].w};
        uint32_t term[3][4];
#pragma unroll
        for (int e = 0; e < 8; e += 2) {
            uint32_t pair[3] = {0u, 0u, 0u};
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                float r = w[e + h];
#pragma unroll
                for (int t = 0; t < 3; ++t) {
                    const uint32_t bits = bf16_bits_rn(r);
                    pair[t] |= bits << (16 * h);
                    r = __fsub_rn(r, __uint_as_float(bits << 16));   // exact: the difference fits fp32
                }
            }
#pragma unroll
            for (int t = 0; t < 3; ++t) term[t][e >> 1] = pair[t];
        }
        const int kb = c >> 3, cc = c & 7;
#pragma unroll
        for (int t = 0; t < 3; ++t) {
            const int r = t * kMix + j;
            *reinterpret_cast<uint4*>(w_ptr + kb * kWBlockBytes + r * 128 + ((cc ^ (r & 7)) << 4)) =
                make_uint4(term[t][0], term[t][1], term[t][2], term[t][3]);
        }
    }
    for (int z = threadIdx.x; z < kKBlocks * (kMixN - 3 * kMix) * 8; z += kMixThreads) {
        const int kb = z / ((kMixN - 3 * kMix) * 8), rest = z % ((kMixN - 3 * kMix) * 8);
        *reinterpret_cast<uint4*>(w_ptr + kb * kWBlockBytes + (3 * kMix) * 128 + rest * 16) = make_uint4(0u, 0u, 0u, 0u);
    }
    fence_proxy_async_smem();   // the generic-proxy stores above are read by the tensor core
    __syncthreads();

    bool alive = mbar_wait(x_full, 0, abort_flag, nullptr, 0);
    if (threadIdx.x == 0 && alive) {
        tc_fence_after();
        constexpr uint32_t idesc = umma_idesc(kMixTile, kMixN, 1, 1);   // bf16 x bf16 -> fp32, both K-major
        uint32_t accumulate = 0;
#pragma unroll
        for (int kb = 0; kb < kKBlocks; ++kb)
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                umma_f16(tmem_base, umma_smem_desc_sw128(x_addr + kb * kXBlockBytes + k * 32),
                         umma_smem_desc_sw128(w_addr + kb * kWBlockBytes + k * 32), idesc, accumulate);
                accumulate = 1;
            }
        umma_commit(mma_done);
    }
    // sum of squares of this thread's token row, from the tile in shared memory, while the MMAs run
    float ss = 0.f;
    if (alive) {
        const int r = threadIdx.x;
#pragma unroll 2
        for (int kb = 0; kb < kKBlocks; ++kb)
#pragma unroll
            for (int cc = 0; cc < 8; ++cc) {
                const uint4 raw = *reinterpret_cast<const uint4*>(x_ptr + kb * kXBlockBytes + r * 128 + ((cc ^ (r & 7)) << 4));
                const uint32_t wv[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float lo = __uint_as_float(wv[i] << 16), hi = __uint_as_float(wv[i] & 0xffff0000u);
                    ss = fmaf(hi, hi, fmaf(lo, lo, ss));
                }
            }
    }
    alive = alive && mbar_wait(mma_done, 0, abort_flag, nullptr, 0);
    const int t = tile * kMixTile + threadIdx.x;
    if (alive) {
        tc_fence_after();
        const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
        uint32_t c[kMixN];
#pragma unroll
        for (int q = 0; q < kMixN / 16; ++q) {
            uint32_t v[16];
            tmem_ld_32x16(tmem_base + lane_base + q * 16, v);
#pragma unroll
            for (int i = 0; i < 16; ++i) c[q * 16 + i] = v[i];
        }
        tmem_ld_wait();
        tc_fence_before();
        if (t < p.m) {
            float* out = p.ws + (static_cast<int64_t>(slice) * p.m + t) * kPart;
#pragma unroll
            for (int j = 0; j < kMix; ++j)
                out[j] = __uint_as_float(c[j]) + (__uint_as_float(c[kMix + j]) + __uint_as_float(c[2 * kMix + j]));
            out[kMix] = ss;
        }
    }
    __syncthreads();
    if (*abort_flag) abort_drain_sleep();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kMixTmemCols);
    }
}

__device__ __forceinline__ float sigmoid(float x) { return __fdiv_rn(1.0f, 1.0f + expf(-x)); }

__device__ __forceinline__ uint32_t pack_e4m3x4(float a, float b, float c, float d) {
    uint16_t lo, hi;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(lo) : "f"(b), "f"(a));
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(hi) : "f"(d), "f"(c));
    return static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
}

// The post gates and the Sinkhorn-normalised comb matrix of one token, by one warp.  `folded` is lane j's mix
// value times r for j < 24 (pre 0..3 | post 4..7 | comb 8..23); lanes 0..3 write post, lanes 0..15 comb
// (row = lane / 4, column = lane % 4): row sums by xor 1, 2; column sums by xor 4, 8.
__device__ __forceinline__ void post_and_comb(float folded, int lane, const float* scale, const float* base, float hc_eps,
                                              float* post, float* comb) {
    const float post_mix = __shfl_sync(0xffffffffu, folded, (lane + kStreams) & 31);
    if (post && lane < kStreams) post[lane] = 2.0f * sigmoid(post_mix * scale[1] + base[kStreams + lane]);
    const float comb_mix = __shfl_sync(0xffffffffu, folded, (lane + 2 * kStreams) & 31);
    const bool live = lane < kStreams * kStreams;
    float v = live ? comb_mix * scale[2] + base[2 * kStreams + lane] : 0.f;
    float mx = v;
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float e = expf(v - mx);
    float rs = e;
    rs += __shfl_xor_sync(0xffffffffu, rs, 1);
    rs += __shfl_xor_sync(0xffffffffu, rs, 2);
    v = __fdiv_rn(e, rs) + hc_eps;
    float cs = v;
    cs += __shfl_xor_sync(0xffffffffu, cs, 4);
    cs += __shfl_xor_sync(0xffffffffu, cs, 8);
    v = __fdiv_rn(v, cs + hc_eps);
    for (int it = 0; it < kSinkhornIters - 1; ++it) {
        rs = v;
        rs += __shfl_xor_sync(0xffffffffu, rs, 1);
        rs += __shfl_xor_sync(0xffffffffu, rs, 2);
        v = __fdiv_rn(v, rs + hc_eps);
        cs = v;
        cs += __shfl_xor_sync(0xffffffffu, cs, 4);
        cs += __shfl_xor_sync(0xffffffffu, cs, 8);
        v = __fdiv_rn(v, cs + hc_eps);
    }
    if (live && comb) comb[lane] = v;
}

// The tail alone: post and comb from exported mixes (one warp per token), for callers that run it behind
// another kernel as the reference does (include/front_mixed_gemm.cuh:438-489).
__global__ void __launch_bounds__(128) mhc_tail_kernel(const float* mix, const float* base, const float* scale, float hc_eps,
                                                       float* pre, float* post, float* comb, int m) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int t = blockIdx.x * 4 + (threadIdx.x >> 5);
    if (t >= m) return;
    const float folded = lane < kMix ? __ldcg(mix + t * kMix + lane) : 0.f;
    if (pre && lane < kStreams) pre[t * kStreams + lane] = sigmoid(folded * scale[0] + base[lane]) + hc_eps;
    post_and_comb(folded, lane, scale, base, hc_eps, post + t * kStreams, comb + t * kStreams * kStreams);
}

// barrier of the eight row warps alone (the ninth warp is busy with the Sinkhorn iterations or gone)
__device__ __forceinline__ void row_warps_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kFinishThreads) : "memory"); }

__global__ void __launch_bounds__(kFinishLaunch) mhc_pre_finish_kernel(Params p) {
    pdl_launch_dependents();
    pdl_wait();   // nothing of global memory is touched before the kernel ahead has finished
    __shared__ float mix[kPart];
    __shared__ float pre_s[kStreams];
    __shared__ float warp_ss[kFinishThreads / 32];
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    constexpr int kMaxVec = 4;                       // hidden <= 4 * 256 * 8 = 8192
    const bool row_warp = threadIdx.x < kFinishThreads;
    const int vectors = (row_warp && (p.collapsed || p.normed || p.x_fp8)) ? p.hidden / 8 : 0;
    // the token's four rows are requested first: their latency hides behind the slice sums, the gates and the
    // Sinkhorn iterations, none of which needs them
    uint4 raw[kMaxVec][kStreams];
#pragma unroll
    for (int k = 0; k < kMaxVec; ++k) {
        const int vi = threadIdx.x + k * kFinishThreads;
#pragma unroll
        for (int h = 0; h < kStreams; ++h)
            raw[k][h] = vi < vectors ? __ldcs(reinterpret_cast<const uint4*>(p.x + (static_cast<int64_t>(t) * kStreams + h) * p.hidden) + vi)
                                     : make_uint4(0u, 0u, 0u, 0u);
    }

    // 25 sums over the slices: 8 groups of threads take every eighth slice each (independent loads), then
    // the 8 group sums are added in order - a fixed tree, so the result does not depend on timing
    __shared__ float group_sum[8][kPart];
    if (threadIdx.x < 8 * kPart) {
        const int j = threadIdx.x % kPart, grp = threadIdx.x / kPart;
        float s = 0.f;
        for (int sl = grp; sl < p.slices; sl += 8) s += p.ws[(static_cast<int64_t>(sl) * p.m + t) * kPart + j];
        group_sum[grp][j] = s;
    }
    __syncthreads();
    if (threadIdx.x < kPart) {
        float s = group_sum[0][threadIdx.x];
#pragma unroll
        for (int grp = 1; grp < 8; ++grp) s += group_sum[grp][threadIdx.x];
        mix[threadIdx.x] = s;
    }
    __syncthreads();
    // The collapse needs the four pre gates only; the post gates and the Sinkhorn-normalised comb matrix - twenty
    // rounds of shuffles and divisions that nothing in this kernel reads - are the ninth warp's, beside the row work.
    if (warp == 0 || !row_warp) {
        const float r = __fdiv_rn(1.0f, __fsqrt_rn(__fdiv_rn(mix[kMix], static_cast<float>(kStreams * p.hidden)) + p.rms_eps));
        if (row_warp) {
            if (lane < kStreams) {
                const float v = sigmoid(mix[lane] * r * p.scale[0] + p.base[lane]) + p.hc_eps;
                pre_s[lane] = v;
                if (p.pre) p.pre[t * kStreams + lane] = v;
            }
            if (p.mix_out && lane < kMix) p.mix_out[t * kMix + lane] = mix[lane] * r;
        } else {
            post_and_comb(lane < kMix ? mix[lane] * r : 0.f, lane, p.scale, p.base, p.hc_eps,
                          p.post ? p.post + t * kStreams : nullptr, p.comb ? p.comb + t * kStreams * kStreams : nullptr);
        }
    }
    if (!row_warp) return;
    row_warps_sync();
    if (!p.collapsed && !p.normed && !p.x_fp8) return;

    // collapse: a thread owns the 8-value vectors tid, tid + 256, ..; a 128-block of the row is 16
    // consecutive vectors, i.e. 16 consecutive threads
    const float pr[kStreams] = {pre_s[0], pre_s[1], pre_s[2], pre_s[3]};
    float y[kMaxVec][8];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < kMaxVec; ++k) {
        const int vi = threadIdx.x + k * kFinishThreads;
        if (vi < vectors) {
            float acc[8];
#pragma unroll
            for (int h = 0; h < kStreams; ++h) {
                const uint32_t wv[4] = {raw[k][h].x, raw[k][h].y, raw[k][h].z, raw[k][h].w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float lo = __fmul_rn(pr[h], __uint_as_float(wv[i] << 16));
                    const float hi = __fmul_rn(pr[h], __uint_as_float(wv[i] & 0xffff0000u));
                    acc[2 * i] = h == 0 ? lo : __fadd_rn(acc[2 * i], lo);
                    acc[2 * i + 1] = h == 0 ? hi : __fadd_rn(acc[2 * i + 1], hi);
                }
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                y[k][i] = __bfloat162float(__float2bfloat16_rn(acc[i]));
                ss = fmaf(y[k][i], y[k][i], ss);
            }
            if (p.collapsed) {
                uint4 o;
                uint32_t* ow = &o.x;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    __nv_bfloat162 b = __floats2bfloat162_rn(y[k][2 * i], y[k][2 * i + 1]);
                    ow[i] = *reinterpret_cast<uint32_t*>(&b);
                }
                *(reinterpret_cast<uint4*>(p.collapsed + static_cast<int64_t>(t) * p.hidden) + vi) = o;
            }
        }
    }
    if (!p.normed && !p.x_fp8) return;
    ss = warp_sum(ss);
    if (lane == 0) warp_ss[warp] = ss;
    row_warps_sync();
    float total = 0.f;
#pragma unroll
    for (int i = 0; i < kFinishThreads / 32; ++i) total += warp_ss[i];
    const float rn = __fdiv_rn(1.0f, __fsqrt_rn(__fdiv_rn(total, static_cast<float>(p.hidden)) + p.norm_eps));
#pragma unroll
    for (int k = 0; k < kMaxVec; ++k) {
        const int vi = threadIdx.x + k * kFinishThreads;
        const bool on = vi < vectors;              // uniform over every group of 16 threads (vectors % 16 == 0)
        float v[8];
        float amax = 0.f;
        uint4 o = make_uint4(0, 0, 0, 0);
        if (on) {
            const uint4 graw = __ldg(reinterpret_cast<const uint4*>(p.gamma) + vi);
            const uint32_t gw[4] = {graw.x, graw.y, graw.z, graw.w};
            uint32_t* ow = &o.x;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float a = __fmul_rn(__fmul_rn(y[k][2 * i], rn), __uint_as_float(gw[i] << 16));
                const float b = __fmul_rn(__fmul_rn(y[k][2 * i + 1], rn), __uint_as_float(gw[i] & 0xffff0000u));
                __nv_bfloat162 bb = __floats2bfloat162_rn(a, b);
                ow[i] = *reinterpret_cast<uint32_t*>(&bb);
                v[2 * i] = __uint_as_float(ow[i] << 16);
                v[2 * i + 1] = __uint_as_float(ow[i] & 0xffff0000u);
                amax = fmaxf(amax, fmaxf(fabsf(v[2 * i]), fabsf(v[2 * i + 1])));
            }
            if (p.normed) *(reinterpret_cast<uint4*>(p.normed + static_cast<int64_t>(t) * p.hidden) + vi) = o;
        }
        if (p.x_fp8) {
#pragma unroll
            for (int s = 8; s > 0; s >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, s));
            if (on) {
                const uint32_t bits = __float_as_uint(fmaxf(__fdiv_rn(amax, 448.f), 1e-4f));
                const int e = static_cast<int>((bits >> 23) & 0xff) - 127 + ((bits & 0x7fffffu) ? 1 : 0);
                const float inv = __uint_as_float(static_cast<uint32_t>(127 - e) << 23);
                const uint2 q = make_uint2(pack_e4m3x4(v[0] * inv, v[1] * inv, v[2] * inv, v[3] * inv),
                                           pack_e4m3x4(v[4] * inv, v[5] * inv, v[6] * inv, v[7] * inv));
                *(reinterpret_cast<uint2*>(p.x_fp8 + static_cast<int64_t>(t) * p.hidden) + vi) = q;
                if ((threadIdx.x & 15) == 0)
                    p.x_scales[static_cast<int64_t>(t) * (p.hidden / 128) + vi / 16] =
                        __uint_as_float(static_cast<uint32_t>(e + 127) << 23);
            }
        }
    }
}

}  // namespace mhcpre
}  // namespace wuda

extern "C" int64_t wuda_mhc_pre_workspace_bytes(int m, int hidden) {
    if (m < 1 || hidden < 8) return -1;
    const int64_t slices = (4LL * hidden + wuda::mhcpre::kSlice - 1) / wuda::mhcpre::kSlice;
    return slices * m * wuda::mhcpre::kPart * 4;
}

namespace {

int fill_params(wuda::mhcpre::Params& p, const void* hidden_states, const float* weight, const float* base, const float* scale,
                const void* gamma, float hc_eps, float rms_eps, float norm_eps, float* pre, float* post, float* comb,
                float* mix_out, void* collapsed_bf16, void* normed_bf16, void* x_fp8, float* x_scales, void* workspace, int m,
                int hidden) {
    using namespace wuda;
    using namespace wuda::mhcpre;
    WUDA_REQUIRE(m >= 1, "m must be >= 1 (got %d)", m);
    WUDA_REQUIRE(hidden >= 128 && hidden % 128 == 0 && hidden <= 8192,
                 "hidden must be a multiple of 128 in [128, 8192] (got %d)", hidden);
    WUDA_REQUIRE(hidden_states && workspace, "hidden and workspace are required");
    WUDA_REQUIRE((!normed_bf16 && !x_fp8) || gamma, "the norm weight is required with normed or x_fp8");
    WUDA_REQUIRE(!x_fp8 || x_scales, "x_scales is required with x_fp8");
    WUDA_REQUIRE(aligned16(hidden_states) && aligned16(weight) && aligned16(gamma) && aligned16(collapsed_bf16) &&
                     aligned16(normed_bf16) && aligned16(x_fp8),
                 "hidden, weight, gamma and the row outputs must be 16-byte aligned");
    p.x = static_cast<const __nv_bfloat16*>(hidden_states);
    p.weight = weight;
    p.base = base;
    p.scale = scale;
    p.gamma = static_cast<const __nv_bfloat16*>(gamma);
    p.ws = static_cast<float*>(workspace);
    p.pre = pre;
    p.post = post;
    p.comb = comb;
    p.mix_out = mix_out;
    p.collapsed = static_cast<__nv_bfloat16*>(collapsed_bf16);
    p.normed = static_cast<__nv_bfloat16*>(normed_bf16);
    p.x_fp8 = static_cast<uint8_t*>(x_fp8);
    p.x_scales = x_scales;
    p.m = m;
    p.hidden = hidden;
    p.slices = (kStreams * hidden + kSlice - 1) / kSlice;
    p.hc_eps = hc_eps;
    p.rms_eps = rms_eps;
    p.norm_eps = norm_eps;
    return WUDA_OK;
}

// The mix kernel: the residual streams as a [m, 4 * hidden] bf16 tensor map with 64 x 128 boxes in the 128-byte
// swizzle; a tile's rows beyond m read as zeros.
int launch_mix(const wuda::mhcpre::Params& p, cudaStream_t stream) {
    using namespace wuda;
    using namespace wuda::mhcpre;
    WUDA_REQUIRE(static_cast<int64_t>(p.m) <= 65535ll * kMixTile, "m is too large (got %d)", p.m);
    CUtensorMap x_map;
    const uint64_t K = static_cast<uint64_t>(kStreams) * p.hidden;
    const uint64_t dims[2] = {K, static_cast<uint64_t>(p.m)};
    const uint64_t strides[1] = {K * 2};
    const uint32_t box[2] = {64u, static_cast<uint32_t>(kMixTile)};
    int st = encode_tensor_map(&x_map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, p.x, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B,
                               CU_TENSOR_MAP_L2_PROMOTION_L2_128B);
    if (st != WUDA_OK) return st;
    WUDA_CUDA(cudaFuncSetAttribute(mhc_pre_mix_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kMixSmemBytes));
    const dim3 grid(p.slices, (p.m + kMixTile - 1) / kMixTile);
    WUDA_CUDA(launch_pdl(mhc_pre_mix_kernel, grid, dim3(kMixThreads), kMixSmemBytes, stream, x_map, p));
    return WUDA_OK;
}

}  // namespace

extern "C" int wuda_mhc_pre(const void* hidden_states, const float* weight, const float* base, const float* scale,
                            const void* attn_norm_gamma, float hc_eps, float rms_eps, float norm_eps, float* pre,
                            float* post, float* comb, void* collapsed_bf16, void* normed_bf16, void* x_fp8,
                            float* x_scales, void* workspace, int64_t workspace_bytes, int m, int hidden,
                            void* stream) {
    using namespace wuda;
    using namespace wuda::mhcpre;
    clear_error();
    WUDA_REQUIRE(weight && base && scale, "weight, base and scale are required");
    Params p;
    int st = fill_params(p, hidden_states, weight, base, scale, attn_norm_gamma, hc_eps, rms_eps, norm_eps, pre, post, comb,
                         nullptr, collapsed_bf16, normed_bf16, x_fp8, x_scales, workspace, m, hidden);
    if (st != WUDA_OK) return st;
    const int64_t need = wuda_mhc_pre_workspace_bytes(m, hidden);
    WUDA_REQUIRE(workspace_bytes >= need, "workspace holds %lld bytes; %lld are needed (wuda_mhc_pre_workspace_bytes)",
                 static_cast<long long>(workspace_bytes), static_cast<long long>(need));
    st = launch_mix(p, static_cast<cudaStream_t>(stream));
    if (st != WUDA_OK) return st;
    WUDA_CUDA(launch_pdl(mhc_pre_finish_kernel, dim3(m), dim3(kFinishLaunch), 0, static_cast<cudaStream_t>(stream), p));
    return WUDA_OK;
}

extern "C" int wuda_mhc_pre_mix(const void* hidden_states, const float* weight, void* workspace, int64_t workspace_bytes,
                                int m, int hidden, void* stream) {
    using namespace wuda;
    using namespace wuda::mhcpre;
    clear_error();
    WUDA_REQUIRE(weight, "weight is required");
    Params p;
    int st = fill_params(p, hidden_states, weight, nullptr, nullptr, nullptr, 0.f, 0.f, 0.f, nullptr, nullptr, nullptr, nullptr,
                         nullptr, nullptr, nullptr, nullptr, workspace, m, hidden);
    if (st != WUDA_OK) return st;
    const int64_t need = wuda_mhc_pre_workspace_bytes(m, hidden);
    WUDA_REQUIRE(workspace_bytes >= need, "workspace holds %lld bytes; %lld are needed (wuda_mhc_pre_workspace_bytes)",
                 static_cast<long long>(workspace_bytes), static_cast<long long>(need));
    st = launch_mix(p, static_cast<cudaStream_t>(stream));
    if (st != WUDA_OK) return st;
    return WUDA_OK;
}

extern "C" int wuda_mhc_pre_finish(const void* hidden_states, const float* partials, int splits, const float* base,
                                   const float* scale, const void* attn_norm_gamma, float hc_eps, float rms_eps,
                                   float norm_eps, float* pre, float* post, float* comb, float* mix_out,
                                   void* collapsed_bf16, void* normed_bf16, void* x_fp8, float* x_scales, int m, int hidden,
                                   void* stream) {
    using namespace wuda;
    using namespace wuda::mhcpre;
    clear_error();
    WUDA_REQUIRE(base && scale, "base and scale are required");
    WUDA_REQUIRE(splits >= 1, "splits must be >= 1 (got %d)", splits);
    Params p;
    int st = fill_params(p, hidden_states, nullptr, base, scale, attn_norm_gamma, hc_eps, rms_eps, norm_eps, pre, post, comb,
                         mix_out, collapsed_bf16, normed_bf16, x_fp8, x_scales, const_cast<float*>(partials), m, hidden);
    if (st != WUDA_OK) return st;
    p.slices = splits;
    WUDA_CUDA(launch_pdl(mhc_pre_finish_kernel, dim3(m), dim3(kFinishLaunch), 0, static_cast<cudaStream_t>(stream), p));
    return WUDA_OK;
}

extern "C" int wuda_mhc_tail(const float* mix, const float* base, const float* scale, float hc_eps, float* post, float* comb,
                             int m, void* stream) {
    using namespace wuda;
    using namespace wuda::mhcpre;
    clear_error();
    WUDA_REQUIRE(m >= 1 && mix && base && scale && post && comb, "m >= 1 and every pointer are required");
    WUDA_CUDA(launch_pdl(mhc_tail_kernel, dim3((m + 3) / 4), dim3(128), 0, static_cast<cudaStream_t>(stream), mix, base, scale,
                         hc_eps, static_cast<float*>(nullptr), post, comb, m));
    return WUDA_OK;
}

extern "C" int wuda_hc_split_sinkhorn(const float* mixes, const float* scale, const float* base, float hc_eps, float* pre, float* post,
                                      float* comb, int64_t tokens, void* stream) {
    using namespace wuda;
    using namespace wuda::mhcpre;
    clear_error();
    WUDA_REQUIRE(tokens >= 0 && tokens <= 0x7fffffff / 32, "tokens out of range");
    if (tokens == 0) return WUDA_OK;
    WUDA_REQUIRE(mixes && base && scale && pre && post && comb, "every pointer is required");
    const int m = static_cast<int>(tokens);
    WUDA_CUDA(launch_pdl(mhc_tail_kernel, dim3((m + 3) / 4), dim3(128), 0, static_cast<cudaStream_t>(stream), mixes, base, scale,
                         hc_eps, pre, post, comb, m));
    return WUDA_OK;
}
