// FRONT-EMIT: what the front projection of a decode step publishes besides the raw query.
// The front GEMM's output row of a token is [q 1536 | win 512] from the FP8 segment and
// [main 2048 | idx 512 | w64 64] from the BF16 segment
// (dsv4_megakernel/megakernel/include/front_mixed_gemm.cuh:390-425).  This kernel scatters
//   win  -> win_y2 [M, 512]   as fp32(bf16(acc))        (the window projection's output is bf16)
//   main -> the token's MAIN state-ring entry, fp32;  the score half (+1024..2047) gets + ape[pos % 4]
//   idx  -> the token's indexer state-ring entry, fp32; the score half (+256..511) gets + idx_ape[pos % 4]
//   w64  -> w64 [M, 64]       as fp32(bf16(acc))        (the head-weight projection's output is bf16)
// State rows are block * ring + pos % ring, computed by the host; a negative row skips the token.
// The reference does this inside the GEMM epilogue; here the BF16 segment is produced in fp32 by
// wuda_gemm_bf16 and scattered by one small launch (3136 fp32 values per token).
#include <cuda_bf16.h>

#include "host.h"

namespace wuda {
namespace femit {

constexpr int kQ = 1536, kWin = 512, kMain = 2048, kIdx = 512, kW64 = 64;
constexpr int kN8 = kQ + kWin, kN16 = kMain + kIdx + kW64;
constexpr int kThreads = 256;

struct Params {
    const __nv_bfloat16* y8;    // [m, 2048]
    const float* y16;           // [m, 2624]
    const int64_t* pos;
    float* main_state;
    const float* ape;           // [4, 1024]
    const int64_t* main_row;
    float* idx_state;
    const float* idx_ape;       // [4, 256]
    const int64_t* idx_row;
    float* win_y2;
    float* w64;
    int64_t state_rows_total;
    int32_t* status;
};

__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

__global__ void __launch_bounds__(kThreads) front_emit_kernel(Params p) {
    pdl_launch_dependents();
    pdl_wait();   // nothing of global memory is touched before the kernel ahead has finished
    // grid (tokens, 4): blockIdx.y = 0, 1 the two halves of the MAIN entry, 2 the indexer entry, 3 win_y2 + w64
    const int t = blockIdx.x;
    const int part = blockIdx.y;
    const int phase = static_cast<int>(p.pos[t] & 3);
    const float* y16 = p.y16 + static_cast<int64_t>(t) * kN16;
    if (part == 3) {
        if (p.win_y2)
            for (int c = threadIdx.x; c < kWin; c += kThreads)
                p.win_y2[static_cast<int64_t>(t) * kWin + c] = __bfloat162float(p.y8[static_cast<int64_t>(t) * kN8 + kQ + c]);
        if (p.w64 && threadIdx.x < kW64)
            p.w64[static_cast<int64_t>(t) * kW64 + threadIdx.x] = bf16_round(y16[kMain + kIdx + threadIdx.x]);
    } else if (part < 2) {
        if (!p.main_state) return;
        const int64_t row = p.main_row[t];
        if (row >= p.state_rows_total) {
            if (threadIdx.x == 0 && p.status) atomicCAS(p.status, 0, WUDA_DEV_BAD_STATE_ROW);
        } else if (row >= 0) {
            // 1024 values as float4: the kv half is copied, the score half gets + ape
            const float4* src = reinterpret_cast<const float4*>(y16 + part * (kMain / 2));
            float4* dst = reinterpret_cast<float4*>(p.main_state + row * kMain + part * (kMain / 2));
            const float4* add = reinterpret_cast<const float4*>(p.ape + phase * (kMain / 2));
            float4 v = src[threadIdx.x];
            if (part == 1) {
                const float4 a = __ldg(add + threadIdx.x);
                v = make_float4(__fadd_rn(v.x, a.x), __fadd_rn(v.y, a.y), __fadd_rn(v.z, a.z), __fadd_rn(v.w, a.w));
            }
            dst[threadIdx.x] = v;
        }
    } else {
        if (!p.idx_state) return;
        const int64_t row = p.idx_row[t];
        if (row >= p.state_rows_total) {
            if (threadIdx.x == 0 && p.status) atomicCAS(p.status, 0, WUDA_DEV_BAD_STATE_ROW);
        } else if (row >= 0) {
            float* dst = p.idx_state + row * kIdx;
            for (int c = threadIdx.x; c < kIdx; c += kThreads)
                dst[c] = c < kIdx / 2 ? y16[kMain + c]
                                      : __fadd_rn(y16[kMain + c], __ldg(p.idx_ape + phase * (kIdx / 2) + c - kIdx / 2));
        }
    }
}

}  // namespace femit
}  // namespace wuda

extern "C" int wuda_front_emit(const void* y8_bf16, const float* y16_f32, const int64_t* pos, float* main_state,
                               const float* ape, const int64_t* main_state_row, float* idx_state, const float* idx_ape,
                               const int64_t* idx_state_row, float* win_y2, float* w64, int64_t state_rows_total, int m,
                               int32_t* status_word, void* stream) {
    using namespace wuda;
    using namespace wuda::femit;
    clear_error();
    WUDA_REQUIRE(m >= 0, "m must be >= 0 (got %d)", m);
    if (m == 0) return WUDA_OK;
    WUDA_REQUIRE(y16_f32 && pos, "the BF16 segment's output and pos are required");
    WUDA_REQUIRE(!win_y2 || y8_bf16, "win_y2 needs the FP8 segment's output");
    WUDA_REQUIRE(!main_state || (ape && main_state_row), "main_state needs ape and main_state_row");
    WUDA_REQUIRE(aligned16(y16_f32) && aligned16(main_state) && aligned16(ape), "y16, main_state and ape must be 16-byte aligned");
    WUDA_REQUIRE(!idx_state || (idx_ape && idx_state_row), "idx_state needs idx_ape and idx_state_row");
    WUDA_REQUIRE((!main_state && !idx_state) || state_rows_total >= 1, "state_rows_total must be >= 1");
    Params p;
    p.y8 = static_cast<const __nv_bfloat16*>(y8_bf16);
    p.y16 = y16_f32;
    p.pos = pos;
    p.main_state = main_state;
    p.ape = ape;
    p.main_row = main_state_row;
    p.idx_state = idx_state;
    p.idx_ape = idx_ape;
    p.idx_row = idx_state_row;
    p.win_y2 = win_y2;
    p.w64 = w64;
    p.state_rows_total = state_rows_total;
    p.status = status_word;
    WUDA_CUDA(launch_pdl(front_emit_kernel, dim3(dim3(m, 4)), dim3(kThreads), 0, static_cast<cudaStream_t>(stream), p));
    return WUDA_OK;
}
