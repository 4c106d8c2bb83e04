// MoE router: from a token's fp32 expert logits to its top-k experts and routing weights.
//   score  = softmax(logits) | sigmoid(logits) | sqrt(softplus(logits))
//   select = the k largest of score + bias (the bias steers the choice only), ties to the lower expert
//   weight = score[selected], divided by their sum unless softmax, times route_scale
// After the origin's Gate.forward (dsv4_megakernel/origin/model.py:563-584); the logits themselves are
// the bf16 x fp32 -> fp32 projection `linear(x.float(), weight.float())`, which wuda_gemm_bf16 produces
// with fp32 output.  One warp per token: a lane holds experts lane, lane + 32, ..; k rounds of a
// warp arg-max pick the experts in descending order.
#include "host.h"

namespace wuda {
namespace route {

constexpr int kMaxPerLane = 16;   // up to 512 experts
constexpr int kWarpsPerCta = 4;

struct Params {
    const float* logits;   // [tokens, experts]
    const float* bias;     // [experts] or nullptr
    float* weights;        // [tokens, k]
    int32_t* indices;      // [tokens, k]
    int tokens, experts, k, score_func;
    float route_scale;
};

__global__ void __launch_bounds__(32 * kWarpsPerCta) moe_route_kernel(Params p) {
    pdl_launch_dependents();
    pdl_wait();   // nothing of global memory is touched before the kernel ahead has finished
    const int lane = threadIdx.x & 31;
    const int t = blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
    if (t >= p.tokens) return;                         // whole warps
    const float* row = p.logits + static_cast<int64_t>(t) * p.experts;
    float score[kMaxPerLane], pick[kMaxPerLane];
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j) {
        const int e = lane + 32 * j;
        score[j] = e < p.experts ? row[e] : -INFINITY;
        mx = fmaxf(mx, score[j]);
    }
    if (p.score_func == 0) {                           // softmax over all experts
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        float sum = 0.f;
#pragma unroll
        for (int j = 0; j < kMaxPerLane; ++j) {
            score[j] = lane + 32 * j < p.experts ? expf(score[j] - mx) : 0.f;
            sum += score[j];
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
#pragma unroll
        for (int j = 0; j < kMaxPerLane; ++j) score[j] = __fdiv_rn(score[j], sum);
    } else {
#pragma unroll
        for (int j = 0; j < kMaxPerLane; ++j) {
            const float x = score[j];
            if (p.score_func == 1) {
                score[j] = __fdiv_rn(1.0f, 1.0f + expf(-x));
            } else {                                    // sqrt(softplus(x)), softplus as log1p(exp(x)) with the usual cut
                const float sp = x > 20.f ? x : log1pf(expf(x));
                score[j] = __fsqrt_rn(sp);
            }
        }
    }
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j) {
        const int e = lane + 32 * j;
        pick[j] = e < p.experts ? (p.bias ? score[j] + __ldg(p.bias + e) : score[j]) : -INFINITY;
    }
    float wsum = 0.f, mine = 0.f;                      // lane r keeps the r-th selected weight
    int mine_e = 0;
    for (int r = 0; r < p.k; ++r) {
        float best = -INFINITY;
        int best_e = 0x7fffffff, best_j = 0;
#pragma unroll
        for (int j = 0; j < kMaxPerLane; ++j)
            if (pick[j] > best) {                       // strict: the lower expert wins inside a lane
                best = pick[j];
                best_e = lane + 32 * j;
                best_j = j;
            }
        float v = best;
        int e = best_e;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, v, o);
            const int oe = __shfl_xor_sync(0xffffffffu, e, o);
            if (ov > v || (ov == v && oe < e)) {
                v = ov;
                e = oe;
            }
        }
        const bool owner = e == best_e && best > -INFINITY;
        float s = 0.f;
        if (owner) {
#pragma unroll
            for (int j = 0; j < kMaxPerLane; ++j)
                if (j == best_j) {
                    s = score[j];
                    pick[j] = -INFINITY;
                }
        }
        s = __shfl_sync(0xffffffffu, s, e & 31);
        wsum += s;
        if (lane == r) {
            mine = s;
            mine_e = e;
        }
    }
    if (lane < p.k) {
        float w = p.score_func == 0 ? mine : __fdiv_rn(mine, wsum);
        p.weights[static_cast<int64_t>(t) * p.k + lane] = w * p.route_scale;
        p.indices[static_cast<int64_t>(t) * p.k + lane] = mine_e;
    }
}

}  // namespace route
}  // namespace wuda

extern "C" int wuda_moe_route(const float* logits, const float* bias, float* weights, int32_t* indices, int tokens,
                              int experts, int k, int score_func, float route_scale, void* stream) {
    using namespace wuda;
    using namespace wuda::route;
    clear_error();
    WUDA_REQUIRE(tokens >= 0, "tokens must be >= 0 (got %d)", tokens);
    WUDA_REQUIRE(experts >= 1 && experts <= 32 * kMaxPerLane, "experts must be in [1, %d] (got %d)", 32 * kMaxPerLane,
                 experts);
    WUDA_REQUIRE(k >= 1 && k <= 32 && k <= experts, "k must be in [1, min(32, experts)] (got %d)", k);
    WUDA_REQUIRE(score_func >= 0 && score_func <= 2, "score_func must be 0 (softmax), 1 (sigmoid) or 2 (sqrt softplus)");
    if (tokens == 0) return WUDA_OK;
    WUDA_REQUIRE(logits && weights && indices, "logits, weights and indices must not be NULL");
    Params p;
    p.logits = logits;
    p.bias = bias;
    p.weights = weights;
    p.indices = indices;
    p.tokens = tokens;
    p.experts = experts;
    p.k = k;
    p.score_func = score_func;
    p.route_scale = route_scale;
    WUDA_CUDA(launch_pdl(moe_route_kernel, dim3((tokens + kWarpsPerCta - 1) / kWarpsPerCta), dim3(32 * kWarpsPerCta), 0, static_cast<cudaStream_t>(stream), p));
    return WUDA_OK;
}
