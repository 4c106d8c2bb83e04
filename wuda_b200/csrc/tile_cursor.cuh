// The walk of a persistent CTA over the flat list of (request, token tile) work items of a paged
// attention-score kernel: the list is cut into equal contiguous chunks inside the kernel (a warp-parallel
// prefix over the context lengths, no host schedule), and every warp role keeps its own cursor into the
// CTA's chunk and advances it identically.  NEXT_N = score rows per request, TILE = tokens per item.
#pragma once
#include <cstdint>

#include "ptx.cuh"

namespace wuda {
namespace tiles {

// A context length as the kernel uses it: negative values count as 0, values beyond what a row of the
// logits / block table holds are cut to that (the math warps report the cut as kDevBadContextLen).
__device__ __forceinline__ int clamp_ctx(int v, int max_ctx) { return min(max(v, 0), max_ctx); }

// Max context over the next_n rows of request b (its tile count follows from it).
template <int NEXT_N>
__device__ __forceinline__ int request_ctx(const int32_t* ctx, int b, int max_ctx) {
    int m = 0;
#pragma unroll
    for (int j = 0; j < NEXT_N; ++j) m = max(m, clamp_ctx(__ldg(ctx + b * NEXT_N + j), max_ctx));
    return m;
}

// The position of one CTA in the flat tile list. Every warp keeps its own copy and
// advances it identically, so no shared-memory broadcast is needed.
struct TileCursor {
    int b;         // request
    int j;         // tile inside the request
    int tiles_b;   // tiles of request b
    int ctx_b;     // max context of request b
    int count;     // tiles this CTA owns
};

template <int NEXT_N, int TILE>
__device__ __forceinline__ TileCursor make_cursor(const int32_t* ctx, int batch, int max_ctx) {
    const uint32_t lane = lane_id();
    long long total = 0;
    for (int base = 0; base < batch; base += 32) {
        int b = base + lane;
        int t = (b < batch) ? ((request_ctx<NEXT_N>(ctx, b, max_ctx) + TILE - 1) / TILE) : 0;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
        total += t;
    }
    const long long start = total * blockIdx.x / gridDim.x;
    const long long end = total * (blockIdx.x + 1) / gridDim.x;
    TileCursor c;
    c.count = static_cast<int>(end - start);
    c.b = batch;
    c.j = 0;
    c.tiles_b = 0;
    c.ctx_b = 0;
    if (c.count == 0) return c;
    long long prefix = 0;
    for (int base = 0; base < batch; base += 32) {
        int b = base + lane;
        int cx = (b < batch) ? request_ctx<NEXT_N>(ctx, b, max_ctx) : 0;
        int t = (cx + TILE - 1) / TILE;
        int incl = t;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            int v = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += v;
        }
        const long long incl_g = prefix + incl;
        const unsigned hit = __ballot_sync(0xffffffffu, incl_g > start);
        if (hit) {
            const int src = __ffs(hit) - 1;
            const long long incl_src = __shfl_sync(0xffffffffu, incl_g, src);
            const int t_src = __shfl_sync(0xffffffffu, t, src);
            c.b = base + src;
            c.tiles_b = t_src;
            c.ctx_b = __shfl_sync(0xffffffffu, cx, src);
            c.j = static_cast<int>(start - (incl_src - t_src));
            return c;
        }
        prefix += __shfl_sync(0xffffffffu, incl, 31);
    }
    c.count = 0;  // unreachable when the two passes see the same lengths
    return c;
}

// Moves the cursor forward by k tiles.  on_enter(cursor) is called once for every
// request entered on the way (requests without tiles are skipped by every role alike),
// including the one the cursor lands in.  The caller never moves past the CTA's range.
template <int NEXT_N, int TILE, typename F>
__device__ __forceinline__ void advance_by(TileCursor& c, int k, const int32_t* ctx, int batch, int max_ctx,
                                           F&& on_enter) {
    c.j += k;
    while (c.j >= c.tiles_b) {
        c.j -= c.tiles_b;
        do {
            ++c.b;
            if (c.b >= batch) {      // cannot happen inside the range; keeps the loop finite
                c.tiles_b = 0x3fffffff;
                c.ctx_b = 0;
                return;
            }
            c.ctx_b = request_ctx<NEXT_N>(ctx, c.b, max_ctx);
            c.tiles_b = (c.ctx_b + TILE - 1) / TILE;
        } while (c.tiles_b == 0);
        on_enter(c);
    }
}

// Ring position that advances without integer division.
struct Ring {
    int idx = 0;
    uint32_t phase = 0;
    __device__ __forceinline__ void step(int n, int size) {   // n <= size
        idx += n;
        if (idx >= size) {
            idx -= size;
            phase ^= 1u;
        }
    }
};

}  // namespace tiles
}  // namespace wuda
