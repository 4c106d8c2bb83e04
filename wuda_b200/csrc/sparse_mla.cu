// Sparse MLA decode attention over gathered FP8 cache records.
//
// Per request, one query token with `heads` heads of 512 dims attends to a list of keys named
// by index: first the sliding-window entries of one pool, then the top-k compressed entries of
// a second pool.  A key is a 584-byte "MODEL1" record (448 e4m3 values with one power-of-two
// scale byte per 64, then 64 bf16 rotary values); the value vector of a key is the key itself.
//   logit[h, t] = softmax_scale * sum_d q[h, d] * k[t, d]
//   out[h, :]   = sum_t exp(logit[h, t]) * k[t, :] / (sum_t exp(logit[h, t]) + exp(sink[h]))
// This is the role the reference gives to a third-party kernel at
// dsv4_megakernel/megakernel/test/test_e2e_decode.py:719-728; the arithmetic is the torch twin
// ref_flash_attn (:377-392) over records dequantised as deq_model1_row (:346-356), the same
// online-softmax form as dsv4_megakernel/origin/kernel.py:276-352.
//
// One CTA owns one request and one 256-dim half of the output (the 512 fp32 accumulator
// columns of a full row do not fit beside the scores in tensor memory); both halves compute
// the full scores.  An MMA of this shape costs about 70 cycles however few keys it covers, so
// Q K^T runs over blocks of 64 keys (32 MMAs per block); the tensor memory that leaves beside the
// output half (256 columns) and one score block (64) holds the first 384 dims of the query as
// the A operand (192 columns of fp16 pairs), the last 128 dims are a shared-memory operand.  Roles:
//   warps 0-3   softmax: thread = head row = tensor-memory lane.  Scores of a 64-key block are
//               read from tensor memory, scaled, masked, exponentiated against a running
//               reference maximum and written to shared memory as fp16 probabilities.  The
//               accumulator is rescaled only when the maximum grows by more than 2^8 (the final
//               division uses the same reference, so the result does not depend on when).
//   warps 4-11  key producers: gather records with plain loads (8 lanes per key), expand e4m3 *
//               2^E to fp16 (exact for E in [-15, 7], two instructions per pair; the query, the
//               rotary values and the probabilities are fp16 as well) and store the block in the
//               128-byte-swizzled operand layout.
//               The same bytes serve as the K-major operand of Q K^T and as the MN-major
//               operand of P V.
//   warps 12-13 issue Q K^T, of the even and of the odd blocks: a thread gets one MMA out about every hundred
//               cycles and spends as long again on the commit, the loop and its waits, so one of the two is
//               already waiting for the score tile when the other's MMAs retire;
//   warp 14     issues P V of a block as soon as its probabilities are stored.
// Every wait is bounded; a wait that runs out leaves a code in the status word and the CTA
// exits normally.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "host.h"
#include "ptx.cuh"

namespace wuda {
namespace mla {

constexpr int kDim = 512;          // key / query / value dims
constexpr int kNope = 448;         // e4m3 part
constexpr int kBody = 576;         // 448 + 64 * 2 bytes
constexpr int kScaleRec = 8;       // 7 scale bytes + 1 pad
constexpr int kRows = 128;         // UMMA M: head rows, zero-padded
constexpr int kBlock = 64;         // keys per block
constexpr int kPass = 32;          // keys the producer warps convert at a time (4 per warp)
constexpr int kHalf = 256;         // output dims per CTA
constexpr int kSoftmaxWarps = 4;
constexpr int kProducerWarps = 8;
constexpr int kIssuerWarp = kSoftmaxWarps + kProducerWarps;   // two warps issue Q K^T, of the even and of the odd blocks
constexpr int kIssuerWarpPV = kIssuerWarp + 2;                 // issues P V
constexpr int kThreads = (kIssuerWarpPV + 1) * 32;
constexpr float kLog2e = 1.4426950408889634f;
constexpr int kAhead = 3;             // passes whose records are in flight ahead of the one being stored
constexpr int kMaxSplits = 32;        // CTAs that may share one request's keys (per output half)
constexpr float kRescaleStep = 8.0f;   // log2 units the block maximum may exceed the reference by

// shared memory, offsets from a 1024-byte aligned base
// A key block's own output half (4 of its 8 chunks) is needed until P V of the block has run, its other half
// only until Q K^T has: two rings of different depth let the producers run a block further ahead than
// whole-block stages of the same total size would.
constexpr int kOwnStages = 3;
constexpr int kOthStages = 2;
constexpr int kQTmemChunks = 6;                         // 64-dim chunks of the query held in tensor memory
constexpr uint32_t kQChunk = kRows * 128;               // one 64-dim chunk of the query: [128 rows][128 B]
constexpr uint32_t kQSmemBytes = (8 - kQTmemChunks) * kQChunk;
constexpr uint32_t kKChunk = kBlock * 128;              // one 64-dim chunk of a key block: [64 keys][128 B]
constexpr uint32_t kHalfStageBytes = 4 * kKChunk;
constexpr uint32_t kPBytes = kRows * kBlock * 2;        // 8 pieces of [128 rows][16 B]
constexpr uint32_t kPPiece = kRows * 16;
constexpr uint32_t kOffQ = 0;
constexpr uint32_t kOffOwn = kOffQ + kQSmemBytes;
constexpr uint32_t kOffOth = kOffOwn + kOwnStages * kHalfStageBytes;
constexpr uint32_t kOffP = kOffOth + kOthStages * kHalfStageBytes;
constexpr uint32_t kOffValid = kOffP + 2 * kPBytes;     // kOwnStages x 16 bytes: per pass and producer warp, 4 valid bits
constexpr uint32_t kOffBars = kOffValid + kOwnStages * 16;
constexpr uint32_t kNumBars = 2 * kOwnStages + kOthStages + 8;
constexpr uint32_t kOffMisc = kOffBars + kNumBars * 8;
constexpr uint32_t kSmemBytes = kOffMisc + 16 + 1024;

constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColQ = 0, kColO = kQTmemChunks * 32, kColS = kColO + kHalf;   // query pairs | output half | scores
static_assert(kColS + kBlock <= kTmemCols, "tensor memory columns");

struct Pool {
    const uint8_t* data;
    int64_t stride;
    int pages, epb;
    int epb_shift;            // log2(epb) when epb is a power of two, else -1
    const int32_t* indices;   // [batch, capacity]
    const int32_t* lengths;   // [batch]
    int capacity;
};

struct Params {
    const __nv_bfloat16* q;   // [batch, heads, 512]
    Pool swa, cmp;
    const float* sink;        // [heads] or nullptr
    float scale_log2;         // softmax_scale * log2(e)
    __nv_bfloat16* out;       // [batch, heads, 512]
    int heads;
    int* status;
    float* part_o;            // [batch, splits, heads, 512] unnormalised sums, when a request is split
    float* part_ml;           // [batch, splits, heads, 2] reference maximum (log2 units) and sum
};

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// The MMAs run on fp16 operands: e4m3 * 2^E is exact in fp16 for E in [-15, 7] (every value from
// 2^-9 * 2^-15 = 2^-24 up to 448 * 2^7 < 65504), which costs two instructions per pair of values where
// the way to bf16 costs six; the cache writers clamp their scales at 1e-4 (E >= -13) and E > 7 would
// mean activations beyond 57344.  A scale byte outside that range is clamped into it and reported.
constexpr int kScaleExpLo = -15, kScaleExpHi = 7;

// 2^E as a pair of fp16, E = byte - 127 clamped to the exact range; `*clamped` is raised when it was
__device__ __forceinline__ uint32_t scale_f16x2(uint32_t byte, bool* clamped) {
    const int raw = static_cast<int>(byte) - 127;
    const int e = min(max(raw, kScaleExpLo), kScaleExpHi);
    *clamped |= e != raw;
    const uint32_t h = e >= -14 ? static_cast<uint32_t>(e + 15) << 10 : 0x0200u;   // 2^-15 is subnormal
    return h | (h << 16);
}

__device__ __forceinline__ uint32_t e4m3x2_to_f16x2(uint32_t pair, uint32_t scale2) {
    uint32_t h2, r;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(static_cast<unsigned short>(pair)));
    asm("mul.f16x2 %0, %1, %2;" : "=r"(r) : "r"(h2), "r"(scale2));
    return r;
}

// two bf16 -> two fp16, saturating at the largest finite fp16 (exact for normal-range values)
__device__ __forceinline__ uint32_t bf16x2_to_f16x2(uint32_t v) {
    const float lo = fminf(fmaxf(__uint_as_float(v << 16), -65504.0f), 65504.0f);
    const float hi = fminf(fmaxf(__uint_as_float(v & 0xffff0000u), -65504.0f), 65504.0f);
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
}
__device__ __forceinline__ uint4 bf16x8_to_f16x8(uint4 v) {
    return make_uint4(bf16x2_to_f16x2(v.x), bf16x2_to_f16x2(v.y), bf16x2_to_f16x2(v.z), bf16x2_to_f16x2(v.w));
}

__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint4 v) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                 : "memory");
}

// One key's share of a lane: 8 e4m3 of each of the 7 scaled tiles, 8 rotary bf16, the scale bytes.
struct KeyRegs {
    uint2 nope[7];
    uint4 rope;
    uint2 scales;
    int valid;
};

// The pool entry of key position g of request b (window entries first), -1 past the end.  Loaded one
// pass before the record loads that depend on it, so that those are not held up by its latency.
__device__ __forceinline__ int fetch_index(const Params& p, int b, int g, int n_swa, int n_total) {
    if (g >= n_total) return -1;
    const bool window = g < n_swa;
    const Pool& pool = window ? p.swa : p.cmp;
    // (read-only loads are sound here although the top-k entries, this step's cache records and the query come from
    // kernels of the same chain: this kernel is launched without the programmatic-launch attribute, i.e. only
    // after those kernels have finished)
    return __ldg(pool.indices + static_cast<int64_t>(b) * pool.capacity + (window ? g : g - n_swa));
}

__device__ __forceinline__ void fetch_key(const Params& p, int g, int n_swa, int idx, int piece, KeyRegs& r, bool* bad) {
    r.valid = 0;
    if (idx < 0) return;
    const Pool& pool = g < n_swa ? p.swa : p.cmp;
    const int page = pool.epb_shift >= 0 ? idx >> pool.epb_shift : idx / pool.epb, off = idx - page * pool.epb;
    if (page >= pool.pages) {
        *bad = true;
        return;
    }
    const uint8_t* base = pool.data + static_cast<int64_t>(page) * pool.stride;
    const uint8_t* rec = base + static_cast<int64_t>(off) * kBody;
#pragma unroll
    for (int c = 0; c < 7; ++c) r.nope[c] = __ldg(reinterpret_cast<const uint2*>(rec + c * 64) + piece);
    r.rope = __ldg(reinterpret_cast<const uint4*>(rec + kNope) + piece);
    r.scales = __ldg(reinterpret_cast<const uint2*>(base + static_cast<int64_t>(pool.epb) * kBody + off * kScaleRec));
    r.valid = 1;
}

// `lo_addr` / `hi_addr`: where dims 0-255 / 256-511 of the block go (4 chunks each)
__device__ __forceinline__ void store_key(uint32_t lo_addr, uint32_t hi_addr, int row, int piece, const KeyRegs& r,
                                          bool* clamped) {
    const uint32_t in_chunk = row * 128 + ((piece ^ (row & 7)) << 4);
    if (!r.valid) {
#pragma unroll
        for (int c = 0; c < 8; ++c)
            st_shared_v4((c < 4 ? lo_addr : hi_addr) + (c & 3) * kKChunk + in_chunk, make_uint4(0, 0, 0, 0));
        return;
    }
#pragma unroll
    for (int c = 0; c < 7; ++c) {
        const uint32_t byte = ((c < 4 ? r.scales.x : r.scales.y) >> ((c & 3) * 8)) & 0xffu;
        const uint32_t s = scale_f16x2(byte, clamped);
        uint4 v;
        v.x = e4m3x2_to_f16x2(r.nope[c].x & 0xffffu, s);
        v.y = e4m3x2_to_f16x2(r.nope[c].x >> 16, s);
        v.z = e4m3x2_to_f16x2(r.nope[c].y & 0xffffu, s);
        v.w = e4m3x2_to_f16x2(r.nope[c].y >> 16, s);
        st_shared_v4((c < 4 ? lo_addr : hi_addr) + (c & 3) * kKChunk + in_chunk, v);
    }
    st_shared_v4(hi_addr + 3 * kKChunk + in_chunk, bf16x8_to_f16x8(r.rope));
}

__global__ void __launch_bounds__(kThreads, 1) sparse_mla_kernel(const Params p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t base = (raw_addr + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (base - raw_addr);
    const uint32_t bars = base + kOffBars;
    // per stage: key block stored / its weighted sum complete; scores complete / read; per
    // probability buffer: probabilities stored / weighted sum complete
    const uint32_t k_full = bars, own_free = bars + kOwnStages * 8, oth_free = bars + 2 * kOwnStages * 8,
                   s_full = oth_free + kOthStages * 8, s_empty = s_full + 16, p_full = s_full + 32, pv_done = s_full + 48;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(base_ptr + kOffMisc);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(base_ptr + kOffMisc + 4);
    volatile uint8_t* valid_bytes = base_ptr + kOffValid;

    const int warp = threadIdx.x >> 5;
    const int lane = static_cast<int>(lane_id());
    const int half = blockIdx.x, b = blockIdx.y;

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int i = 0; i < kOwnStages; ++i) {
            mbar_init(k_full + i * 8, kProducerWarps);   // every producer warp, once per block
            mbar_init(own_free + i * 8, 1);
        }
        for (int i = 0; i < kOthStages; ++i) mbar_init(oth_free + i * 8, 1);
        for (int i = 0; i < 2; ++i) {   // one pair per score issuer (blocks of even / odd number)
            mbar_init(s_full + i * 8, 1);
            mbar_init(s_empty + i * 8, kSoftmaxWarps);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(p_full + i * 8, kSoftmaxWarps);
            mbar_init(pv_done + i * 8, 1);
        }
        fence_mbar_init();
    }
    if (warp == kIssuerWarp) {
        tmem_alloc(smem_u32(tmem_slot), kTmemCols);
        tmem_relinquish();
    }
    pdl_launch_dependents();   // the kernel behind this one may set itself up early; this one was launched in order

    const int n_swa = p.swa.capacity > 0 ? min(max(__ldg(p.swa.lengths + b), 0), p.swa.capacity) : 0;
    const int n_cmp = p.cmp.capacity > 0 ? min(max(__ldg(p.cmp.lengths + b), 0), p.cmp.capacity) : 0;
    const int n_total = n_swa + n_cmp;
    // the CTAs of a request that share an output half each take a contiguous run of its key blocks
    const int all_blocks = (n_total + kBlock - 1) / kBlock;
    const int per_split = (all_blocks + static_cast<int>(gridDim.z) - 1) / static_cast<int>(gridDim.z);
    const int first = static_cast<int>(blockIdx.z) * per_split;
    const int blocks = min(max(all_blocks - first, 0), per_split);

    tc_fence_before();
    __syncthreads();   // the tensor-memory base address is published
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // the query rows, zero-padded to 128: rotary dims to shared memory in the swizzled K-major operand
    // layout, scaled dims to tensor memory (row = lane, column = a pair of dims)
    constexpr int kQSmemPieces = (8 - kQTmemChunks) * 8;
    for (int i = threadIdx.x; i < kRows * kQSmemPieces; i += kThreads) {
        const int row = i / kQSmemPieces, piece = i % kQSmemPieces;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (row < p.heads)
            v = __ldg(reinterpret_cast<const uint4*>(p.q + (static_cast<int64_t>(b) * p.heads + row) * kDim +
                                                     kQTmemChunks * 64) + piece);
        st_shared_v4(base + kOffQ + (piece >> 3) * kQChunk + row * 128 + (((piece & 7) ^ (row & 7)) << 4), bf16x8_to_f16x8(v));
    }
    if (warp < kSoftmaxWarps) {
        const int row = warp * 32 + lane;
        const uint4* src = reinterpret_cast<const uint4*>(p.q + (static_cast<int64_t>(b) * p.heads + row) * kDim);
#pragma unroll 1
        for (int c = 0; c < kQTmemChunks; ++c) {
            uint32_t w[32];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const uint4 v = bf16x8_to_f16x8(row < p.heads ? __ldg(src + c * 8 + i) : make_uint4(0, 0, 0, 0));
                w[4 * i] = v.x, w[4 * i + 1] = v.y, w[4 * i + 2] = v.z, w[4 * i + 3] = v.w;
            }
            tmem_st_32x32(tmem_base + (static_cast<uint32_t>(warp * 32) << 16) + kColQ + c * 32, w);
        }
        tmem_st_wait();
    }
    fence_proxy_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();

    if (warp >= kSoftmaxWarps && warp < kIssuerWarp) {
        // ------------------------------------------------------------ key producers
        const int pw = warp - kSoftmaxWarps;
        const int row = pw * 4 + (lane >> 3), piece = lane & 7;
        bool bad = false, clamped = false;
        // a block's records are requested kAhead blocks before they are converted: a gather from
        // random pages takes far longer than one block's turn through the pipeline
        KeyRegs ring[kAhead + 1];
        constexpr int kPasses = kBlock / kPass;
        const int passes = blocks * kPasses, first_key = first * kBlock;
#pragma unroll
        for (int u = 0; u < kAhead; ++u) {
            const int g = first_key + u * kPass + row;
            fetch_key(p, g, n_swa, fetch_index(p, b, g, n_swa, n_total), piece, ring[u], &bad);
        }
        int next_idx = fetch_index(p, b, first_key + kAhead * kPass + row, n_swa, n_total);
        bool alive = true;
        for (int q0 = 0; q0 < passes && alive; q0 += kAhead + 1) {
#pragma unroll
            for (int u = 0; u <= kAhead; ++u) {
                const int q = q0 + u;
                if (q >= passes) break;
                const int j = q / kPasses, sub = q % kPasses;
                const int s = j % kOwnStages, t = j % kOthStages;
                const int g_ahead = first_key + (q + kAhead) * kPass + row;
                fetch_key(p, g_ahead, n_swa, next_idx, piece, ring[(u + kAhead) % (kAhead + 1)], &bad);
                next_idx = fetch_index(p, b, g_ahead + kPass, n_swa, n_total);
                if (sub == 0) {
                    if (j >= kOwnStages)
                        alive = mbar_wait_warp(own_free + s * 8, (j / kOwnStages - 1) & 1u, abort_flag, p.status,
                                               kDevTimeoutMlaOutput);
                    if (alive && j >= kOthStages)
                        alive = mbar_wait_warp(oth_free + t * 8, (j / kOthStages - 1) & 1u, abort_flag, p.status,
                                               kDevTimeoutMlaScores);
                }
                if (!alive) break;
                const uint32_t own_addr = base + kOffOwn + s * kHalfStageBytes, oth_addr = base + kOffOth + t * kHalfStageBytes;
                store_key(half == 0 ? own_addr : oth_addr, half == 0 ? oth_addr : own_addr, sub * kPass + row, piece, ring[u],
                          &clamped);
                const uint32_t bits = __ballot_sync(0xffffffffu, ring[u].valid != 0);
                if (lane == 0)
                    valid_bytes[s * 16 + sub * 8 + pw] = static_cast<uint8_t>(
                        (bits & 1u) | ((bits >> 7) & 2u) | ((bits >> 14) & 4u) | ((bits >> 21) & 8u));
                if (sub == kPasses - 1) {   // the block's last pass: one fence and one arrival cover both passes' stores
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(k_full + s * 8);
                }
            }
        }
        if (bad && p.status) atomicCAS(p.status, 0, static_cast<int>(kDevBadPageIndex));
        if (clamped && p.status) atomicCAS(p.status, 0, static_cast<int>(kDevMlaScaleRange));
    } else if (warp == kIssuerWarp || warp == kIssuerWarp + 1) {
        // ------------------------------------------------------------ score issuers
        // A block's 32 MMAs keep their issuing thread busy for longer than they keep the tensor pipe, and the commit,
        // the loop and the two waits behind them cost that thread as much again while the other warps of its scheduler
        // compute; so two threads take the blocks alternately: one is already waiting for the score tile to be read
        // when the other's MMAs retire.  Each has its own pair of barriers, so that it sees every phase of the ones it
        // waits on.
        const int me = warp - kIssuerWarp;
        constexpr uint32_t idesc_qk = umma_idesc(kRows, kBlock, 0, 0);     // fp16 operands
        bool alive = true;
        for (int j = me; j < blocks && alive; j += 2) {
            {
                const int s = j % kOwnStages, t = j % kOthStages;
                alive = mbar_wait_lane0(k_full + s * 8, (j / kOwnStages) & 1u, abort_flag, p.status, kDevTimeoutMlaKeys);
                if (alive && j >= 1)
                    alive = mbar_wait_lane0(s_empty + (me ^ 1) * 8, ((j - 1) >> 1) & 1u, abort_flag, p.status,
                                            kDevTimeoutMlaScoresRead);   // the block before, the other issuer's
                if (!alive) break;
                tc_fence_after();
                if (lane == 0) {
                    const uint32_t own_addr = base + kOffOwn + s * kHalfStageBytes, oth_addr = base + kOffOth + t * kHalfStageBytes;
                    // descriptors differ only in their 14-bit address field: one add per MMA
                    const uint64_t own_desc = umma_smem_desc_sw128(own_addr), oth_desc = umma_smem_desc_sw128(oth_addr);
                    const uint64_t q_desc = umma_smem_desc_sw128(base + kOffQ);
#pragma unroll
                    for (int c = 0; c < 8; ++c)
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            const uint64_t k_desc = ((c >> 2) == half ? own_desc : oth_desc) + (((c & 3) * kKChunk + k * 32) >> 4);
                            if (c < kQTmemChunks)
                                umma_f16_ta(tmem_base + kColS, tmem_base + kColQ + c * 32 + k * 8, k_desc, idesc_qk, (c | k) != 0);
                            else
                                umma_f16(tmem_base + kColS, q_desc + (((c - kQTmemChunks) * kQChunk + k * 32) >> 4), k_desc,
                                         idesc_qk, 1u);
                        }
                    umma_commit(s_full + me * 8);   // (the other half's ring stage is released by the softmax, which sees this commit)
                }
                __syncwarp();
            }
        }
    } else if (warp == kIssuerWarpPV) {
        // ------------------------------------------------------------ weighted-sum issuer
        // A thread issues an MMA about every hundred cycles whatever its size; with the weighted sums on a thread of
        // their own the score issuer goes straight on to the next block.
        constexpr uint32_t idesc_pv = umma_idesc_b_mn(kRows, kHalf, 0, 0);
        bool alive = true;
        for (int j = 0; j < blocks && alive; ++j) {
            const int t = j & 1, s = j % kOwnStages;
            alive = mbar_wait_lane0(p_full + t * 8, (j >> 1) & 1u, abort_flag, p.status, kDevTimeoutMlaProbs);
            if (!alive) break;
            tc_fence_after();
            if (lane == 0) {
                const uint32_t p_addr = base + kOffP + t * kPBytes;
                const uint32_t v_addr = base + kOffOwn + s * kHalfStageBytes;
#pragma unroll
                for (int k = 0; k < kBlock / 16; ++k)   // 16 keys each
                    umma_f16(tmem_base + kColO, umma_smem_desc_noswz(p_addr + k * 2 * kPPiece, kPPiece, 128),
                             umma_smem_desc_mn_sw128(v_addr + k * 16 * 128, kKChunk), idesc_pv, j > 0 || k > 0);
                umma_commit(pv_done + t * 8);   // the probability buffer and the accumulator
                umma_commit(own_free + s * 8);  // this half of the key block
            }
            __syncwarp();
        }
    } else {
        // ------------------------------------------------------------ softmax and output
        const int row = warp * 32 + lane;
        const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
        float m_ref = -INFINITY, l = 0.0f;
        bool alive = true;
        for (int j = 0; j < blocks && alive; ++j) {
            const int s = j & 1, stage = j % kOwnStages;
            alive = mbar_wait_warp(s_full + (j & 1) * 8, (j >> 1) & 1u, abort_flag, p.status, kDevTimeoutMlaScores);
            // the scores are complete: the half of the key block that only they needed may be refilled (a second
            // tcgen05.commit would hold the issuing thread for several hundred cycles)
            if (alive && warp == 0 && lane == 0) mbar_arrive(oth_free + (j % kOthStages) * 8);
            if (!alive) break;
            tc_fence_after();
            // the block's valid bits were published before its keys were announced, and its stage is
            // not refilled before this block's weighted sum has run
            const volatile uint32_t* vw = reinterpret_cast<const volatile uint32_t*>(valid_bytes + stage * 16);
            float x[kBlock], bm[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};   // four chains, not one of 64
            {   // raw scores into registers, then the score buffer goes back to the issuer at once
                uint32_t* raw = reinterpret_cast<uint32_t*>(x);
                tmem_ld_32x32(lane_addr + kColS, *reinterpret_cast<uint32_t(*)[32]>(raw));
                tmem_ld_32x32(lane_addr + kColS + 32, *reinterpret_cast<uint32_t(*)[32]>(raw + 32));
                tmem_ld_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(s_empty + (j & 1) * 8);
            }
            // A block whose 64 keys all exist (every block but a request's last) needs no masks: the maximum is taken
            // over the raw scores and the scale rides in the exponent's multiply-add.  Otherwise missing keys become
            // -inf and the scores are scaled in place.
            const bool all_valid = (vw[0] & vw[1] & vw[2] & vw[3]) == 0x0f0f0f0fu;   // the same word for every thread
            float sc = p.scale_log2;
            if (all_valid) {
#pragma unroll
                for (int i = 0; i < kBlock; ++i) bm[i & 3] = fmaxf(bm[i & 3], x[i]);
#pragma unroll
                for (int c = 0; c < 4; ++c) bm[c] *= p.scale_log2;
            } else {
                sc = 1.0f;
#pragma unroll
                for (int h2 = 0; h2 < kBlock / 32; ++h2) {
                    const uint2 vb = make_uint2(vw[2 * h2], vw[2 * h2 + 1]);
                    uint32_t mask = 0;
#pragma unroll
                    for (int w = 0; w < 4; ++w) {
                        mask |= ((vb.x >> (8 * w)) & 0xfu) << (4 * w);
                        mask |= ((vb.y >> (8 * w)) & 0xfu) << (16 + 4 * w);
                    }
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        x[h2 * 32 + i] = (mask >> i) & 1u ? x[h2 * 32 + i] * p.scale_log2 : -INFINITY;
                        bm[i & 3] = fmaxf(bm[i & 3], x[h2 * 32 + i]);
                    }
                }
            }
            const float bmax = fmaxf(fmaxf(bm[0], bm[1]), fmaxf(bm[2], bm[3]));
            const bool grow = bmax > m_ref + kRescaleStep;   // also the first finite maximum
            if (__any_sync(0xffffffffu, grow)) {
                const float m_new = grow ? bmax : m_ref;
                const float f = grow ? ex2(m_ref - m_new) : 1.0f;   // 0 on the first finite maximum
                if (j > 0) {
                    alive = mbar_wait_warp(pv_done + ((j - 1) & 1) * 8, ((j - 1) >> 1) & 1u, abort_flag, p.status,
                                           kDevTimeoutMlaOutput);
                    if (!alive) break;
                    tc_fence_after();
#pragma unroll 1
                    for (int c = 0; c < kHalf; c += 32) {
                        uint32_t o[32];
                        tmem_ld_32x32(lane_addr + kColO + c, o);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * f);
                        tmem_st_32x32(lane_addr + kColO + c, o);
                    }
                    tmem_st_wait();
                    tc_fence_before();
                }
                l *= f;
                m_ref = m_new;
            }
            // while the reference is still -inf every score of the row is -inf too: 2^(-inf - 0) = 0
            const float m_use = m_ref == -INFINITY ? 0.0f : m_ref;
            float sm[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            uint32_t pk[kBlock / 2];
#pragma unroll
            for (int i = 0; i < kBlock; i += 2) {
                const float e0 = ex2(fmaf(x[i], sc, -m_use)), e1 = ex2(fmaf(x[i + 1], sc, -m_use));
                sm[(i >> 1) & 3] += e0 + e1;
                const __half2 h = __floats2half2_rn(e0, e1);
                pk[i >> 1] = *reinterpret_cast<const uint32_t*>(&h);
            }
            l += (sm[0] + sm[1]) + (sm[2] + sm[3]);
            if (j >= 2) {   // the weighted sum of block j-2 has read this probability buffer
                alive = mbar_wait_warp(pv_done + s * 8, ((j >> 1) - 1) & 1u, abort_flag, p.status, kDevTimeoutMlaOutput);
                if (!alive) break;
            }
            const uint32_t p_addr = base + kOffP + s * kPBytes + row * 16;
#pragma unroll
            for (int c = 0; c < kBlock / 8; ++c)
                st_shared_v4(p_addr + c * kPPiece, make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]));
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full + s * 8);
        }
        if (alive && blocks > 0)
            alive = mbar_wait_warp(pv_done + ((blocks - 1) & 1) * 8, ((blocks - 1) >> 1) & 1u, abort_flag, p.status,
                                   kDevTimeoutMlaOutput);
        if (alive && gridDim.z > 1) {
            // partial result of this run of blocks: the unnormalised sums with their reference maximum
            tc_fence_after();
            const int64_t slot = (static_cast<int64_t>(b) * gridDim.z + blockIdx.z) * p.heads + row;
            if (row < p.heads && half == 0) {
                p.part_ml[slot * 2] = blocks > 0 ? m_ref : -INFINITY;
                p.part_ml[slot * 2 + 1] = blocks > 0 ? l : 0.0f;
            }
            if (blocks > 0) {   // the combine step skips partials whose maximum is -inf
                float* dst = p.part_o + slot * kDim + half * kHalf;
#pragma unroll 1
                for (int c = 0; c < kHalf; c += 32) {
                    uint32_t o[32];
                    tmem_ld_32x32(lane_addr + kColO + c, o);
                    tmem_ld_wait();
                    if (row < p.heads) {
#pragma unroll
                        for (int i = 0; i < 32; i += 4)
                            *reinterpret_cast<uint4*>(dst + c + i) = make_uint4(o[i], o[i + 1], o[i + 2], o[i + 3]);
                    }
                }
            }
            tc_fence_before();
        } else if (alive) {
            tc_fence_after();
            const bool any = blocks > 0 && m_ref != -INFINITY;
            float inv = 0.0f;
            if (any) {
                const float sink = (p.sink && row < p.heads) ? ex2(__ldg(p.sink + row) * kLog2e - m_ref) : 0.0f;
                inv = 1.0f / (l + sink);   // an overwhelming sink gives 1 / inf = 0
            }
            __nv_bfloat16* dst = p.out + (static_cast<int64_t>(b) * p.heads + row) * kDim + half * kHalf;
#pragma unroll 1
            for (int c = 0; c < kHalf; c += 32) {
                uint32_t o[32];
                if (blocks > 0) {   // warp-uniform: without a block the accumulator was never written
                    tmem_ld_32x32(lane_addr + kColO + c, o);
                    tmem_ld_wait();
                }
                if (row < p.heads) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        uint32_t w[4];
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            const float lo = any ? __uint_as_float(o[i + 2 * k]) * inv : 0.0f;
                            const float hi = any ? __uint_as_float(o[i + 2 * k + 1]) * inv : 0.0f;
                            const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
                            w[k] = *reinterpret_cast<const uint32_t*>(&h);
                        }
                        *reinterpret_cast<uint4*>(dst + c + i) = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                }
            }
            tc_fence_before();
        }
    }

    __syncthreads();
    if (*abort_flag) abort_drain_sleep();
    __syncthreads();
    if (warp == kIssuerWarp) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

// Merges the partial results of a split request: weights 2^(m_z - max m), the sink in the denominator.
__global__ void __launch_bounds__(128) sparse_mla_combine_kernel(const Params p, int splits) {
    pdl_launch_dependents();
    pdl_wait();
    const int h = blockIdx.x, b = blockIdx.y;
    const int64_t first = (static_cast<int64_t>(b) * splits) * p.heads + h;
    float m = -INFINITY;
    for (int z = 0; z < splits; ++z) m = fmaxf(m, p.part_ml[(first + static_cast<int64_t>(z) * p.heads) * 2]);
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    float den = 0.0f;
    if (m != -INFINITY) {
        for (int z = 0; z < splits; ++z) {
            const int64_t slot = first + static_cast<int64_t>(z) * p.heads;
            const float mz = p.part_ml[slot * 2];
            if (mz == -INFINITY) continue;
            const float w = ex2(mz - m);
            den += w * p.part_ml[slot * 2 + 1];
            const float4 o = *reinterpret_cast<const float4*>(p.part_o + slot * kDim + threadIdx.x * 4);
            acc.x += w * o.x, acc.y += w * o.y, acc.z += w * o.z, acc.w += w * o.w;
        }
        if (p.sink) den += ex2(__ldg(p.sink + h) * kLog2e - m);
    }
    const float inv = m != -INFINITY ? 1.0f / den : 0.0f;
    const __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x * inv, acc.y * inv), hi = __floats2bfloat162_rn(acc.z * inv, acc.w * inv);
    uint2 v;
    v.x = *reinterpret_cast<const uint32_t*>(&lo);
    v.y = *reinterpret_cast<const uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p.out + (static_cast<int64_t>(b) * p.heads + h) * kDim + threadIdx.x * 4) = v;
}

// CTAs per request and output half: enough to give every SM one, at least two key blocks each.
static int splits_for(int batch, int key_capacity, int num_sms) {
    const int blocks = (key_capacity + kBlock - 1) / kBlock;
    int s = num_sms / (2 * batch);
    if (s > blocks / 2) s = blocks / 2;
    if (s > kMaxSplits) s = kMaxSplits;
    return s < 1 ? 1 : s;
}

static int check_pool(const char* name, const void* data, int64_t stride, int pages, int epb, const int32_t* indices,
                      const int32_t* lengths, int capacity, Pool* out) {
    WUDA_REQUIRE(capacity >= 0, "%s_capacity must be >= 0 (got %d)", name, capacity);
    out->capacity = capacity;
    if (capacity == 0) {
        out->data = nullptr, out->indices = nullptr, out->lengths = nullptr;
        out->stride = 0, out->pages = 0, out->epb = 1, out->epb_shift = 0;
        return WUDA_OK;
    }
    WUDA_REQUIRE(data && indices && lengths, "%s pool, indices and lengths must not be NULL when its capacity is > 0", name);
    WUDA_REQUIRE(pages >= 1 && epb >= 1, "%s pages and entries_per_block must be >= 1", name);
    WUDA_REQUIRE(aligned16(data) && stride % 16 == 0, "%s pool base and page stride must be multiples of 16 bytes", name);
    WUDA_REQUIRE(stride >= static_cast<int64_t>(epb) * (kBody + kScaleRec),
                 "%s page stride %lld is smaller than %d records of 584 bytes", name, static_cast<long long>(stride), epb);
    WUDA_REQUIRE((static_cast<int64_t>(epb) * kBody) % 8 == 0, "%s scale records must start on an 8-byte boundary", name);
    out->data = static_cast<const uint8_t*>(data);
    out->stride = stride;
    out->pages = pages;
    out->epb = epb;
    out->epb_shift = -1;
    for (int sft = 0; sft < 24; ++sft)
        if ((1 << sft) == epb) out->epb_shift = sft;
    out->indices = indices;
    out->lengths = lengths;
    return WUDA_OK;
}

}  // namespace mla
}  // namespace wuda

extern "C" int64_t wuda_sparse_mla_workspace_bytes(int batch, int heads, int key_capacity) {
    using namespace wuda;
    using namespace wuda::mla;
    if (batch < 1 || heads < 1 || heads > kRows || key_capacity < 0) return -1;
    DeviceInfo dev;
    if (current_device_info(&dev) != WUDA_OK) return -1;
    const int splits = splits_for(batch, key_capacity, dev.num_sms);
    if (splits <= 1) return 0;
    return static_cast<int64_t>(batch) * splits * heads * (kDim + 2) * 4;
}

extern "C" int wuda_sparse_mla_decode(const wuda_sparse_mla_args* a, int32_t* status_word, void* stream) {
    using namespace wuda;
    using namespace wuda::mla;
    clear_error();
    WUDA_REQUIRE(a != nullptr, "args must not be NULL");
    WUDA_REQUIRE(a->batch >= 0, "batch must be >= 0 (got %d)", a->batch);
    WUDA_REQUIRE(a->heads >= 1 && a->heads <= kRows, "heads must be in [1, 128] (got %d)", a->heads);
    if (a->batch == 0) return WUDA_OK;
    WUDA_REQUIRE(a->batch <= 65535, "batch must be <= 65535 (got %d)", a->batch);
    WUDA_REQUIRE(a->q && a->out, "q and out must not be NULL");
    WUDA_REQUIRE(aligned16(a->q) && aligned16(a->out), "q and out must be 16-byte aligned");
    WUDA_REQUIRE(a->softmax_scale > 0.0f && a->softmax_scale < 1e30f, "softmax_scale must be positive and finite");
    Params p;
    int st = check_pool("swa", a->swa_pool, a->swa_stride, a->swa_pages, a->swa_entries_per_block, a->swa_indices,
                        a->swa_lengths, a->swa_capacity, &p.swa);
    if (st != WUDA_OK) return st;
    st = check_pool("cmp", a->cmp_pool, a->cmp_stride, a->cmp_pages, a->cmp_entries_per_block, a->cmp_indices,
                    a->cmp_lengths, a->cmp_capacity, &p.cmp);
    if (st != WUDA_OK) return st;
    p.q = static_cast<const __nv_bfloat16*>(a->q);
    p.sink = a->attn_sink;
    p.scale_log2 = a->softmax_scale * kLog2e;
    p.out = static_cast<__nv_bfloat16*>(a->out);
    p.heads = a->heads;
    p.status = status_word;

    DeviceInfo dev;
    st = current_device_info(&dev);
    if (st != WUDA_OK) return st;
    if (static_cast<int>(kSmemBytes) > dev.smem_optin)
        return fail(WUDA_ERR_UNSUPPORTED, "device offers %d bytes of shared memory per block; the kernel needs %u",
                    dev.smem_optin, kSmemBytes);
    int splits = a->workspace ? splits_for(a->batch, a->swa_capacity + a->cmp_capacity, dev.num_sms) : 1;
    if (splits > 1) {
        const int64_t need = wuda_sparse_mla_workspace_bytes(a->batch, a->heads, a->swa_capacity + a->cmp_capacity);
        WUDA_REQUIRE(a->workspace_bytes >= need, "workspace holds %lld bytes; %lld are needed (wuda_sparse_mla_workspace_bytes)",
                     static_cast<long long>(a->workspace_bytes), static_cast<long long>(need));
        WUDA_REQUIRE(aligned16(a->workspace), "workspace must be 16-byte aligned");
        p.part_o = static_cast<float*>(a->workspace);
        p.part_ml = p.part_o + static_cast<int64_t>(a->batch) * splits * a->heads * kDim;
    } else {
        p.part_o = p.part_ml = nullptr;
    }
    WUDA_CUDA(cudaFuncSetAttribute(sparse_mla_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
    // An ordinary launch, not a programmatic one: the kernel gathers its records through the read-only path, which
    // is only sound for data that nobody writes while the kernel is resident - and the cache writers and the query
    // tail of the same step could still be running under an early launch.  (Coherent loads instead cost 10 % of
    // the kernel's time; the early launch it gives up is worth 2-3 us.)
    sparse_mla_kernel<<<dim3(2, a->batch, splits), dim3(kThreads), kSmemBytes, static_cast<cudaStream_t>(stream)>>>(p);
    WUDA_CUDA(cudaGetLastError());
    if (splits > 1)
        WUDA_CUDA(launch_pdl(sparse_mla_combine_kernel, dim3(a->heads, a->batch), dim3(128), 0,
                             static_cast<cudaStream_t>(stream), p, splits));
    return WUDA_OK;
}
