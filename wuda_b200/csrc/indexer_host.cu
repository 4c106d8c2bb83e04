// Host-buffer form of the indexer step (paged MQA logits -> top-k): the call a host
// program makes when its tensors live in host memory.  A plan owns the device-side
// staging buffers (allocated once, sized for the largest call); each call copies the
// inputs host->device on the caller's stream, launches the two kernels, copies the
// selected indices (and optionally the logits) back and synchronises the stream.
#include <cuda_runtime.h>

#include <new>

#include "host.h"

struct wuda_indexer_plan {
    int max_batch, next_n, num_blocks, epb, bt_stride, k, device;
    int64_t page_stride, logits_stride;
    uint8_t* q = nullptr;
    uint8_t* kv = nullptr;
    float* weights = nullptr;
    int32_t* ctx = nullptr;
    int32_t* bt = nullptr;
    float* logits = nullptr;
    int32_t* indices = nullptr;
    int32_t* status = nullptr;
};

extern "C" int wuda_indexer_plan_destroy(wuda_indexer_plan* plan) {
    if (!plan) return WUDA_OK;
    cudaFree(plan->q);
    cudaFree(plan->kv);
    cudaFree(plan->weights);
    cudaFree(plan->ctx);
    cudaFree(plan->bt);
    cudaFree(plan->logits);
    cudaFree(plan->indices);
    cudaFree(plan->status);
    delete plan;
    return WUDA_OK;
}

extern "C" int wuda_indexer_plan_create(wuda_indexer_plan** out, int max_batch, int next_n, int num_blocks,
                                        int entries_per_block, int64_t page_stride_bytes,
                                        int block_table_stride, int64_t logits_stride, int k) {
    using namespace wuda;
    clear_error();
    WUDA_REQUIRE(out, "plan output pointer must not be NULL");
    *out = nullptr;
    WUDA_REQUIRE(max_batch >= 1 && (next_n == 1 || next_n == 2) && num_blocks >= 1 && k >= 1,
                 "max_batch, num_blocks, k must be >= 1 and next_n 1 or 2");
    WUDA_REQUIRE(entries_per_block == 32 || entries_per_block == 64 || entries_per_block == 128,
                 "entries_per_block must be 32, 64 or 128");
    WUDA_REQUIRE(page_stride_bytes >= static_cast<int64_t>(entries_per_block) * 132 && page_stride_bytes % 16 == 0,
                 "page_stride_bytes must be a multiple of 16 and >= entries_per_block * 132");
    WUDA_REQUIRE(block_table_stride >= 1 && logits_stride >= 1 && logits_stride % 4 == 0,
                 "block_table_stride >= 1 and logits_stride a positive multiple of 4 are required");
    wuda_indexer_plan* p = new (std::nothrow) wuda_indexer_plan();
    if (!p) return fail(WUDA_ERR_CUDA, "out of host memory");
    p->max_batch = max_batch;
    p->next_n = next_n;
    p->num_blocks = num_blocks;
    p->epb = entries_per_block;
    p->bt_stride = block_table_stride;
    p->k = k;
    p->page_stride = page_stride_bytes;
    p->logits_stride = logits_stride;
    const int64_t rows = static_cast<int64_t>(max_batch) * next_n;
    cudaError_t e = cudaGetDevice(&p->device);
    if (e == cudaSuccess) e = cudaMalloc(&p->q, rows * 64 * 128);
    if (e == cudaSuccess) e = cudaMalloc(&p->kv, static_cast<size_t>(num_blocks) * page_stride_bytes);
    if (e == cudaSuccess) e = cudaMalloc(&p->weights, rows * 64 * sizeof(float));
    if (e == cudaSuccess) e = cudaMalloc(&p->ctx, rows * sizeof(int32_t));
    if (e == cudaSuccess) e = cudaMalloc(&p->bt, static_cast<size_t>(max_batch) * block_table_stride * sizeof(int32_t));
    if (e == cudaSuccess) e = cudaMalloc(&p->logits, rows * logits_stride * sizeof(float));
    if (e == cudaSuccess) e = cudaMalloc(&p->indices, rows * k * sizeof(int32_t));
    if (e == cudaSuccess) e = cudaMalloc(&p->status, sizeof(int32_t));
    if (e != cudaSuccess) {
        cudaGetLastError();
        wuda_indexer_plan_destroy(p);
        return fail(WUDA_ERR_CUDA, "indexer plan allocation failed: %s", cudaGetErrorString(e));
    }
    *out = p;
    return WUDA_OK;
}

namespace {

// Everything between the first enqueue and the final synchronisation; a failure in here must not
// return to the caller while copies from (or to) its host buffers are still in flight.
int indexer_topk_enqueue(wuda_indexer_plan* plan, const void* q_host, const void* kv_pages_host,
                         const int32_t* dirty_pages_host, int n_dirty, const float* weights_host, const int32_t* context_lens_host, const int32_t* block_table_host,
                         int32_t* page_indices_host, float* logits_host, int batch, int32_t* dev_status, cudaStream_t s) {
    using namespace wuda;
    const int64_t rows = static_cast<int64_t>(batch) * plan->next_n;
    WUDA_CUDA(cudaMemsetAsync(plan->status, 0, sizeof(int32_t), s));
    WUDA_CUDA(cudaMemcpyAsync(plan->q, q_host, rows * 64 * 128, cudaMemcpyHostToDevice, s));
    if (kv_pages_host && dirty_pages_host) {
        // only the pages the host names, one copy per run of consecutive page numbers
        for (int i = 0; i < n_dirty;) {
            int j = i + 1;
            while (j < n_dirty && dirty_pages_host[j] == dirty_pages_host[j - 1] + 1) ++j;
            const size_t at = static_cast<size_t>(dirty_pages_host[i]) * plan->page_stride;
            WUDA_CUDA(cudaMemcpyAsync(static_cast<uint8_t*>(plan->kv) + at, static_cast<const uint8_t*>(kv_pages_host) + at,
                                      static_cast<size_t>(j - i) * plan->page_stride, cudaMemcpyHostToDevice, s));
            i = j;
        }
    } else if (kv_pages_host) {
        WUDA_CUDA(cudaMemcpyAsync(plan->kv, kv_pages_host, static_cast<size_t>(plan->num_blocks) * plan->page_stride,
                                  cudaMemcpyHostToDevice, s));
    }
    WUDA_CUDA(cudaMemcpyAsync(plan->weights, weights_host, rows * 64 * sizeof(float), cudaMemcpyHostToDevice, s));
    WUDA_CUDA(cudaMemcpyAsync(plan->ctx, context_lens_host, rows * sizeof(int32_t), cudaMemcpyHostToDevice, s));
    WUDA_CUDA(cudaMemcpyAsync(plan->bt, block_table_host,
                              static_cast<size_t>(batch) * plan->bt_stride * sizeof(int32_t),
                              cudaMemcpyHostToDevice, s));
    int st = wuda_mqa_logits_fp8(plan->q, plan->kv, plan->weights, plan->ctx, plan->bt, plan->logits, batch,
                                 plan->next_n, plan->num_blocks, plan->epb, plan->page_stride, plan->bt_stride,
                                 plan->logits_stride, plan->status, s);
    if (st != WUDA_OK) return st;
    st = wuda_topk(plan->logits, plan->ctx, plan->bt, plan->indices, nullptr, static_cast<int>(rows),
                   plan->logits_stride, plan->bt_stride, plan->next_n, plan->k, plan->epb, s);
    if (st != WUDA_OK) return st;
    WUDA_CUDA(cudaMemcpyAsync(page_indices_host, plan->indices, rows * plan->k * sizeof(int32_t),
                              cudaMemcpyDeviceToHost, s));
    if (logits_host)
        WUDA_CUDA(cudaMemcpyAsync(logits_host, plan->logits, rows * plan->logits_stride * sizeof(float),
                                  cudaMemcpyDeviceToHost, s));
    WUDA_CUDA(cudaMemcpyAsync(dev_status, plan->status, sizeof(int32_t), cudaMemcpyDeviceToHost, s));
    return WUDA_OK;
}

}  // namespace

extern "C" int wuda_indexer_topk_host_pages(wuda_indexer_plan* plan, const void* q_host, const void* kv_pages_host,
                                            const int32_t* dirty_pages_host, int n_dirty, const float* weights_host,
                                            const int32_t* context_lens_host, const int32_t* block_table_host,
                                            int32_t* page_indices_host, float* logits_host, int batch, void* stream) {
    using namespace wuda;
    clear_error();
    WUDA_REQUIRE(n_dirty >= 0 && (n_dirty == 0 || (dirty_pages_host && kv_pages_host)),
                 "n_dirty must be >= 0, and a list of pages needs both the list and the host pool");
    if (plan)
        for (int i = 0; i < n_dirty; ++i)
            WUDA_REQUIRE(dirty_pages_host[i] >= 0 && dirty_pages_host[i] < plan->num_blocks, "dirty page %d is outside the pool of %d",
                         dirty_pages_host[i], plan->num_blocks);
    WUDA_REQUIRE(plan, "plan must not be NULL");
    WUDA_REQUIRE(batch >= 0 && batch <= plan->max_batch, "batch %d exceeds the plan's max_batch %d", batch,
                 plan->max_batch);
    if (batch == 0) return WUDA_OK;
    WUDA_REQUIRE(q_host && weights_host && context_lens_host && block_table_host && page_indices_host,
                 "host input and output pointers must not be NULL (only kv_pages_host may be: pool unchanged)");
    int dev = -1;
    WUDA_CUDA(cudaGetDevice(&dev));
    WUDA_REQUIRE(dev == plan->device, "the plan was created on device %d but device %d is current", plan->device, dev);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    int32_t dev_status = 0;
    const int st = indexer_topk_enqueue(plan, q_host, kv_pages_host, dirty_pages_host, n_dirty, weights_host, context_lens_host, block_table_host,
                                        page_indices_host, logits_host, batch, &dev_status, s);
    // on every path: no copy may outlive this call, the caller is free to reuse its host buffers
    const cudaError_t sync = cudaStreamSynchronize(s);
    if (st != WUDA_OK) return st;      // the message of the first failure stands
    if (sync != cudaSuccess) return fail(WUDA_ERR_CUDA, "cudaStreamSynchronize failed: %s", cudaGetErrorString(sync));
    if (dev_status != 0) return fail(WUDA_ERR_DEVICE_STATUS, "kernel reported device status %d", dev_status);
    return WUDA_OK;
}

extern "C" int wuda_indexer_topk_host(wuda_indexer_plan* plan, const void* q_host, const void* kv_pages_host,
                                      const float* weights_host, const int32_t* context_lens_host,
                                      const int32_t* block_table_host, int32_t* page_indices_host,
                                      float* logits_host, int batch, void* stream) {
    return wuda_indexer_topk_host_pages(plan, q_host, kv_pages_host, nullptr, 0, weights_host, context_lens_host, block_table_host,
                                        page_indices_host, logits_host, batch, stream);
}
