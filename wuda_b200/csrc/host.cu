#include "host.h"

#include <cstdio>
#include <cstring>
#include <mutex>

namespace wuda {

static thread_local char g_error[512] = "";

int fail(int status, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    return status;
}
void clear_error() { g_error[0] = '\0'; }

static thread_local int g_gemm_sm_limit = 0;
int gemm_sms(const DeviceInfo& dev) {
    return g_gemm_sm_limit > 0 && g_gemm_sm_limit < dev.num_sms ? g_gemm_sm_limit : dev.num_sms;
}

int current_device_info(DeviceInfo* out) {
    static std::mutex mu;
    static DeviceInfo cache[64];
    static bool have[64] = {};
    int dev = -1;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) {
        cudaGetLastError();
        return fail(WUDA_ERR_NO_DEVICE, "cudaGetDevice failed: %s", cudaGetErrorString(err));
    }
    if (dev < 0 || dev >= 64) return fail(WUDA_ERR_UNSUPPORTED, "device ordinal %d out of range", dev);
    std::lock_guard<std::mutex> lock(mu);
    if (!have[dev]) {
        DeviceInfo info;
        info.device = dev;
        WUDA_CUDA(cudaDeviceGetAttribute(&info.num_sms, cudaDevAttrMultiProcessorCount, dev));
        WUDA_CUDA(cudaDeviceGetAttribute(&info.smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
        WUDA_CUDA(cudaDeviceGetAttribute(&info.cc_major, cudaDevAttrComputeCapabilityMajor, dev));
        cache[dev] = info;
        have[dev] = true;
    }
    *out = cache[dev];
    if (out->cc_major != 10)
        return fail(WUDA_ERR_NO_DEVICE, "device %d is compute capability %d.x; this library is sm_100a only",
                    dev, out->cc_major);
    return WUDA_OK;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

static EncodeTiledFn resolve_encode() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
        cudaError_t err = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
        if (err == cudaSuccess && q == cudaDriverEntryPointSuccess) fn = reinterpret_cast<EncodeTiledFn>(p);
        else cudaGetLastError();
    });
    return fn;
}

int encode_tensor_map(CUtensorMap* map, CUtensorMapDataType dtype, int rank, const void* base,
                      const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                      CUtensorMapSwizzle swizzle, CUtensorMapL2promotion promo) {
    EncodeTiledFn fn = resolve_encode();
    if (!fn) return fail(WUDA_ERR_NO_DEVICE, "cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t d[5];
    cuuint64_t s[4];
    cuuint32_t b[5];
    cuuint32_t e[5];
    for (int i = 0; i < rank; ++i) {
        d[i] = dims[i];
        b[i] = box[i];
        e[i] = 1;
    }
    for (int i = 0; i + 1 < rank; ++i) s[i] = strides_bytes[i];
    CUresult r = fn(map, dtype, static_cast<cuuint32_t>(rank), const_cast<void*>(base), d, s, b, e,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, promo, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(WUDA_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", static_cast<int>(r));
    return WUDA_OK;
}

}  // namespace wuda

extern "C" {

int wuda_version(void) { return 100; }

const char* wuda_last_error(void) { return wuda::g_error; }

int wuda_num_sms(void) {
    wuda::DeviceInfo info;
    int st = wuda::current_device_info(&info);
    if (st != WUDA_OK) return -st;
    return info.num_sms;
}

}  // extern "C"

extern "C" int wuda_gemm_sm_limit(int max_sms) {
    const int before = wuda::g_gemm_sm_limit;
    wuda::g_gemm_sm_limit = max_sms > 0 ? max_sms : 0;
    return before;
}
