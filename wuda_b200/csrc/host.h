// Host-side helpers shared by the entry points: status codes and the per-thread error
// message, argument checks, and TMA tensor-map encoding through the driver entry point
// (resolved at run time, so the library has no link-time dependency on libcuda and
// loads on a machine without a GPU).
#pragma once
#include <cstdarg>
#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>

#include "../../include/wuda_b200.h"

namespace wuda {

int fail(int status, const char* fmt, ...);
void clear_error();

#define WUDA_REQUIRE(cond, ...)                                         \
    do {                                                                \
        if (!(cond)) return ::wuda::fail(WUDA_ERR_INVALID_ARGUMENT, __VA_ARGS__); \
    } while (0)

#define WUDA_CUDA(expr)                                                                   \
    do {                                                                                  \
        cudaError_t err__ = (expr);                                                       \
        if (err__ != cudaSuccess)                                                         \
            return ::wuda::fail(WUDA_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(err__)); \
    } while (0)

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Device properties cached per device (SM count, opt-in shared memory).
struct DeviceInfo {
    int device = -1;
    int num_sms = 0;
    int smem_optin = 0;
    int cc_major = 0;
};
int current_device_info(DeviceInfo* out);
// SMs the GEMM launches of the calling thread may cover: all of the device's, or fewer after wuda_gemm_sm_limit
int gemm_sms(const DeviceInfo& dev);

// rank-`rank` tiled tensor map. dims/box are innermost-first; strides_bytes has rank-1
// entries (stride of dims 1..rank-1). Returns a wuda_status.
int encode_tensor_map(CUtensorMap* map, CUtensorMapDataType dtype, int rank, const void* base,
                      const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                      CUtensorMapSwizzle swizzle, CUtensorMapL2promotion promo);

// ---- programmatic dependent launch.  Every kernel of the library is launched with the attribute
// that lets it start while the kernel before it in the stream is still running; it then runs its
// prologue (barrier set-up, TMEM allocation, descriptor prefetch) and stops at pdl_wait() until
// the earlier kernel has completed and its writes are visible, before its first access to global memory.
// pdl_launch_dependents() is called at the start, so the next kernel gets the same head start.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

#ifdef __CUDACC__
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
#endif

}  // namespace wuda
