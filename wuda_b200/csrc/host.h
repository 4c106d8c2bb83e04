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

// rank-`rank` tiled tensor map. dims/box are innermost-first; strides_bytes has rank-1
// entries (stride of dims 1..rank-1). Returns a wuda_status.
int encode_tensor_map(CUtensorMap* map, CUtensorMapDataType dtype, int rank, const void* base,
                      const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                      CUtensorMapSwizzle swizzle, CUtensorMapL2promotion promo);

}  // namespace wuda
