// Host-side helpers shared by the entry points: error reporting through the
// C ABI's (code, message) pair, a device guard and launch plumbing.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "../../include/halops_b200.h"

namespace hq {

inline int fail(char* err, size_t errlen, int code, const char* fmt, ...) {
    if (err != nullptr && errlen > 0) {
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(err, errlen, fmt, ap);
        va_end(ap);
    }
    return code;
}

#define HQ_CUDA_TRY(expr)                                                  \
    do {                                                                   \
        const cudaError_t hq_e_ = (expr);                                  \
        if (hq_e_ != cudaSuccess) {                                        \
            return ::hq::fail(err, errlen, HQ_ERR_CUDA, "CUDA error: %s",  \
                              cudaGetErrorString(hq_e_));                  \
        }                                                                  \
    } while (0)

// Makes `device` current for the lifetime of the object and restores the
// previous device afterwards (the reference's CudaDeviceGuard,
// csrc/common/cuda_utils.h:38-57).
class DeviceGuard {
  public:
    explicit DeviceGuard(int device) {
        if (device < 0) return;
        if (cudaGetDevice(&prev_) != cudaSuccess) return;
        if (prev_ != device) {
            ok_ = cudaSetDevice(device) == cudaSuccess;
            restore_ = ok_;
        }
    }
    ~DeviceGuard() {
        if (restore_) cudaSetDevice(prev_);
    }
    DeviceGuard(const DeviceGuard&) = delete;
    DeviceGuard& operator=(const DeviceGuard&) = delete;
    bool ok() const { return ok_; }

  private:
    int prev_ = -1;
    bool restore_ = false;
    bool ok_ = true;
};

inline bool aligned(const void* p, size_t a) {
    return (reinterpret_cast<uintptr_t>(p) % a) == 0;
}

// One launch with optional programmatic stream serialisation (PDL) and an
// optional cluster shape.
template <typename... KArgs, typename... Args>
inline cudaError_t launch(void (*kernel)(KArgs...), dim3 grid, dim3 block,
                          size_t smem, cudaStream_t stream, bool pdl,
                          unsigned cluster_x, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attrs[2];
    unsigned n = 0;
    if (pdl) {
        attrs[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attrs[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    if (cluster_x > 1) {
        attrs[n].id = cudaLaunchAttributeClusterDimension;
        attrs[n].val.clusterDim.x = cluster_x;
        attrs[n].val.clusterDim.y = 1;
        attrs[n].val.clusterDim.z = 1;
        ++n;
    }
    cfg.attrs = attrs;
    cfg.numAttrs = n;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

}  // namespace hq
