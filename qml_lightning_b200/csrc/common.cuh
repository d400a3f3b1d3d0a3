// Shared helpers for the qmlb200 kernels (error reporting, launch checks, small device utilities).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "qmlb200.h"

namespace qmlb {

// Stores a printf-style message in a thread-local buffer returned by qmlb_last_error().
void set_error(const char *fmt, ...);

// Returns QMLB_OK or records the pending CUDA launch error under `what`.
int check_launch(const char *what);

inline cudaStream_t as_stream(qmlb_stream_t s) { return reinterpret_cast<cudaStream_t>(s); }

// Opt a kernel into more than 48 KB of dynamic shared memory when needed.
template <typename K>
inline int ensure_smem(K kernel, size_t bytes, const char *what) {
    if (bytes > 227 * 1024) {
        set_error("%s: needs %zu bytes of shared memory per block, above the 227 KB limit", what, bytes);
        return QMLB_ERR_UNSUPPORTED;
    }
    if (bytes > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
        if (e != cudaSuccess) {
            set_error("%s: cudaFuncSetAttribute(%zu): %s", what, bytes, cudaGetErrorString(e));
            return QMLB_ERR_CUDA;
        }
    }
    return QMLB_OK;
}

}  // namespace qmlb

#define QMLB_REQUIRE(cond, ...)              \
    do {                                     \
        if (!(cond)) {                       \
            qmlb::set_error(__VA_ARGS__);    \
            return QMLB_ERR_INVALID;         \
        }                                    \
    } while (0)

#define QMLB_FULL_MASK 0xffffffffu

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(QMLB_FULL_MASK, v, o);
    return v;
}
