// Warp-level fast Walsh-Hadamard transform shared by the unfused SORF operators and the training kernels.
#pragma once

#include "common.cuh"

// Unnormalised transform of a vector of N = 32 * E floats held by one warp, lane l owning elements l*E .. l*E+E-1:
// the low log2(E) butterfly stages run in registers, the five lane bits through warp shuffles.
template <int E>
__device__ __forceinline__ void warp_fwht(float (&u)[E], int lane) {
#pragma unroll
    for (int h = 1; h < E; h <<= 1)
#pragma unroll
        for (int i = 0; i < E; ++i)
            if ((i & h) == 0) {
                const float a = u[i], b = u[i | h];
                u[i] = a + b;
                u[i | h] = a - b;
            }
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float sgn = (lane & o) ? -1.0f : 1.0f;
#pragma unroll
        for (int i = 0; i < E; ++i) {
            const float other = __shfl_xor_sync(QMLB_FULL_MASK, u[i], o);
            u[i] = fmaf(sgn, u[i], other);
        }
    }
}
