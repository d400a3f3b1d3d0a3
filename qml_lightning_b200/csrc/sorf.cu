// Unfused SORF operators with the upstream operator semantics (materialised coefficient tensors):
//   qmlb_sorf_coefficients / _backward   <- hadamard_kernel / hadamard_kernel_backwards (cuda/hadamard_kernel.cu:5-102, 204-312)
//   qmlb_cos_features / _backward        <- compute_cos_features_kernel / compute_cos_derivative_features_kernel (:778-854)
// They back the TorchScript operators qml_lightning_sorf::get_SORF_coefficients and ::get_cos_features, which saved
// upstream models call directly; new code uses the fused kernel in sorf_fused.cu.
//
// One warp transforms one (row, stack) vector: N/32 registers per lane hold consecutive elements, the low bits
// of the transform run in registers and the five lane bits through warp shuffles, so the [n,S,N] tensor is read
// or written exactly once with 128-bit coalesced accesses.  Vectors shorter than 32 or longer than 1024 fall
// back to a shared-memory butterfly with one block per row.
#include <math.h>

#include "common.cuh"
#include "fwht.cuh"

namespace {

template <int E>
__device__ __forceinline__ void load_e(float (&v)[E], const float *p) {
    if (E >= 4) {
#pragma unroll
        for (int q = 0; q < E / 4; ++q) {
            const float4 t = *reinterpret_cast<const float4 *>(p + 4 * q);
            v[4 * q] = t.x; v[4 * q + 1] = t.y; v[4 * q + 2] = t.z; v[4 * q + 3] = t.w;
        }
    } else {
#pragma unroll
        for (int q = 0; q < E; ++q) v[q] = p[q];
    }
}

template <int E>
__device__ __forceinline__ void store_e(const float (&v)[E], float *p) {
    if (E >= 4) {
#pragma unroll
        for (int q = 0; q < E / 4; ++q)
            *reinterpret_cast<float4 *>(p + 4 * q) = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
    } else {
#pragma unroll
        for (int q = 0; q < E; ++q) p[q] = v[q];
    }
}

// forward: out[r,s,:] = norm * (H D_{T-1,s} ... H D_{0,s}) u[r,:]      (norm includes N^(-T/2))
template <int E>
__global__ void __launch_bounds__(256)
sorf_coeff_warp_kernel(const float *__restrict__ u, const float *__restrict__ D, long n, int S, int T, float norm,
                       float *__restrict__ out) {
    constexpr int N = 32 * E;
    const int lane = threadIdx.x & 31;
    const long wid = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (wid >= n * S) return;
    const long r = wid / S;
    const int s = (int)(wid % S);
    float v[E], d[E];
    load_e<E>(v, u + r * N + lane * E);
    for (int m = 0; m < T; ++m) {
        load_e<E>(d, D + ((size_t)m * S + s) * N + lane * E);
#pragma unroll
        for (int i = 0; i < E; ++i) v[i] *= d[i];
        warp_fwht<E>(v, lane);
    }
#pragma unroll
    for (int i = 0; i < E; ++i) v[i] *= norm;
    store_e<E>(v, out + ((size_t)r * S + s) * N + lane * E);
}

// backward: out[r,:] = norm * sum_s (D_0 H ... D_{T-1} H) grad[r,s,:]
template <int E>
__global__ void __launch_bounds__(256)
sorf_coeff_bwd_warp_kernel(const float *__restrict__ grad, const float *__restrict__ D, long n, int S, int T, float norm,
                           float *__restrict__ out) {
    constexpr int N = 32 * E;
    const int lane = threadIdx.x & 31;
    const long r = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (r >= n) return;
    float acc[E];
#pragma unroll
    for (int i = 0; i < E; ++i) acc[i] = 0.f;
    for (int s = 0; s < S; ++s) {
        float v[E], d[E];
        load_e<E>(v, grad + ((size_t)r * S + s) * N + lane * E);
        for (int m = T - 1; m >= 0; --m) {
            warp_fwht<E>(v, lane);
            load_e<E>(d, D + ((size_t)m * S + s) * N + lane * E);
#pragma unroll
            for (int i = 0; i < E; ++i) v[i] *= d[i];
        }
#pragma unroll
        for (int i = 0; i < E; ++i) acc[i] += v[i];
    }
#pragma unroll
    for (int i = 0; i < E; ++i) acc[i] *= norm;
    store_e<E>(acc, out + (size_t)r * N + lane * E);
}

// generic shared-memory version, one block per row
__device__ void block_fwht(float *s, int N) {
    for (int h = 1; h < N; h <<= 1) {
        __syncthreads();
        for (int p = threadIdx.x; p < N / 2; p += blockDim.x) {
            const int i0 = ((p / h) * 2 * h) + (p % h), i1 = i0 + h;
            const float a = s[i0], b = s[i1];
            s[i0] = a + b;
            s[i1] = a - b;
        }
    }
    __syncthreads();
}

__global__ void sorf_coeff_block_kernel(const float *__restrict__ u, const float *__restrict__ D, int N, int S, int T,
                                        float norm, float *__restrict__ out) {
    extern __shared__ float sm[];
    const size_t r = blockIdx.x;
    for (int s = 0; s < S; ++s) {
        for (int p = threadIdx.x; p < N; p += blockDim.x) sm[p] = u[r * N + p];
        for (int m = 0; m < T; ++m) {
            __syncthreads();
            for (int p = threadIdx.x; p < N; p += blockDim.x) sm[p] *= D[((size_t)m * S + s) * N + p];
            block_fwht(sm, N);
        }
        for (int p = threadIdx.x; p < N; p += blockDim.x) out[(r * S + s) * N + p] = norm * sm[p];
        __syncthreads();
    }
}

__global__ void sorf_coeff_bwd_block_kernel(const float *__restrict__ grad, const float *__restrict__ D, int N, int S,
                                            int T, float norm, float *__restrict__ out) {
    extern __shared__ float sm[];
    float *acc = sm + N;
    const size_t r = blockIdx.x;
    for (int p = threadIdx.x; p < N; p += blockDim.x) acc[p] = 0.f;
    for (int s = 0; s < S; ++s) {
        __syncthreads();
        for (int p = threadIdx.x; p < N; p += blockDim.x) sm[p] = grad[(r * S + s) * N + p];
        for (int m = T - 1; m >= 0; --m) {
            block_fwht(sm, N);
            for (int p = threadIdx.x; p < N; p += blockDim.x) sm[p] *= D[((size_t)m * S + s) * N + p];
        }
        __syncthreads();
        for (int p = threadIdx.x; p < N; p += blockDim.x) acc[p] += sm[p];
    }
    __syncthreads();
    for (int p = threadIdx.x; p < N; p += blockDim.x) out[r * N + p] = norm * acc[p];
}

// cos features: thread = one feature column over a chunk of consecutive rows; rows of the same molecule are summed
// in registers and flushed with one atomic per run, so sorted batch_indexes (the usual case) need few atomics.
constexpr int COS_ROWS = 32;
__global__ void __launch_bounds__(256)
cos_features_kernel(const float *__restrict__ coeffs, const float *__restrict__ bias, const int *__restrict__ mol,
                    long n, int F, int nmol, float normf, float *__restrict__ out) {
    const int f = blockIdx.x * blockDim.x + threadIdx.x;
    if (f >= F) return;
    const long r0 = (long)blockIdx.y * COS_ROWS, r1 = min(n, r0 + COS_ROWS);
    const float b = bias[f];
    int cur = -1;
    float acc = 0.f;
    for (long r = r0; r < r1; ++r) {
        const int m = mol[r];
        if (m != cur) {
            if (cur >= 0 && cur < nmol) atomicAdd(out + (size_t)cur * F + f, acc);
            cur = m;
            acc = 0.f;
        }
        acc += cosf(coeffs[(size_t)r * F + f] + b) * normf;
    }
    if (cur >= 0 && cur < nmol) atomicAdd(out + (size_t)cur * F + f, acc);
}

__global__ void __launch_bounds__(256)
cos_features_bwd_kernel(const float *__restrict__ grads, const float *__restrict__ coeffs, const float *__restrict__ bias,
                        const int *__restrict__ mol, long n, int F, float normf, float *__restrict__ out) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)n * F) return;
    const size_t r = idx / F;
    const int f = (int)(idx % F);
    out[idx] = grads[(size_t)mol[r] * F + f] * -sinf(coeffs[idx] + bias[f]) * normf;
}

int ilog2_exact(int n) {
    int l = 0;
    while ((1 << l) < n && l < 30) ++l;
    return (1 << l) == n ? l : -1;
}

}  // namespace

extern "C" int qmlb_sorf_coefficients(const float *u, const float *D, int n, int N, int S, int T, float normalisation,
                                      float *out, qmlb_stream_t stream) {
    QMLB_REQUIRE(u && D && out, "qmlb_sorf_coefficients: null tensor");
    QMLB_REQUIRE(ilog2_exact(N) >= 0, "input size must be power of 2.");  // message of hadamard_kernel.cu:730
    QMLB_REQUIRE(n >= 0 && S > 0 && T > 0, "qmlb_sorf_coefficients: bad sizes");
    if (n == 0) return QMLB_OK;
    const float norm = normalisation * (float)pow((double)N, -0.5 * T);
    cudaStream_t st = qmlb::as_stream(stream);
    const long warps = (long)n * S;
    const unsigned grid = (unsigned)((warps + 7) / 8);
    switch (N) {
        case 32: sorf_coeff_warp_kernel<1><<<grid, 256, 0, st>>>(u, D, n, S, T, norm, out); break;
        case 64: sorf_coeff_warp_kernel<2><<<grid, 256, 0, st>>>(u, D, n, S, T, norm, out); break;
        case 128: sorf_coeff_warp_kernel<4><<<grid, 256, 0, st>>>(u, D, n, S, T, norm, out); break;
        case 256: sorf_coeff_warp_kernel<8><<<grid, 256, 0, st>>>(u, D, n, S, T, norm, out); break;
        case 512: sorf_coeff_warp_kernel<16><<<grid, 256, 0, st>>>(u, D, n, S, T, norm, out); break;
        case 1024: sorf_coeff_warp_kernel<32><<<grid, 256, 0, st>>>(u, D, n, S, T, norm, out); break;
        default: {
            QMLB_REQUIRE(N <= 8192, "qmlb_sorf_coefficients: N up to 8192 supported");
            const int threads = N / 2 < 32 ? 32 : (N / 2 > 256 ? 256 : N / 2);
            sorf_coeff_block_kernel<<<n, threads, N * sizeof(float), st>>>(u, D, N, S, T, norm, out);
        }
    }
    return qmlb::check_launch("qmlb_sorf_coefficients");
}

extern "C" int qmlb_sorf_coefficients_backward(const float *grad, const float *D, int n, int N, int S, int T,
                                               float normalisation, float *out, qmlb_stream_t stream) {
    QMLB_REQUIRE(grad && D && out, "qmlb_sorf_coefficients_backward: null tensor");
    QMLB_REQUIRE(ilog2_exact(N) >= 0, "input size must be power of 2.");
    QMLB_REQUIRE(n >= 0 && S > 0 && T > 0, "qmlb_sorf_coefficients_backward: bad sizes");
    if (n == 0) return QMLB_OK;
    const float norm = normalisation * (float)pow((double)N, -0.5 * T);
    cudaStream_t st = qmlb::as_stream(stream);
    const unsigned grid = (unsigned)(((long)n + 7) / 8);
    switch (N) {
        case 32: sorf_coeff_bwd_warp_kernel<1><<<grid, 256, 0, st>>>(grad, D, n, S, T, norm, out); break;
        case 64: sorf_coeff_bwd_warp_kernel<2><<<grid, 256, 0, st>>>(grad, D, n, S, T, norm, out); break;
        case 128: sorf_coeff_bwd_warp_kernel<4><<<grid, 256, 0, st>>>(grad, D, n, S, T, norm, out); break;
        case 256: sorf_coeff_bwd_warp_kernel<8><<<grid, 256, 0, st>>>(grad, D, n, S, T, norm, out); break;
        case 512: sorf_coeff_bwd_warp_kernel<16><<<grid, 256, 0, st>>>(grad, D, n, S, T, norm, out); break;
        case 1024: sorf_coeff_bwd_warp_kernel<32><<<grid, 256, 0, st>>>(grad, D, n, S, T, norm, out); break;
        default: {
            QMLB_REQUIRE(N <= 8192, "qmlb_sorf_coefficients_backward: N up to 8192 supported");
            const int threads = N / 2 < 32 ? 32 : (N / 2 > 256 ? 256 : N / 2);
            sorf_coeff_bwd_block_kernel<<<n, threads, 2 * N * sizeof(float), st>>>(grad, D, N, S, T, norm, out);
        }
    }
    return qmlb::check_launch("qmlb_sorf_coefficients_backward");
}

extern "C" int qmlb_cos_features(const float *coeffs, const float *bias, const int *batch_indexes, int n, int F,
                                 int nmol, float *out, qmlb_stream_t stream) {
    QMLB_REQUIRE(coeffs && bias && batch_indexes && out, "qmlb_cos_features: null tensor");
    QMLB_REQUIRE(n >= 0 && F > 0 && nmol >= 0, "qmlb_cos_features: bad sizes");
    cudaStream_t st = qmlb::as_stream(stream);
    if (nmol == 0) return QMLB_OK;
    if (cudaMemsetAsync(out, 0, sizeof(float) * (size_t)nmol * F, st) != cudaSuccess)
        return qmlb::check_launch("qmlb_cos_features(memset)");
    if (n == 0) return QMLB_OK;
    const float normf = (float)sqrt(2.0 / (double)F);
    dim3 grid((unsigned)((F + 255) / 256), (unsigned)(((long)n + COS_ROWS - 1) / COS_ROWS));
    QMLB_REQUIRE(grid.y <= 65535u, "qmlb_cos_features: at most %d rows per call", 65535 * COS_ROWS);
    cos_features_kernel<<<grid, 256, 0, st>>>(coeffs, bias, batch_indexes, n, F, nmol, normf, out);
    return qmlb::check_launch("qmlb_cos_features");
}

extern "C" int qmlb_cos_features_backward(const float *grads, const float *coeffs, const float *bias,
                                          const int *batch_indexes, int n, int F, float *out, qmlb_stream_t stream) {
    QMLB_REQUIRE(grads && coeffs && bias && batch_indexes && out, "qmlb_cos_features_backward: null tensor");
    QMLB_REQUIRE(n >= 0 && F > 0, "qmlb_cos_features_backward: bad sizes");
    if (n == 0) return QMLB_OK;
    const size_t tot = (size_t)n * F;
    cos_features_bwd_kernel<<<(unsigned)((tot + 255) / 256), 256, 0, qmlb::as_stream(stream)>>>(
        grads, coeffs, bias, batch_indexes, n, F, (float)sqrt(2.0 / (double)F), out);
    return qmlb::check_launch("qmlb_cos_features_backward");
}
