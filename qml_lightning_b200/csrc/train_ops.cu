// Fine-grained SORF training operators with the semantics of the upstream extension module `sorf_gpu`
// (cuda/hadamard_cuda.cpp:77-126): they work on the rows of ONE element, take the molecule of every row from an
// `ordering` array and ACCUMULATE into caller-owned float64 tensors.  Scripts written against upstream's
// calculate_features (models/hadamard_features.py:66-80) keep working through them; the model classes themselves use
// qmlb_sorf_train_features, which covers all elements of a batch in two launches.
//
//   qmlb_hadamard_features_accumulate        <- compute_featurisation_kernel          (cuda/hadamard_kernel.cu:541-563)
//   qmlb_partial_feature_derivatives         <- compute_sin_coeffs_kernel             (:565-585)
//   qmlb_featurization_derivative_accumulate <- compute_featurisation_derivative_kernel (:587-717)
#include <math.h>

#include "common.cuh"
#include "fwht.cuh"

namespace {

// features[ordering[a], f] += sqrt(2/F) cos(coeffs[a,f] + bias[f]); the term is formed in float as upstream does and
// added with a float64 atomic (rows of one molecule collide, their order is not fixed: float64 makes that harmless).
__global__ void __launch_bounds__(256)
hadamard_features_kernel(const float *__restrict__ coeffs, const float *__restrict__ bias, const int *__restrict__ ordering,
                         int F, float normf, double *__restrict__ features) {
    const size_t a = blockIdx.y;
    const int mol = ordering[a];
    for (int f = blockIdx.x * blockDim.x + threadIdx.x; f < F; f += gridDim.x * blockDim.x)
        atomicAdd(features + (size_t)mol * F + f, (double)(cosf(coeffs[a * F + f] + bias[f]) * normf));
}

__global__ void __launch_bounds__(256)
sin_coeffs_kernel(const float *__restrict__ coeffs, const float *__restrict__ bias, size_t total, int F, float normf,
                  double *__restrict__ out) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
        out[i] = (double)(sinf(coeffs[i] + bias[i % F]) * normf);
}

// One warp per (row a, derivative atom j, axis, stack): u = N^(-T/2) (H D_{T-1} ... H D_0) dx[a,j,axis,:], then
// G[ordering[a], j, axis, s*N + p] += normalisation * sinc[a, s*N + p] * u[p].
template <int E>
__global__ void __launch_bounds__(256)
featurization_derivative_kernel(const double *__restrict__ sinc, double normalisation, const float *__restrict__ D,
                                const float *__restrict__ dx, const int *__restrict__ ordering, long n, int A, int S, int T,
                                float normh, double *__restrict__ G) {
    constexpr int N = 32 * E;
    const int lane = threadIdx.x & 31;
    const long wid = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (wid >= n * A * 3 * S) return;
    const int s = (int)(wid % S);
    const int xd = (int)((wid / S) % 3);
    const int j = (int)((wid / ((long)S * 3)) % A);
    const long a = wid / ((long)S * 3 * A);
    const float *src = dx + (((size_t)a * A + j) * 3 + xd) * N + lane * E;
    float v[E];
    bool nz = false;
#pragma unroll
    for (int i = 0; i < E; ++i) {
        v[i] = src[i];
        nz |= v[i] != 0.f;
    }
    if (!__any_sync(QMLB_FULL_MASK, nz)) return;   // atom j does not move the representation of atom a
    for (int m = 0; m < T; ++m) {
        const float *d = D + ((size_t)m * S + s) * N + lane * E;
#pragma unroll
        for (int i = 0; i < E; ++i) v[i] *= d[i];
        warp_fwht<E>(v, lane);
#pragma unroll
        for (int i = 0; i < E; ++i) v[i] *= normh;
    }
    const size_t F = (size_t)S * N;
    const double *sc = sinc + (size_t)a * F + (size_t)s * N + lane * E;
    double *dst = G + (((size_t)ordering[a] * A + j) * 3 + xd) * F + (size_t)s * N + lane * E;
#pragma unroll
    for (int i = 0; i < E; ++i) atomicAdd(dst + i, normalisation * sc[i] * (double)v[i]);
}

}  // namespace

extern "C" int qmlb_hadamard_features_accumulate(const float *coeffs, const float *bias, const int *ordering, int n, int F,
                                                 double *features, qmlb_stream_t stream) {
    QMLB_REQUIRE(coeffs && bias && ordering && features, "qmlb_hadamard_features_accumulate: null tensor");
    QMLB_REQUIRE(n >= 0 && n < 65536 * 32 && F > 0, "qmlb_hadamard_features_accumulate: bad sizes");
    if (n == 0) return QMLB_OK;
    const float normf = (float)sqrt(2.0 / (double)F);
    for (int a0 = 0; a0 < n; a0 += 65535) {      // gridDim.y limit
        const int rows = n - a0 < 65535 ? n - a0 : 65535;
        dim3 grid((unsigned)((F + 1023) / 1024), (unsigned)rows);
        hadamard_features_kernel<<<grid, 256, 0, qmlb::as_stream(stream)>>>(coeffs + (size_t)a0 * F, bias, ordering + a0, F, normf,
                                                                           features);
    }
    return qmlb::check_launch("qmlb_hadamard_features_accumulate");
}

extern "C" int qmlb_partial_feature_derivatives(const float *coeffs, const float *bias, int n, int F, double *out,
                                                qmlb_stream_t stream) {
    QMLB_REQUIRE(coeffs && bias && out, "qmlb_partial_feature_derivatives: null tensor");
    QMLB_REQUIRE(n >= 0 && F > 0, "qmlb_partial_feature_derivatives: bad sizes");
    if (n == 0) return QMLB_OK;
    const size_t total = (size_t)n * F;
    const unsigned blocks = (unsigned)((total + 1023) / 1024 < 148 * 64 ? (total + 1023) / 1024 : 148 * 64);
    sin_coeffs_kernel<<<blocks, 256, 0, qmlb::as_stream(stream)>>>(coeffs, bias, total, F, (float)sqrt(2.0 / (double)F), out);
    return qmlb::check_launch("qmlb_partial_feature_derivatives");
}

extern "C" int qmlb_featurization_derivative_accumulate(const double *partial_derivatives, double normalisation, const float *D,
                                                        const float *input_derivatives, const int *ordering, int n, int A,
                                                        int N, int S, int T, double *feature_derivatives,
                                                        qmlb_stream_t stream) {
    QMLB_REQUIRE(partial_derivatives && D && input_derivatives && ordering && feature_derivatives,
                 "qmlb_featurization_derivative_accumulate: null tensor");
    QMLB_REQUIRE(n >= 0 && A > 0 && S > 0 && T > 0, "qmlb_featurization_derivative_accumulate: bad sizes");
    if (n == 0) return QMLB_OK;
    const long warps = (long)n * A * 3 * S;
    QMLB_REQUIRE((warps + 7) / 8 < (1L << 31), "qmlb_featurization_derivative_accumulate: batch too large");
    const float normh = (float)(1.0 / sqrt((double)N));
    const unsigned grid = (unsigned)((warps + 7) / 8);
    cudaStream_t st = qmlb::as_stream(stream);
#define QMLB_FD(EE)                                                                                                            \
    featurization_derivative_kernel<EE><<<grid, 256, 0, st>>>(partial_derivatives, normalisation, D, input_derivatives, ordering, \
                                                              (long)n, A, S, T, normh, feature_derivatives);                  \
    break
    switch (N) {
        case 32: QMLB_FD(1);
        case 64: QMLB_FD(2);
        case 128: QMLB_FD(4);
        case 256: QMLB_FD(8);
        case 512: QMLB_FD(16);
        case 1024: QMLB_FD(32);
        default:
            qmlb::set_error("qmlb_featurization_derivative_accumulate: npcas must be a power of two in [32, 1024], got %d", N);
            return QMLB_ERR_UNSUPPORTED;
    }
#undef QMLB_FD
    return qmlb::check_launch("qmlb_featurization_derivative_accumulate");
}
