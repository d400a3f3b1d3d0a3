// Training rows of the SORF model: per molecule the feature vector Z[m,:] and the force features
// G[m,j,x,:] = -dZ[m,:]/dr_{j,x}, both float64, as consumed by the normal equations.
//
// Upstream: sorf_matrix_kernel + compute_featurisation_kernel + compute_sin_coeffs_kernel +
// compute_featurisation_derivative_kernel (cuda/hadamard_kernel.cu:424-717), driven by calculate_features
// (models/hadamard_features.py:66-80) once per element.  Here two launches cover all elements of a batch:
//   1. one warp per (atom row, stack): coefficients c = (sqrt(N)/sigma) N^(-T/2) (HD)^T x, then
//      Z[mol, f] += sqrt(2/F) cos(c + b)   (float64 atomics, like upstream) and  sinc[row, f] = sqrt(2/F) sin(c + b);
//   2. one warp per (molecule, derivative atom j, axis, stack): loops over the centre atoms i of the molecule,
//      transforms the projected Jacobian row dx[row_i, j, axis, :] and accumulates sinc[row_i] * (HD)^T dx in registers;
//      every G element is written exactly once (no atomics, no zero-initialisation by the caller).
// The transform is the warp-shuffle FWHT (N/32 registers per lane), N in [32, 1024].
#include <math.h>

#include "common.cuh"
#include "fwht.cuh"

namespace {

__device__ __forceinline__ int element_of_row(long row, const int *group_start, int nel) {
    int e = 0;
    while (e + 1 < nel && row >= group_start[e + 1]) ++e;
    return e;
}

template <int E>
__global__ void __launch_bounds__(256)
train_features_kernel(const float *__restrict__ x, const float *__restrict__ Dmat, const float *__restrict__ bias,
                      const int *__restrict__ group_start, const int *__restrict__ slot_of_row, int nel, int A, int S, int T,
                      float scale, float normf, double *__restrict__ Zout, float *__restrict__ sinc) {
    constexpr int N = 32 * E;
    const int lane = threadIdx.x & 31;
    const long wid = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const long row = wid / S;
    const int s = (int)(wid % S);
    if (row >= group_start[nel]) return;
    const int slot = slot_of_row[row];
    if (slot < 0) return;
    const int el = element_of_row(row, group_start, nel);
    const size_t F = (size_t)S * N;
    float v[E];
#pragma unroll
    for (int i = 0; i < E; ++i) v[i] = x[(size_t)row * N + lane * E + i];
    for (int m = 0; m < T; ++m) {
        const float *d = Dmat + (((size_t)el * T + m) * S + s) * N + lane * E;
#pragma unroll
        for (int i = 0; i < E; ++i) v[i] *= d[i];
        warp_fwht<E>(v, lane);
    }
    const int mol = slot / A;
#pragma unroll
    for (int i = 0; i < E; ++i) {
        const size_t f = (size_t)s * N + lane * E + i;
        const float arg = fmaf(v[i], scale, bias[(size_t)el * F + f]);
        float sn, cs;
        sincosf(arg, &sn, &cs);
        atomicAdd(Zout + (size_t)mol * F + f, (double)(cs * normf));
        sinc[(size_t)row * F + f] = sn * normf;
    }
}

template <int E>
__global__ void __launch_bounds__(256)
train_derivative_kernel(const float *__restrict__ dx, const float *__restrict__ sinc, const float *__restrict__ Dmat,
                        const int *__restrict__ row_of_slot, const int *__restrict__ group_start,
                        const int *__restrict__ atom_counts, int nel, int nb, int A, int S, int T, float scale,
                        double *__restrict__ G) {
    constexpr int N = 32 * E;
    const int lane = threadIdx.x & 31;
    const long wid = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const long total = (long)nb * A * 3 * S;
    if (wid >= total) return;
    const int s = (int)(wid % S);
    const int xd = (int)((wid / S) % 3);
    const int j = (int)((wid / ((long)S * 3)) % A);
    const int mol = (int)(wid / ((long)S * 3 * A));
    const size_t F = (size_t)S * N;
    double *dst = G + (((size_t)mol * A + j) * 3 + xd) * F + (size_t)s * N + lane * E;
    int natoms = atom_counts[mol];
    natoms = natoms > A ? A : natoms;
    float acc[E];
#pragma unroll
    for (int i = 0; i < E; ++i) acc[i] = 0.f;
    if (j < natoms) {
        for (int ia = 0; ia < natoms; ++ia) {
            const int row = row_of_slot[(size_t)mol * A + ia];
            if (row < 0) continue;
            float v[E];
            const float *src = dx + (((size_t)row * A + j) * 3 + xd) * N + lane * E;
            bool nz = false;
#pragma unroll
            for (int i = 0; i < E; ++i) {
                v[i] = src[i];
                nz |= v[i] != 0.f;
            }
            if (!__any_sync(QMLB_FULL_MASK, nz)) continue;   // atom j is not a neighbour of atom ia
            const int el = element_of_row(row, group_start, nel);
            for (int m = 0; m < T; ++m) {
                const float *d = Dmat + (((size_t)el * T + m) * S + s) * N + lane * E;
#pragma unroll
                for (int i = 0; i < E; ++i) v[i] *= d[i];
                warp_fwht<E>(v, lane);
            }
            const float *sc = sinc + (size_t)row * F + (size_t)s * N + lane * E;
#pragma unroll
            for (int i = 0; i < E; ++i) acc[i] = fmaf(sc[i], v[i], acc[i]);
        }
    }
#pragma unroll
    for (int i = 0; i < E; ++i) dst[i] = (double)(acc[i] * scale);
}

template <int E>
int launch_train(const float *x, const float *dx, const float *Dmat, const float *bias, const int *group_start,
                 const int *slot_of_row, const int *row_of_slot, const int *atom_counts, int nel, int nb, int A,
                 size_t rows_cap, int S, int T, float scale, float normf, double *Zout, double *G, float *sinc,
                 cudaStream_t st) {
    const long w1 = (long)rows_cap * S;
    train_features_kernel<E><<<(unsigned)((w1 + 7) / 8), 256, 0, st>>>(x, Dmat, bias, group_start, slot_of_row, nel, A, S, T,
                                                                      scale, normf, Zout, sinc);
    if (int rc = qmlb::check_launch("qmlb_sorf_train_features")) return rc;
    if (dx && G) {
        const long w2 = (long)nb * A * 3 * S;
        train_derivative_kernel<E><<<(unsigned)((w2 + 7) / 8), 256, 0, st>>>(dx, sinc, Dmat, row_of_slot, group_start,
                                                                            atom_counts, nel, nb, A, S, T, scale, G);
        return qmlb::check_launch("qmlb_sorf_train_features(derivative)");
    }
    return QMLB_OK;
}

}  // namespace

extern "C" int qmlb_sorf_train_features(const float *x, const float *dx, const float *Dmat, const float *bias,
                                        const int *group_start, const int *slot_of_row, const int *row_of_slot,
                                        const int *atom_counts, int nelements, int nb, int A, size_t rows_cap, int N, int S,
                                        int T, float sigma, double *Zout, double *G, float *sinc_scratch,
                                        qmlb_stream_t stream) {
    QMLB_REQUIRE(x && Dmat && bias && group_start && slot_of_row && row_of_slot && atom_counts && Zout && sinc_scratch,
                 "qmlb_sorf_train_features: null tensor");
    QMLB_REQUIRE((dx == nullptr) == (G == nullptr), "qmlb_sorf_train_features: dx and G go together");
    QMLB_REQUIRE(nelements > 0 && nb > 0 && A > 0 && S > 0 && T > 0 && sigma > 0.f, "qmlb_sorf_train_features: bad sizes");
    QMLB_REQUIRE((long)rows_cap * S / 8 < (1L << 31) && (long)nb * A * 3 * S / 8 < (1L << 31), "qmlb_sorf_train_features: batch too large");
    cudaStream_t st = qmlb::as_stream(stream);
    const size_t F = (size_t)S * N;
    if (cudaMemsetAsync(Zout, 0, sizeof(double) * (size_t)nb * F, st) != cudaSuccess)
        return qmlb::check_launch("qmlb_sorf_train_features(memset)");
    const float scale = (float)(sqrt((double)N) / (double)sigma * pow((double)N, -0.5 * (double)T));
    const float normf = (float)sqrt(2.0 / (double)F);
#define QMLB_TRAIN(EE) \
    return launch_train<EE>(x, dx, Dmat, bias, group_start, slot_of_row, row_of_slot, atom_counts, nelements, nb, A, rows_cap, S, T, scale, normf, Zout, G, sinc_scratch, st)
    switch (N) {
        case 32: QMLB_TRAIN(1);
        case 64: QMLB_TRAIN(2);
        case 128: QMLB_TRAIN(4);
        case 256: QMLB_TRAIN(8);
        case 512: QMLB_TRAIN(16);
        case 1024: QMLB_TRAIN(32);
        default:
            qmlb::set_error("qmlb_sorf_train_features: npcas must be a power of two in [32, 1024], got %d", N);
            return QMLB_ERR_UNSUPPORTED;
    }
#undef QMLB_TRAIN
}
