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
// Step 1 uses the warp-shuffle FWHT (N/32 registers per lane), N in [32, 512].  Step 2, where nearly all the transforms
// are (atoms x 3 A per atom and stack), uses the register-tile FWHT of the prediction kernel (16 registers
// per lane, one shared-memory transposition instead of five shuffle stages per element) and handles the three axes of a
// derivative atom in one warp, so that the sin coefficients of a centre atom are read once for the three of them.
#include <math.h>

#include "common.cuh"
#include "fwht.cuh"
#include "fwht_tile.cuh"

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

constexpr int TD_WARPS = 4;

// Element index of register e of lane-in-vector l after `transforms` flips, starting from the natural order.
template <int LOG2N>
__device__ __forceinline__ int tile_index(int l, int e, bool layout_b) {
    return layout_b ? qmlb_fwht::layoutB_n(LOG2N, l * 16 + e) : l * 16 + e;
}

// A vector in natural order from global memory into layout A (lane l: elements 16 l .. 16 l + 15).  Reading 64
// consecutive bytes per lane straight from global memory costs 16 L1 wavefronts per 128-bit instruction; here the
// vector's lanes read consecutive 16-byte pieces (4 wavefronts per instruction) and exchange them through the warp's
// transposition slab.  `nonzero` reports whether this lane saw a non-zero value.
template <int LOG2N>
__device__ __forceinline__ void stage_rows(const float *__restrict__ src, float *slab, int l, bool &nonzero) {
    using C = qmlb_fwht::Cfg<LOG2N>;
    using X = qmlb_fwht::Xpose<LOG2N>;
    nonzero = false;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const int n0 = (q * C::L + l) * 4;
        const float4 t = __ldg(reinterpret_cast<const float4 *>(src + n0));
        nonzero |= (t.x != 0.f) | (t.y != 0.f) | (t.z != 0.f) | (t.w != 0.f);
        *reinterpret_cast<float4 *>(slab + X::a_base(n0 >> 4) + (n0 & 15)) = t;
    }
}
template <int LOG2N>
__device__ __forceinline__ void read_row_a(float (&v)[16], const float *slab, int l) {
    const float4 *r = reinterpret_cast<const float4 *>(slab + qmlb_fwht::Xpose<LOG2N>::a_base(l));
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const float4 t = r[q];
        v[4 * q] = t.x; v[4 * q + 1] = t.y; v[4 * q + 2] = t.z; v[4 * q + 3] = t.w;
    }
}

// One warp per (molecule, derivative atom j, group of V stacks); the three axes in turn.  Shared memory per warp: the
// transposition slab and, when `cache_d`, the first sign diagonal of every element for the warp's stacks (in slab-row
// format, read back with conflict-free 128-bit loads).
template <int LOG2N>
__global__ void __launch_bounds__(TD_WARPS * 32, 4)
train_derivative_tile_kernel(const float *__restrict__ dx, const float *__restrict__ sinc, const float *__restrict__ Dmat,
                             const int *__restrict__ row_of_slot, const int *__restrict__ group_start,
                             const int *__restrict__ atom_counts, int nel, int nb, int A, int S, int T, float scale,
                             int cache_d, double *__restrict__ G) {
    using C = qmlb_fwht::Cfg<LOG2N>;
    constexpr int N = C::N;
    extern __shared__ __align__(16) float smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane / C::L, l = lane % C::L;
    const int per_warp = (cache_d ? 1 + nel : 1) * C::WARP_FLOATS;
    float *slab = smem + warp * per_warp + g * C::SLAB;
    const int SG = (S + C::V - 1) / C::V;
    const long wid = (long)blockIdx.x * TD_WARPS + warp;
    if (wid >= (long)nb * A * SG) return;
    const int sg = (int)(wid % SG);
    const int j = (int)((wid / SG) % A);
    const int mol = (int)(wid / ((long)SG * A));
    const int s_raw = sg * C::V + g;
    const bool s_live = s_raw < S;
    const int s = s_live ? s_raw : S - 1;     // lanes beyond the last stack repeat it and do not store
    const size_t F = (size_t)S * N;
    const bool final_b = (T & 1) != 0;
    int natoms = atom_counts[mol];
    natoms = natoms > A ? A : natoms;
    if (j >= natoms) {     // padding atom: its rows are zero
        if (s_live)
            for (int xd = 0; xd < 3; ++xd) {
                double *dst = G + (((size_t)mol * A + j) * 3 + xd) * F + (size_t)s * N;
#pragma unroll
                for (int e = 0; e < 16; ++e) dst[tile_index<LOG2N>(l, e, final_b)] = 0.0;
            }
        return;
    }
    if (cache_d) {
        bool unused;
        for (int el = 0; el < nel; ++el)
            stage_rows<LOG2N>(Dmat + (((size_t)el * T) * S + s) * N, slab + (1 + el) * C::WARP_FLOATS, l, unused);
        __syncwarp();
    }
    float acc[3][16];
#pragma unroll
    for (int xd = 0; xd < 3; ++xd)
#pragma unroll
        for (int e = 0; e < 16; ++e) acc[xd][e] = 0.f;
    for (int ia = 0; ia < natoms; ++ia) {
        const int row = row_of_slot[(size_t)mol * A + ia];
        if (row < 0) continue;
        float sc[16];
        bool have_sc = false;
        int el = 0;
#pragma unroll
        for (int xd = 0; xd < 3; ++xd) {
            bool nz;
            stage_rows<LOG2N>(dx + (((size_t)row * A + j) * 3 + xd) * N, slab, l, nz);
            if (!__any_sync(QMLB_FULL_MASK, nz)) continue;   // atom j does not move this component of atom ia's row
            __syncwarp();
            float v[16];
            read_row_a<LOG2N>(v, slab, l);
            __syncwarp();
            if (!have_sc) {
                el = element_of_row(row, group_start, nel);
                const float *sp = sinc + (size_t)row * F + (size_t)s * N;
#pragma unroll
                for (int e = 0; e < 16; ++e) sc[e] = __ldg(sp + tile_index<LOG2N>(l, e, final_b));
                have_sc = true;
            }
            for (int m = 0; m < T; ++m) {
                const bool in_b = (m & 1) != 0;
                if (m == 0 && cache_d) {
                    float d[16];
                    read_row_a<LOG2N>(d, slab + (1 + el) * C::WARP_FLOATS, l);
#pragma unroll
                    for (int e = 0; e < 16; ++e) v[e] *= d[e];
                } else {
                    const float *d = Dmat + (((size_t)el * T + m) * S + s) * N;
#pragma unroll
                    for (int e = 0; e < 16; ++e) v[e] *= __ldg(d + tile_index<LOG2N>(l, e, in_b));
                }
                qmlb_fwht::fwht_flip<LOG2N>(v, slab, l, lane, !in_b);
            }
#pragma unroll
            for (int e = 0; e < 16; ++e) acc[xd][e] = fmaf(sc[e], v[e], acc[xd][e]);
        }
    }
    if (!s_live) return;
#pragma unroll
    for (int xd = 0; xd < 3; ++xd) {
        double *dst = G + (((size_t)mol * A + j) * 3 + xd) * F + (size_t)s * N;
#pragma unroll
        for (int e = 0; e < 16; ++e) dst[tile_index<LOG2N>(l, e, final_b)] = (double)(acc[xd][e] * scale);
    }
}

template <int LOG2N>
int launch_derivative_tile(const float *dx, const float *sinc, const float *Dmat, const int *row_of_slot, const int *group_start,
                           const int *atom_counts, int nel, int nb, int A, int S, int T, float scale, double *G, cudaStream_t st) {
    using C = qmlb_fwht::Cfg<LOG2N>;
    const long items = (long)nb * A * ((S + C::V - 1) / C::V);
    size_t smem = sizeof(float) * TD_WARPS * (1 + (size_t)nel) * C::WARP_FLOATS;
    const int cache_d = smem <= 72 * 1024 ? 1 : 0;     // up to five elements at any width: three blocks per SM stay resident
    if (!cache_d) smem = sizeof(float) * TD_WARPS * C::WARP_FLOATS;
    if (int rc = qmlb::ensure_smem(train_derivative_tile_kernel<LOG2N>, smem, "qmlb_sorf_train_features")) return rc;
    train_derivative_tile_kernel<LOG2N><<<(unsigned)((items + TD_WARPS - 1) / TD_WARPS), TD_WARPS * 32, smem, st>>>(
        dx, sinc, Dmat, row_of_slot, group_start, atom_counts, nel, nb, A, S, T, scale, cache_d, G);
    return qmlb::check_launch("qmlb_sorf_train_features(derivative)");
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
        switch (E) {   // register-tile transform for N = 32 ... 512
            case 1: return launch_derivative_tile<5>(dx, sinc, Dmat, row_of_slot, group_start, atom_counts, nel, nb, A, S, T, scale, G, st);
            case 2: return launch_derivative_tile<6>(dx, sinc, Dmat, row_of_slot, group_start, atom_counts, nel, nb, A, S, T, scale, G, st);
            case 4: return launch_derivative_tile<7>(dx, sinc, Dmat, row_of_slot, group_start, atom_counts, nel, nb, A, S, T, scale, G, st);
            case 8: return launch_derivative_tile<8>(dx, sinc, Dmat, row_of_slot, group_start, atom_counts, nel, nb, A, S, T, scale, G, st);
            case 16: return launch_derivative_tile<9>(dx, sinc, Dmat, row_of_slot, group_start, atom_counts, nel, nb, A, S, T, scale, G, st);
            default: break;
        }
        qmlb::set_error("qmlb_sorf_train_features: force rows need npcas in [32, 512]");
        return QMLB_ERR_UNSUPPORTED;
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
    QMLB_REQUIRE((long)rows_cap * S / 8 < (1L << 31) && (long)nb * A * S / 4 < (1L << 31), "qmlb_sorf_train_features: batch too large");
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
        default:
            qmlb::set_error("qmlb_sorf_train_features: npcas must be a power of two in [32, 512], got %d", N);
            return QMLB_ERR_UNSUPPORTED;
    }
#undef QMLB_TRAIN
}
