// Training rows of the RFF model in one fused float64 kernel: per molecule the feature vector Z[m,:] and the force
// features G[m,j,x,:] = -dZ[m,:]/dr_{j,x}.
//
// Upstream: random_fourrier_features_kernel / _derivative (cuda/random_features_kernel.cu:5-94) via get_rff /
// get_rff_derivatives (cuda/random_features.cpp:11-33), driven once per element by calculate_features
// (models/random_features.py:60-67) with W.double() and b.double(): every dot product x.W and dx.W is a serial float64
// sum of float32 inputs, and the results are added to Z and G with float64 atomics.  Same arithmetic here (float32
// inputs promoted to float64, float64 accumulation, float64 sin/cos), reorganised as
//
//   G[m, (j,x), f] = sum over the atoms i of m of  sinc[i,f] * ( dx[i,(j,x),:] . W_e(i)[:,f] )
//
// i.e. per molecule a [3A x K] x [K x D] product per atom whose result is scaled column-wise by sinc[i,:] and summed
// over the atoms.  One block owns (molecule, 64 features, 64 derivative rows): the W tile of one element stays in
// shared memory while the block walks the atoms of that element; per atom it forms arg = x.W + b for its 64 features
// (plain DFMA), sin/cos, then streams the atom's dx rows through a double-buffered cp.async ring and multiplies them
// with the W tile on the double-precision tensor-core path (mma.sync.m8n8k4.f64), folding sinc * product into the
// block's G accumulators in registers.  Every Z and G element is written exactly once: no atomics, no zero-filled
// outputs, and none of the [rows, D] / [rows, 3A, D] intermediates of the unfused form.
#include <math.h>

#include "common.cuh"

namespace {

constexpr int FT = 64;           // features per block
constexpr int MTILE = 64;        // derivative rows (j,x) per block
constexpr int KS = 32;           // k per dx slice
constexpr int THREADS = 256;     // 8 warps: 4 (16 rows each) x 2 (32 features each)
constexpr int LDW = FT + 8;      // W tile row stride in floats: (8k + n) mod 32 distinct over a warp's B fragment
constexpr int LDD = KS + 4;      // dx slice row stride in floats: (4m + k) mod 32 distinct over a warp's A fragment

__device__ __forceinline__ void cp_async16(void *dst, const void *src, bool valid) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N)); }

__device__ __forceinline__ void dmma(double &d0, double &d1, double a, double b) {
    asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0,%1}, {%2}, {%3}, {%0,%1};"
                 : "+d"(d0), "+d"(d1)
                 : "d"(a), "d"(b));
}

__device__ __forceinline__ int element_of_row(long row, const int *group_start, int nel) {
    int e = 0;
    while (e + 1 < nel && row >= group_start[e + 1]) ++e;
    return e;
}

struct Smem {
    float *W;        // [Kpad][LDW]
    float *dx;       // [2][MTILE][LDD]
    float *x;        // [Kpad]
    double *red;     // [4][FT]
    double *sinc;    // [FT]
};

__device__ __forceinline__ Smem carve(unsigned char *base, int Kpad) {
    Smem s;
    s.red = reinterpret_cast<double *>(base);
    s.sinc = s.red + 4 * FT;
    s.W = reinterpret_cast<float *>(s.sinc + FT);
    s.dx = s.W + (size_t)Kpad * LDW;
    s.x = s.dx + 2 * MTILE * LDD;
    return s;
}

__host__ __device__ inline size_t smem_bytes(int Kpad) {
    return sizeof(double) * 5 * FT + sizeof(float) * ((size_t)Kpad * LDW + 2 * MTILE * LDD + Kpad);
}

// dx rows [jx0, jx0 + MTILE) of one atom, k in [k0, k0 + KS), into one buffer; rows >= nrows and k >= K become zero.
__device__ __forceinline__ void load_dx_slice(float *buf, const float *__restrict__ dxrow, int nrows, int K, int jx0, int k0) {
#pragma unroll
    for (int q = 0; q < MTILE * (KS / 4) / THREADS; ++q) {
        const int idx = q * THREADS + threadIdx.x;
        const int r = idx / (KS / 4), c = (idx % (KS / 4)) * 4;
        const bool ok = jx0 + r < nrows && k0 + c + 4 <= K;
        cp_async16(buf + r * LDD + c, dxrow + (ok ? (size_t)(jx0 + r) * K + k0 + c : 0), ok);
    }
}

__global__ void __launch_bounds__(THREADS, 2)
rff_train_kernel(const float *__restrict__ x, const float *__restrict__ dx, const float *__restrict__ W,
                 const float *__restrict__ b, const int *__restrict__ group_start, const int *__restrict__ row_of_slot,
                 const int *__restrict__ atom_counts, int nel, int A, int K, int Kpad, int D, double normf,
                 double *__restrict__ Zout, double *__restrict__ G) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const Smem S = carve(smem_raw, Kpad);
    const int f0 = blockIdx.x * FT, mol = blockIdx.y, jx0 = blockIdx.z * MTILE;
    const int nrows = 3 * A;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int wm = warp & 3, wn = warp >> 2;
    const int lk = lane & 3, lm = lane >> 2;
    int natoms = atom_counts[mol];
    natoms = natoms < 0 ? 0 : (natoms > A ? A : natoms);
    const bool with_grad = dx != nullptr;

    double zacc = 0.0;                      // threads 0..FT-1: feature f0 + threadIdx.x
    double gacc[2][4][2];
#pragma unroll
    for (int a = 0; a < 2; ++a)
#pragma unroll
        for (int c = 0; c < 4; ++c) gacc[a][c][0] = gacc[a][c][1] = 0.0;

    for (int e = 0; e < nel; ++e) {
        bool present = false;
        for (int i = 0; i < natoms; ++i) {
            const int row = row_of_slot[(size_t)mol * A + i];
            present |= row >= 0 && element_of_row(row, group_start, nel) == e;
        }
        if (!present) continue;             // uniform over the block
        __syncthreads();                    // the previous element's tile is no longer read
        for (int idx = threadIdx.x; idx < Kpad * FT; idx += THREADS) {
            const int k = idx / FT, f = idx % FT;
            S.W[k * LDW + f] = (k < K && f0 + f < D) ? W[((size_t)e * K + k) * D + f0 + f] : 0.f;
        }
        for (int i = 0; i < natoms; ++i) {
            const int row = row_of_slot[(size_t)mol * A + i];
            if (row < 0 || element_of_row(row, group_start, nel) != e) continue;
            const float *dxrow = with_grad ? dx + (size_t)row * nrows * K : nullptr;
            if (with_grad) {                // first slice in flight while the features of this atom are formed
                load_dx_slice(S.dx, dxrow, nrows, K, jx0, 0);
                cp_async_commit();
            }
            __syncthreads();                // W tile visible; x / red / sinc of the previous atom no longer read
            for (int k = threadIdx.x; k < Kpad; k += THREADS) S.x[k] = k < K ? x[(size_t)row * K + k] : 0.f;
            __syncthreads();
            {
                // arg[f] = sum_k x[k] W[k][f]: four threads per feature, each a quarter of k, serial float64 sums
                const int f = threadIdx.x % FT, part = threadIdx.x / FT;
                const int kq = (Kpad + 3) / 4, k_lo = part * kq, k_hi = min(Kpad, k_lo + kq);
                double s = 0.0;
                for (int k = k_lo; k < k_hi; ++k) s = fma((double)S.x[k], (double)S.W[k * LDW + f], s);
                S.red[part * FT + f] = s;
            }
            __syncthreads();
            if (threadIdx.x < FT) {
                const int f = threadIdx.x;
                double sn = 0.0, cs = 0.0;
                if (f0 + f < D) {
                    const double arg = ((S.red[f] + S.red[FT + f]) + (S.red[2 * FT + f] + S.red[3 * FT + f])) + (double)b[(size_t)e * D + f0 + f];
                    sincos(arg, &sn, &cs);
                }
                zacc += normf * cs;
                S.sinc[f] = normf * sn;
            }
            if (!with_grad) continue;       // uniform
            double acc[2][4][2];
#pragma unroll
            for (int a = 0; a < 2; ++a)
#pragma unroll
                for (int c = 0; c < 4; ++c) acc[a][c][0] = acc[a][c][1] = 0.0;
            const int nslices = Kpad / KS;
            for (int ks = 0; ks < nslices; ++ks) {
                if (ks + 1 < nslices) load_dx_slice(S.dx + ((ks + 1) & 1) * MTILE * LDD, dxrow, nrows, K, jx0, (ks + 1) * KS);
                cp_async_commit();
                cp_async_wait<1>();
                __syncthreads();            // slice ks landed for everybody (also publishes sinc on the first pass)
                const float *As = S.dx + (ks & 1) * MTILE * LDD + (wm * 16 + lm) * LDD + lk;
                const float *Bs = S.W + (size_t)(ks * KS + lk) * LDW + wn * 32 + lm;
#pragma unroll
                for (int kk = 0; kk < KS / 4; ++kk) {
                    double a[2], bb[4];
#pragma unroll
                    for (int mt = 0; mt < 2; ++mt) a[mt] = (double)As[mt * 8 * LDD + kk * 4];
#pragma unroll
                    for (int n8 = 0; n8 < 4; ++n8) bb[n8] = (double)Bs[(size_t)kk * 4 * LDW + n8 * 8];
#pragma unroll
                    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
                        for (int n8 = 0; n8 < 4; ++n8) dmma(acc[mt][n8][0], acc[mt][n8][1], a[mt], bb[n8]);
                }
                __syncthreads();            // everybody is done with slice ks before its buffer is refilled
            }
#pragma unroll
            for (int mt = 0; mt < 2; ++mt)
#pragma unroll
                for (int n8 = 0; n8 < 4; ++n8) {
                    const int n = wn * 32 + n8 * 8 + lk * 2;
                    gacc[mt][n8][0] = fma(S.sinc[n], acc[mt][n8][0], gacc[mt][n8][0]);
                    gacc[mt][n8][1] = fma(S.sinc[n + 1], acc[mt][n8][1], gacc[mt][n8][1]);
                }
        }
    }
    if (blockIdx.z == 0 && threadIdx.x < FT && f0 + threadIdx.x < D) Zout[(size_t)mol * D + f0 + threadIdx.x] = zacc;
    if (with_grad) {
#pragma unroll
        for (int mt = 0; mt < 2; ++mt) {
            const int jx = jx0 + wm * 16 + mt * 8 + lm;
            if (jx >= nrows) continue;
            double *dst = G + ((size_t)mol * nrows + jx) * D + f0;
#pragma unroll
            for (int n8 = 0; n8 < 4; ++n8) {
                const int n = wn * 32 + n8 * 8 + lk * 2;
                if (f0 + n < D) dst[n] = gacc[mt][n8][0];
                if (f0 + n + 1 < D) dst[n + 1] = gacc[mt][n8][1];
            }
        }
    }
}

}  // namespace

extern "C" int qmlb_rff_train_features(const float *x, const float *dx, const float *W, const float *b,
                                       const int *group_start, const int *slot_of_row, const int *row_of_slot,
                                       const int *atom_counts, int nelements, int nb, int A, size_t rows_cap, int K, int D,
                                       double *Zout, double *G, qmlb_stream_t stream) {
    (void)slot_of_row;
    (void)rows_cap;
    QMLB_REQUIRE(x && W && b && group_start && row_of_slot && atom_counts && Zout, "qmlb_rff_train_features: null tensor");
    QMLB_REQUIRE((dx == nullptr) == (G == nullptr), "qmlb_rff_train_features: dx and G go together");
    QMLB_REQUIRE(nelements > 0 && nb > 0 && A > 0 && K > 0 && D > 0, "qmlb_rff_train_features: bad sizes");
    QMLB_REQUIRE(K % 4 == 0 && (((uintptr_t)dx) & 15) == 0, "qmlb_rff_train_features: npcas must be a multiple of 4 and dx 16-byte aligned");
    QMLB_REQUIRE(nb < 65536, "qmlb_rff_train_features: at most 65535 molecules per call");
    const int Kpad = (K + KS - 1) / KS * KS;
    const size_t smem = smem_bytes(Kpad);
    if (int rc = qmlb::ensure_smem(rff_train_kernel, smem, "qmlb_rff_train_features")) return rc;
    dim3 grid((unsigned)((D + FT - 1) / FT), (unsigned)nb, dx ? (unsigned)((3 * A + MTILE - 1) / MTILE) : 1u);
    rff_train_kernel<<<grid, THREADS, smem, qmlb::as_stream(stream)>>>(x, dx, W, b, group_start, row_of_slot, atom_counts,
                                                                      nelements, A, K, Kpad, D, sqrt(2.0 / (double)D), Zout, G);
    return qmlb::check_launch("qmlb_rff_train_features");
}
