// FCHL19 atom-centred representation for sm_100a: element typing, neighbour lists, forward,
// vector-Jacobian product (coordinate gradient) and explicit Jacobian.
//
// Work decomposition: one thread block per molecule, one warp per centre atom (warps stride over the atoms of
// the molecule).  The coordinates of the molecule live in shared memory; every warp builds the neighbour list of
// its centre atom in its own shared-memory slab (ballot compaction keeps neighbours in ascending index order),
// accumulates the representation row in shared memory and writes it out once.  No global atomics are used and
// no output needs to be zero-initialised by the caller.
//
// Arithmetic follows the upstream kernels (cuda/fchl_cuda_kernel.cu:476-674 forward, :1325-1714 backward):
// per-neighbour quantities (log-normal parameters, decay, cut-off) are evaluated in double precision, where
// upstream promotes implicitly through double literals; the per-grid-point loops run in float.
#include <math.h>

#include "common.cuh"

namespace {

#ifndef QMLB_FCHL_WARPS
#define QMLB_FCHL_WARPS 4
#endif
constexpr int FCHL_WARPS = QMLB_FCHL_WARPS;
constexpr int FCHL_THREADS = FCHL_WARPS * 32;
constexpr float ZETA2 = 0.014383766711652736f;  // 2 * exp(-pi^2 / 2)

struct FchlK {
    int nb, A, nel, nRs2, nRs3, repsize, pbc;
    float eta2, eta3, d2, w3, d3, rcut;
};

// ---- shared-memory carve-up ----------------------------------------------------------------------------------
// block : x[A] y[A] z[A] et[A] | Rs2[nRs2] logRs2[nRs2] invRs2[nRs2] Rs3[nRs3] | cell[9] icell[9] | logRs2_lo[nRs2] (+pad)
// ln Rs2 and mu are kept as float pairs (hi + lo): the log-normal exponent (ln Rs2 - mu)^2 / (2 sigma^2) amplifies
// the rounding of its argument by up to 1/sigma^2 ~ 100, which would otherwise cost a digit of the representation.
// warp  : NB_FIELDS arrays of A entries | row[repsize] | (backward) force[3A] | 32 x float4 triplet staging
constexpr int NB_FIELDS = 16;
enum { F_IDX = 0, F_DX, F_DY, F_DZ, F_R, F_FC, F_DFC, F_ET, F_MU, F_MULO, F_I2S, F_PREF, F_C0, F_C1, F_C2, F_IR };

__host__ __device__ inline int align4(int v) { return (v + 3) & ~3; }

struct Layout {
    int block_floats, warp_floats, off_row, off_force, off_stage;
    __host__ __device__ Layout(int A, int nRs2, int nRs3, int repsize, bool backward) {
        block_floats = align4(4 * A + 4 * nRs2 + nRs3 + 18);
        off_row = align4(NB_FIELDS * A);
        off_force = off_row + align4(repsize);
        off_stage = off_force + (backward ? align4(3 * A) : 0);
        warp_floats = off_stage + 128;   // 32 staged triplets x float4
    }
    __host__ __device__ size_t bytes() const { return sizeof(float) * ((size_t)block_floats + (size_t)FCHL_WARPS * warp_floats); }
};

__device__ __forceinline__ void min_image(float &dx, float &dy, float &dz, const float *cell, const float *icell) {
    // s = inv_cell . d ; s -= round(s) ; d = cell . s   (cuda/fchl_cuda_kernel.cu:16-49)
    float s0 = icell[0] * dx + icell[1] * dy + icell[2] * dz;
    float s1 = icell[3] * dx + icell[4] * dy + icell[5] * dz;
    float s2 = icell[6] * dx + icell[7] * dy + icell[8] * dz;
    s0 -= roundf(s0);
    s1 -= roundf(s1);
    s2 -= roundf(s2);
    dx = cell[0] * s0 + cell[1] * s1 + cell[2] * s2;
    dy = cell[3] * s0 + cell[4] * s1 + cell[5] * s2;
    dz = cell[6] * s0 + cell[7] * s1 + cell[8] * s2;
}

// The same in double for the FCHL19 kernels: the stored coordinates of a periodic system may lie several cell lengths
// apart, so r_i - r_j and its reduction are formed in double (both are exact or nearly so) and rounded to float once;
// the reduced vector then carries the same relative rounding as in the non-periodic case.
__device__ __forceinline__ void min_image_d(double &dx, double &dy, double &dz, const float *cell, const float *icell) {
    double s0 = (double)icell[0] * dx + (double)icell[1] * dy + (double)icell[2] * dz;
    double s1 = (double)icell[3] * dx + (double)icell[4] * dy + (double)icell[5] * dz;
    double s2 = (double)icell[6] * dx + (double)icell[7] * dy + (double)icell[8] * dz;
    s0 -= round(s0);
    s1 -= round(s1);
    s2 -= round(s2);
    dx = (double)cell[0] * s0 + (double)cell[1] * s1 + (double)cell[2] * s2;
    dy = (double)cell[3] * s0 + (double)cell[4] * s1 + (double)cell[5] * s2;
    dz = (double)cell[6] * s0 + (double)cell[7] * s1 + (double)cell[8] * s2;
}

__device__ __forceinline__ int species_index(float z, const float *species, int nel) {
    // upstream truncates the charge to int and keeps the last match (fchl_cuda_kernel.cu:1730-1737)
    float q = (float)(int)z;
    int idx = -1;
    for (int j = 0; j < nel; ++j)
        if (q == species[j]) idx = j;
    return idx;
}

// Loads one molecule into shared memory; returns its atom count.
__device__ int stage_molecule(const float *X, const float *Z, const int *counts, const float *species,
                              const float *Rs2, const float *Rs3, const float *cell, const float *icell,
                              const FchlK &K, int mol, float *sm) {
    const int A = K.A;
    float *sx = sm, *sy = sm + A, *sz = sm + 2 * A;
    int *set = reinterpret_cast<int *>(sm + 3 * A);
    float *sRs2 = sm + 4 * A, *sLog2 = sRs2 + K.nRs2, *sInv2 = sLog2 + K.nRs2, *sRs3 = sInv2 + K.nRs2;
    float *scell = sRs3 + K.nRs3;
    int natoms = counts[mol];
    natoms = natoms < 0 ? 0 : (natoms > A ? A : natoms);
    for (int a = threadIdx.x; a < A; a += blockDim.x) {
        const float *xp = X + ((size_t)mol * A + a) * 3;
        sx[a] = xp[0];
        sy[a] = xp[1];
        sz[a] = xp[2];
        set[a] = a < natoms ? species_index(Z[(size_t)mol * A + a], species, K.nel) : -1;
    }
    for (int z = threadIdx.x; z < K.nRs2; z += blockDim.x) {
        float r = Rs2[z];
        sRs2[z] = r;
        const double lg = log((double)r);
        sLog2[z] = (float)lg;
        scell[18 + z] = (float)(lg - (double)(float)lg);
        sInv2[z] = 1.0f / r;
    }
    for (int z = threadIdx.x; z < K.nRs3; z += blockDim.x) sRs3[z] = Rs3[z];
    if (K.pbc && threadIdx.x < 18)
        scell[threadIdx.x] = threadIdx.x < 9 ? cell[(size_t)mol * 9 + threadIdx.x] : icell[(size_t)mol * 9 + threadIdx.x - 9];
    __syncthreads();
    return natoms;
}

// Builds the neighbour slab of centre atom i for one warp; returns the neighbour count.
// Per neighbour: index, d = r_i - r_j, r, cut-off fc and its derivative, element, and the two-body scalars
//   mu, i2s = log2(e)/(2 sigma^2) (the radial term is evaluated as 2^(-t^2 i2s)), pref = r^-d2 / (sigma sqrt(2 pi))
//   (without cut-off),
//   c0,c1,c2: d ln(radial_z)/dr = c0 + c1 t + c2 t^2 with t = ln Rs2[z] - mu (used by the backward pass).
__device__ int build_neighbours(const float *sm, float *ws, const FchlK &K, int natoms, int i, int lane) {
    const int A = K.A;
    const float *sx = sm, *sy = sm + A, *sz = sm + 2 * A;
    const int *set = reinterpret_cast<const int *>(sm + 3 * A);
    const float *scell = sm + 4 * A + 3 * K.nRs2 + K.nRs3;
    int *n_idx = reinterpret_cast<int *>(ws + F_IDX * A);
    int *n_et = reinterpret_cast<int *>(ws + F_ET * A);
    const float xi = sx[i], yi = sy[i], zi = sz[i];
    const float rcut2 = K.rcut * K.rcut;
    int nn = 0;
    for (int j0 = 0; j0 < natoms; j0 += 32) {
        const int j = j0 + lane;
        bool ok = false;
        float dx = 0.f, dy = 0.f, dz = 0.f, r2 = 0.f;
        if (j < natoms && j != i && set[j] >= 0) {
            if (K.pbc) {
                double ddx = (double)xi - (double)sx[j], ddy = (double)yi - (double)sy[j], ddz = (double)zi - (double)sz[j];
                min_image_d(ddx, ddy, ddz, scell, scell + 9);
                dx = (float)ddx;
                dy = (float)ddy;
                dz = (float)ddz;
            } else {
                dx = xi - sx[j];
                dy = yi - sy[j];
                dz = zi - sz[j];
            }
            r2 = dx * dx + dy * dy + dz * dz;
            ok = r2 < rcut2 && r2 > 0.f;  // cuda/pairlist_kernel.cu:386
        }
        const unsigned m = __ballot_sync(QMLB_FULL_MASK, ok);
        if (ok) {
            const int pos = nn + __popc(m & ((1u << lane) - 1u));
            // Distance and the two logarithms of the log-normal parameters in double (their rounding is amplified
            // by 1/sigma^2 in the exponent); everything else is well conditioned and stays in float.
            const double r2d = (double)dx * dx + (double)dy * dy + (double)dz * dz;
            const float r = sqrtf((float)r2d);
            const float inv_rcut = 1.0f / K.rcut;
            float sarg, carg;
            sincospif(r * inv_rcut, &sarg, &carg);
            const float fc = 0.5f * (carg + 1.0f);
            const float dfc = -0.5f * sarg * 3.14159265358979f * inv_rcut;
            // sigma^2 = ln(1 + eta2 / r^2) = ln(r^2 + eta2) - ln(r^2) ;  mu = ln r - sigma^2 / 2 = ln(r^2) - ln(r^2 + eta2) / 2:
            // two double logarithms of r^2 and r^2 + eta2 replace sqrt, division, log1p and log of the direct form
            const double la = log(r2d), lb = log(r2d + (double)K.eta2);
            const double s2 = lb - la;
            const double mu = la - 0.5 * lb;
            const float rf2 = r * r;
            const float s2f = (float)s2;
            const float ds2 = -2.0f * K.eta2 / (r * (rf2 + K.eta2));
            const float dmu = (rf2 + 2.0f * K.eta2) / (r * (rf2 + K.eta2));
            n_idx[pos] = j;
            n_et[pos] = set[j];
            ws[F_DX * A + pos] = dx;
            ws[F_DY * A + pos] = dy;
            ws[F_DZ * A + pos] = dz;
            ws[F_R * A + pos] = r;
            ws[F_IR * A + pos] = 1.0f / r;
            ws[F_FC * A + pos] = fc;
            ws[F_DFC * A + pos] = dfc;
            ws[F_MU * A + pos] = (float)mu;
            ws[F_MULO * A + pos] = (float)(mu - (double)(float)mu);
            ws[F_I2S * A + pos] = 0.5f * 1.4426950408889634f / s2f;
            ws[F_PREF * A + pos] = powf(r, -K.d2) * rsqrtf(s2f) * 0.3989422804014327f;  // 1 / (sigma sqrt(2 pi))
            ws[F_C0 * A + pos] = -0.5f * ds2 / s2f - K.d2 / r;
            ws[F_C1 * A + pos] = dmu / s2f;
            ws[F_C2 * A + pos] = ds2 / (2.0f * s2f * s2f);
        }
        nn += __popc(m);
    }
    __syncwarp();
    return nn;
}

// 2^x on the SFU without the denormal-range fix-up that exp2f() adds (results below 2^-126 flush to zero, which is
// what a Gaussian tail of that size is worth here); saves three instructions per grid point in the radial loops.
__device__ __forceinline__ float ex2_fast(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Row-major enumeration of pairs j<k of n items: t -> (j,k).
__device__ __forceinline__ void decode_pair(int t, int n, int &j, int &k) {
    const float b = (float)(2 * n - 1);
    int jj = (int)((b - sqrtf(fmaxf(b * b - 8.0f * (float)t, 0.f))) * 0.5f);
    jj = jj < 0 ? 0 : (jj > n - 2 ? n - 2 : jj);
    while (jj > 0 && (jj * (2 * n - jj - 1)) / 2 > t) --jj;
    while (((jj + 1) * (2 * n - jj - 2)) / 2 <= t) ++jj;
    j = jj;
    k = t - (jj * (2 * n - jj - 1)) / 2 + jj + 1;
}

// Scalars of one triplet (i; j,k) that the backward pass needs on top of the forward amplitudes.
struct TripletGeom {
    float a, b, c;          // r_ij, r_ik, r_jk
    float ia, ib, ic;       // their reciprocals
    float ci, cj, ck;       // cosines at i, j, k
    float cth, sth, w;      // clamped cos(theta_i), sin(theta_i), regularised 1/sin factor
    float T, R, Fij, Fik;   // ksi3 = w3*T*R ; cut-offs
    float dFij, dFik;
    float ejk[3];           // (r_j - r_k)/r_jk
};

__device__ __forceinline__ void triplet_geometry(const float *ws, int A, int j, int k, const FchlK &K, TripletGeom &g) {
    const float dxj = ws[F_DX * A + j], dyj = ws[F_DY * A + j], dzj = ws[F_DZ * A + j];
    const float dxk = ws[F_DX * A + k], dyk = ws[F_DY * A + k], dzk = ws[F_DZ * A + k];
    g.a = ws[F_R * A + j];
    g.b = ws[F_R * A + k];
    const float jx = dxk - dxj, jy = dyk - dyj, jz = dzk - dzj;  // r_j - r_k
    const float c2 = jx * jx + jy * jy + jz * jz;
    const float inv_c = rsqrtf(c2);   // SFU reciprocal square root (2 ulp): r_jk only enters well-conditioned factors
    g.c = c2 * inv_c;
    g.ejk[0] = jx * inv_c;
    g.ejk[1] = jy * inv_c;
    g.ejk[2] = jz * inv_c;
    const float vi = dxj * dxk + dyj * dyk + dzj * dzk;           // (ri-rj).(ri-rk)
    const float vk = jx * dxk + jy * dyk + jz * dzk;              // (rj-rk).(ri-rk)
    const float vj = -(dxj * jx + dyj * jy + dzj * jz);           // (ri-rj).(rk-rj)
    const float inv_a = ws[F_IR * A + j], inv_b = ws[F_IR * A + k];   // 1/r per neighbour, divided once
    g.ci = vi * inv_a * inv_b;
    g.cj = vj * inv_a * inv_c;
    g.ck = vk * inv_b * inv_c;
    g.cth = fminf(1.0f, fmaxf(-1.0f, g.ci));
    // sin(theta_i) from the cross product |d_ij x d_ik| = r_ij r_ik sin(theta): unlike sqrt(1 - cos^2) (what
    // sinf(acosf(c)) amounts to upstream) it does not cancel for nearly collinear triplets, whose d sin/d cos =
    // -cos/sin is large.  Upstream regularises 1/(r_ij r_ik sin) as 1/sqrt(max(1e-10, r_ij^2 r_ik^2 - vi^2))
    // (:1578-1579); r_ij^2 r_ik^2 - vi^2 is the squared cross product, so the same floor (1e-5) is applied to it.
    const float cx = dyj * dzk - dzj * dyk, cy = dzj * dxk - dxj * dzk, cz = dxj * dyk - dyj * dxk;
    const float sab = sqrtf(cx * cx + cy * cy + cz * cz);
    const float ab = g.a * g.b;
    g.sth = fminf(1.0f, sab * inv_a * inv_b);
    g.w = ab / fmaxf(sab, 1e-5f);
    g.ia = inv_a; g.ib = inv_b; g.ic = inv_c;
    g.T = 1.0f + 3.0f * g.ci * g.cj * g.ck;
    g.R = ex2_fast(-K.d3 * __log2f(g.a * g.b * g.c));  // (r_ij r_ik r_jk)^-d3; the SFU log2 is exact to ~2e-7 relative here
    g.Fij = ws[F_FC * A + j];
    g.Fik = ws[F_FC * A + k];
    g.dFij = ws[F_DFC * A + j];
    g.dFik = ws[F_DFC * A + k];
}

__device__ __forceinline__ int pair_block(int ej, int ek, const FchlK &K) {
    const int p = ej < ek ? ej : ek, q = ej < ek ? ek : ej;
    return K.nel * K.nRs2 + 2 * K.nRs3 * (q + K.nel * p - (p * (p + 1)) / 2);  // fchl_cuda_kernel.cu:661
}

// ---- forward -------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(FCHL_THREADS)
fchl_forward_kernel(const float *__restrict__ X, const float *__restrict__ Z, const int *__restrict__ counts,
                    const float *__restrict__ species, const float *__restrict__ Rs2, const float *__restrict__ Rs3,
                    const float *__restrict__ cell, const float *__restrict__ icell, FchlK K,
                    const int *__restrict__ row_of_slot, float *__restrict__ out) {
    extern __shared__ __align__(16) float sm[];
    const int mol = blockIdx.x, A = K.A;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const Layout L(A, K.nRs2, K.nRs3, K.repsize, false);
    const int natoms = stage_molecule(X, Z, counts, species, Rs2, Rs3, cell, icell, K, mol, sm);
    const float *sLog2 = sm + 4 * A + K.nRs2, *sInv2 = sLog2 + K.nRs2, *sRs3 = sInv2 + K.nRs2;
    const float *sLog2lo = sRs3 + K.nRs3 + 18;
    float *ws = sm + L.block_floats + (size_t)warp * L.warp_floats;
    float *acc = ws + L.off_row;
    const int *n_et = reinterpret_cast<const int *>(ws + F_ET * A);

    for (int i = warp; i < A; i += FCHL_WARPS) {
        long row = row_of_slot ? (long)row_of_slot[(size_t)mol * A + i] : (long)mol * A + i;
        if (row < 0) continue;
        float *dst = out + (size_t)row * K.repsize;
        if (i >= natoms) {
            if (!row_of_slot)
                for (int c = lane; c < K.repsize; c += 32) dst[c] = 0.f;
            continue;
        }
        const int nn = build_neighbours(sm, ws, K, natoms, i, lane);
        for (int c = lane; c < K.repsize; c += 32) acc[c] = 0.f;
        __syncwarp();

        // two-body (fchl_cuda_kernel.cu:586-603): lanes over grid points, neighbours serial
        for (int jn = 0; jn < nn; ++jn) {
            const float mu = ws[F_MU * A + jn], mulo = ws[F_MULO * A + jn], i2s = ws[F_I2S * A + jn];
            const float pref = ws[F_PREF * A + jn] * ws[F_FC * A + jn];
            float *blk = acc + n_et[jn] * K.nRs2;
            for (int z = lane; z < K.nRs2; z += 32) {
                const float t = (sLog2[z] - mu) + (sLog2lo[z] - mulo);
                blk[z] += pref * sInv2[z] * ex2_fast(-t * t * i2s);
            }
        }

        // three-body (fchl_cuda_kernel.cu:605-672): 32 triplets at a time, one per lane for the scalar part; their
        // (rbar, amplitudes, block offset) go to a small per-warp staging area, then each triplet is read back as
        // one broadcast 128-bit load and the lanes cover the radial grid (exp2 with the constant folded in).
        const int ntrip = nn * (nn - 1) / 2;
        float4 *stage = reinterpret_cast<float4 *>(ws + L.off_stage);
        // exp(-eta3 d^2) = 2^-(kk d)^2 with kk = sqrt(eta3 log2 e): the triplet's mean distance and the grid are both
        // scaled by kk once, so a grid point costs one subtraction, one negated square and the exp2
        const float kk = sqrtf(K.eta3 * 1.4426950408889634f);
        const bool pair_ok = ((K.nel * K.nRs2) & 1) == 0;   // (cos, sin) columns 8-byte aligned
        for (int t0 = 0; t0 < ntrip; t0 += 32) {
            const int t = t0 + lane;
            float4 tr = make_float4(0.f, 0.f, 0.f, 0.f);
            if (t < ntrip) {
                int j, k;
                decode_pair(t, nn, j, k);
                TripletGeom g;
                triplet_geometry(ws, A, j, k, K, g);
                const float amp = ZETA2 * K.w3 * g.T * g.R * g.Fij * g.Fik;
                tr.x = kk * (0.5f * (g.a + g.b));
                tr.y = amp * g.cth;
                tr.z = amp * g.sth;
                tr.w = __int_as_float(pair_block(n_et[j], n_et[k], K));
            }
            stage[lane] = tr;
            __syncwarp();
            const int cnt = min(32, ntrip - t0);
            if (K.nRs3 <= 32 && pair_ok) {
                const float rs = lane < K.nRs3 ? kk * sRs3[lane] : 0.f;
                for (int q = 0; q < cnt; ++q) {
                    const float4 b = stage[q];
                    if (lane < K.nRs3) {
                        const float d = b.x - rs;
                        const float radial = ex2_fast(-d * d);
                        float2 *p2 = reinterpret_cast<float2 *>(acc + __float_as_int(b.w)) + lane;
                        *p2 = __ffma2_rn(make_float2(radial, radial), make_float2(b.y, b.z), *p2);
                    }
                }
            } else {
                for (int q = 0; q < cnt; ++q) {
                    const float4 b = stage[q];
                    const int sidx = __float_as_int(b.w);
                    for (int l = lane; l < K.nRs3; l += 32) {
                        const float d = b.x - kk * sRs3[l];
                        const float radial = ex2_fast(-d * d);
                        acc[sidx + 2 * l] += radial * b.y;
                        acc[sidx + 2 * l + 1] += radial * b.z;
                    }
                }
            }
            __syncwarp();
        }
        __syncwarp();
        for (int c = lane; c < K.repsize; c += 32) dst[c] = acc[c];
        __syncwarp();
    }
}

// ---- backward (vector-Jacobian product) ----------------------------------------------------------------------
// For centre atom i with incoming gradient row g (length repsize) every term of the representation is a function
// of the three distances of a triplet (or the one distance of a pair), so the chain rule is carried out on
// (r_ij, r_ik, r_jk) and mapped to the three atoms along the unit vectors.
// The kernel is latency bound (dependent shared-memory loads and exp2 in the per-triplet loops), so it is compiled for
// 8 resident blocks per SM (64 registers, one 4-byte spill) and the radial loop is unrolled twice: 2.05 -> 1.66 ms on
// 10,000 21-atom molecules; 5 / 6 / 7 blocks gave 1.87 / 1.82 / 1.75 ms.
constexpr int BWD_UNROLL = 2;
__global__ void __launch_bounds__(FCHL_THREADS, 32 / FCHL_WARPS)
fchl_backward_kernel(const float *__restrict__ X, const float *__restrict__ Z, const int *__restrict__ counts,
                     const float *__restrict__ species, const float *__restrict__ Rs2, const float *__restrict__ Rs3,
                     const float *__restrict__ cell, const float *__restrict__ icell, FchlK K,
                     const int *__restrict__ row_of_slot, const float *__restrict__ grad_rep,
                     float *__restrict__ grad_X, const float *__restrict__ atom_energy, float *__restrict__ mol_energy) {
    extern __shared__ __align__(16) float sm[];
    const int mol = blockIdx.x, A = K.A;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const Layout L(A, K.nRs2, K.nRs3, K.repsize, true);
    const int natoms = stage_molecule(X, Z, counts, species, Rs2, Rs3, cell, icell, K, mol, sm);
    const float *sLog2 = sm + 4 * A + K.nRs2, *sInv2 = sLog2 + K.nRs2, *sRs3 = sInv2 + K.nRs2;
    const float *sLog2lo = sRs3 + K.nRs3 + 18;
    float *ws = sm + L.block_floats + (size_t)warp * L.warp_floats;
    float *grow = ws + L.off_row;
    float *force = ws + L.off_force;  // this warp's contribution to d/dr of every atom of the molecule
    const int *n_et = reinterpret_cast<const int *>(ws + F_ET * A);
    const int *n_idx = reinterpret_cast<const int *>(ws + F_IDX * A);

    for (int c = lane; c < 3 * A; c += 32) force[c] = 0.f;
    __syncwarp();

    for (int i = warp; i < natoms; i += FCHL_WARPS) {
        const long row = row_of_slot ? (long)row_of_slot[(size_t)mol * A + i] : (long)mol * A + i;
        if (row < 0) continue;
        const int nn = build_neighbours(sm, ws, K, natoms, i, lane);
        const float *src = grad_rep + (size_t)row * K.repsize;
        for (int c = lane; c < K.repsize; c += 32) grow[c] = src[c];
        __syncwarp();

        float fi0 = 0.f, fi1 = 0.f, fi2 = 0.f;

        // two-body: one neighbour per lane, grid points serial
        for (int j0 = 0; j0 < nn; j0 += 32) {
            const int jn = j0 + lane;
            if (jn < nn) {
                const float mu = ws[F_MU * A + jn], mulo = ws[F_MULO * A + jn], i2s = ws[F_I2S * A + jn];
                const float pref = ws[F_PREF * A + jn];
                const float fc = ws[F_FC * A + jn], dfc = ws[F_DFC * A + jn];
                const float c0 = ws[F_C0 * A + jn], c1 = ws[F_C1 * A + jn], c2 = ws[F_C2 * A + jn];
                const float *gb = grow + n_et[jn] * K.nRs2;
                float gr = 0.f;
                for (int z = 0; z < K.nRs2; ++z) {
                    const float t = (sLog2[z] - mu) + (sLog2lo[z] - mulo);
                    const float base = pref * sInv2[z] * ex2_fast(-t * t * i2s);
                    gr += gb[z] * base * (fc * (c0 + t * (c1 + t * c2)) + dfc);
                }
                const float inv_r = ws[F_IR * A + jn];
                const float ex = ws[F_DX * A + jn] * inv_r, ey = ws[F_DY * A + jn] * inv_r, ez = ws[F_DZ * A + jn] * inv_r;
                fi0 += gr * ex;
                fi1 += gr * ey;
                fi2 += gr * ez;
                float *fj = force + 3 * n_idx[jn];  // distinct atoms per lane: no conflict
                fj[0] -= gr * ex;
                fj[1] -= gr * ey;
                fj[2] -= gr * ez;
            }
        }
        __syncwarp();

        // three-body: one triplet per lane, radial grid serial.  Triplets are enumerated row-major in (j,k), so the
        // lanes that share j form one contiguous run per warp: their contributions to atom j are combined with a
        // segmented shuffle reduction and added once by the run's first lane (runs have distinct j, so no atomics);
        // contributions to atom k collide at most between runs and use shared-memory atomics.
        const int ntrip = nn * (nn - 1) / 2;
        // exp(-eta3 d^2) = 2^-(kk d)^2 with kk = sqrt(eta3 log2 e); the loop works on kk d (one fused multiply-add from the
        // grid point) and the factor 1/kk of the d-weighted sums is applied once per triplet
        const float kk = sqrtf(K.eta3 * 1.4426950408889634f), inv_kk = 1.0f / kk;
        const bool pair_ok = ((K.nel * K.nRs2) & 1) == 0;   // (cos, sin) gradient columns 8-byte aligned
        for (int t0 = 0; t0 < ntrip; t0 += 32) {
            const int t = t0 + lane;
            const bool active = t < ntrip;
            int j = 0, k = 1;
            float fj0 = 0.f, fj1 = 0.f, fj2 = 0.f;
            if (active) {
                decode_pair(t, nn, j, k);
                TripletGeom g;
                triplet_geometry(ws, A, j, k, K, g);
                const float Kk = K.w3 * g.T * g.R * g.Fij * g.Fik;
                const float a_cos = ZETA2 * Kk * g.cth, a_sin = ZETA2 * Kk * g.sth;
                const float rbar = 0.5f * (g.a + g.b);
                const float *gb = grow + pair_block(n_et[j], n_et[k], K);
                float Gc = 0.f, Gs = 0.f, Gcd = 0.f, Gsd = 0.f;   // sums of g radial and of g radial (rbar - Rs3)
                const float krbar = kk * rbar;
                if (pair_ok) {
                    const float2 *gb2 = reinterpret_cast<const float2 *>(gb);
                    float2 G2 = make_float2(0.f, 0.f), Gd2 = make_float2(0.f, 0.f);   // (cos, sin) columns side by side
#pragma unroll BWD_UNROLL
                    for (int l = 0; l < K.nRs3; ++l) {
                        const float d = fmaf(-kk, sRs3[l], krbar);
                        const float radial = ex2_fast(-d * d);
                        const float2 g2 = __fmul2_rn(gb2[l], make_float2(radial, radial));
                        G2 = __fadd2_rn(G2, g2);
                        Gd2 = __ffma2_rn(g2, make_float2(d, d), Gd2);
                    }
                    Gc = G2.x; Gs = G2.y;
                    Gcd = Gd2.x * inv_kk; Gsd = Gd2.y * inv_kk;
                } else {
                    for (int l = 0; l < K.nRs3; ++l) {
                        const float d = fmaf(-kk, sRs3[l], krbar);
                        const float radial = ex2_fast(-d * d);
                        const float gc = gb[2 * l] * radial, gs = gb[2 * l + 1] * radial;
                        Gc += gc;
                        Gs += gs;
                        Gcd = fmaf(gc, d, Gcd);
                        Gsd = fmaf(gs, d, Gsd);
                    }
                    Gcd *= inv_kk; Gsd *= inv_kk;
                }
                // the amplitudes are constant over the grid: d/d(rbar) of the radial factor, summed first
                const float Gr = -2.0f * K.eta3 * fmaf(a_cos, Gcd, a_sin * Gsd);
                // d/d(cos theta_i), d/dK
                float g_ci = ZETA2 * Kk * g.w * (Gc * g.sth - Gs * g.cth);
                const float g_K = ZETA2 * (Gc * g.cth + Gs * g.sth);
                const float w3FF = K.w3 * g.Fij * g.Fik;
                const float g_T = g_K * w3FF * g.R;
                const float g_R = g_K * w3FF * g.T;
                const float g_Fij = g_K * K.w3 * g.T * g.R * g.Fik;
                const float g_Fik = g_K * K.w3 * g.T * g.R * g.Fij;
                g_ci += g_T * 3.0f * g.cj * g.ck;
                const float g_cj = g_T * 3.0f * g.ci * g.ck;
                const float g_ck = g_T * 3.0f * g.ci * g.cj;
                const float inv_a = g.ia, inv_b = g.ib, inv_c = g.ic;
                const float dR = -K.d3 * g.R * g_R;
                float ga = dR * inv_a + g_Fij * g.dFij + 0.5f * Gr;
                float gbb = dR * inv_b + g_Fik * g.dFik + 0.5f * Gr;
                float gcc = dR * inv_c;
                // cosines as functions of the three distances (law of cosines)
                ga += g_ci * (inv_b - g.ci * inv_a) + g_cj * (inv_c - g.cj * inv_a) - g_ck * g.a * inv_b * inv_c;
                gbb += g_ci * (inv_a - g.ci * inv_b) - g_cj * g.b * inv_a * inv_c + g_ck * (inv_c - g.ck * inv_b);
                gcc += -g_ci * g.c * inv_a * inv_b + g_cj * (inv_a - g.cj * inv_c) + g_ck * (inv_b - g.ck * inv_c);
                const float eij0 = ws[F_DX * A + j] * inv_a, eij1 = ws[F_DY * A + j] * inv_a, eij2 = ws[F_DZ * A + j] * inv_a;
                const float eik0 = ws[F_DX * A + k] * inv_b, eik1 = ws[F_DY * A + k] * inv_b, eik2 = ws[F_DZ * A + k] * inv_b;
                fi0 += ga * eij0 + gbb * eik0;
                fi1 += ga * eij1 + gbb * eik1;
                fi2 += ga * eij2 + gbb * eik2;
                fj0 = -ga * eij0 + gcc * g.ejk[0];
                fj1 = -ga * eij1 + gcc * g.ejk[1];
                fj2 = -ga * eij2 + gcc * g.ejk[2];
                float *fk = force + 3 * n_idx[k];
                atomicAdd(fk + 0, -gbb * eik0 - gcc * g.ejk[0]);
                atomicAdd(fk + 1, -gbb * eik1 - gcc * g.ejk[1]);
                atomicAdd(fk + 2, -gbb * eik2 - gcc * g.ejk[2]);
            }
            __syncwarp();
            // segmented reduction over the run of lanes with equal j
            const bool head = active && (lane == 0 || k == j + 1);
            const unsigned heads = __ballot_sync(QMLB_FULL_MASK, head || !active);
            const unsigned above = lane == 31 ? 0u : (heads & ~((2u << lane) - 1u));
            const int last = above ? __ffs(above) - 2 : 31;
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                const float o0 = __shfl_down_sync(QMLB_FULL_MASK, fj0, off);
                const float o1 = __shfl_down_sync(QMLB_FULL_MASK, fj1, off);
                const float o2 = __shfl_down_sync(QMLB_FULL_MASK, fj2, off);
                if (lane + off <= last) {
                    fj0 += o0;
                    fj1 += o1;
                    fj2 += o2;
                }
            }
            if (head) {
                float *fj = force + 3 * n_idx[j];
                atomicAdd(fj + 0, fj0);   // uncontended: one head per j in this pass
                atomicAdd(fj + 1, fj1);
                atomicAdd(fj + 2, fj2);
            }
            __syncwarp();
        }
        fi0 = warp_sum(fi0);
        fi1 = warp_sum(fi1);
        fi2 = warp_sum(fi2);
        __syncwarp();
        if (lane == 0) {
            force[3 * i + 0] += fi0;
            force[3 * i + 1] += fi1;
            force[3 * i + 2] += fi2;
        }
        __syncwarp();
    }
    // an atom that found no row because the caller's row capacity was too small poisons its molecule: NaN energy and
    // gradient instead of a silently incomplete sum
    int lost = 0;
    if (row_of_slot)
        for (int a = threadIdx.x; a < natoms; a += blockDim.x) lost |= row_of_slot[(size_t)mol * A + a] == QMLB_ROW_OVERFLOW;
    lost = __syncthreads_or(lost);
    const float poison = lost ? __int_as_float(0x7fc00000) : 0.f;
    // fixed-order reduction over the warps' partial gradients
    for (int c = threadIdx.x; c < 3 * A; c += blockDim.x) {
        float s = 0.f;
        if (c < 3 * natoms) {
#pragma unroll
            for (int w = 0; w < FCHL_WARPS; ++w) s += sm[L.block_floats + (size_t)w * L.warp_floats + L.off_force + c];
            s += poison;
        }
        grad_X[(size_t)mol * 3 * A + c] = s;
    }
    if (atom_energy && mol_energy && warp == 0) {
        float e = 0.f;
        for (int a = lane; a < natoms; a += 32) {
            const long row = row_of_slot ? (long)row_of_slot[(size_t)mol * A + a] : (long)mol * A + a;
            if (row >= 0) e += atom_energy[row];
        }
        e = warp_sum(e) + poison;
        if (lane == 0) mol_energy[mol] = e;
    }
}

// ---- explicit Jacobian -----------------------------------------------------------------------------------------
// One warp per centre atom owns jac[m,i,:,:,:]; it zero-fills the slab and then adds term by term.  The same lane
// always updates the same column, so plain read-modify-write in global memory is race free.
__global__ void __launch_bounds__(FCHL_THREADS)
fchl_jacobian_kernel(const float *__restrict__ X, const float *__restrict__ Z, const int *__restrict__ counts,
                     const float *__restrict__ species, const float *__restrict__ Rs2, const float *__restrict__ Rs3,
                     const float *__restrict__ cell, const float *__restrict__ icell, FchlK K,
                     const int *__restrict__ row_of_slot, float *__restrict__ rep, float *__restrict__ jac) {
    extern __shared__ __align__(16) float sm[];
    const int mol = blockIdx.x, A = K.A;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const Layout L(A, K.nRs2, K.nRs3, K.repsize, false);
    const int natoms = stage_molecule(X, Z, counts, species, Rs2, Rs3, cell, icell, K, mol, sm);
    const float *sLog2 = sm + 4 * A + K.nRs2, *sInv2 = sLog2 + K.nRs2, *sRs3 = sInv2 + K.nRs2;
    const float *sLog2lo = sRs3 + K.nRs3 + 18;
    float *ws = sm + L.block_floats + (size_t)warp * L.warp_floats;
    float *acc = ws + L.off_row;
    const int *n_et = reinterpret_cast<const int *>(ws + F_ET * A);
    const int *n_idx = reinterpret_cast<const int *>(ws + F_IDX * A);
    const size_t R = K.repsize;

    for (int i = warp; i < A; i += FCHL_WARPS) {
        const long row = row_of_slot ? (long)row_of_slot[(size_t)mol * A + i] : (long)mol * A + i;
        if (row < 0) continue;
        float *dst = rep + (size_t)row * R;
        float *J = jac + (size_t)row * (size_t)A * 3 * R;  // [a][x][c]
        for (size_t c = lane; c < (size_t)A * 3 * R; c += 32) J[c] = 0.f;
        if (i >= natoms) {
            for (int c = lane; c < K.repsize; c += 32) dst[c] = 0.f;
            continue;
        }
        const int nn = build_neighbours(sm, ws, K, natoms, i, lane);
        for (int c = lane; c < K.repsize; c += 32) acc[c] = 0.f;
        __syncwarp();
        float *Ji = J + (size_t)i * 3 * R;

        for (int jn = 0; jn < nn; ++jn) {
            const float mu = ws[F_MU * A + jn], mulo = ws[F_MULO * A + jn], i2s = ws[F_I2S * A + jn];
            const float pref = ws[F_PREF * A + jn];
            const float fc = ws[F_FC * A + jn], dfc = ws[F_DFC * A + jn];
            const float c0 = ws[F_C0 * A + jn], c1 = ws[F_C1 * A + jn], c2 = ws[F_C2 * A + jn];
            const float inv_r = ws[F_IR * A + jn];
            const float e[3] = {ws[F_DX * A + jn] * inv_r, ws[F_DY * A + jn] * inv_r, ws[F_DZ * A + jn] * inv_r};
            const int col0 = n_et[jn] * K.nRs2;
            float *Jj = J + (size_t)n_idx[jn] * 3 * R;
            for (int z = lane; z < K.nRs2; z += 32) {
                const float t = (sLog2[z] - mu) + (sLog2lo[z] - mulo);
                const float base = pref * sInv2[z] * ex2_fast(-t * t * i2s);
                acc[col0 + z] += base * fc;
                const float dr = base * (fc * (c0 + t * (c1 + t * c2)) + dfc);
#pragma unroll
                for (int x = 0; x < 3; ++x) {
                    Ji[x * R + col0 + z] += dr * e[x];
                    Jj[x * R + col0 + z] -= dr * e[x];
                }
            }
        }

        const int ntrip = nn * (nn - 1) / 2;
        for (int t = 0; t < ntrip; ++t) {
            int j, k;
            decode_pair(t, nn, j, k);
            TripletGeom g;
            triplet_geometry(ws, A, j, k, K, g);
            const float Kk = K.w3 * g.T * g.R * g.Fij * g.Fik;
            const float rbar = 0.5f * (g.a + g.b);
            const int sidx = pair_block(n_et[j], n_et[k], K);
            const float inv_a = g.ia, inv_b = g.ib, inv_c = g.ic;
            // derivatives of ci, cj, ck, K with respect to (a, b, c)
            const float dci[3] = {inv_b - g.ci * inv_a, inv_a - g.ci * inv_b, -g.c * inv_a * inv_b};
            const float dcj[3] = {inv_c - g.cj * inv_a, -g.b * inv_a * inv_c, inv_a - g.cj * inv_c};
            const float dck[3] = {-g.a * inv_b * inv_c, inv_c - g.ck * inv_b, inv_b - g.ck * inv_c};
            const float w3FF = K.w3 * g.Fij * g.Fik;
            const float invr[3] = {inv_a, inv_b, inv_c};
            float dK[3], dcos[3], dsin[3];
#pragma unroll
            for (int q = 0; q < 3; ++q) {
                const float dT = 3.0f * (dci[q] * g.cj * g.ck + g.ci * dcj[q] * g.ck + g.ci * g.cj * dck[q]);
                dK[q] = w3FF * (g.R * dT - K.d3 * g.R * invr[q] * g.T);
                dcos[q] = g.sth * g.w * dci[q];
                dsin[q] = -g.cth * g.w * dci[q];
            }
            dK[0] += K.w3 * g.T * g.R * g.dFij * g.Fik;
            dK[1] += K.w3 * g.T * g.R * g.Fij * g.dFik;
            const float eij[3] = {ws[F_DX * A + j] * inv_a, ws[F_DY * A + j] * inv_a, ws[F_DZ * A + j] * inv_a};
            const float eik[3] = {ws[F_DX * A + k] * inv_b, ws[F_DY * A + k] * inv_b, ws[F_DZ * A + k] * inv_b};
            float *Jj = J + (size_t)n_idx[j] * 3 * R;
            float *Jk = J + (size_t)n_idx[k] * 3 * R;
            for (int l = lane; l < K.nRs3; l += 32) {
                const float d = rbar - sRs3[l];
                const float radial = expf(-K.eta3 * d * d);
                const float drad = -K.eta3 * d * radial;  // d radial / d a = d radial / d b (rbar = (a+b)/2)
                acc[sidx + 2 * l] += radial * ZETA2 * Kk * g.cth;
                acc[sidx + 2 * l + 1] += radial * ZETA2 * Kk * g.sth;
                float vc[3], vs[3];  // derivative of the two outputs with respect to (a, b, c)
#pragma unroll
                for (int q = 0; q < 3; ++q) {
                    const float dr = q < 2 ? drad : 0.f;
                    vc[q] = ZETA2 * (dr * Kk * g.cth + radial * (dK[q] * g.cth + Kk * dcos[q]));
                    vs[q] = ZETA2 * (dr * Kk * g.sth + radial * (dK[q] * g.sth + Kk * dsin[q]));
                }
                const int cc = sidx + 2 * l;
#pragma unroll
                for (int x = 0; x < 3; ++x) {
                    Ji[x * R + cc] += vc[0] * eij[x] + vc[1] * eik[x];
                    Ji[x * R + cc + 1] += vs[0] * eij[x] + vs[1] * eik[x];
                    Jj[x * R + cc] += -vc[0] * eij[x] + vc[2] * g.ejk[x];
                    Jj[x * R + cc + 1] += -vs[0] * eij[x] + vs[2] * g.ejk[x];
                    Jk[x * R + cc] += -vc[1] * eik[x] - vc[2] * g.ejk[x];
                    Jk[x * R + cc + 1] += -vs[1] * eik[x] - vs[2] * g.ejk[x];
                }
            }
        }
        __syncwarp();
        for (int c = lane; c < K.repsize; c += 32) dst[c] = acc[c];
        __syncwarp();
    }
}

// ---- element types / neighbour lists (API compatibility) -----------------------------------------------------
__global__ void element_types_kernel(const float *__restrict__ Z, const int *__restrict__ counts,
                                     const float *__restrict__ species, int nel, int nb, int A, int *__restrict__ out) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)nb * A) return;
    const int m = (int)(idx / A), a = (int)(idx % A);
    out[idx] = a < counts[m] ? species_index(Z[idx], species, nel) : 0;
}

template <bool WRITE_LIST>
__global__ void neighbours_kernel(const float *__restrict__ X, const int *__restrict__ counts, int nb, int A, float rcut2,
                                  const float *__restrict__ cell, const float *__restrict__ icell, int max_nb,
                                  int *__restrict__ out, int A_out) {
    // one warp per (molecule, atom); lanes scan the candidate neighbours with ballot compaction (ascending j)
    const int lane = threadIdx.x & 31;
    const size_t wid = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (wid >= (size_t)nb * A_out) return;
    const int m = (int)(wid / A_out), i = (int)(wid % A_out);
    int natoms = counts[m];
    natoms = natoms > A ? A : natoms;
    int *dst = WRITE_LIST ? out + wid * (size_t)max_nb : out + wid;
    if (WRITE_LIST)
        for (int c = lane; c < max_nb; c += 32) dst[c] = -1;
    if (i >= natoms) {
        if (!WRITE_LIST && lane == 0) *dst = 0;
        return;
    }
    __syncwarp();
    const float *xm = X + (size_t)m * A * 3;
    const float xi = xm[3 * i], yi = xm[3 * i + 1], zi = xm[3 * i + 2];
    float c9[18];
    const bool pbc = cell != nullptr;
    if (pbc)
        for (int q = 0; q < 18; ++q) c9[q] = q < 9 ? cell[(size_t)m * 9 + q] : icell[(size_t)m * 9 + q - 9];
    int nn = 0;
    for (int j0 = 0; j0 < natoms; j0 += 32) {
        const int j = j0 + lane;
        bool ok = false;
        if (j < natoms) {
            float dx = xi - xm[3 * j], dy = yi - xm[3 * j + 1], dz = zi - xm[3 * j + 2];
            if (pbc) min_image(dx, dy, dz, c9, c9 + 9);
            const float r2 = dx * dx + dy * dy + dz * dz;
            ok = r2 < rcut2 && r2 > 0.f;
        }
        const unsigned msk = __ballot_sync(QMLB_FULL_MASK, ok);
        if (WRITE_LIST && ok) {
            const int pos = nn + __popc(msk & ((1u << lane) - 1u));
            if (pos < max_nb) dst[pos] = j;
        }
        nn += __popc(msk);
    }
    if (!WRITE_LIST && lane == 0) *dst = nn;
}

int make_K(const qmlb_fchl_params *p, int nb, int A, const float *cell, const float *inv_cell, FchlK &K) {
    QMLB_REQUIRE(p && p->species && p->Rs2 && p->Rs3, "fchl19: null parameter block or grids");
    QMLB_REQUIRE(p->nspecies > 0 && p->nRs2 > 0 && p->nRs3 > 0, "fchl19: nspecies, nRs2 and nRs3 must be positive");
    QMLB_REQUIRE(nb >= 0 && A > 0, "fchl19: bad batch shape nb=%d A=%d", nb, A);
    QMLB_REQUIRE((cell == nullptr) == (inv_cell == nullptr), "fchl19: cell and inv_cell must be given together");
    QMLB_REQUIRE(p->rcut > 0.f, "fchl19: rcut must be positive");
    K.nb = nb;
    K.A = A;
    K.nel = p->nspecies;
    K.nRs2 = p->nRs2;
    K.nRs3 = p->nRs3;
    K.repsize = qmlb_fchl19_repsize(p->nspecies, p->nRs2, p->nRs3);
    K.pbc = cell != nullptr;
    K.eta2 = p->eta2;
    K.eta3 = p->eta3;
    K.d2 = p->two_body_decay;
    K.w3 = p->three_body_weight;
    K.d3 = p->three_body_decay;
    K.rcut = p->rcut;
    return QMLB_OK;
}

}  // namespace

extern "C" int qmlb_fchl19_repsize(int nspecies, int nRs2, int nRs3) {
    return nspecies * nRs2 + nspecies * (nspecies + 1) * nRs3;
}

extern "C" int qmlb_fchl19_forward(const float *X, const float *Z, const int *atom_counts, int nb, int A,
                                   const qmlb_fchl_params *p, const float *cell, const float *inv_cell,
                                   const int *row_of_slot, float *rep, qmlb_stream_t stream) {
    FchlK K;
    if (int rc = make_K(p, nb, A, cell, inv_cell, K)) return rc;
    QMLB_REQUIRE(X && Z && atom_counts && rep, "qmlb_fchl19_forward: null tensor");
    if (nb == 0) return QMLB_OK;
    const Layout L(A, K.nRs2, K.nRs3, K.repsize, false);
    if (int rc = qmlb::ensure_smem(fchl_forward_kernel, L.bytes(), "qmlb_fchl19_forward")) return rc;
    fchl_forward_kernel<<<nb, FCHL_THREADS, L.bytes(), qmlb::as_stream(stream)>>>(
        X, Z, atom_counts, p->species, p->Rs2, p->Rs3, cell, inv_cell, K, row_of_slot, rep);
    return qmlb::check_launch("qmlb_fchl19_forward");
}

extern "C" int qmlb_fchl19_backward(const float *X, const float *Z, const int *atom_counts, int nb, int A,
                                    const qmlb_fchl_params *p, const float *cell, const float *inv_cell,
                                    const int *row_of_slot, const float *grad_rep, float *grad_X,
                                    const float *atom_energy, float *mol_energy, qmlb_stream_t stream) {
    FchlK K;
    if (int rc = make_K(p, nb, A, cell, inv_cell, K)) return rc;
    QMLB_REQUIRE(X && Z && atom_counts && grad_rep && grad_X, "qmlb_fchl19_backward: null tensor");
    if (nb == 0) return QMLB_OK;
    const Layout L(A, K.nRs2, K.nRs3, K.repsize, true);
    if (int rc = qmlb::ensure_smem(fchl_backward_kernel, L.bytes(), "qmlb_fchl19_backward")) return rc;
    fchl_backward_kernel<<<nb, FCHL_THREADS, L.bytes(), qmlb::as_stream(stream)>>>(
        X, Z, atom_counts, p->species, p->Rs2, p->Rs3, cell, inv_cell, K, row_of_slot, grad_rep, grad_X, atom_energy,
        mol_energy);
    return qmlb::check_launch("qmlb_fchl19_backward");
}

extern "C" int qmlb_fchl19_forward_jacobian(const float *X, const float *Z, const int *atom_counts, int nb, int A,
                                            const qmlb_fchl_params *p, const float *cell, const float *inv_cell,
                                            const int *row_of_slot, float *rep, float *jac, qmlb_stream_t stream) {
    FchlK K;
    if (int rc = make_K(p, nb, A, cell, inv_cell, K)) return rc;
    QMLB_REQUIRE(X && Z && atom_counts && rep && jac, "qmlb_fchl19_forward_jacobian: null tensor");
    if (nb == 0) return QMLB_OK;
    const Layout L(A, K.nRs2, K.nRs3, K.repsize, false);
    if (int rc = qmlb::ensure_smem(fchl_jacobian_kernel, L.bytes(), "qmlb_fchl19_forward_jacobian")) return rc;
    fchl_jacobian_kernel<<<nb, FCHL_THREADS, L.bytes(), qmlb::as_stream(stream)>>>(
        X, Z, atom_counts, p->species, p->Rs2, p->Rs3, cell, inv_cell, K, row_of_slot, rep, jac);
    return qmlb::check_launch("qmlb_fchl19_forward_jacobian");
}

extern "C" int qmlb_element_types(const float *Z, const int *atom_counts, const float *species, int nspecies, int nb,
                                  int A, int *element_types, qmlb_stream_t stream) {
    QMLB_REQUIRE(Z && atom_counts && species && element_types, "qmlb_element_types: null tensor");
    QMLB_REQUIRE(nspecies > 0 && nb >= 0 && A > 0, "qmlb_element_types: bad sizes");
    if (nb == 0) return QMLB_OK;
    const size_t n = (size_t)nb * A;
    element_types_kernel<<<(unsigned)((n + 255) / 256), 256, 0, qmlb::as_stream(stream)>>>(Z, atom_counts, species,
                                                                                          nspecies, nb, A, element_types);
    return qmlb::check_launch("qmlb_element_types");
}

extern "C" int qmlb_num_neighbours(const float *X, const int *atom_counts, int nb, int A, float rcut, const float *cell,
                                   const float *inv_cell, int *num_neighbours, int A_out, qmlb_stream_t stream) {
    QMLB_REQUIRE(X && atom_counts && num_neighbours, "qmlb_num_neighbours: null tensor");
    QMLB_REQUIRE(nb >= 0 && A > 0 && A_out > 0 && A_out <= A, "qmlb_num_neighbours: bad sizes");
    QMLB_REQUIRE((cell == nullptr) == (inv_cell == nullptr), "qmlb_num_neighbours: cell and inv_cell go together");
    if (nb == 0) return QMLB_OK;
    const size_t warps = (size_t)nb * A_out;
    neighbours_kernel<false><<<(unsigned)((warps + 7) / 8), 256, 0, qmlb::as_stream(stream)>>>(
        X, atom_counts, nb, A, rcut * rcut, cell, inv_cell, 0, num_neighbours, A_out);
    return qmlb::check_launch("qmlb_num_neighbours");
}

extern "C" int qmlb_neighbour_list(const float *X, const int *atom_counts, int nb, int A, float rcut, const float *cell,
                                   const float *inv_cell, int max_neighbours, int *neighbour_list, int A_out,
                                   qmlb_stream_t stream) {
    QMLB_REQUIRE(X && atom_counts && neighbour_list, "qmlb_neighbour_list: null tensor");
    QMLB_REQUIRE(nb >= 0 && A > 0 && A_out > 0 && A_out <= A && max_neighbours >= 0, "qmlb_neighbour_list: bad sizes");
    QMLB_REQUIRE((cell == nullptr) == (inv_cell == nullptr), "qmlb_neighbour_list: cell and inv_cell go together");
    if (nb == 0 || max_neighbours == 0) return QMLB_OK;
    const size_t warps = (size_t)nb * A_out;
    neighbours_kernel<true><<<(unsigned)((warps + 7) / 8), 256, 0, qmlb::as_stream(stream)>>>(
        X, atom_counts, nb, A, rcut * rcut, cell, inv_cell, max_neighbours, neighbour_list, A_out);
    return qmlb::check_launch("qmlb_neighbour_list");
}
