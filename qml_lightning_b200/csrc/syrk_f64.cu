// Float64 normal-equation accumulation  ZTZ += M^T M  (row-major upper triangle) and  ZTy += M^T y  for a row block
// M f64[rows, F] of one training batch, hand-written for sm_100a.
//
// Upstream: torch.matmul(Ztrain.T, Ztrain) and torch.matmul(Ztrain.T, targets) in build_Z_components
// (models/kernel.py:172-192), a full float64 GEMM per batch.  Float64 has no tcgen05 kind, so the product runs on
// the double-precision tensor-core path mma.sync.m8n8k4.f64: one block owns a 128 x 128 tile of the upper triangle,
// eight warps hold 32 x 64 accumulators each, and the two 128-column panels of M stream through a four-stage
// cp.async ring in slices of 16 rows.  Tiles below the diagonal are never computed (half the flops of the upstream
// product); tiles are numbered band by band so that blocks running at the same time share their panels in L2.
#include <stdlib.h>

#include "common.cuh"

namespace {

constexpr int BN = 128;
constexpr int LD = BN + 4;                       // row stride in doubles: (4k + m) mod 16 distinct over a half warp
constexpr int BAND = 8;                          // tile rows per band

__device__ __forceinline__ void cp_async16(void *dst, const void *src, bool valid) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void cp_async8(void *dst, const void *src, bool valid) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    const int bytes = valid ? 8 : 0;
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;" ::"r"(d), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N)); }

__device__ __forceinline__ void dmma(double &d0, double &d1, double a, double b) {
    asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0,%1}, {%2}, {%3}, {%0,%1};"
                 : "+d"(d0), "+d"(d1)
                 : "d"(a), "d"(b));
}

// Linear tile number -> (I, J), I <= J.  Tile rows are taken in bands of BAND; inside a band the tiles are ordered by
// column J, so consecutive blocks share one column panel and the few row panels of the band.
__device__ __forceinline__ void decode_tile(long t, int nt, int &I, int &J) {
    int i0 = 0;
    for (;;) {
        const int h = min(BAND, nt - i0);
        const long tri = (long)h * (h + 1) / 2;
        const long cnt = tri + (long)h * (nt - i0 - h);
        if (t < cnt) {
            if (t < tri) {
                int c = 0;
                while ((long)(c + 1) * (c + 2) / 2 <= t) ++c;     // column c of the band's triangle holds c+1 tiles
                J = i0 + c;
                I = i0 + (int)(t - (long)c * (c + 1) / 2);
            } else {
                const long r = t - tri;
                J = i0 + h + (int)(r / h);
                I = i0 + (int)(r % h);
            }
            return;
        }
        t -= cnt;
        i0 += h;
    }
}

// Loads rows [r0, r0+BK) of the two panels (columns I*BM.. and J*BN..) into one stage; out-of-range parts are zero.
// m16n8k8: A 16x8 row-major (a0..a3: row = lane/4 + 8*(i&1), k = lane%4 + 4*(i>>1)), B 8x8 (b0,b1: k = lane%4 + 4*i,
// n = lane/4), C 16x8 (c0,c1: row lane/4, cols 2*(lane%4)+{0,1}; c2,c3: row + 8).
__device__ __forceinline__ void dmma16x8x8(double (&c)[4], const double (&a)[4], const double (&b)[2]) {
    asm volatile("mma.sync.aligned.m16n8k8.row.col.f64.f64.f64.f64 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+d"(c[0]), "+d"(c[1]), "+d"(c[2]), "+d"(c[3])
                 : "d"(a[0]), "d"(a[1]), "d"(a[2]), "d"(a[3]), "d"(b[0]), "d"(b[1]));
}

// m16n8k16: as m16n8k8 with a0..a7 (k = lane%4 + 4*(i>>1)) and b0..b3 (k = lane%4 + 4*i).
__device__ __forceinline__ void dmma16x8x16(double (&c)[4], const double (&a)[8], const double (&b)[4]) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f64.f64.f64.f64 {%0,%1,%2,%3}, {%4,%5,%6,%7,%8,%9,%10,%11}, {%12,%13,%14,%15}, {%0,%1,%2,%3};"
                 : "+d"(c[0]), "+d"(c[1]), "+d"(c[2]), "+d"(c[3])
                 : "d"(a[0]), "d"(a[1]), "d"(a[2]), "d"(a[3]), "d"(a[4]), "d"(a[5]), "d"(a[6]), "d"(a[7]), "d"(b[0]), "d"(b[1]),
                   "d"(b[2]), "d"(b[3]));
}

template <bool VEC16, int BK, int WIDTH, int THREADS>
__device__ __forceinline__ void load_panel(double *dst, const double *__restrict__ M, int rows, int F, int r0, int c0) {
    constexpr int W = VEC16 ? 2 : 1;                       // doubles per copy
    constexpr int PER_ROW = WIDTH / W;
    constexpr int COPIES = BK * PER_ROW;
#pragma unroll
    for (int q = 0; q < COPIES / THREADS; ++q) {
        const int idx = q * THREADS + threadIdx.x;
        const int r = idx / PER_ROW, c = (idx % PER_ROW) * W;
        const bool ok = r0 + r < rows && c0 + c + W <= F;
        const double *src = M + (ok ? (size_t)(r0 + r) * F + c0 + c : 0);
        if (VEC16) cp_async16(dst + r * LD + c, src, ok);
        else cp_async8(dst + r * LD + c, src, ok);
    }
}

template <bool VEC16, int BK, int BM, int THREADS>
__device__ __forceinline__ void load_stage(double *stage, const double *__restrict__ M, int rows, int F, int r0, int ci, int cj) {
    load_panel<VEC16, BK, BM, THREADS>(stage, M, rows, F, r0, ci);
    load_panel<VEC16, BK, BN, THREADS>(stage + BK * LD, M, rows, F, r0, cj);
}

template <bool VEC16, int BK, int STAGES, int SHAPE, int BM, int WTN>
__global__ void __launch_bounds__(BM / 32 * (BN / WTN) * 32, 128 / BM)
syrk_f64_kernel(const double *__restrict__ M, int rows, int F, double *__restrict__ C, int nt, int c_vec) {
    constexpr int STAGE_DOUBLES = 2 * BK * LD;
    constexpr int THREADS = BM / 32 * (BN / WTN) * 32, WM = BM / 32, NT8 = WTN / 8;
    extern __shared__ __align__(16) double smem[];
    int I, J;
    decode_tile(blockIdx.x / (128 / BM), nt, I, J);
    const int ci = I * 128 + (BM == 64 ? (int)(blockIdx.x & 1) * 64 : 0), cj = J * BN;
    if (ci >= F) return;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int wm = warp % WM, wn = warp / WM;              // WM x (BN / WTN) warps, 32 x WTN each
    const int lk = lane & 3, lm = lane >> 2;

    double acc[4][NT8][2];
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < NT8; ++b) acc[a][b][0] = acc[a][b][1] = 0.0;

    const int nk = (rows + BK - 1) / BK;
#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) {
        if (s < nk) load_stage<VEC16, BK, BM, THREADS>(smem + s * STAGE_DOUBLES, M, rows, F, s * BK, ci, cj);
        cp_async_commit();
    }
    for (int kt = 0; kt < nk; ++kt) {
        cp_async_wait<STAGES - 2>();
        __syncthreads();
        const int nxt = kt + STAGES - 1;
        if (nxt < nk) load_stage<VEC16, BK, BM, THREADS>(smem + (nxt % STAGES) * STAGE_DOUBLES, M, rows, F, nxt * BK, ci, cj);
        cp_async_commit();
        const double *As = smem + (kt % STAGES) * STAGE_DOUBLES + wm * 32 + lm;
        const double *Bs = smem + (kt % STAGES) * STAGE_DOUBLES + BK * LD + wn * WTN + lm;
        if (SHAPE == 4) {
#pragma unroll
            for (int kk = 0; kk < BK / 4; ++kk) {
                double a[4], b[NT8];
#pragma unroll
                for (int mt = 0; mt < 4; ++mt) a[mt] = As[(kk * 4 + lk) * LD + mt * 8];
#pragma unroll
                for (int nt8 = 0; nt8 < NT8; ++nt8) b[nt8] = Bs[(kk * 4 + lk) * LD + nt8 * 8];
#pragma unroll
                for (int mt = 0; mt < 4; ++mt)
#pragma unroll
                    for (int nt8 = 0; nt8 < NT8; ++nt8) dmma(acc[mt][nt8][0], acc[mt][nt8][1], a[mt], b[nt8]);
            }
        } else if (SHAPE == 16) {
#pragma unroll
            for (int kk = 0; kk < BK / 16; ++kk) {
                double a[2][8];
#pragma unroll
                for (int p = 0; p < 2; ++p)
#pragma unroll
                    for (int q = 0; q < 8; ++q) a[p][q] = As[(kk * 16 + lk + 4 * (q >> 1)) * LD + p * 16 + 8 * (q & 1)];
#pragma unroll
                for (int nt8 = 0; nt8 < NT8; ++nt8) {
                    double b[4];
#pragma unroll
                    for (int q = 0; q < 4; ++q) b[q] = Bs[(kk * 16 + lk + 4 * q) * LD + nt8 * 8];
#pragma unroll
                    for (int p = 0; p < 2; ++p) {
                        double c[4] = {acc[2 * p][nt8][0], acc[2 * p][nt8][1], acc[2 * p + 1][nt8][0], acc[2 * p + 1][nt8][1]};
                        dmma16x8x16(c, a[p], b);
                        acc[2 * p][nt8][0] = c[0]; acc[2 * p][nt8][1] = c[1];
                        acc[2 * p + 1][nt8][0] = c[2]; acc[2 * p + 1][nt8][1] = c[3];
                    }
                }
            }
        } else {
            // m16n8k8: accumulators of row tiles (2p, 2p+1) form one 16-row tile: {acc[2p][n][0..1], acc[2p+1][n][0..1]}
#pragma unroll
            for (int kk = 0; kk < BK / 8; ++kk) {
                double a[2][4], b[NT8][2];
#pragma unroll
                for (int p = 0; p < 2; ++p)
#pragma unroll
                    for (int q = 0; q < 4; ++q) a[p][q] = As[(kk * 8 + lk + 4 * (q >> 1)) * LD + p * 16 + 8 * (q & 1)];
#pragma unroll
                for (int nt8 = 0; nt8 < NT8; ++nt8)
#pragma unroll
                    for (int q = 0; q < 2; ++q) b[nt8][q] = Bs[(kk * 8 + lk + 4 * q) * LD + nt8 * 8];
#pragma unroll
                for (int p = 0; p < 2; ++p)
#pragma unroll
                    for (int nt8 = 0; nt8 < NT8; ++nt8) {
                        double c[4] = {acc[2 * p][nt8][0], acc[2 * p][nt8][1], acc[2 * p + 1][nt8][0], acc[2 * p + 1][nt8][1]};
                        dmma16x8x8(c, a[p], b[nt8]);
                        acc[2 * p][nt8][0] = c[0]; acc[2 * p][nt8][1] = c[1];
                        acc[2 * p + 1][nt8][0] = c[2]; acc[2 * p + 1][nt8][1] = c[3];
                    }
            }
        }
    }
    cp_async_wait<0>();

    // C[i][j] += acc for j >= i (row-major upper triangle); every element belongs to exactly one thread
    const bool interior = c_vec && J > I && ci + BM <= F && cj + BN <= F;
#pragma unroll
    for (int mt = 0; mt < 4; ++mt) {
        const int i = ci + wm * 32 + mt * 8 + lm;
#pragma unroll
        for (int nt8 = 0; nt8 < NT8; ++nt8) {
            const int j = cj + wn * WTN + nt8 * 8 + lk * 2;
            if (interior) {
                double2 *p = reinterpret_cast<double2 *>(C + (size_t)i * F + j);
                double2 v = *p;
                v.x += acc[mt][nt8][0];
                v.y += acc[mt][nt8][1];
                *p = v;
            } else if (i < F) {
                if (j < F && j >= i) C[(size_t)i * F + j] += acc[mt][nt8][0];
                if (j + 1 < F && j + 1 >= i) C[(size_t)i * F + j + 1] += acc[mt][nt8][1];
            }
        }
    }
}

// ---- decoupled variant --------------------------------------------------------------------------------------------
// The kernel above keeps its warps in lock step: one __syncthreads per 16-row slice drains the DMMA pipe of all of them
// at once (measured: 0.87 of the cuBLAS DSYRK rate with one block per SM, 0.93 with two).  Here a 64 x 128 tile belongs
// to four warps that are only coupled through mbarriers: `full[s]` completes when the cp.async copies of all threads
// for stage s have landed (cp.async.mbarrier.arrive.noinc), `empty[s]` when all four warps have read it.  A slice is
// requested two iterations ahead into the stage that was read two iterations ago, so a warp may run a whole slice
// ahead of the slowest one before it has to wait, and two such blocks share an SM.  Every wait is bounded; a block
// that gives up skips its update and counts the event.
constexpr int A_BM = 64, A_BK = 16, A_STAGES = 4, A_DIST = 2, A_THREADS = 128, A_WARPS = 4;
constexpr int A_LDA = A_BM + 4;                          // same bank argument as LD
constexpr int A_STAGE_DOUBLES = A_BK * (A_LDA + LD);
constexpr size_t A_SMEM = sizeof(double) * A_STAGES * A_STAGE_DOUBLES;
constexpr int SYRK_WAIT_LIMIT = 1 << 24;
__device__ int g_syrk_timeouts = 0;

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_on_copies(uint32_t bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (int it = 0; it < SYRK_WAIT_LIMIT; ++it) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(bar), "r"(parity)
            : "memory");
        if (ok) return true;
    }
    return false;
}

template <bool VEC16>
__device__ __forceinline__ void load_stage_async(double *stage, const double *__restrict__ M, int rows, int F, int r0, int ci,
                                                 int cj) {
    constexpr int W = VEC16 ? 2 : 1;
#pragma unroll
    for (int q = 0; q < A_BK * (A_BM / W) / A_THREADS; ++q) {
        const int idx = q * A_THREADS + threadIdx.x;
        const int r = idx / (A_BM / W), c = (idx % (A_BM / W)) * W;
        const bool ok = r0 + r < rows && ci + c + W <= F;
        const double *src = M + (ok ? (size_t)(r0 + r) * F + ci + c : 0);
        if (VEC16) cp_async16(stage + r * A_LDA + c, src, ok);
        else cp_async8(stage + r * A_LDA + c, src, ok);
    }
    double *sb = stage + A_BK * A_LDA;
#pragma unroll
    for (int q = 0; q < A_BK * (BN / W) / A_THREADS; ++q) {
        const int idx = q * A_THREADS + threadIdx.x;
        const int r = idx / (BN / W), c = (idx % (BN / W)) * W;
        const bool ok = r0 + r < rows && cj + c + W <= F;
        const double *src = M + (ok ? (size_t)(r0 + r) * F + cj + c : 0);
        if (VEC16) cp_async16(sb + r * LD + c, src, ok);
        else cp_async8(sb + r * LD + c, src, ok);
    }
}

template <bool VEC16>
__global__ void __launch_bounds__(A_THREADS, 2)
syrk_f64_async_kernel(const double *__restrict__ M, int rows, int F, double *__restrict__ C, int nt, int c_vec) {
    extern __shared__ __align__(16) double smem[];
    __shared__ __align__(8) unsigned long long bars[2 * A_STAGES];
    int I, J;
    decode_tile(blockIdx.x >> 1, nt, I, J);
    const int ci = I * 128 + (int)(blockIdx.x & 1) * A_BM, cj = J * BN;
    if (ci >= F) return;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int wm = warp & 1, wn = warp >> 1;               // 2 x 2 warps, 32 x 64 each
    const int lk = lane & 3, lm = lane >> 2;
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + A_STAGES);
    if (threadIdx.x == 0) {
        for (int s = 0; s < A_STAGES; ++s) {
            mbar_init(full0 + 8 * s, A_THREADS);
            mbar_init(empty0 + 8 * s, A_WARPS);
        }
    }
    __syncthreads();

    double acc[4][8][2];
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < 8; ++b) acc[a][b][0] = acc[a][b][1] = 0.0;

    const int nk = (rows + A_BK - 1) / A_BK;
    for (int t = 0; t < A_DIST && t < nk; ++t) {
        load_stage_async<VEC16>(smem + t * A_STAGE_DOUBLES, M, rows, F, t * A_BK, ci, cj);
        mbar_arrive_on_copies(full0 + 8 * t);
    }
    bool ok = true;
    for (int kt = 0; kt < nk; ++kt) {
        const int nxt = kt + A_DIST;
        if (nxt < nk) {
            const int ns = nxt % A_STAGES, fill = nxt / A_STAGES;
            if (fill >= 1) ok = mbar_wait(empty0 + 8 * ns, (uint32_t)(fill - 1) & 1u);
            ok = __all_sync(QMLB_FULL_MASK, ok);
            if (!ok) break;
            load_stage_async<VEC16>(smem + ns * A_STAGE_DOUBLES, M, rows, F, nxt * A_BK, ci, cj);
            mbar_arrive_on_copies(full0 + 8 * ns);
        }
        const int cs = kt % A_STAGES;
        ok = __all_sync(QMLB_FULL_MASK, mbar_wait(full0 + 8 * cs, (uint32_t)(kt / A_STAGES) & 1u));
        if (!ok) break;
        const double *As = smem + cs * A_STAGE_DOUBLES + wm * 32 + lm;
        const double *Bs = smem + cs * A_STAGE_DOUBLES + A_BK * A_LDA + wn * 64 + lm;
#pragma unroll
        for (int kk = 0; kk < A_BK / 8; ++kk) {
            double a[2][4], b[8][2];
#pragma unroll
            for (int p = 0; p < 2; ++p)
#pragma unroll
                for (int q = 0; q < 4; ++q) a[p][q] = As[(kk * 8 + lk + 4 * (q >> 1)) * A_LDA + p * 16 + 8 * (q & 1)];
#pragma unroll
            for (int n8 = 0; n8 < 8; ++n8)
#pragma unroll
                for (int q = 0; q < 2; ++q) b[n8][q] = Bs[(kk * 8 + lk + 4 * q) * LD + n8 * 8];
#pragma unroll
            for (int p = 0; p < 2; ++p)
#pragma unroll
                for (int n8 = 0; n8 < 8; ++n8) {
                    double c[4] = {acc[2 * p][n8][0], acc[2 * p][n8][1], acc[2 * p + 1][n8][0], acc[2 * p + 1][n8][1]};
                    dmma16x8x8(c, a[p], b[n8]);
                    acc[2 * p][n8][0] = c[0]; acc[2 * p][n8][1] = c[1];
                    acc[2 * p + 1][n8][0] = c[2]; acc[2 * p + 1][n8][1] = c[3];
                }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty0 + 8 * cs);
    }
    cp_async_wait<0>();                                    // nothing of this thread is in flight when the block leaves
    if (!ok) {
        if (lane == 0) atomicAdd(&g_syrk_timeouts, 1);
        return;
    }
    const bool interior = c_vec && J > I && ci + A_BM <= F && cj + BN <= F;
#pragma unroll
    for (int mt = 0; mt < 4; ++mt) {
        const int i = ci + wm * 32 + mt * 8 + lm;
#pragma unroll
        for (int n8 = 0; n8 < 8; ++n8) {
            const int j = cj + wn * 64 + n8 * 8 + lk * 2;
            if (interior) {
                double2 *p = reinterpret_cast<double2 *>(C + (size_t)i * F + j);
                double2 v = *p;
                v.x += acc[mt][n8][0];
                v.y += acc[mt][n8][1];
                *p = v;
            } else if (i < F) {
                if (j < F && j >= i) C[(size_t)i * F + j] += acc[mt][n8][0];
                if (j + 1 < F && j + 1 >= i) C[(size_t)i * F + j + 1] += acc[mt][n8][1];
            }
        }
    }
}

// ZTy[f] += sum_r M[r][f] y[r]: columns across the threads (coalesced), the rows split over blockIdx.y, four independent
// partial sums per thread, one float64 atomic per (thread, row split).
constexpr int GEMV_SPLIT_ROWS = 128;
__global__ void __launch_bounds__(256)
gemv_t_kernel(const double *__restrict__ M, int rows, int F, const double *__restrict__ y, double *__restrict__ out) {
    const int f = blockIdx.x * blockDim.x + threadIdx.x;
    if (f >= F) return;
    const int r0 = blockIdx.y * GEMV_SPLIT_ROWS, r1 = min(rows, r0 + GEMV_SPLIT_ROWS);
    double s0 = 0.0, s1 = 0.0, s2 = 0.0, s3 = 0.0;
    int r = r0;
    for (; r + 3 < r1; r += 4) {
        s0 = fma(M[(size_t)r * F + f], y[r], s0);
        s1 = fma(M[(size_t)(r + 1) * F + f], y[r + 1], s1);
        s2 = fma(M[(size_t)(r + 2) * F + f], y[r + 2], s2);
        s3 = fma(M[(size_t)(r + 3) * F + f], y[r + 3], s3);
    }
    for (; r < r1; ++r) s0 = fma(M[(size_t)r * F + f], y[r], s0);
    atomicAdd(out + f, (s0 + s1) + (s2 + s3));
}

template <bool VEC16, int BK, int STAGES, int SHAPE, int BM = 128, int WTN = 64>
int launch_syrk(const double *M, int rows, int F, double *ZTZ, int nt, long tiles, int c_vec, cudaStream_t st) {
    constexpr size_t smem = sizeof(double) * STAGES * 2 * BK * LD;
    if (int rc = qmlb::ensure_smem(syrk_f64_kernel<VEC16, BK, STAGES, SHAPE, BM, WTN>, smem, "qmlb_syrk_f64")) return rc;
    syrk_f64_kernel<VEC16, BK, STAGES, SHAPE, BM, WTN><<<(unsigned)(tiles * (128 / BM)), BM / 32 * (BN / WTN) * 32, smem, st>>>(M, rows, F, ZTZ, nt, c_vec);
    return qmlb::check_launch("qmlb_syrk_f64");
}

}  // namespace

extern "C" int qmlb_syrk_f64(const double *M, int rows, int F, double *ZTZ, qmlb_stream_t stream) {
    QMLB_REQUIRE(M && ZTZ, "qmlb_syrk_f64: null tensor");
    QMLB_REQUIRE(rows >= 0 && F > 0, "qmlb_syrk_f64: bad sizes");
    if (rows == 0) return QMLB_OK;
    const int nt = (F + BN - 1) / BN;
    const long tiles = (long)nt * (nt + 1) / 2;
    QMLB_REQUIRE(tiles < (1L << 31), "qmlb_syrk_f64: too many features");
    const bool vec16 = (F % 2 == 0) && (((uintptr_t)M & 15) == 0);
    const int c_vec = (F % 2 == 0) && (((uintptr_t)ZTZ & 15) == 0);
    cudaStream_t st = qmlb::as_stream(stream);
    if (!vec16) return launch_syrk<false, 16, 4, 4>(M, rows, F, ZTZ, nt, tiles, c_vec, st);
    const char *v = getenv("QMLB_SYRK_VARIANT");
    const int variant = v ? atoi(v) : 0;
    switch (variant) {
        case 1: return launch_syrk<true, 32, 3, 4>(M, rows, F, ZTZ, nt, tiles, c_vec, st);
        case 2: return launch_syrk<true, 16, 4, 8>(M, rows, F, ZTZ, nt, tiles, c_vec, st);
        case 3: return launch_syrk<true, 32, 3, 8>(M, rows, F, ZTZ, nt, tiles, c_vec, st);
        case 4: return launch_syrk<true, 16, 3, 4, 64>(M, rows, F, ZTZ, nt, tiles, c_vec, st);
        case 5: return launch_syrk<true, 16, 3, 8, 64>(M, rows, F, ZTZ, nt, tiles, c_vec, st);
        case 6: return launch_syrk<true, 16, 3, 16, 64>(M, rows, F, ZTZ, nt, tiles, c_vec, st);
        case 7: return launch_syrk<true, 16, 4, 16, 128>(M, rows, F, ZTZ, nt, tiles, c_vec, st);
        case 9: return launch_syrk<true, 16, 3, 8, 64, 32>(M, rows, F, ZTZ, nt, tiles, c_vec, st);
        case 10: return launch_syrk<true, 16, 3, 4, 64, 32>(M, rows, F, ZTZ, nt, tiles, c_vec, st);
        case 11: return launch_syrk<true, 32, 3, 8, 64, 32>(M, rows, F, ZTZ, nt, tiles, c_vec, st);
        case 8: {
            if (int rc = qmlb::ensure_smem(syrk_f64_async_kernel<true>, A_SMEM, "qmlb_syrk_f64")) return rc;
            syrk_f64_async_kernel<true><<<(unsigned)(tiles * 2), A_THREADS, A_SMEM, st>>>(M, rows, F, ZTZ, nt, c_vec);
            return qmlb::check_launch("qmlb_syrk_f64");
        }
        case 12: return launch_syrk<true, 16, 4, 4>(M, rows, F, ZTZ, nt, tiles, c_vec, st);
        default: return launch_syrk<true, 16, 3, 8, 64>(M, rows, F, ZTZ, nt, tiles, c_vec, st);
    }
}

extern "C" int qmlb_gemv_t_f64(const double *M, int rows, int F, const double *y, double *ZTy, qmlb_stream_t stream) {
    QMLB_REQUIRE(M && y && ZTy, "qmlb_gemv_t_f64: null tensor");
    QMLB_REQUIRE(rows >= 0 && F > 0, "qmlb_gemv_t_f64: bad sizes");
    if (rows == 0) return QMLB_OK;
    dim3 grid((unsigned)((F + 255) / 256), (unsigned)((rows + GEMV_SPLIT_ROWS - 1) / GEMV_SPLIT_ROWS));
    QMLB_REQUIRE(grid.y < 65536, "qmlb_gemv_t_f64: too many rows per call");
    gemv_t_kernel<<<grid, 256, 0, qmlb::as_stream(stream)>>>(M, rows, F, y, ZTy);
    return qmlb::check_launch("qmlb_gemv_t_f64");
}
