// Float64 normal-equation accumulation  ZTZ += M^T M  (row-major upper triangle) and  ZTy += M^T y  for a row block
// M f64[rows, F] of one training batch, hand-written for sm_100a.
//
// Upstream: torch.matmul(Ztrain.T, Ztrain) and torch.matmul(Ztrain.T, targets) in build_Z_components
// (models/kernel.py:172-192), a full float64 GEMM per batch.  Float64 has no tcgen05 kind, so the product runs on
// the double-precision tensor-core path mma.sync.m8n8k4.f64.  The matrix is cut into 128 x 128 super-tiles of the
// upper triangle, numbered band by band so that blocks running at the same time share their panels of M in L2; a
// block owns a BM x BN part of one super-tile, its warps WTM x WTN accumulators each, and the two column panels of M
// stream through a cp.async ring in slices of BK rows.  Parts below the diagonal are never computed (half the flops
// of the upstream product).  The DMMA pipe needs about four resident warps per scheduler to stay busy, so the
// default is many small blocks (64 x 64, four warps, four blocks per SM) rather than a few large ones.
#include "common.cuh"

namespace {

constexpr int SUPER = 128;                       // super-tile edge
constexpr int BAND = 8;                          // super-tile rows per band

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

// A 8x4 row-major (a: row lane/4, k lane%4), B 4x8 (b: k lane%4, n lane/4), C 8x8 (c0,c1: row lane/4, cols 2*(lane%4)+{0,1}).
__device__ __forceinline__ void dmma(double &d0, double &d1, double a, double b) {
    asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0,%1}, {%2}, {%3}, {%0,%1};"
                 : "+d"(d0), "+d"(d1)
                 : "d"(a), "d"(b));
}

// Linear super-tile number -> (I, J), I <= J.  Rows are taken in bands of BAND; inside a band the tiles are ordered by
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

// Rows [r0, r0+BK) x columns [c0, c0+WIDTH) of M into a panel with row stride LDP; out-of-range parts become zero.
template <bool VEC16, int BK, int WIDTH, int LDP, int THREADS>
__device__ __forceinline__ void load_panel(double *dst, const double *__restrict__ M, int rows, int F, int r0, int c0) {
    constexpr int W = VEC16 ? 2 : 1;                       // doubles per copy
    constexpr int PER_ROW = WIDTH / W;
    constexpr int COPIES = BK * PER_ROW;
#pragma unroll
    for (int q = 0; q < (COPIES + THREADS - 1) / THREADS; ++q) {
        const int idx = q * THREADS + threadIdx.x;
        if (COPIES % THREADS != 0 && idx >= COPIES) break;
        const int r = idx / PER_ROW, c = (idx % PER_ROW) * W;
        const bool ok = r0 + r < rows && c0 + c + W <= F;
        const double *src = M + (ok ? (size_t)(r0 + r) * F + c0 + c : 0);
        if (VEC16) cp_async16(dst + r * LDP + c, src, ok);
        else cp_async8(dst + r * LDP + c, src, ok);
    }
}

// C[i][j] += sum_r P[r][i] Q[r][j] for P f64[rows, Fi], Q f64[rows, Fj], C f64[Fi, Fj].  UPPER: P == Q and only j >= i is
// computed and stored (the normal equations); otherwise the whole product (the general matmul_and_reduce form).
template <int BM, int BN, int WTM, int WTN, int BK, int STAGES, int MINBLOCKS, bool VEC16, bool UPPER>
__global__ void __launch_bounds__((BM / WTM) * (BN / WTN) * 32, MINBLOCKS)
syrk_f64_kernel(const double *__restrict__ P, const double *__restrict__ Q, int rows, int Fi, int Fj, double *__restrict__ C,
                int nt, int c_vec) {
    constexpr int THREADS = (BM / WTM) * (BN / WTN) * 32;
    constexpr int LDA = BM + 4, LDB = BN + 4;              // (4k + m) mod 16 distinct over a half warp: no bank conflicts
    constexpr int STAGE_DOUBLES = BK * (LDA + LDB);
    constexpr int SUB_M = SUPER / BM, SUB_N = SUPER / BN, MT = WTM / 8, NT = WTN / 8;
    extern __shared__ __align__(16) double smem[];
    int I, J;
    const int sub = blockIdx.x % (SUB_M * SUB_N);
    if (UPPER) {
        decode_tile(blockIdx.x / (SUB_M * SUB_N), nt, I, J);
    } else {                                               // nt super-tile rows; consecutive blocks share a column panel
        const long t = blockIdx.x / (SUB_M * SUB_N);
        I = (int)(t % nt);
        J = (int)(t / nt);
    }
    const int ci = I * SUPER + (sub / SUB_N) * BM, cj = J * SUPER + (sub % SUB_N) * BN;
    if (ci >= Fi || cj >= Fj || (UPPER && cj + BN <= ci)) return;   // outside the matrix or entirely below the diagonal
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int wm = warp % (BM / WTM), wn = warp / (BM / WTM);
    const int lk = lane & 3, lm = lane >> 2;

    double acc[MT][NT][2];
#pragma unroll
    for (int a = 0; a < MT; ++a)
#pragma unroll
        for (int b = 0; b < NT; ++b) acc[a][b][0] = acc[a][b][1] = 0.0;

    const int nk = (rows + BK - 1) / BK;
#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) {
        if (s < nk) {
            load_panel<VEC16, BK, BM, LDA, THREADS>(smem + s * STAGE_DOUBLES, P, rows, Fi, s * BK, ci);
            load_panel<VEC16, BK, BN, LDB, THREADS>(smem + s * STAGE_DOUBLES + BK * LDA, Q, rows, Fj, s * BK, cj);
        }
        cp_async_commit();
    }
    for (int kt = 0; kt < nk; ++kt) {
        cp_async_wait<STAGES - 2>();
        __syncthreads();
        const int nxt = kt + STAGES - 1;
        if (nxt < nk) {
            double *st = smem + (nxt % STAGES) * STAGE_DOUBLES;
            load_panel<VEC16, BK, BM, LDA, THREADS>(st, P, rows, Fi, nxt * BK, ci);
            load_panel<VEC16, BK, BN, LDB, THREADS>(st + BK * LDA, Q, rows, Fj, nxt * BK, cj);
        }
        cp_async_commit();
        const double *As = smem + (kt % STAGES) * STAGE_DOUBLES + wm * WTM + lm;
        const double *Bs = smem + (kt % STAGES) * STAGE_DOUBLES + BK * LDA + wn * WTN + lm;
#pragma unroll
        for (int kk = 0; kk < BK / 4; ++kk) {
            double a[MT], b[NT];
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) a[mt] = As[(kk * 4 + lk) * LDA + mt * 8];
#pragma unroll
            for (int n8 = 0; n8 < NT; ++n8) b[n8] = Bs[(kk * 4 + lk) * LDB + n8 * 8];
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int n8 = 0; n8 < NT; ++n8) dmma(acc[mt][n8][0], acc[mt][n8][1], a[mt], b[n8]);
        }
    }
    cp_async_wait<0>();

    // C[i][j] += acc for j >= i (row-major upper triangle); every element belongs to exactly one thread
    const bool interior = c_vec && (!UPPER || cj >= ci + BM) && ci + BM <= Fi && cj + BN <= Fj;
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
        const int i = ci + wm * WTM + mt * 8 + lm;
#pragma unroll
        for (int n8 = 0; n8 < NT; ++n8) {
            const int j = cj + wn * WTN + n8 * 8 + lk * 2;
            if (interior) {
                double2 *p = reinterpret_cast<double2 *>(C + (size_t)i * Fj + j);
                double2 v = *p;
                v.x += acc[mt][n8][0];
                v.y += acc[mt][n8][1];
                *p = v;
            } else if (i < Fi) {
                if (j < Fj && (!UPPER || j >= i)) C[(size_t)i * Fj + j] += acc[mt][n8][0];
                if (j + 1 < Fj && (!UPPER || j + 1 >= i)) C[(size_t)i * Fj + j + 1] += acc[mt][n8][1];
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

template <bool VEC16, bool UPPER>
int launch_product(const double *P, const double *Q, int rows, int Fi, int Fj, double *C, const char *who, cudaStream_t st) {
    // 64 x 64 blocks of four warps (32 x 32 each), 16-row slices, three stages, four blocks per SM.  Measured on a
    // 4096 x 16384 row block against cuBLAS DSYRK in the same process (35.8 TFLOP/s on the triangle): this shape 0.951;
    // 64 x 128 / 8 warps / 2 per SM 0.92; 128 x 128 / 8 warps / 1 per SM 0.87; 64 x 32 / 4 warps / 4 per SM 0.86;
    // m16n8k8 and m16n8k16 instruction shapes and an mbarrier-decoupled pipeline changed nothing.
    constexpr int BM = 64, BN = 64, WTM = 32, WTN = 32, BK = 16, STAGES = 3, MINB = 4;
    constexpr size_t smem = sizeof(double) * STAGES * BK * (BM + 4 + BN + 4);
    constexpr int threads = (BM / WTM) * (BN / WTN) * 32, subs = (SUPER / BM) * (SUPER / BN);
    const int nti = (Fi + SUPER - 1) / SUPER, ntj = (Fj + SUPER - 1) / SUPER;
    const long tiles = UPPER ? (long)nti * (nti + 1) / 2 : (long)nti * ntj;
    if (tiles * subs >= (1L << 31)) {
        qmlb::set_error("%s: too many features", who);
        return QMLB_ERR_INVALID;
    }
    const int c_vec = (Fj % 2 == 0) && (((uintptr_t)C & 15) == 0);
    auto kernel = syrk_f64_kernel<BM, BN, WTM, WTN, BK, STAGES, MINB, VEC16, UPPER>;
    if (int rc = qmlb::ensure_smem(kernel, smem, who)) return rc;
    kernel<<<(unsigned)(tiles * subs), threads, smem, st>>>(P, Q, rows, Fi, Fj, C, nti, c_vec);
    return qmlb::check_launch(who);
}

}  // namespace

extern "C" int qmlb_syrk_f64(const double *M, int rows, int F, double *ZTZ, qmlb_stream_t stream) {
    QMLB_REQUIRE(M && ZTZ, "qmlb_syrk_f64: null tensor");
    QMLB_REQUIRE(rows >= 0 && F > 0, "qmlb_syrk_f64: bad sizes");
    if (rows == 0) return QMLB_OK;
    const bool vec16 = (F % 2 == 0) && (((uintptr_t)M & 15) == 0);
    cudaStream_t st = qmlb::as_stream(stream);
    if (vec16) return launch_product<true, true>(M, M, rows, F, F, ZTZ, "qmlb_syrk_f64", st);
    return launch_product<false, true>(M, M, rows, F, F, ZTZ, "qmlb_syrk_f64", st);
}

extern "C" int qmlb_gemm_tn_f64(const double *P, const double *Q, int rows, int Fi, int Fj, double *C, qmlb_stream_t stream) {
    QMLB_REQUIRE(P && Q && C, "qmlb_gemm_tn_f64: null tensor");
    QMLB_REQUIRE(rows >= 0 && Fi > 0 && Fj > 0, "qmlb_gemm_tn_f64: bad sizes");
    if (rows == 0) return QMLB_OK;
    const bool vec16 = (Fi % 2 == 0) && (Fj % 2 == 0) && ((((uintptr_t)P | (uintptr_t)Q) & 15) == 0);
    cudaStream_t st = qmlb::as_stream(stream);
    if (vec16) return launch_product<true, false>(P, Q, rows, Fi, Fj, C, "qmlb_gemm_tn_f64", st);
    return launch_product<false, false>(P, Q, rows, Fi, Fj, C, "qmlb_gemm_tn_f64", st);
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
