// Per-element PCA projection on element-grouped rows:  out[r,:] = in[r,:] . P_e  (or . P_e^T for the backward).
//
// Upstream gathers the rows of one element with a boolean mask and calls torch.matmul per element
// (representations/dimensionality_reduction.py:47-58, models/hadamard_features.py:99-111).  Here the rows are
// already grouped by element and padded to QMLB_ROW_TILE, so one launch covers all elements: a 64-row tile
// belongs to exactly one element and picks its projection matrix from group_start.
//
// fp32 FFMA tiles (64x64x16, 4x4 per thread).  The product feeds cos() with arguments of order 10, so single-pass
// TF32 would not hold the 1e-5 energy tolerance; full fp32 accumulation is used.
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, PAD = 4;  // BM divides QMLB_ROW_TILE

template <bool TRANS>
__global__ void __launch_bounds__(256)
pca_gemm_kernel(const float *__restrict__ in, const float *__restrict__ P, const int *__restrict__ group_start, int nel,
                int K, int Nout, int npcas, size_t p_stride, int sub_rows, float *__restrict__ out) {
    __shared__ __align__(16) float As[BK][BM + PAD];
    __shared__ __align__(16) float Bs[BK][BN + PAD];
    // `sub_rows` matrix rows belong to every grouped row (1 for representations, 3*natoms for Jacobians), so the group
    // boundaries scale with it and stay tile aligned.
    const long row0 = (long)blockIdx.x * BM;
    const int col0 = blockIdx.y * BN;
    if (row0 >= (long)group_start[nel] * sub_rows) return;
    int e = 0;
    while (e + 1 < nel && row0 >= (long)group_start[e + 1] * sub_rows) ++e;
    const float *Pe = P + (size_t)e * p_stride;
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    float acc[4][4] = {};
    const bool a_vec = (K & 3) == 0;

    for (int k0 = 0; k0 < K; k0 += BK) {
        {   // A tile: 64 rows x 16 k ; thread -> (row = tid/4, 4 consecutive k)
            const int r = tid >> 2, kk = (tid & 3) * 4;
            const float *src = in + (size_t)(row0 + r) * K + k0 + kk;
            float v[4];
            if (a_vec && k0 + kk + 3 < K) {
                const float4 t = *reinterpret_cast<const float4 *>(src);
                v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
            } else {
#pragma unroll
                for (int q = 0; q < 4; ++q) v[q] = (k0 + kk + q < K) ? src[q] : 0.f;
            }
#pragma unroll
            for (int q = 0; q < 4; ++q) As[kk + q][r] = v[q];
        }
        if (!TRANS) {  // B[k][n] = Pe[k*npcas + n] : thread -> (k = tid/16, 4 consecutive n)
            const int k = tid >> 4, n = (tid & 15) * 4;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int kk = k0 + k, nn = col0 + n + q;
                Bs[k][n + q] = (kk < K && nn < Nout) ? Pe[(size_t)kk * npcas + nn] : 0.f;
            }
        } else {       // B[k][n] = Pe[n*npcas + k] : thread -> (n = tid/4, 4 consecutive k)
            const int n = tid >> 2, kk = (tid & 3) * 4;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int k = k0 + kk + q, nn = col0 + n;
                Bs[kk + q][n] = (k < K && nn < Nout) ? Pe[(size_t)nn * npcas + k] : 0.f;
            }
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            const float4 a = *reinterpret_cast<const float4 *>(&As[kk][ty * 4]);
            const float4 b = *reinterpret_cast<const float4 *>(&Bs[kk][tx * 4]);
            const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float *dst = out + (size_t)(row0 + ty * 4 + i) * Nout + col0 + tx * 4;
#pragma unroll
        for (int j = 0; j < 4; ++j)
            if (col0 + tx * 4 + j < Nout) dst[j] = acc[i][j];
    }
}

}  // namespace

extern "C" int qmlb_pca_project(const float *in, const float *reductors, const int *group_start, int nelements,
                                size_t rows_cap, int repsize, int npcas, int transpose, float *out,
                                qmlb_stream_t stream) {
    QMLB_REQUIRE(in && reductors && group_start && out, "qmlb_pca_project: null tensor");
    QMLB_REQUIRE(nelements > 0 && repsize > 0 && npcas > 0, "qmlb_pca_project: bad sizes");
    QMLB_REQUIRE(rows_cap % BM == 0, "qmlb_pca_project: rows_cap must be a multiple of %d", BM);
    if (rows_cap == 0) return QMLB_OK;
    const int K = transpose ? npcas : repsize, Nout = transpose ? repsize : npcas;
    dim3 grid((unsigned)(rows_cap / BM), (unsigned)((Nout + BN - 1) / BN));
    const size_t p_stride = (size_t)repsize * npcas;
    if (transpose)
        pca_gemm_kernel<true><<<grid, 256, 0, qmlb::as_stream(stream)>>>(in, reductors, group_start, nelements, K, Nout,
                                                                         npcas, p_stride, 1, out);
    else
        pca_gemm_kernel<false><<<grid, 256, 0, qmlb::as_stream(stream)>>>(in, reductors, group_start, nelements, K, Nout,
                                                                          npcas, p_stride, 1, out);
    return qmlb::check_launch("qmlb_pca_project");
}

extern "C" int qmlb_pca_project_jacobian(const float *jac_rows, const float *reductors, const int *group_start,
                                         int nelements, size_t rows_cap, int sub_rows, int repsize, int npcas, float *out,
                                         qmlb_stream_t stream) {
    QMLB_REQUIRE(jac_rows && reductors && group_start && out, "qmlb_pca_project_jacobian: null tensor");
    QMLB_REQUIRE(nelements > 0 && repsize > 0 && npcas > 0 && sub_rows > 0, "qmlb_pca_project_jacobian: bad sizes");
    QMLB_REQUIRE(rows_cap % BM == 0, "qmlb_pca_project_jacobian: rows_cap must be a multiple of %d", BM);
    if (rows_cap == 0) return QMLB_OK;
    const size_t mrows = rows_cap * (size_t)sub_rows;
    QMLB_REQUIRE(mrows / BM < ((size_t)1 << 31), "qmlb_pca_project_jacobian: too many rows");
    dim3 grid((unsigned)(mrows / BM), (unsigned)((npcas + BN - 1) / BN));
    pca_gemm_kernel<false><<<grid, 256, 0, qmlb::as_stream(stream)>>>(jac_rows, reductors, group_start, nelements, repsize,
                                                                      npcas, npcas, (size_t)repsize * npcas, sub_rows, out);
    return qmlb::check_launch("qmlb_pca_project_jacobian");
}
