// Normal-equation accumulation  ZTZ += M^T M ,  ZTy += M^T y  in float64 for row blocks M = [Z; G] of one batch.
//
// Upstream: torch.matmul(Ztrain.T, Ztrain) and torch.matmul(Ztrain.T, targets) in build_Z_components
// (models/kernel.py:172-192).  This is a plain dense contraction, so it goes to the library: cuBLAS DSYRK computes
// only one triangle (half the flops of the upstream DGEMM), DGEMV the right-hand side; a small kernel mirrors the
// triangle before the solve.  One cuBLAS handle per device, bound to the caller's stream on every call.
#include <cublas_v2.h>

#include <mutex>

#include "common.cuh"

namespace {

constexpr int MAX_DEVICES = 64;
cublasHandle_t g_handles[MAX_DEVICES] = {};
std::mutex g_handle_mutex;

int get_handle(cublasHandle_t *out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) {
        qmlb::set_error("normal equations: cannot query the current device");
        return QMLB_ERR_CUDA;
    }
    std::lock_guard<std::mutex> lock(g_handle_mutex);
    if (g_handles[dev] == nullptr) {
        if (cublasCreate(&g_handles[dev]) != CUBLAS_STATUS_SUCCESS) {
            g_handles[dev] = nullptr;
            qmlb::set_error("normal equations: cublasCreate failed");
            return QMLB_ERR_CUDA;
        }
    }
    *out = g_handles[dev];
    return QMLB_OK;
}

__global__ void mirror_kernel(double *C, int F) {
    // row-major upper triangle (i <= j) -> lower
    const int j = blockIdx.x * blockDim.x + threadIdx.x, i = blockIdx.y * blockDim.y + threadIdx.y;
    if (i < F && j < F && j > i) C[(size_t)j * F + i] = C[(size_t)i * F + j];
}

}  // namespace

extern "C" int qmlb_normal_equations_accumulate(const double *M, int rows, int F, const double *y, double *ZTZ,
                                                double *ZTy, qmlb_stream_t stream) {
    QMLB_REQUIRE(M && ZTZ, "qmlb_normal_equations_accumulate: null tensor");
    QMLB_REQUIRE((y == nullptr) == (ZTy == nullptr), "qmlb_normal_equations_accumulate: y and ZTy go together");
    QMLB_REQUIRE(rows >= 0 && F > 0, "qmlb_normal_equations_accumulate: bad sizes");
    if (rows == 0) return QMLB_OK;
    cublasHandle_t h;
    if (int rc = get_handle(&h)) return rc;
    if (cublasSetStream(h, qmlb::as_stream(stream)) != CUBLAS_STATUS_SUCCESS) {
        qmlb::set_error("qmlb_normal_equations_accumulate: cublasSetStream failed");
        return QMLB_ERR_CUDA;
    }
    const double one = 1.0;
    // Row-major M[rows,F] is the column-major matrix Mc[F,rows] (lda = F); M^T M = Mc Mc^T.  The column-major LOWER
    // triangle is the row-major UPPER triangle of ZTZ.
    cublasStatus_t st = cublasDsyrk(h, CUBLAS_FILL_MODE_LOWER, CUBLAS_OP_N, F, rows, &one, M, F, &one, ZTZ, F);
    if (st != CUBLAS_STATUS_SUCCESS) {
        qmlb::set_error("qmlb_normal_equations_accumulate: cublasDsyrk failed with status %d", (int)st);
        return QMLB_ERR_CUDA;
    }
    if (y) {
        st = cublasDgemv(h, CUBLAS_OP_N, F, rows, &one, M, F, y, 1, &one, ZTy, 1);
        if (st != CUBLAS_STATUS_SUCCESS) {
            qmlb::set_error("qmlb_normal_equations_accumulate: cublasDgemv failed with status %d", (int)st);
            return QMLB_ERR_CUDA;
        }
    }
    return QMLB_OK;
}

extern "C" int qmlb_symmetrize_upper(double *ZTZ, int F, qmlb_stream_t stream) {
    QMLB_REQUIRE(ZTZ && F > 0, "qmlb_symmetrize_upper: bad arguments");
    dim3 block(32, 8), grid((F + 31) / 32, (F + 7) / 8);
    mirror_kernel<<<grid, block, 0, qmlb::as_stream(stream)>>>(ZTZ, F);
    return qmlb::check_launch("qmlb_symmetrize_upper");
}
