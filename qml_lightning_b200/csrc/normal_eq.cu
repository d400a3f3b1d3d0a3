// Normal-equation accumulation  ZTZ += M^T M ,  ZTy += M^T y  in float64 for row blocks M = [Z; G] of one batch.
//
// Upstream: torch.matmul(Ztrain.T, Ztrain) and torch.matmul(Ztrain.T, targets) in build_Z_components
// (models/kernel.py:172-192).  qmlb_normal_equations_accumulate runs the in-tree kernels of syrk_f64.cu;
// qmlb_normal_equations_accumulate_cublas is the same update through cuBLAS DSYRK + DGEMV, kept as the library
// yardstick the in-tree kernel is timed against (one handle per device, bound to the caller's stream on every call).
// Small kernels mirror the triangle before the solve and pack / unpack it for the exchange between ranks.
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

// Row i of the packed triangle starts at i*F - i*(i-1)/2 and holds columns i..F-1: both sides of the copy are contiguous.
__device__ __forceinline__ size_t packed_row_start(size_t i, size_t F) { return i * F - (i * (i - 1)) / 2; }

template <bool PACK>
__global__ void triangle_copy_kernel(double *C, double *packed, int F) {
    const size_t i = blockIdx.y;
    const size_t j = i + (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= (size_t)F) return;
    const size_t a = i * (size_t)F + j, b = packed_row_start(i, F) + (j - i);
    if (PACK) packed[b] = C[a];
    else C[a] = packed[b];
}

}  // namespace

extern "C" size_t qmlb_packed_upper_elements(int F) { return F > 0 ? (size_t)F * ((size_t)F + 1) / 2 : 0; }

extern "C" int qmlb_pack_upper(const double *ZTZ, int F, double *packed, qmlb_stream_t stream) {
    QMLB_REQUIRE(ZTZ && packed && F > 0 && F <= 65535, "qmlb_pack_upper: bad arguments");
    dim3 block(256), grid((F + 255) / 256, F);
    triangle_copy_kernel<true><<<grid, block, 0, qmlb::as_stream(stream)>>>(const_cast<double *>(ZTZ), packed, F);
    return qmlb::check_launch("qmlb_pack_upper");
}

extern "C" int qmlb_unpack_upper(const double *packed, int F, double *ZTZ, qmlb_stream_t stream) {
    QMLB_REQUIRE(ZTZ && packed && F > 0 && F <= 65535, "qmlb_unpack_upper: bad arguments");
    dim3 block(256), grid((F + 255) / 256, F);
    triangle_copy_kernel<false><<<grid, block, 0, qmlb::as_stream(stream)>>>(ZTZ, const_cast<double *>(packed), F);
    if (int rc = qmlb::check_launch("qmlb_unpack_upper")) return rc;
    return qmlb_symmetrize_upper(ZTZ, F, stream);
}

extern "C" int qmlb_normal_equations_accumulate(const double *M, int rows, int F, const double *y, double *ZTZ,
                                                double *ZTy, qmlb_stream_t stream) {
    QMLB_REQUIRE(M && ZTZ, "qmlb_normal_equations_accumulate: null tensor");
    QMLB_REQUIRE((y == nullptr) == (ZTy == nullptr), "qmlb_normal_equations_accumulate: y and ZTy go together");
    if (int rc = qmlb_syrk_f64(M, rows, F, ZTZ, stream)) return rc;
    return y ? qmlb_gemv_t_f64(M, rows, F, y, ZTy, stream) : QMLB_OK;
}

extern "C" int qmlb_normal_equations_accumulate_cublas(const double *M, int rows, int F, const double *y, double *ZTZ,
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
