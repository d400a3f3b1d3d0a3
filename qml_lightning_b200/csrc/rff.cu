// Fused random-Fourier-feature energy + gradient kernel.
//
// Replaces, per element, the ATen chain of the upstream RFF model
//   Ztest.index_add_(0, mol, sqrt(2/D) cos(x @ W_e + b_e)) ; E = Ztest @ alpha        (models/random_features.py:98-100)
// and the autograd backward it builds (g = -alpha sqrt(2/D) sin(arg) ; grad_x = g @ W_e^T) by one kernel that keeps a
// 64-row tile of x and its gradient accumulators on chip and streams W_e once per tile in chunks of 64 features:
//   chunk:  arg = x W_c + b_c  ->  E_row += alpha_c . cos(arg) ;  G = -alpha_c sin(arg)  ->  grad_x += G W_c^T
// so neither the [atoms, D] feature matrix nor its gradient ever reaches HBM.  Both contractions use the same
// shared-memory copy of the W chunk.  fp32 FFMA with fp32 accumulation (the arguments feed cos(), a single-pass
// TF32 product would miss the energy tolerance).
#include <math.h>

#include "common.cuh"
#include "sincos.cuh"

namespace {

constexpr int BM = 64;             // rows per block (divides QMLB_ROW_TILE, so a block never straddles two elements)
constexpr int BN = 64;             // features per chunk
constexpr int XS = BM + 4;         // row stride of the transposed x tile   Xs[k][row]
constexpr int WS = BN + 1;         // row stride of the W chunk             Wc[k][feature]  (odd: conflict-free columns)
constexpr int GS = BM + 4;         // row stride of the transposed G tile   Gt[feature][row]

template <int KC>
__host__ __device__ constexpr size_t rff_smem_floats() {
    return (size_t)(16 * KC) * XS + (size_t)(16 * KC) * WS + (size_t)BN * GS;
}

// KC = npcas / 16: every thread owns 4 rows x KC columns (k = q*16 + tx) of the gradient tile.
template <int KC, bool FAST>
__global__ void __launch_bounds__(256)
rff_energy_grad_kernel(const float *__restrict__ x, const int *__restrict__ group_start,
                       const int *__restrict__ slot_of_row, int nel, int D, const float *__restrict__ W,
                       const float *__restrict__ b, const float *__restrict__ alpha, float normf,
                       float *__restrict__ atom_energy, float *__restrict__ grad_x) {
    constexpr int K = 16 * KC;
    extern __shared__ __align__(16) float sm[];
    float *Xs = sm;                      // [K][XS]
    float *Wc = Xs + (size_t)K * XS;     // [K][WS]
    float *Gt = Wc + (size_t)K * WS;     // [BN][GS]
    const int row0 = blockIdx.x * BM;
    if (row0 >= group_start[nel]) return;
    int el = 0;
    while (el + 1 < nel && row0 >= group_start[el + 1]) ++el;
    const float *We = W + (size_t)el * K * D;
    const float *be = b + (size_t)el * D;
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;

    // x tile, transposed; padding rows of the element group are read as zeros
    for (int idx = tid; idx < BM * (K / 4); idx += 256) {
        const int r = idx / (K / 4), k4 = (idx % (K / 4)) * 4;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (slot_of_row[row0 + r] >= 0) v = *reinterpret_cast<const float4 *>(x + (size_t)(row0 + r) * K + k4);
        Xs[(k4 + 0) * XS + r] = v.x;
        Xs[(k4 + 1) * XS + r] = v.y;
        Xs[(k4 + 2) * XS + r] = v.z;
        Xs[(k4 + 3) * XS + r] = v.w;
    }

    float gacc[4][KC];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int q = 0; q < KC; ++q) gacc[i][q] = 0.f;
    float eacc[4] = {0.f, 0.f, 0.f, 0.f};

    for (int f0 = 0; f0 < D; f0 += BN) {
        __syncthreads();  // previous chunk fully consumed (and the x tile visible on the first pass)
        // W chunk: K rows of 64 consecutive features
        for (int idx = tid; idx < K * (BN / 4); idx += 256) {
            const int k = idx / (BN / 4), c4 = (idx % (BN / 4)) * 4;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (f0 + c4 + 3 < D) v = __ldg(reinterpret_cast<const float4 *>(We + (size_t)k * D + f0 + c4));
            else
                for (int q = 0; q < 4; ++q)
                    if (f0 + c4 + q < D) (&v.x)[q] = We[(size_t)k * D + f0 + c4 + q];
            float *dst = Wc + (size_t)k * WS + c4;
            dst[0] = v.x; dst[1] = v.y; dst[2] = v.z; dst[3] = v.w;
        }
        __syncthreads();

        // arg tile: rows ty*4.., features tx + 16c
        float acc[4][4] = {};
#pragma unroll 8
        for (int k = 0; k < K; ++k) {
            const float4 a = *reinterpret_cast<const float4 *>(Xs + (size_t)k * XS + ty * 4);
            const float av[4] = {a.x, a.y, a.z, a.w};
            float wv[4];
#pragma unroll
            for (int c = 0; c < 4; ++c) wv[c] = Wc[(size_t)k * WS + tx + 16 * c];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int c = 0; c < 4; ++c) acc[i][c] = fmaf(av[i], wv[c], acc[i][c]);
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const int f = f0 + tx + 16 * c;
            const float bf = f < D ? be[f] : 0.f;
            const float af = f < D ? alpha[f] * normf : 0.f;
            float g[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                float sn, cs;
                if (FAST) __sincosf(acc[i][c] + bf, &sn, &cs);
                else qmlb_sincos::sincos_one(acc[i][c] + bf, sn, cs);
                eacc[i] = fmaf(af, cs, eacc[i]);
                g[i] = -af * sn;
            }
            *reinterpret_cast<float4 *>(Gt + (size_t)(tx + 16 * c) * GS + ty * 4) = make_float4(g[0], g[1], g[2], g[3]);
        }
        __syncthreads();

        // gradient tile: grad_x[r][k] += sum_j G[r][j] W[k][j]
#pragma unroll 4
        for (int j = 0; j < BN; ++j) {
            const float4 gv = *reinterpret_cast<const float4 *>(Gt + (size_t)j * GS + ty * 4);
            const float g4[4] = {gv.x, gv.y, gv.z, gv.w};
#pragma unroll
            for (int q = 0; q < KC; ++q) {
                const float w = Wc[(size_t)(q * 16 + tx) * WS + j];
#pragma unroll
                for (int i = 0; i < 4; ++i) gacc[i][q] = fmaf(g4[i], w, gacc[i][q]);
            }
        }
    }

#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = row0 + ty * 4 + i;
        float e = eacc[i];
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) e += __shfl_xor_sync(QMLB_FULL_MASK, e, o);  // the 16 tx lanes of one row group
        const bool live = slot_of_row[r] >= 0;
        if (tx == 0) atom_energy[r] = live ? e : 0.f;
#pragma unroll
        for (int q = 0; q < KC; ++q) grad_x[(size_t)r * K + q * 16 + tx] = live ? gacc[i][q] : 0.f;
    }
}

template <int KC>
int launch_rff(const float *x, const int *group_start, const int *slot_of_row, int nel, size_t rows_cap, int D,
               const float *W, const float *b, const float *alpha, int fast, float *atom_energy, float *grad_x,
               cudaStream_t st) {
    const size_t smem = sizeof(float) * rff_smem_floats<KC>();
    const float normf = (float)sqrt(2.0 / (double)D);
    const unsigned grid = (unsigned)(rows_cap / BM);
    if (fast) {
        if (int rc = qmlb::ensure_smem(rff_energy_grad_kernel<KC, true>, smem, "qmlb_rff_energy_grad")) return rc;
        rff_energy_grad_kernel<KC, true><<<grid, 256, smem, st>>>(x, group_start, slot_of_row, nel, D, W, b, alpha, normf,
                                                                  atom_energy, grad_x);
    } else {
        if (int rc = qmlb::ensure_smem(rff_energy_grad_kernel<KC, false>, smem, "qmlb_rff_energy_grad")) return rc;
        rff_energy_grad_kernel<KC, false><<<grid, 256, smem, st>>>(x, group_start, slot_of_row, nel, D, W, b, alpha, normf,
                                                                   atom_energy, grad_x);
    }
    return qmlb::check_launch("qmlb_rff_energy_grad");
}

}  // namespace

extern "C" int qmlb_rff_energy_grad(const float *x, const int *group_start, const int *slot_of_row, int nelements,
                                    size_t rows_cap, int npcas, int nfeatures, const float *W, const float *b,
                                    const float *alpha, int fast_math, float *atom_energy, float *grad_x,
                                    qmlb_stream_t stream) {
    QMLB_REQUIRE(x && group_start && slot_of_row && W && b && alpha && atom_energy && grad_x,
                 "qmlb_rff_energy_grad: null tensor");
    QMLB_REQUIRE(nelements > 0 && nfeatures > 0, "qmlb_rff_energy_grad: bad sizes");
    QMLB_REQUIRE(rows_cap % BM == 0, "qmlb_rff_energy_grad: rows_cap must be a multiple of %d", BM);
    if (rows_cap == 0) return QMLB_OK;
    cudaStream_t st = qmlb::as_stream(stream);
    switch (npcas) {
        case 32: return launch_rff<2>(x, group_start, slot_of_row, nelements, rows_cap, nfeatures, W, b, alpha, fast_math, atom_energy, grad_x, st);
        case 64: return launch_rff<4>(x, group_start, slot_of_row, nelements, rows_cap, nfeatures, W, b, alpha, fast_math, atom_energy, grad_x, st);
        case 128: return launch_rff<8>(x, group_start, slot_of_row, nelements, rows_cap, nfeatures, W, b, alpha, fast_math, atom_energy, grad_x, st);
        case 256: return launch_rff<16>(x, group_start, slot_of_row, nelements, rows_cap, nfeatures, W, b, alpha, fast_math, atom_energy, grad_x, st);
        default:
            qmlb::set_error("qmlb_rff_energy_grad: npcas must be 32, 64, 128 or 256, got %d", npcas);
            return QMLB_ERR_UNSUPPORTED;
    }
}
