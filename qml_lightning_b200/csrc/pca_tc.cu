// Tensor-core version of the per-element PCA projection: tcgen05.mma (kind::tf32) with the accumulator in tensor
// memory and a 3xTF32 split, so that the result keeps fp32 accuracy.
//
//   out[r, n] = sum_k in[r, k] * B_e[n, k],   B_e[n,k] = P_e[k,n] (projection) or P_e[n,k] (its transpose)
//
// Every fp32 operand is split as x = hi + lo with hi = tf32(x) and lo = tf32(x - hi); the product is accumulated as
// hi*hi + hi*lo + lo*hi in fp32 (the dropped lo*lo term is ~2^-22 relative).  A single-pass TF32 product would lose
// three digits and break the 1e-5 energy tolerance, because the projected vector feeds cos().
//
// One block (128 threads) owns a 128-row x 128-column output tile:
//   * all threads stage K-chunks of 16 for A (hi, lo) and B (hi, lo) into shared memory in the canonical K-major,
//     no-swizzle UMMA layout (8-row x 16-byte core matrices; LBO = distance between the 4-element K chunks,
//     SBO = 128 B between 8-row groups), double buffered;
//   * one thread issues 2 k-steps x 3 products of tcgen05.mma M=128, N=128, K=8 per chunk and commits them to the
//     stage's mbarrier; the loaders of chunk c+2 wait on that barrier before overwriting the stage;
//   * after the last commit the four warps read their 32 accumulator lanes with tcgen05.ld and store the tile.
// The tensor core adds into its fp32 accumulator with truncation, about one ulp of the running sum per MMA and
// always towards zero, so a long K loop accumulates a bias (measured 3.5x the error of an fp32 FFMA loop at K = 336).
// For the projection the K loop is therefore cut into groups of FWD_GROUP_CHUNKS chunks: every group starts a fresh
// accumulator in tensor memory and is added to per-thread fp32 registers (round to nearest) when it completes, which
// keeps the running sums small where the truncation happens (measured: below the FFMA loop's error).  The
// transposed product has a short K (npcas) and feeds only the force chain rule; it accumulates in one go.
// Every wait is bounded; on a time-out the block records it in a device counter (qmlb_tc_timeouts), skips its
// stores, releases its tensor memory and returns.
#include "common.cuh"

namespace {

constexpr int BM = 128, BN = 128, BK = 16, STAGES = 2;
constexpr int TILE_FLOATS = BM * BK;                  // one operand tile (hi or lo) of one stage
constexpr int STAGE_FLOATS = 4 * TILE_FLOATS;         // A_hi, A_lo, B_hi, B_lo
constexpr uint32_t LBO_BYTES = BM * 16;               // next 4-element K chunk of the same rows
constexpr uint32_t SBO_BYTES = 128;                   // next 8-row group
constexpr int WAIT_LIMIT = 1 << 22;
#ifndef QMLB_FWD_GROUP_CHUNKS
#define QMLB_FWD_GROUP_CHUNKS 2
#endif
constexpr int FWD_GROUP_CHUNKS = QMLB_FWD_GROUP_CHUNKS;  // projection: K = 32 per tensor-memory accumulation group

__device__ int g_tc_timeouts = 0;

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ uint64_t make_desc(uint32_t saddr) {
    // start address, leading byte offset, stride byte offset (all >> 4), descriptor version 1, no swizzle
    return (uint64_t)((saddr >> 4) & 0x3FFF) | ((uint64_t)(LBO_BYTES >> 4) << 16) | ((uint64_t)(SBO_BYTES >> 4) << 32) |
           ((uint64_t)1 << 46);
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}

// Bounded parity wait; false on time-out.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (int it = 0; it < WAIT_LIMIT; ++it) {
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

__device__ __forceinline__ void mma_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        :
        : "r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}

__device__ __forceinline__ void split_tf32(float x, float &hi, float &lo) {
    uint32_t h;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(h) : "f"(x));
    hi = __uint_as_float(h);
    const float r = x - hi;  // exact in fp32
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(h) : "f"(r));  // round (the tensor core would truncate)
    lo = __uint_as_float(h);
}

// element (row r, k) of an operand tile in the canonical layout, as a float offset
__device__ __forceinline__ int tile_offset(int r, int k) { return (k >> 2) * (BM * 4) + (r >> 3) * 32 + (r & 7) * 4 + (k & 3); }

// GROUP_CHUNKS > 0: flush the tensor-memory accumulator into registers every GROUP_CHUNKS chunks (used for the
// projection, whose result feeds cos()); GROUP_CHUNKS == 0: one accumulation over all of K (used for the transposed
// product, whose K = npcas is short and whose result only feeds the force chain rule).
template <bool TRANS, int GROUP_CHUNKS>
__global__ void __launch_bounds__(128)
pca_tc_kernel(const float *__restrict__ in, const float *__restrict__ P, const int *__restrict__ group_start, int nel, int K,
              int Nout, int npcas, size_t p_stride, int sub_rows, float *__restrict__ out) {
    extern __shared__ __align__(128) float smem[];
    __shared__ __align__(8) uint64_t bars[STAGES];
    __shared__ uint32_t tmem_slot;
    __shared__ int failed;

    const long row0 = (long)blockIdx.x * BM;
    const int col0 = blockIdx.y * BN;
    if (row0 >= (long)group_start[nel] * sub_rows) return;
    int e = 0;
    while (e + 1 < nel && row0 >= (long)group_start[e + 1] * sub_rows) ++e;
    const float *Pe = P + (size_t)e * p_stride;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) mbar_init(smem_u32(&bars[s]), 1);
        failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(BN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_d = tmem_slot;

    // instruction descriptor: D = F32, A = B = TF32, both K-major, N = 128, M = 128
    const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
    const int nchunks = (K + BK - 1) / BK;
    bool ok = true;
    constexpr bool GROUPED = GROUP_CHUNKS > 0;
    constexpr int GC = GROUPED ? GROUP_CHUNKS : 1;
    float racc[GROUPED ? BN : 1];  // this thread's output row (lane of the accumulator), summed over the K groups in fp32
#pragma unroll
    for (int i = 0; i < (GROUPED ? BN : 1); ++i) racc[i] = 0.f;
    uint32_t phase[STAGES] = {0u, 0u};  // parity of the next completion of each stage barrier

    // Register prefetch: the global loads of chunk c+1 are issued before chunk c is handed to the tensor core, so
    // their latency overlaps the barrier, the MMA issue and the next stage wait.
    float4 ra[BK / 4];
    float rb[BK];
    auto fetch = [&](int c) {
        const int k0 = c * BK;
        const float *src = in + (size_t)(row0 + tid) * K + k0;
#pragma unroll
        for (int q = 0; q < BK / 4; ++q) {
            if ((K & 3) == 0 && k0 + 4 * q + 3 < K) {
                ra[q] = *reinterpret_cast<const float4 *>(src + 4 * q);
            } else {
                float v[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) v[i] = (k0 + 4 * q + i < K) ? src[4 * q + i] : 0.f;
                ra[q] = make_float4(v[0], v[1], v[2], v[3]);
            }
        }
        const int n = col0 + tid;
        if (TRANS && (npcas & 3) == 0 && n < Nout && k0 + BK <= K) {
            // B[n][k] = P[n][k]: the thread's 16 values are contiguous
            const float4 *bsrc = reinterpret_cast<const float4 *>(Pe + (size_t)n * npcas + k0);
#pragma unroll
            for (int q = 0; q < BK / 4; ++q) {
                const float4 t = __ldg(bsrc + q);
                rb[4 * q] = t.x; rb[4 * q + 1] = t.y; rb[4 * q + 2] = t.z; rb[4 * q + 3] = t.w;
            }
        } else {
#pragma unroll
            for (int i = 0; i < BK; ++i) {
                const int k = k0 + i;
                rb[i] = (n < Nout && k < K) ? (TRANS ? Pe[(size_t)n * npcas + k] : Pe[(size_t)k * npcas + n]) : 0.f;
            }
        }
    };
    fetch(0);

    for (int c = 0; c < nchunks; ++c) {
        const int s = c & 1;
        float *stage = smem + (size_t)s * STAGE_FLOATS;
        const bool group_start_chunk = GROUPED ? (c % GC) == 0 : c == 0;
        const bool group_end_chunk = (GROUPED && ((c + 1) % GC) == 0) || c == nchunks - 1;
        // The MMAs that read this stage two chunks ago must have completed, unless a group flush already waited
        // for everything issued so far.
        if (c >= STAGES && (!GROUPED || (((c - 1) % GC) != GC - 1 && ((c - 2) % GC) != GC - 1))) {
            if (!mbar_wait(smem_u32(&bars[s]), phase[s])) ok = false;
            phase[s] ^= 1u;
        }
        // split the prefetched operands and store them in the canonical layout (thread = A row = B column)
#pragma unroll
        for (int q = 0; q < BK / 4; ++q) {
            const float v[4] = {ra[q].x, ra[q].y, ra[q].z, ra[q].w};
            float hi[4], lo[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) split_tf32(v[i], hi[i], lo[i]);
            const int off = tile_offset(tid, 4 * q);
            *reinterpret_cast<float4 *>(stage + off) = make_float4(hi[0], hi[1], hi[2], hi[3]);
            *reinterpret_cast<float4 *>(stage + TILE_FLOATS + off) = make_float4(lo[0], lo[1], lo[2], lo[3]);
#pragma unroll
            for (int i = 0; i < 4; ++i) split_tf32(rb[4 * q + i], hi[i], lo[i]);
            *reinterpret_cast<float4 *>(stage + 2 * TILE_FLOATS + off) = make_float4(hi[0], hi[1], hi[2], hi[3]);
            *reinterpret_cast<float4 *>(stage + 3 * TILE_FLOATS + off) = make_float4(lo[0], lo[1], lo[2], lo[3]);
        }
        if (c + 1 < nchunks) fetch(c + 1);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy stores -> visible to the MMA unit
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        if (tid == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t a_hi = smem_u32(stage), a_lo = a_hi + TILE_FLOATS * 4, b_hi = a_hi + 2 * TILE_FLOATS * 4,
                           b_lo = a_hi + 3 * TILE_FLOATS * 4;
#pragma unroll
            for (int ks = 0; ks < BK / 8; ++ks) {
                const uint32_t koff = ks * 2 * LBO_BYTES;  // two 4-element chunks per k-step
                // small cross terms first, the large hi*hi term last
                mma_tf32(tmem_d, make_desc(a_hi + koff), make_desc(b_lo + koff), idesc, (group_start_chunk && ks == 0) ? 0u : 1u);
                mma_tf32(tmem_d, make_desc(a_lo + koff), make_desc(b_hi + koff), idesc, 1u);
                mma_tf32(tmem_d, make_desc(a_hi + koff), make_desc(b_hi + koff), idesc, 1u);
            }
            // arrives on the stage barrier when these (and all earlier) MMAs have finished
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&bars[s])) : "memory");
        }
        if (group_end_chunk) {
            // wait for the whole group, then fold the tensor-memory accumulator into the register row
            if (!mbar_wait(smem_u32(&bars[s]), phase[s])) ok = false;
            phase[s] ^= 1u;
            // the other stage's last commit (if any since its last wait) has completed too: consume its phase
            if (c >= 1 && (!GROUPED || ((c - 1) % GC) != GC - 1)) {
                if (!mbar_wait(smem_u32(&bars[s ^ 1]), phase[s ^ 1])) ok = false;
                phase[s ^ 1] ^= 1u;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (GROUPED) {
#pragma unroll
                for (int cc = 0; cc < BN; cc += 16) {
                    uint32_t v[16];
                    const uint32_t taddr = tmem_d + ((uint32_t)(warp * 32) << 16) + (uint32_t)cc;
                    asm volatile(
                        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
                          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
                        : "r"(taddr));
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int i = 0; i < 16; ++i) racc[cc + i] += __uint_as_float(v[i]);
                }
                // the next group's first MMA overwrites the accumulator: order it after these loads
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncthreads();
            }
        }
    }
    if (!ok) failed = 1;  // benign race: every writer stores 1
    __syncthreads();

    if (!failed) {
        const long r = row0 + warp * 32 + lane;
        float *dst = out + (size_t)r * Nout + col0;
        const bool full = col0 + BN <= Nout && (Nout & 3) == 0;
        if (GROUPED) {
            if (full) {
#pragma unroll
                for (int cc = 0; cc < BN; cc += 4)
                    *reinterpret_cast<float4 *>(dst + cc) = make_float4(racc[cc], racc[cc + 1], racc[cc + 2], racc[cc + 3]);
            } else {
#pragma unroll
                for (int cc = 0; cc < BN; ++cc)
                    if (col0 + cc < Nout) dst[cc] = racc[cc];
            }
        } else {
#pragma unroll 1
            for (int cc = 0; cc < BN; cc += 16) {
                uint32_t v[16];
                const uint32_t taddr = tmem_d + ((uint32_t)(warp * 32) << 16) + (uint32_t)cc;
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                    : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
                      "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
                    : "r"(taddr));
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (full) {
#pragma unroll
                    for (int q = 0; q < 4; ++q)
                        *reinterpret_cast<float4 *>(dst + cc + 4 * q) =
                            make_float4(__uint_as_float(v[4 * q]), __uint_as_float(v[4 * q + 1]), __uint_as_float(v[4 * q + 2]),
                                        __uint_as_float(v[4 * q + 3]));
                } else {
#pragma unroll
                    for (int i = 0; i < 16; ++i)
                        if (col0 + cc + i < Nout) dst[cc + i] = __uint_as_float(v[i]);
                }
            }
        }
    } else if (tid == 0) {
        atomicAdd(&g_tc_timeouts, 1);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(BN) : "memory");
    }
}

}  // namespace

namespace qmlb {
int rff_tc_timeouts();   // rff_tc.cu
int pca_tc2_timeouts();  // pca_tc2.cu
}

extern "C" int qmlb_tc_timeouts(void) {
    int v = -1;
    if (cudaMemcpyFromSymbol(&v, g_tc_timeouts, sizeof(int)) != cudaSuccess) return -1;
    const int w = qmlb::rff_tc_timeouts(), u = qmlb::pca_tc2_timeouts();
    return (w < 0 || u < 0) ? -1 : v + w + u;
}

extern "C" int qmlb_pca_project_tc(const float *in, const float *reductors, const int *group_start, int nelements,
                                   size_t rows_cap, int sub_rows, int repsize, int npcas, int transpose, float *out,
                                   qmlb_stream_t stream) {
    QMLB_REQUIRE(in && reductors && group_start && out, "qmlb_pca_project_tc: null tensor");
    QMLB_REQUIRE(nelements > 0 && repsize > 0 && npcas > 0 && sub_rows > 0, "qmlb_pca_project_tc: bad sizes");
    const size_t mrows = rows_cap * (size_t)sub_rows;
    QMLB_REQUIRE(mrows % BM == 0, "qmlb_pca_project_tc: rows_cap * sub_rows must be a multiple of %d", BM);
    if (mrows == 0) return QMLB_OK;
    const int K = transpose ? npcas : repsize, Nout = transpose ? repsize : npcas;
    dim3 grid((unsigned)(mrows / BM), (unsigned)((Nout + BN - 1) / BN));
    const size_t smem = sizeof(float) * STAGES * STAGE_FLOATS + 128;
    const size_t p_stride = (size_t)repsize * npcas;
    if (transpose) {
        if (int rc = qmlb::ensure_smem(pca_tc_kernel<true, 0>, smem, "qmlb_pca_project_tc")) return rc;
        pca_tc_kernel<true, 0><<<grid, 128, smem, qmlb::as_stream(stream)>>>(in, reductors, group_start, nelements, K, Nout, npcas,
                                                                        p_stride, sub_rows, out);
    } else {
        if (int rc = qmlb::ensure_smem(pca_tc_kernel<false, FWD_GROUP_CHUNKS>, smem, "qmlb_pca_project_tc")) return rc;
        pca_tc_kernel<false, FWD_GROUP_CHUNKS><<<grid, 128, smem, qmlb::as_stream(stream)>>>(in, reductors, group_start, nelements, K, Nout, npcas,
                                                                         p_stride, sub_rows, out);
    }
    return qmlb::check_launch("qmlb_pca_project_tc");
}
