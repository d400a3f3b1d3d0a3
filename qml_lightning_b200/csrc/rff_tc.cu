// Tensor-core version of the fused random-Fourier-feature energy + gradient kernel (tcgen05.mma kind::f16, accumulators
// in tensor memory, weights streamed by bulk asynchronous copies).
//
// Per element group the upstream chain (models/random_features.py:98-100 and the autograd backward it builds) is
//   arg = x W_e + b_e ;  E_row = sum_f a_f cos(arg_f) ;  grad_x = -(a * sin(arg)) W_e^T ,   a = alpha sqrt(2/D).
// Both contractions run on the tensor cores with fp32 accuracy: every fp32 operand v is written as hi + lo with
// hi = fp16(s v), lo = fp16(s v - hi) (s a power of two that brings the largest operand to 2^13..2^14, so the pair
// carries 22 significant bits like a TF32 pair but moves half the bytes and multiplies at twice the rate), and the
// product is hi*hi + hi*lo + lo*hi accumulated in fp32.
//
// One block owns 128 rows of one element group and loops over all features in chunks of 32:
//   * x (hi, lo) of the tile stays in shared memory for the whole loop (A operand of the first product, K-major);
//   * the weights are re-packed once per model (qmlb_rff_pack) into per-chunk blobs that already have the shared-memory
//     image: 8x8 fp16 core matrices [8 k][8 features], blocks ordered (feature block, k block).  The same image is the
//     B operand of the first product (MN-major: N = features) and of the second (K-major: N = k, K = features), so a
//     chunk is fetched once, by one cp.async.bulk of 32.4 KB issued by a producer thread, and used twice;
//   * one thread issues the MMAs: arg chunk (M=128, N=32, K=npcas) into one of two tensor-memory buffers, and
//     grad (M=128, N=npcas, K=32) into a persistent tensor-memory accumulator;
//   * four warps (one tensor-memory lane = one row per thread) read the arg chunk, evaluate sin/cos, add the energy
//     and write G = -a sin(arg) (hi, lo) to shared memory as the A operand of the second product.
// Chunks are processed in pairs (arg c, arg c+1, grad c, grad c+1) so that the sin/cos work of one chunk hides behind
// the MMAs of its neighbour and a weight buffer is refilled while the other one is in use.
//
// The tensor core adds into its fp32 accumulator with truncation (towards zero, up to one ulp of the running sum per
// MMA).  The small cross terms of the first product are therefore issued first and the hi*hi terms are split over two
// accumulators; the gradient accumulator is folded into fp32 global memory (round to nearest, red.global.add) every
// FLUSH_CHUNKS chunks and restarted.
//
// Every wait is bounded.  A thread that times out marks the block as failed; the block then skips its stores, waits
// (bounded) for its copies and MMAs in flight, releases its tensor memory and counts the event (qmlb_tc_timeouts).
// A block that finds parameters packed for other sizes does nothing and counts itself the same way.
#include <cuda_fp16.h>
#include <math.h>

#include "common.cuh"

namespace {

constexpr int BM = 128;            // rows per block = QMLB_ROW_TILE
constexpr int FC = 32;             // features per chunk
constexpr int NTHREADS = 192;      // warps 0-3: sin/cos + flush, warp 4: MMA issue, warp 5: weight copies
#ifndef QMLB_RFF_FLUSH_CHUNKS
#define QMLB_RFF_FLUSH_CHUNKS 16
#endif
constexpr int FLUSH_CHUNKS = QMLB_RFF_FLUSH_CHUNKS;  // gradient accumulator folded into global memory every this many chunks (even)
constexpr int WAIT_LIMIT = 1 << 22;
constexpr size_t HEADER_BYTES = 256;
constexpr int EXP_CLAMP = 40;

static_assert(BM == QMLB_ROW_TILE, "a block must cover exactly one row tile");
static_assert(FLUSH_CHUNKS % 2 == 0, "flush groups must hold whole chunk pairs");

struct PackHeader {
    unsigned max_w_bits;   // bit pattern of max |W|
    unsigned max_a_bits;   // bit pattern of max |alpha| sqrt(2/D)
    int npcas, nfeatures, nchunks, nelements;
};

__device__ int g_rff_tc_timeouts = 0;

__host__ __device__ constexpr size_t chunk_bytes(int K) { return (size_t)2 * K * FC * 2 + 3 * FC * 4; }

// floor(log2(v)) of a positive float given by its bits, clamped; 0 for v == 0
__device__ __forceinline__ int exponent_of(unsigned bits) {
    if (bits == 0u) return 0;
    int e = (int)((bits >> 23) & 0xFFu) - 127;
    return max(-EXP_CLAMP, min(EXP_CLAMP, e));
}
__device__ __forceinline__ float pow2i(int e) { return __uint_as_float((unsigned)(127 + e) << 23); }

__device__ __forceinline__ void split_half(float v, __half &hi, __half &lo) {
    hi = __float2half_rn(v);
    lo = __float2half_rn(v - __half2float(hi));
}
// two values at once (one packed conversion each way instead of two scalar ones)
__device__ __forceinline__ void split_half2(float a, float b, __half2 &hi, __half2 &lo) {
    hi = __floats2half2_rn(a, b);
    const float2 h = __half22float2(hi);
    lo = __floats2half2_rn(a - h.x, b - h.y);
}

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ uint64_t make_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    // start address, leading (K direction) and stride (M/N direction) byte offsets between 8x16-byte core matrices,
    // all >> 4; descriptor version 1; no swizzle
    return (uint64_t)((saddr >> 4) & 0x3FFF) | ((uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16) |
           ((uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32) | ((uint64_t)1 << 46);
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
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
#ifdef RFF_DBG_PROFILE
__device__ unsigned long long g_prof[16];
__device__ __forceinline__ bool mbar_wait_prof(uint32_t bar, uint32_t parity, int slot, bool rec) {
    const long long t0 = clock64();
    const bool r = mbar_wait(bar, parity);
    if (rec) g_prof[slot] += (unsigned long long)(clock64() - t0);
    return r;
}
#define MBAR_WAIT(bar, parity, slot) mbar_wait_prof(bar, parity, slot, blockIdx.x == 0 && (threadIdx.x & 31) == 0 && (threadIdx.x < 32 || threadIdx.x >= 128))
#define PROF_STAMP(t) const long long t = clock64()
#define PROF_ADD(slot, t) do { if (blockIdx.x == 0 && threadIdx.x == 0) g_prof[slot] += (unsigned long long)(clock64() - t); } while (0)
#else
#define MBAR_WAIT(bar, parity, slot) mbar_wait(bar, parity)
#define PROF_STAMP(t)
#define PROF_ADD(slot, t)
#endif
__device__ __forceinline__ void bulk_copy(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(__cvta_generic_to_global(src)), "r"(bytes), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void mma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        :
        : "r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
          "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr));
}
// fire-and-forget fp32 add of four consecutive floats (16-byte aligned); all adds to one address come from one thread,
// in program order, so the result does not depend on scheduling
__device__ __forceinline__ void red_add4(float *p, float a, float b, float c, float d) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ---------------------------------------------------------------------------------------------------------------
// packing
// ---------------------------------------------------------------------------------------------------------------

__global__ void rff_pack_max_kernel(const float *__restrict__ W, size_t nW, const float *__restrict__ alpha, int D,
                                    float normf, PackHeader *hdr) {
    float mw = 0.f, ma = 0.f;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < nW; i += (size_t)gridDim.x * blockDim.x) {
        const float v = fabsf(W[i]);
        if (v < INFINITY) mw = fmaxf(mw, v);
    }
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < (size_t)D; i += (size_t)gridDim.x * blockDim.x) {
        const float v = fabsf(alpha[i] * normf);
        if (v < INFINITY) ma = fmaxf(ma, v);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        mw = fmaxf(mw, __shfl_xor_sync(QMLB_FULL_MASK, mw, o));
        ma = fmaxf(ma, __shfl_xor_sync(QMLB_FULL_MASK, ma, o));
    }
    if ((threadIdx.x & 31) == 0) {  // non-negative floats order like their bit patterns
        atomicMax(&hdr->max_w_bits, __float_as_uint(mw));
        atomicMax(&hdr->max_a_bits, __float_as_uint(ma));
    }
}

// One thread per (element, k, block of 8 features): 16 bytes of hi and of lo in the chunk image.
template <int K>
__global__ void rff_pack_weights_kernel(const float *__restrict__ W, int nel, int D, int nchunks, unsigned char *packed) {
    constexpr int KB = K / 8;
    const PackHeader *hdr = reinterpret_cast<const PackHeader *>(packed);
    const float sw = pow2i(13 - exponent_of(hdr->max_w_bits));
    const int fblocks = nchunks * (FC / 8);
    const size_t total = (size_t)nel * K * fblocks;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int fbg = (int)(i % fblocks);         // global feature block (consecutive threads: consecutive features)
        const int k = (int)((i / fblocks) % K);
        const int e = (int)(i / ((size_t)fblocks * K));
        const int c = fbg / (FC / 8), fb = fbg % (FC / 8);
        __align__(16) __half hi[8], lo[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            const int f = fbg * 8 + q;
            const float v = f < D ? W[((size_t)e * K + k) * D + f] * sw : 0.f;
            split_half(v, hi[q], lo[q]);
        }
        unsigned char *blob = packed + HEADER_BYTES + ((size_t)e * nchunks + c) * chunk_bytes(K);
        const size_t off = ((size_t)(fb * KB + (k >> 3)) * 128) + (size_t)(k & 7) * 16;
        *reinterpret_cast<uint4 *>(blob + off) = *reinterpret_cast<const uint4 *>(hi);
        *reinterpret_cast<uint4 *>(blob + (size_t)K * FC * 2 + off) = *reinterpret_cast<const uint4 *>(lo);
    }
}

// One thread per (element, padded feature): bias, energy weight a_f, scaled gradient weight -a_f s_a.
template <int K>
__global__ void rff_pack_params_kernel(const float *__restrict__ b, const float *__restrict__ alpha, int nel, int D,
                                       int nchunks, float normf, unsigned char *packed) {
    const PackHeader *hdr = reinterpret_cast<const PackHeader *>(packed);
    const float sa = pow2i(13 - exponent_of(hdr->max_a_bits));
    const int Dp = nchunks * FC;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= nel * Dp) return;
    const int e = i / Dp, f = i % Dp, c = f / FC, j = f % FC;
    float *prm = reinterpret_cast<float *>(packed + HEADER_BYTES + ((size_t)e * nchunks + c) * chunk_bytes(K) + (size_t)2 * K * FC * 2);
    const float a = f < D ? alpha[f] * normf : 0.f;
    prm[j] = f < D ? b[(size_t)e * D + f] : 0.f;
    prm[FC + j] = a;
    prm[2 * FC + j] = -a * sa;
}

__global__ void rff_pack_header_kernel(PackHeader *hdr, int K, int D, int nchunks, int nel) {
    hdr->npcas = K; hdr->nfeatures = D; hdr->nchunks = nchunks; hdr->nelements = nel;
}

// ---------------------------------------------------------------------------------------------------------------
// main kernel
// ---------------------------------------------------------------------------------------------------------------

// barrier slots
enum { W_FULL = 0, W_FREE = 2, ARG_FULL = 4, ARG_FREE = 6, G_FULL = 8, G_FREE = 10, GRAD_FULL = 12, GRAD_FREE = 13, ALL_DONE = 14, NBARS = 15 };

template <int K>
struct Smem {
    static constexpr uint32_t X_HALF = BM * K * 2;              // x hi (or lo) image
    static constexpr uint32_t W_HALF = K * FC * 2;              // weight hi (or lo) image of one chunk
    static constexpr uint32_t CHUNK = (uint32_t)chunk_bytes(K);
    static constexpr uint32_t G_HALF = BM * FC * 2;             // G hi (or lo) image
    static constexpr uint32_t OFF_XH = 0, OFF_XL = X_HALF, OFF_W = 2 * X_HALF, OFF_G = OFF_W + 2 * CHUNK;
    static constexpr uint32_t TOTAL = OFF_G + 4 * G_HALF;
    static_assert(CHUNK % 128 == 0, "chunk images must keep 128-byte alignment");
};

template <int K, bool FAST>
__global__ void __launch_bounds__(NTHREADS, 1)
rff_tc_kernel(const float *__restrict__ x, const int *__restrict__ group_start, const int *__restrict__ slot_of_row, int nel,
              const unsigned char *__restrict__ packed, float *__restrict__ atom_energy, float *__restrict__ grad_x) {
    using S = Smem<K>;
    constexpr int KB = K / 8;
    constexpr uint32_t TMEM_COLS = 512;
    constexpr uint32_t COL_GRAD = 128;            // columns 0..127: two arg buffers x two partial accumulators x 32
    extern __shared__ unsigned char smem_dyn[];
    __shared__ __align__(8) uint64_t bars[NBARS];
    __shared__ uint32_t tmem_slot;
    __shared__ unsigned xmax_bits;
    __shared__ int failed;

    const int row0 = blockIdx.x * BM;
    if (row0 >= group_start[nel]) return;
    int e = 0;
    while (e + 1 < nel && row0 >= group_start[e + 1]) ++e;

    const PackHeader *hdr = reinterpret_cast<const PackHeader *>(packed);
    if (hdr->npcas != K || hdr->nelements != nel) {  // parameters packed for another model: refuse, and say so
        if (threadIdx.x == 0) atomicAdd(&g_rff_tc_timeouts, 1);
        return;
    }
    const int nchunks = hdr->nchunks;
    const int ew = exponent_of(hdr->max_w_bits), ea = exponent_of(hdr->max_a_bits);
    const unsigned char *blobs = packed + HEADER_BYTES + (size_t)e * nchunks * S::CHUNK;

    const uint32_t sbase = (smem_u32(smem_dyn) + 127u) & ~127u;
    unsigned char *sptr = smem_dyn + (sbase - smem_u32(smem_dyn));
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    auto bar = [&](int i) { return smem_u32(&bars[i]); };

    if (tid == 0) {
        mbar_init(bar(W_FULL), 1); mbar_init(bar(W_FULL + 1), 1);
        mbar_init(bar(W_FREE), 1); mbar_init(bar(W_FREE + 1), 1);
        mbar_init(bar(ARG_FULL), 1); mbar_init(bar(ARG_FULL + 1), 1);
        mbar_init(bar(ARG_FREE), 4); mbar_init(bar(ARG_FREE + 1), 4);
        mbar_init(bar(G_FULL), 4); mbar_init(bar(G_FULL + 1), 4);
        mbar_init(bar(G_FREE), 1); mbar_init(bar(G_FREE + 1), 1);
        mbar_init(bar(GRAD_FULL), 1); mbar_init(bar(GRAD_FREE), 4); mbar_init(bar(ALL_DONE), 1);
        failed = 0;
        xmax_bits = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 4) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    __syncthreads();

    // the gradient rows of the tile start at zero: the accumulator is folded into them with reductions
    for (int i = tid; i < BM * (K / 4); i += NTHREADS)
        *reinterpret_cast<float4 *>(grad_x + (size_t)row0 * K + (size_t)i * 4) = make_float4(0.f, 0.f, 0.f, 0.f);

    // ---- x tile: scale, split, canonical K-major image (8 rows x 8 k core matrices, k blocks outermost) ----
    {
        float m = 0.f;
        for (int i = tid; i < BM * (K / 4); i += NTHREADS) {
            const int r = i / (K / 4), k4 = (i % (K / 4)) * 4;
            if (slot_of_row[row0 + r] >= 0) {
                const float4 v = *reinterpret_cast<const float4 *>(x + (size_t)(row0 + r) * K + k4);
                m = fmaxf(m, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(QMLB_FULL_MASK, m, o));
        if (lane == 0 && m < INFINITY) atomicMax(&xmax_bits, __float_as_uint(m));
    }
    __syncthreads();
    const int ex = exponent_of(xmax_bits);
    {
        const float sx = pow2i(13 - ex);
        for (int i = tid; i < BM * KB; i += NTHREADS) {
            const int r = i % BM, kb = i / BM;
            __align__(16) __half hi[8], lo[8];
            float v[8];
            if (slot_of_row[row0 + r] >= 0) {
                const float4 a = *reinterpret_cast<const float4 *>(x + (size_t)(row0 + r) * K + kb * 8);
                const float4 c = *reinterpret_cast<const float4 *>(x + (size_t)(row0 + r) * K + kb * 8 + 4);
                v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = c.x; v[5] = c.y; v[6] = c.z; v[7] = c.w;
            } else {
#pragma unroll
                for (int q = 0; q < 8; ++q) v[q] = 0.f;
            }
#pragma unroll
            for (int q = 0; q < 8; ++q) split_half(v[q] * sx, hi[q], lo[q]);
            const uint32_t off = (uint32_t)(kb * 16 + (r >> 3)) * 128u + (uint32_t)(r & 7) * 16u;
            *reinterpret_cast<uint4 *>(sptr + S::OFF_XH + off) = *reinterpret_cast<const uint4 *>(hi);
            *reinterpret_cast<uint4 *>(sptr + S::OFF_XL + off) = *reinterpret_cast<const uint4 *>(lo);
        }
    }
    fence_async_smem();
    fence_before();
    __syncthreads();
    fence_after();
    const uint32_t tmem = tmem_slot;
    const float arg_scale = pow2i(ex - 13) * pow2i(ew - 13);     // undoes the operand scales of the first product
    const float grad_scale = pow2i(ea - 13) * pow2i(ew - 13);    // and of the second

#ifdef RFF_DBG_PROFILE
    const long long t_role0 = clock64();
#endif
    if (warp < 4) {
        // ------------------------------------------------------------------ sin/cos warps: one row per thread
        const int r = warp * 32 + lane;
        const bool live = slot_of_row[row0 + r] >= 0;
        const uint32_t lane_field = (uint32_t)(warp * 32) << 16;
        const uint32_t g_off = (uint32_t)(r >> 3) * 128u + (uint32_t)(r & 7) * 16u;
        float eacc = 0.f, ecomp = 0.f;  // energy of the row, summed over the chunks with compensation
        bool ok = true;
        for (int c = 0; c < nchunks && ok; ++c) {
            const int s = c & 1;
            const uint32_t par = (uint32_t)(c >> 1) & 1u;
            if (!MBAR_WAIT(bar(ARG_FULL + s), par, 0)) { ok = false; break; }
            fence_after();
            PROF_STAMP(t0);
            float arg[FC];
#pragma unroll
            for (int h = 0; h < FC / 16; ++h) {
                uint32_t v0[16], v1[16];
                tmem_ld16(tmem + lane_field + (uint32_t)(s * 64 + h * 16), v0);
                tmem_ld16(tmem + lane_field + (uint32_t)(s * 64 + 32 + h * 16), v1);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 16; ++i) arg[h * 16 + i] = __uint_as_float(v0[i]) + __uint_as_float(v1[i]);
            }
            fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(ARG_FREE + s));
            PROF_ADD(12, t0);
            // the chunk image (already complete: the MMAs above read it) also carries this chunk's bias and weights;
            // observing its barrier makes the copied bytes visible to this thread's loads
            if (!MBAR_WAIT(bar(W_FULL + s), par, 1)) { ok = false; break; }
            const float *prm = reinterpret_cast<const float *>(sptr + S::OFF_W + s * S::CHUNK + 2 * S::W_HALF);
            // the previous use of this G buffer (chunk c-2) must have been consumed by its MMAs
            if (c >= 2 && !MBAR_WAIT(bar(G_FREE + s), (uint32_t)((c >> 1) - 1) & 1u, 2)) { ok = false; break; }
            unsigned char *gbuf = sptr + S::OFF_G + s * 2 * S::G_HALF;
            float echunk = 0.f;
            PROF_STAMP(t1);
#pragma unroll
            for (int fb = 0; fb < FC / 8; ++fb) {
                __align__(16) __half2 hi[4], lo[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    float gq[2];
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const int f = fb * 8 + 2 * q + h;
                        const float a = fmaf(arg[f], arg_scale, prm[f]);
                        float sn, cs;
#ifdef RFF_DBG_NO_SINCOS
                        sn = a; cs = a;
#else
                        if (FAST) __sincosf(a, &sn, &cs);
                        else sincosf(a, &sn, &cs);
#endif
                        echunk = fmaf(prm[FC + f], cs, echunk);
                        gq[h] = prm[2 * FC + f] * sn;
                    }
                    split_half2(gq[0], gq[1], hi[q], lo[q]);
                }
                const uint32_t off = (uint32_t)fb * (16u * 128u) + g_off;
                *reinterpret_cast<uint4 *>(gbuf + off) = *reinterpret_cast<const uint4 *>(hi);
                *reinterpret_cast<uint4 *>(gbuf + S::G_HALF + off) = *reinterpret_cast<const uint4 *>(lo);
            }
            PROF_ADD(13, t1);
            PROF_STAMP(t2);
            fence_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(G_FULL + s));
            PROF_ADD(14, t2);
            {   // Kahan step: a plain running sum over nfeatures terms would lose ~sqrt(nfeatures) ulps
                const float y = echunk - ecomp, t = eacc + y;
                ecomp = (t - eacc) - y;
                eacc = t;
            }

            if ((c % FLUSH_CHUNKS) == FLUSH_CHUNKS - 1 || c == nchunks - 1) {
                // fold the gradient accumulator of this group into global memory
                const int group = c / FLUSH_CHUNKS;
                if (!MBAR_WAIT(bar(GRAD_FULL), (uint32_t)group & 1u, 3)) { ok = false; break; }
                fence_after();
                PROF_STAMP(t3);
                float *dst = grad_x + (size_t)(row0 + r) * K;
#pragma unroll 1
                for (int cc = 0; cc < K; cc += 32) {
                    uint32_t v0[16], v1[16];
                    tmem_ld16(tmem + lane_field + COL_GRAD + (uint32_t)cc, v0);
                    tmem_ld16(tmem + lane_field + COL_GRAD + (uint32_t)cc + 16u, v1);
                    tmem_ld_wait();
                    if (live) {  // rows of the padding keep their zeros
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            red_add4(dst + cc + 4 * q, __uint_as_float(v0[4 * q]) * grad_scale, __uint_as_float(v0[4 * q + 1]) * grad_scale,
                                     __uint_as_float(v0[4 * q + 2]) * grad_scale, __uint_as_float(v0[4 * q + 3]) * grad_scale);
                            red_add4(dst + cc + 16 + 4 * q, __uint_as_float(v1[4 * q]) * grad_scale, __uint_as_float(v1[4 * q + 1]) * grad_scale,
                                     __uint_as_float(v1[4 * q + 2]) * grad_scale, __uint_as_float(v1[4 * q + 3]) * grad_scale);
                        }
                    }
                }
                fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(GRAD_FREE));
                PROF_ADD(15, t3);
            }
        }
        if (ok) atom_energy[row0 + r] = live ? eacc : 0.f;
        else failed = 1;  // benign race: every writer stores 1
    } else if (warp == 4) {
        // ------------------------------------------------------------------ MMA issue
        if (lane == 0) {
            // D = F32, A = B = F16; first product: A K-major, B MN-major, N = FC; second: both K-major, N = K
            const uint32_t idesc1 = (1u << 4) | (1u << 16) | ((uint32_t)(FC >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
            const uint32_t idesc2 = (1u << 4) | ((uint32_t)(K >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
            const uint32_t xh = sbase + S::OFF_XH, xl = sbase + S::OFF_XL;
            bool ok = true;
            auto issue_arg = [&](int c) {
                const int s = c & 1;
                if (!MBAR_WAIT(bar(W_FULL + s), (uint32_t)(c >> 1) & 1u, 5)) { ok = false; return; }
                if (c >= 2 && !MBAR_WAIT(bar(ARG_FREE + s), (uint32_t)((c >> 1) - 1) & 1u, 6)) { ok = false; return; }
                fence_after();
                const uint32_t wh = sbase + S::OFF_W + s * S::CHUNK, wl = wh + S::W_HALF;
                const uint32_t acc0 = tmem + (uint32_t)(s * 64), acc1 = acc0 + 32;
                // A: 16 k per step = 2 k blocks of 2048 B; B: 2 k blocks of 128 B
                auto adesc = [&](uint32_t base, int ks) { return make_desc(base + (uint32_t)ks * 4096u, 2048u, 128u); };
                auto bdesc = [&](uint32_t base, int ks) { return make_desc(base + (uint32_t)ks * 256u, 128u, (uint32_t)KB * 128u); };
#ifndef RFF_DBG_NO_CROSS1
                for (int ks = 0; ks < K / 16; ++ks) mma_f16(acc0, adesc(xh, ks), bdesc(wl, ks), idesc1, ks > 0 ? 1u : 0u);
                for (int ks = 0; ks < K / 16; ++ks) mma_f16(acc0, adesc(xl, ks), bdesc(wh, ks), idesc1, 1u);
#endif
                for (int ks = 0; ks < K / 32; ++ks) mma_f16(acc0, adesc(xh, ks), bdesc(wh, ks), idesc1, 1u);
                for (int ks = K / 32; ks < K / 16; ++ks) mma_f16(acc1, adesc(xh, ks), bdesc(wh, ks), idesc1, ks > K / 32 ? 1u : 0u);
                mma_commit(bar(ARG_FULL + s));
            };
            auto issue_grad = [&](int c) {
                const int s = c & 1;
                if (!MBAR_WAIT(bar(G_FULL + s), (uint32_t)(c >> 1) & 1u, 7)) { ok = false; return; }
                const int group = c / FLUSH_CHUNKS;
                const bool first = (c % FLUSH_CHUNKS) == 0;
                if (first && group > 0 && !MBAR_WAIT(bar(GRAD_FREE), (uint32_t)(group - 1) & 1u, 8)) { ok = false; return; }
                fence_after();
                const uint32_t wh = sbase + S::OFF_W + s * S::CHUNK, wl = wh + S::W_HALF;
                const uint32_t gh = sbase + S::OFF_G + s * 2 * S::G_HALF, gl = gh + S::G_HALF;
                // A: 16 features per step = 2 feature blocks of 2048 B; B: 2 feature blocks of KB*128 B
                auto adesc = [&](uint32_t base, int ks) { return make_desc(base + (uint32_t)ks * 4096u, 2048u, 128u); };
                auto bdesc = [&](uint32_t base, int ks) { return make_desc(base + (uint32_t)ks * 2u * KB * 128u, (uint32_t)KB * 128u, 128u); };
#ifndef RFF_DBG_NO_GRAD
                for (int ks = 0; ks < FC / 16; ++ks) {
                    mma_f16(tmem + COL_GRAD, adesc(gh, ks), bdesc(wl, ks), idesc2, (first && ks == 0) ? 0u : 1u);
                    mma_f16(tmem + COL_GRAD, adesc(gl, ks), bdesc(wh, ks), idesc2, 1u);
                    mma_f16(tmem + COL_GRAD, adesc(gh, ks), bdesc(wh, ks), idesc2, 1u);
                }
#endif
                mma_commit(bar(W_FREE + s));
                mma_commit(bar(G_FREE + s));
                if ((c % FLUSH_CHUNKS) == FLUSH_CHUNKS - 1 || c == nchunks - 1) mma_commit(bar(GRAD_FULL));
            };
            for (int c0 = 0; c0 < nchunks && ok; c0 += 2) {
                issue_arg(c0);
                if (ok && c0 + 1 < nchunks) issue_arg(c0 + 1);
                if (ok) issue_grad(c0);
                if (ok && c0 + 1 < nchunks) issue_grad(c0 + 1);
            }
            // everything issued so far must have left the tensor pipe before the tensor memory is released
            mma_commit(bar(ALL_DONE));
            if (!mbar_wait(bar(ALL_DONE), 0u)) ok = false;
            if (!ok) failed = 1;
        }
    } else {
        // ------------------------------------------------------------------ weight copies
        if (lane == 0) {
            bool ok = true;
            int issued = 0;
            for (int c = 0; c < nchunks; ++c) {
                const int s = c & 1;
                if (c >= 2 && !MBAR_WAIT(bar(W_FREE + s), (uint32_t)((c >> 1) - 1) & 1u, 10)) { ok = false; break; }
                mbar_expect_tx(bar(W_FULL + s), S::CHUNK);
                bulk_copy(sbase + S::OFF_W + s * S::CHUNK, blobs + (size_t)c * S::CHUNK, S::CHUNK, bar(W_FULL + s));
                issued = c + 1;
            }
            // no copy may still be in flight when the block leaves
            for (int c = max(0, issued - 2); c < issued; ++c)
                if (!mbar_wait(bar(W_FULL + (c & 1)), (uint32_t)(c >> 1) & 1u)) ok = false;
            if (!ok) failed = 1;
        }
    }
#ifdef RFF_DBG_PROFILE
    if (blockIdx.x == 0 && lane == 0 && (warp == 0 || warp >= 4)) g_prof[warp == 0 ? 4 : (warp == 4 ? 9 : 11)] += (unsigned long long)(clock64() - t_role0);
#endif
    __syncwarp();
    fence_before();
    __syncthreads();
    fence_after();
    if (failed && tid == 0) atomicAdd(&g_rff_tc_timeouts, 1);
    if (warp == 4) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}

template <int K>
int launch_rff_tc(const float *x, const int *group_start, const int *slot_of_row, int nel, size_t rows_cap,
                  const unsigned char *packed, int fast, float *atom_energy, float *grad_x, cudaStream_t st) {
    const size_t smem = Smem<K>::TOTAL + 128;
    const unsigned grid = (unsigned)(rows_cap / BM);
    if (fast) {
        if (int rc = qmlb::ensure_smem(rff_tc_kernel<K, true>, smem, "qmlb_rff_energy_grad_tc")) return rc;
        rff_tc_kernel<K, true><<<grid, NTHREADS, smem, st>>>(x, group_start, slot_of_row, nel, packed, atom_energy, grad_x);
    } else {
        if (int rc = qmlb::ensure_smem(rff_tc_kernel<K, false>, smem, "qmlb_rff_energy_grad_tc")) return rc;
        rff_tc_kernel<K, false><<<grid, NTHREADS, smem, st>>>(x, group_start, slot_of_row, nel, packed, atom_energy, grad_x);
    }
    return qmlb::check_launch("qmlb_rff_energy_grad_tc");
}

template <int K>
int launch_rff_pack(const float *W, const float *b, const float *alpha, int nel, int D, unsigned char *packed, cudaStream_t st) {
    const int nchunks = (D + FC - 1) / FC;
    const float normf = (float)sqrt(2.0 / (double)D);
    PackHeader *hdr = reinterpret_cast<PackHeader *>(packed);
    if (cudaMemsetAsync(packed, 0, HEADER_BYTES, st) != cudaSuccess) {
        qmlb::set_error("qmlb_rff_pack: cudaMemsetAsync failed");
        return QMLB_ERR_CUDA;
    }
    rff_pack_header_kernel<<<1, 1, 0, st>>>(hdr, K, D, nchunks, nel);
    rff_pack_max_kernel<<<296, 256, 0, st>>>(W, (size_t)nel * K * D, alpha, D, normf, hdr);
    rff_pack_weights_kernel<K><<<1184, 256, 0, st>>>(W, nel, D, nchunks, packed);
    const int np = nel * nchunks * FC;
    rff_pack_params_kernel<K><<<(np + 255) / 256, 256, 0, st>>>(b, alpha, nel, D, nchunks, normf, packed);
    return qmlb::check_launch("qmlb_rff_pack");
}

bool supported_npcas(int npcas) { return npcas == 32 || npcas == 64 || npcas == 128 || npcas == 256; }

}  // namespace

#ifdef RFF_DBG_PROFILE
extern "C" int qmlb_dbg_rff_profile(unsigned long long *out, int reset) {
    if (reset) { unsigned long long z[16] = {}; return cudaMemcpyToSymbol(g_prof, z, sizeof(z)) != cudaSuccess; }
    return cudaMemcpyFromSymbol(out, g_prof, 16 * sizeof(unsigned long long)) != cudaSuccess;
}
#endif

namespace qmlb {
int rff_tc_timeouts() {
    int v = -1;
    if (cudaMemcpyFromSymbol(&v, g_rff_tc_timeouts, sizeof(int)) != cudaSuccess) return -1;
    return v;
}
}  // namespace qmlb

extern "C" size_t qmlb_rff_pack_bytes(int nelements, int npcas, int nfeatures) {
    if (nelements <= 0 || nfeatures <= 0 || !supported_npcas(npcas)) return 0;
    const size_t nchunks = ((size_t)nfeatures + FC - 1) / FC;
    return HEADER_BYTES + (size_t)nelements * nchunks * chunk_bytes(npcas);
}

extern "C" int qmlb_rff_pack(const float *W, const float *b, const float *alpha, int nelements, int npcas, int nfeatures,
                             void *packed, size_t packed_bytes, qmlb_stream_t stream) {
    QMLB_REQUIRE(W && b && alpha && packed, "qmlb_rff_pack: null tensor");
    QMLB_REQUIRE(nelements > 0 && nfeatures > 0, "qmlb_rff_pack: bad sizes");
    QMLB_REQUIRE(supported_npcas(npcas), "qmlb_rff_pack: npcas must be 32, 64, 128 or 256, got %d", npcas);
    QMLB_REQUIRE(packed_bytes >= qmlb_rff_pack_bytes(nelements, npcas, nfeatures), "qmlb_rff_pack: packed buffer too small");
    QMLB_REQUIRE(((uintptr_t)packed & 255) == 0, "qmlb_rff_pack: packed buffer must be 256-byte aligned");
    cudaStream_t st = qmlb::as_stream(stream);
    unsigned char *p = static_cast<unsigned char *>(packed);
    switch (npcas) {
        case 32: return launch_rff_pack<32>(W, b, alpha, nelements, nfeatures, p, st);
        case 64: return launch_rff_pack<64>(W, b, alpha, nelements, nfeatures, p, st);
        case 128: return launch_rff_pack<128>(W, b, alpha, nelements, nfeatures, p, st);
        default: return launch_rff_pack<256>(W, b, alpha, nelements, nfeatures, p, st);
    }
}

extern "C" int qmlb_rff_energy_grad_tc(const float *x, const int *group_start, const int *slot_of_row, int nelements,
                                       size_t rows_cap, int npcas, const void *packed, int fast_math, float *atom_energy,
                                       float *grad_x, qmlb_stream_t stream) {
    QMLB_REQUIRE(x && group_start && slot_of_row && packed && atom_energy && grad_x, "qmlb_rff_energy_grad_tc: null tensor");
    QMLB_REQUIRE(nelements > 0, "qmlb_rff_energy_grad_tc: bad sizes");
    QMLB_REQUIRE(supported_npcas(npcas), "qmlb_rff_energy_grad_tc: npcas must be 32, 64, 128 or 256, got %d", npcas);
    QMLB_REQUIRE(rows_cap % BM == 0, "qmlb_rff_energy_grad_tc: rows_cap must be a multiple of %d", BM);
    if (rows_cap == 0) return QMLB_OK;
    cudaStream_t st = qmlb::as_stream(stream);
    const unsigned char *p = static_cast<const unsigned char *>(packed);
    switch (npcas) {
        case 32: return launch_rff_tc<32>(x, group_start, slot_of_row, nelements, rows_cap, p, fast_math, atom_energy, grad_x, st);
        case 64: return launch_rff_tc<64>(x, group_start, slot_of_row, nelements, rows_cap, p, fast_math, atom_energy, grad_x, st);
        case 128: return launch_rff_tc<128>(x, group_start, slot_of_row, nelements, rows_cap, p, fast_math, atom_energy, grad_x, st);
        default: return launch_rff_tc<256>(x, group_start, slot_of_row, nelements, rows_cap, p, fast_math, atom_energy, grad_x, st);
    }
}
