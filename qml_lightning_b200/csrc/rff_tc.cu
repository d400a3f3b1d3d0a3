// Tensor-core version of the fused random-Fourier-feature energy + gradient kernel (tcgen05.mma kind::f16, accumulators
// and the x operand in tensor memory, weights streamed by bulk asynchronous copies).
//
// Per element group the upstream chain (models/random_features.py:98-100 and the autograd backward it builds) is
//   arg = x W_e + b_e ;  E_row = sum_f a_f cos(arg_f) ;  grad_x = -(a * sin(arg)) W_e^T ,   a = alpha sqrt(2/D).
// Both contractions run on the tensor cores with fp32 accuracy: every fp32 operand v is written as hi + lo with
// hi = fp16(s v), lo = fp16(s v - hi) (s a power of two that brings the largest operand to 2^13..2^14, so the pair
// carries 22 significant bits like a TF32 pair but moves half the bytes and multiplies at twice the rate), and the
// product is hi*hi + hi*lo + lo*hi accumulated in fp32.
//
// One block (12 warps) owns 128 rows of one element group and loops over all features in chunks of 32:
//   * x_hi of the tile lives in tensor memory (lane = row, one 32-bit column = two consecutive k) and x_lo in shared
//     memory (canonical K-major image) for the whole loop;
//   * the weights are re-packed once per model (qmlb_rff_pack) into per-chunk blobs that already have the shared-memory
//     image: 8x8 fp16 core matrices [8 k][8 features], blocks ordered (feature block, k block), hi image then lo image,
//     then the chunk's bias and weights.  The same image is the B operand of the first product (MN-major: N = features)
//     and of the second (K-major: N = k, K = features), so a chunk is fetched once, by one cp.async.bulk of 32.4 KB
//     issued by a producer thread into a ring of four stages, and used twice;
//   * first product, per chunk: x_hi [W_hi | W_lo] as npcas/16 MMAs with N = 64 (the lo image continues the hi image at
//     the feature-block stride, so one descriptor covers both) and x_lo W_hi as npcas/16 MMAs with N = 32, into one of
//     two 64-column tensor-memory buffers [hi*hi | cross terms].  Measured: an MMA occupies the tensor pipe for
//     max(its math time, its shared-memory operand bytes / ~64 B per cycle), operands in tensor memory being free, so a
//     small-N MMA with A in shared memory costs 80 cycles for 16 cycles of math; that is why x_hi sits in tensor memory,
//     why the two weight images are multiplied in one instruction, and why two warps issue (even / odd chunks);
//   * eight warps (warps w and w+4 share the rows of a tensor-memory lane quarter and take 16 features each) read the
//     arg chunk, evaluate sin/cos, add the energy (compensated sum) and write G = -a sin(arg) (hi, lo) to shared memory
//     as the A operand of the second product;
//   * second product, per chunk: 6 MMAs with N = npcas (G_hi W_lo, G_lo W_hi, G_hi W_hi for two 16-feature steps) into
//     a persistent tensor-memory accumulator, issued by a third warp.
//
// The tensor core adds into its fp32 accumulator with truncation (towards zero, up to one ulp of the running sum per
// MMA).  For arg the small cross terms have their own columns; the gradient accumulator is folded into fp32 global memory
// (round to nearest, red.global.add) every FLUSH_CHUNKS chunks and restarted (measured relative gradient error
// 1.9e-6 at 16 chunks, 3.5e-6 at 32, 5.5e-5 without folding over 512 chunks).
//
// Tensor memory (all 512 columns): arg 2 x 64, gradient npcas (<= 256), x_hi npcas/2 (<= 128).
// Shared memory at npcas = 256: x_lo 64 KB, weight ring 4 x 32.4 KB, G 16 KB, fold staging 12 KB.
//
// The block is a pipeline of stages that wait on one another (weight copy -> first product -> sin/cos -> second product
// -> stage free), and its period is set by the longest of these loops, not by the tensor pipe (about 55 % busy).  Cycle
// counters around every wait showed the loop through the weight ring to be the longest with three stages: the copy of
// chunk c+3 can only start when the second product of chunk c has released its stage.  The ring therefore has four
// stages, paid for with a single G image instead of two (the sin/cos warps wait for the second product of the previous
// chunk before they store, which is off the critical loop); 106.5 -> 95.9 ms on 2.1 M rows x 16,384 features.
//
// Every wait is bounded.  A thread that times out marks the block as failed; the block then skips its stores, waits
// (bounded) for its copies and MMAs in flight, releases its tensor memory and counts the event (qmlb_tc_timeouts).
// A block that finds parameters packed for other sizes does nothing and counts itself the same way.
#include <cuda_fp16.h>
#include <math.h>

#include <atomic>
#include <type_traits>

#include "common.cuh"
#include "sincos.cuh"

namespace {

constexpr int BM = 128;            // rows per block = QMLB_ROW_TILE
constexpr int FC = 32;             // features per chunk
constexpr int EPI_WARPS = 8;       // warps 0-7: sin/cos + flush (warps w and w+4 share the rows of a tensor-memory lane quarter)
constexpr int MMA_WARP = 8;        // warp 8: MMAs of the first product for even chunks (+ tensor-memory allocation), warp 9: MMAs
constexpr int NTHREADS = 384;      // of the second product, warp 10: weight copies, warp 11: first product for odd chunks
#ifndef QMLB_RFF_STAGES
#define QMLB_RFF_STAGES 4
#endif
#ifndef QMLB_RFF_GBUFS
#define QMLB_RFF_GBUFS 1
#endif
#ifndef QMLB_RFF_FOLD_STAGE
#define QMLB_RFF_FOLD_STAGE 1
#endif
constexpr int NSTAGES = QMLB_RFF_STAGES;   // weight chunks in flight
constexpr int G_BUFS = QMLB_RFF_GBUFS;     // G images in flight between the sin/cos warps and the second product
#ifndef QMLB_RFF_FLUSH_CHUNKS
#define QMLB_RFF_FLUSH_CHUNKS 16
#endif
constexpr int FLUSH_CHUNKS = QMLB_RFF_FLUSH_CHUNKS;  // gradient accumulator folded into global memory every this many chunks
constexpr int FOLD_STRIDE = 12;     // floats per row of the fold's staging slab (8 + 4: conflict-free 128-bit row stores)
constexpr int FLUSH_DELAY = G_BUFS;   // ... this many chunks after the group's last chunk (as many as there are G buffers)
constexpr int WAIT_LIMIT = 1 << 22;
constexpr size_t HEADER_BYTES = 256;
constexpr int EXP_CLAMP = 40;

static_assert(BM == QMLB_ROW_TILE, "a block must cover exactly one row tile");

struct PackHeader {
    unsigned max_w_bits;   // bit pattern of max |W|
    unsigned max_a_bits;   // bit pattern of max |alpha| sqrt(2/D)
    int npcas, nfeatures, nchunks, nelements;
};

__device__ int g_rff_tc_timeouts = 0;
// Sequence number of the last launch in which a block gave up on a wait: the remaining blocks of that launch return at
// once instead of each running into the same bounded waits (a launch that cannot make progress then ends within one
// wave of blocks).  The host passes a fresh number with every launch.
__device__ unsigned g_rff_tc_failed_launch = 0;

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
__device__ __forceinline__ void bulk_copy(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(__cvta_generic_to_global(src)), "r"(bytes), "r"(bar)
                 : "memory");
}
// A shared-memory descriptor is kept as two 32-bit words so that stepping through an operand is one 32-bit add on the
// low word (start address >> 4 in bits 0-13, leading byte offset >> 4 in bits 16-29); the high word (stride byte
// offset >> 4, descriptor version 1 at bit 14, no swizzle) never changes and is a compile-time constant at the call sites.
__device__ __forceinline__ uint32_t desc_lo(uint32_t saddr, uint32_t lbo_bytes) { return ((saddr >> 4) & 0x3FFFu) | ((lbo_bytes >> 4) << 16); }

// D[tmem] (+)= A[smem] * B[smem]
__device__ __forceinline__ void mma_ss(uint32_t tmem_d, uint32_t alo, uint32_t ahi, uint32_t blo, uint32_t bhi, uint32_t idesc,
                                       uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "setp.ne.b32 p, %6, 0;\n\t"
        "mov.b64 da, {%1, %2};\n\t"
        "mov.b64 db, {%3, %4};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t}"
        :
        : "r"(tmem_d), "r"(alo), "r"(ahi), "r"(blo), "r"(bhi), "r"(idesc), "r"(accumulate)
        : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]; A: lane = row, 32-bit column = two consecutive k
__device__ __forceinline__ void mma_ts(uint32_t tmem_d, uint32_t tmem_a, uint32_t blo, uint32_t bhi, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 db;\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t}"
        :
        : "r"(tmem_d), "r"(tmem_a), "r"(blo), "r"(bhi), "r"(idesc), "r"(accumulate)
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
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&v)[8]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr), "r"(v[0]), "r"(v[1]),
                 "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7])
                 : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
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
enum {
    W_FULL = 0, W_FREE = W_FULL + NSTAGES, ARG_FULL = W_FREE + NSTAGES, ARG_FREE = ARG_FULL + 2, G_FULL = ARG_FREE + 2,
    G_FREE = G_FULL + G_BUFS, GRAD_FULL = G_FREE + G_BUFS, GRAD_FREE, ALL_DONE, NBARS
};

// tensor-memory columns (512 allocated)
constexpr uint32_t COL_ARG = 0;      // two arg buffers of 2 FC columns: [x_hi W_hi | x_hi W_lo + x_lo W_hi]
constexpr uint32_t COL_GRAD = 128;   // npcas columns
constexpr uint32_t COL_XH = 384;     // npcas/2 columns of packed x hi pairs
constexpr uint32_t TMEM_COLS = 512;

template <int K>
struct Smem {
    static constexpr uint32_t X_HALF = BM * K * 2;              // x lo image
    static constexpr uint32_t W_HALF = K * FC * 2;              // weight hi (or lo) image of one chunk
    static constexpr uint32_t CHUNK = (uint32_t)chunk_bytes(K);
    static constexpr uint32_t G_HALF = BM * FC * 2;             // G hi (or lo) image
    static constexpr uint32_t OFF_XL = 0, OFF_W = X_HALF, OFF_G = OFF_W + NSTAGES * CHUNK;
    static constexpr uint32_t OFF_FOLD = OFF_G + 2 * G_BUFS * G_HALF;   // staging slabs of the gradient fold, one per sin/cos warp
    static constexpr uint32_t FOLD_WARP = 32 * FOLD_STRIDE * 4;
    static constexpr uint32_t TOTAL = OFF_FOLD + (QMLB_RFF_FOLD_STAGE ? EPI_WARPS * FOLD_WARP : 0);
    static_assert(CHUNK % 128 == 0, "chunk images must keep 128-byte alignment");
};

template <int K, bool FAST>
__global__ void __launch_bounds__(NTHREADS, 1)
rff_tc_kernel(const float *__restrict__ x, const int *__restrict__ group_start, const int *__restrict__ slot_of_row, int nel,
              const unsigned char *__restrict__ packed, float *__restrict__ atom_energy, float *__restrict__ grad_x,
              unsigned launch_seq) {
    using S = Smem<K>;
    constexpr int KB = K / 8;
    extern __shared__ unsigned char smem_dyn[];
    __shared__ __align__(8) uint64_t bars[NBARS];
    __shared__ float energy_half[BM];
    __shared__ uint32_t tmem_slot;
    __shared__ unsigned xmax_bits;
    __shared__ int failed;

    const int row0 = blockIdx.x * BM;
    if (row0 >= group_start[nel]) return;
    // A block that cannot deliver its rows fills them with NaN: the caller reads energies and gradients without asking
    // qmlb_tc_timeouts(), and NaN travels through the remaining stages into the molecules concerned.
    auto poison = [&]() {
        const float nan = __int_as_float(0x7fc00000);
        for (int i = threadIdx.x; i < BM * (K + 1); i += NTHREADS) {
            const int r = i / (K + 1), c = i % (K + 1);
            if (c == K) atom_energy[row0 + r] = nan;
            else grad_x[(size_t)(row0 + r) * K + c] = nan;
        }
    };
    if (*reinterpret_cast<volatile unsigned *>(&g_rff_tc_failed_launch) == launch_seq) {
        poison();
        return;
    }
    int e = 0;
    while (e + 1 < nel && row0 >= group_start[e + 1]) ++e;

    const PackHeader *hdr = reinterpret_cast<const PackHeader *>(packed);
    if (hdr->npcas != K || hdr->nelements != nel) {  // parameters packed for another model: refuse, and say so
        if (threadIdx.x == 0) atomicAdd(&g_rff_tc_timeouts, 1);
        poison();
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
        for (int i = 0; i < NSTAGES; ++i) { mbar_init(bar(W_FULL + i), 1); mbar_init(bar(W_FREE + i), 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(bar(ARG_FULL + i), 1); mbar_init(bar(ARG_FREE + i), EPI_WARPS); }
        for (int i = 0; i < G_BUFS; ++i) { mbar_init(bar(G_FULL + i), EPI_WARPS); mbar_init(bar(G_FREE + i), 1); }
        mbar_init(bar(GRAD_FULL), 1); mbar_init(bar(GRAD_FREE), EPI_WARPS); mbar_init(bar(ALL_DONE), 3);
        failed = 0;
        xmax_bits = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == MMA_WARP) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // the gradient rows of the tile start at zero: the accumulator is folded into them with reductions
    for (int i = tid; i < BM * (K / 4); i += NTHREADS)
        *reinterpret_cast<float4 *>(grad_x + (size_t)row0 * K + (size_t)i * 4) = make_float4(0.f, 0.f, 0.f, 0.f);
    {   // largest |x| of the tile -> power-of-two scale
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
        __syncthreads();   // xmax_bits initialised
        if (lane == 0 && m < INFINITY) atomicMax(&xmax_bits, __float_as_uint(m));
    }
    fence_before();
    __syncthreads();
    fence_after();
    // All 512 columns are allocated, so the allocation can only start at column 0 (checked): tensor-memory addresses are
    // then compile-time constants, which keeps them out of the per-MMA instruction stream.
    const uint32_t tmem_alloc = tmem_slot;
    constexpr uint32_t tmem = 0u;
    const bool tmem_ok = tmem_alloc == 0u;
    const int ex = exponent_of(xmax_bits);
    const float sx = pow2i(13 - ex);

    // ---- x lo: canonical K-major shared-memory image (8 rows x 8 k core matrices, k blocks outermost) ----
    for (int i = tid; i < BM * KB; i += NTHREADS) {
        const int r = i % BM, kb = i / BM;
        __align__(16) __half2 lo[4];
        if (slot_of_row[row0 + r] >= 0) {
            const float4 a = *reinterpret_cast<const float4 *>(x + (size_t)(row0 + r) * K + kb * 8);
            const float4 c = *reinterpret_cast<const float4 *>(x + (size_t)(row0 + r) * K + kb * 8 + 4);
            __half2 hi;
            split_half2(a.x * sx, a.y * sx, hi, lo[0]);
            split_half2(a.z * sx, a.w * sx, hi, lo[1]);
            split_half2(c.x * sx, c.y * sx, hi, lo[2]);
            split_half2(c.z * sx, c.w * sx, hi, lo[3]);
        } else {
#pragma unroll
            for (int q = 0; q < 4; ++q) lo[q] = __floats2half2_rn(0.f, 0.f);
        }
        const uint32_t off = (uint32_t)(kb * 16 + (r >> 3)) * 128u + (uint32_t)(r & 7) * 16u;
        *reinterpret_cast<uint4 *>(sptr + S::OFF_XL + off) = *reinterpret_cast<const uint4 *>(lo);
    }
    // ---- x hi: tensor memory, lane = row, column j = (k = 2j, k = 2j + 1) packed; warps w and w + 4 share a lane quarter
    if (warp < EPI_WARPS && tmem_ok) {
        const int r = (warp & 3) * 32 + lane, h = warp >> 2;
        const bool live = slot_of_row[row0 + r] >= 0;
        const uint32_t lane_field = (uint32_t)((warp & 3) * 32) << 16;
        const float *xr = x + (size_t)(row0 + r) * K + h * (K / 2);
#pragma unroll 1
        for (int j = 0; j < K / 32; ++j) {      // 16 k = 8 columns per store
            uint32_t pk[8];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                if (live) v = *reinterpret_cast<const float4 *>(xr + j * 16 + q * 4);
                __half2 h0, h1, l0;
                split_half2(v.x * sx, v.y * sx, h0, l0);
                split_half2(v.z * sx, v.w * sx, h1, l0);
                pk[2 * q] = *reinterpret_cast<uint32_t *>(&h0);
                pk[2 * q + 1] = *reinterpret_cast<uint32_t *>(&h1);
            }
            tmem_st8(tmem + lane_field + COL_XH + (uint32_t)(h * (K / 4) + j * 8), pk);
        }
        tmem_st_wait();
    }
    fence_async_smem();
    fence_before();
    __syncthreads();
    fence_after();
    const float arg_scale = pow2i(ex - 13) * pow2i(ew - 13);     // undoes the operand scales of the first product
    const float grad_scale = pow2i(ea - 13) * pow2i(ew - 13);    // and of the second

    if (warp < EPI_WARPS) {
        // ------------------------------------------------------------------ sin/cos warps
        // thread = (row r, half h): features [16 h, 16 h + 16) of every chunk, gradient columns [h K/2, (h+1) K/2)
        const int r = (warp & 3) * 32 + lane, h = warp >> 2;
        const bool live = slot_of_row[row0 + r] >= 0;
        const uint32_t lane_field = (uint32_t)((warp & 3) * 32) << 16;
        float eacc = 0.f, ecomp = 0.f;  // energy of the row, summed over the chunks with compensation
        bool ok = tmem_ok;
        int next_fold = 0;
        const int last_group = (nchunks - 1) / FLUSH_CHUNKS;
        const unsigned live_rows = __ballot_sync(QMLB_FULL_MASK, live);
        for (int c = 0; c < nchunks && ok; ++c) {
            const int b = c & 1, s = c % NSTAGES, gb = c % G_BUFS;
            const uint32_t par = (uint32_t)(c >> 1) & 1u;
            if (!mbar_wait(bar(ARG_FULL + b), par)) { ok = false; break; }
            fence_after();
            uint32_t av[16], cv[16];   // hi*hi block and cross-term block of this thread's 16 features
            tmem_ld16(tmem + lane_field + COL_ARG + (uint32_t)(b * 2 * FC + h * 16), av);
            tmem_ld16(tmem + lane_field + COL_ARG + (uint32_t)(b * 2 * FC + FC + h * 16), cv);
            tmem_ld_wait();
            fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(ARG_FREE + b));
            // the chunk image (already complete: the MMAs above read it) also carries this chunk's bias and weights;
            // observing its barrier makes the copied bytes visible to this thread's loads
            if (!mbar_wait(bar(W_FULL + s), (uint32_t)(c / NSTAGES) & 1u)) { ok = false; break; }
            const float *prm = reinterpret_cast<const float *>(sptr + S::OFF_W + s * S::CHUNK + 2 * S::W_HALF) + h * 16;
            float echunk = 0.f;
            uint32_t ghi[8], glo[8];
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                float gq[2];
#pragma unroll
                for (int t = 0; t < 2; ++t) {
                    const int f = 2 * q + t;
                    const float a = fmaf(__uint_as_float(av[f]) + __uint_as_float(cv[f]), arg_scale, prm[f]);
                    float sn, cs;
                    if (FAST) __sincosf(a, &sn, &cs);
                    else qmlb_sincos::sincos_one(a, sn, cs);
                    echunk = fmaf(prm[FC + f], cs, echunk);
                    gq[t] = prm[2 * FC + f] * sn;
                }
                __half2 hi, lo;
                split_half2(gq[0], gq[1], hi, lo);
                ghi[q] = *reinterpret_cast<uint32_t *>(&hi);
                glo[q] = *reinterpret_cast<uint32_t *>(&lo);
            }
            // the previous use of this G buffer (chunk c-2) must have been consumed by its MMAs
            if (c >= G_BUFS && !mbar_wait(bar(G_FREE + gb), (uint32_t)((c / G_BUFS) - 1) & 1u)) { ok = false; break; }
            {   // canonical K-major image (K = features): 8 rows x 8 features per 128-byte core matrix, feature blocks outermost
                unsigned char *gbuf = sptr + S::OFF_G + gb * 2 * S::G_HALF;
                const uint32_t off = (uint32_t)(2 * h) * 2048u + (uint32_t)(r >> 3) * 128u + (uint32_t)(r & 7) * 16u;
                *reinterpret_cast<uint4 *>(gbuf + off) = make_uint4(ghi[0], ghi[1], ghi[2], ghi[3]);
                *reinterpret_cast<uint4 *>(gbuf + off + 2048u) = make_uint4(ghi[4], ghi[5], ghi[6], ghi[7]);
                *reinterpret_cast<uint4 *>(gbuf + S::G_HALF + off) = make_uint4(glo[0], glo[1], glo[2], glo[3]);
                *reinterpret_cast<uint4 *>(gbuf + S::G_HALF + off + 2048u) = make_uint4(glo[4], glo[5], glo[6], glo[7]);
            }
            fence_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(G_FULL + gb));
            {   // Kahan step: a plain running sum over nfeatures terms would lose ~sqrt(nfeatures) ulps
                const float y = echunk - ecomp, t = eacc + y;
                ecomp = (t - eacc) - y;
                eacc = t;
            }

            // Fold finished accumulator groups into global memory.  A group ends at chunk E = min(FLUSH_CHUNKS (g+1), nchunks) - 1;
            // it is folded FLUSH_DELAY chunks later (at the last chunk if that comes first): by then its last MMAs have
            // left the pipe, so the wait below is short, and the first product already runs ahead on the next chunks
            // while this warp reads the accumulator, instead of the whole pipeline draining at every fold.
            while (ok && next_fold <= last_group) {
                const int group_end = min((next_fold + 1) * FLUSH_CHUNKS, nchunks) - 1;
                if (c != nchunks - 1 && c < group_end + FLUSH_DELAY) break;
                if (!mbar_wait(bar(GRAD_FULL), (uint32_t)next_fold & 1u)) { ok = false; break; }
                fence_after();
#if QMLB_RFF_FOLD_STAGE
                // The accumulator arrives one row per thread; adding it from there would send 32 separate 16-byte
                // atomics (rows are K floats apart) per instruction.  The warp's tile goes through a staging slab
                // instead, eight columns at a time, so that two lanes cover a whole 32-byte sector of a row.
                float *stg = reinterpret_cast<float *>(sptr + S::OFF_FOLD + warp * S::FOLD_WARP);
#pragma unroll 1
                for (int cc = 0; cc < K / 2; cc += 16) {
                    uint32_t v0[16];
                    tmem_ld16(tmem + lane_field + COL_GRAD + (uint32_t)(h * (K / 2) + cc), v0);
                    tmem_ld_wait();
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        float4 *own = reinterpret_cast<float4 *>(stg + lane * FOLD_STRIDE);
#pragma unroll
                        for (int q = 0; q < 2; ++q) {
                            const int e = 8 * half + 4 * q;
                            own[q] = make_float4(__uint_as_float(v0[e]) * grad_scale, __uint_as_float(v0[e + 1]) * grad_scale,
                                                 __uint_as_float(v0[e + 2]) * grad_scale, __uint_as_float(v0[e + 3]) * grad_scale);
                        }
                        __syncwarp();
#pragma unroll
                        for (int j = 0; j < 2; ++j) {
                            const int rr = 16 * j + (lane >> 1), c4 = (lane & 1) * 4;
                            const float4 t = *reinterpret_cast<const float4 *>(stg + rr * FOLD_STRIDE + c4);
                            if ((live_rows >> rr) & 1u)   // rows of the padding keep their zeros
                                red_add4(grad_x + (size_t)(row0 + (warp & 3) * 32 + rr) * K + h * (K / 2) + cc + 8 * half + c4, t.x, t.y, t.z, t.w);
                        }
                        __syncwarp();
                    }
                }
#else
                float *dst = grad_x + (size_t)(row0 + r) * K + h * (K / 2);
#pragma unroll 1
                for (int cc = 0; cc < K / 2; cc += 16) {
                    uint32_t v0[16];
                    tmem_ld16(tmem + lane_field + COL_GRAD + (uint32_t)(h * (K / 2) + cc), v0);
                    tmem_ld_wait();
                    if (live) {  // rows of the padding keep their zeros
#pragma unroll
                        for (int q = 0; q < 4; ++q)
                            red_add4(dst + cc + 4 * q, __uint_as_float(v0[4 * q]) * grad_scale, __uint_as_float(v0[4 * q + 1]) * grad_scale,
                                     __uint_as_float(v0[4 * q + 2]) * grad_scale, __uint_as_float(v0[4 * q + 3]) * grad_scale);
                    }
                }
#endif
                fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(GRAD_FREE));
                ++next_fold;
            }
        }
        if (!ok) failed = 1;  // benign race: every writer stores 1
        // the two halves of a row add their energies through shared memory
        if (h == 1) energy_half[r] = eacc;
        asm volatile("bar.sync 1, %0;" ::"n"(EPI_WARPS * 32) : "memory");
        if (h == 0 && ok) atom_energy[row0 + r] = live ? eacc + energy_half[r] : 0.f;
    } else if (warp == MMA_WARP || warp == MMA_WARP + 3) {
        // ------------------------------------------------------------------ MMAs of the first product: arg = x W
        // x_hi multiplies [W_hi | W_lo] in one N = 2 FC instruction (the lo image follows the hi image at the feature-block
        // stride) and x_lo multiplies W_hi with N = FC into the cross-term columns; two warps issue, one the even chunks
        // (arg buffer 0), one the odd chunks (arg buffer 1); the whole warp runs the loop in uniform control flow and only
        // the MMA and commit instructions are left to lane 0.
        // D = F32, A = B = F16, A K-major, B MN-major (N = features)
        constexpr uint32_t idesc_wide = (1u << 4) | (1u << 16) | ((uint32_t)((2 * FC) >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
        constexpr uint32_t idesc_one = (1u << 4) | (1u << 16) | ((uint32_t)(FC >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
        static_assert(Smem<K>::W_HALF == (uint32_t)(FC / 8) * KB * 128u, "the lo image must continue the feature-block stride");
        // A from shared memory: 16 k per step = 2 k blocks 2048 B apart, row groups 128 B apart; from tensor memory:
        // 8 columns per step.  B: 2 k blocks 128 B apart, feature blocks KB*128 B apart
        const uint32_t a_lo = desc_lo(sbase + S::OFF_XL, 2048u);
        constexpr uint32_t a_hi = (128u >> 4) | (1u << 14), b_hi = (((uint32_t)KB * 128u) >> 4) | (1u << 14);
        constexpr uint32_t xh = tmem + COL_XH;
        bool ok = tmem_ok;
        auto chunks_of_parity = [&](auto parity) {
            constexpr int b = decltype(parity)::value;
            constexpr uint32_t acc = tmem + COL_ARG + (uint32_t)(b * 2 * FC);
            for (int c = b; c < nchunks && ok; c += 2) {
                const int s = c % NSTAGES;
                bool w = mbar_wait(bar(W_FULL + s), (uint32_t)(c / NSTAGES) & 1u);
                // arg chunks run up to two ahead of the sin/cos warps
                if (c >= 2) w = mbar_wait(bar(ARG_FREE + b), (uint32_t)((c >> 1) - 1) & 1u) && w;
                if (!__all_sync(QMLB_FULL_MASK, w)) { ok = false; break; }
                fence_after();
                const uint32_t wh_lo = desc_lo(sbase + S::OFF_W + s * S::CHUNK, 128u);
                if (lane == 0) {
#pragma unroll
                    for (int ks = 0; ks < K / 16; ++ks) mma_ts(acc, xh + ks * 8, wh_lo + ks * 16, b_hi, idesc_wide, ks > 0 ? 1u : 0u);
#pragma unroll
                    for (int ks = 0; ks < K / 16; ++ks) mma_ss(acc + FC, a_lo + ks * 256, a_hi, wh_lo + ks * 16, b_hi, idesc_one, 1u);
                    mma_commit(bar(ARG_FULL + b));
                }
                __syncwarp();
            }
        };
        if (warp == MMA_WARP) chunks_of_parity(std::integral_constant<int, 0>{});
        else chunks_of_parity(std::integral_constant<int, 1>{});
        // everything issued by this warp must have left the tensor pipe before the tensor memory is released
        if (lane == 0) mma_commit(bar(ALL_DONE));
        __syncwarp();
        if (!mbar_wait(bar(ALL_DONE), 0u)) ok = false;
        if (!ok) failed = 1;
    } else if (warp == MMA_WARP + 1) {
        // ------------------------------------------------------------------ MMAs of the second product: grad += G W^T
        // both operands K-major (K = features), N = npcas; A = G: 16 features per step = 2 feature blocks 2048 B apart,
        // row groups 128 B apart; B: 2 feature blocks KB*128 B apart, k blocks 128 B apart
        constexpr uint32_t idesc2 = (1u << 4) | ((uint32_t)(K >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
        constexpr uint32_t ab_hi = (128u >> 4) | (1u << 14);
        constexpr uint32_t grad = tmem + COL_GRAD;
        bool ok = tmem_ok;
        for (int c = 0; c < nchunks && ok; ++c) {
            const int s = c % NSTAGES, gb = c % G_BUFS;
            const int group = c / FLUSH_CHUNKS;
            const bool first = (c % FLUSH_CHUNKS) == 0;
            bool w = mbar_wait(bar(G_FULL + gb), (uint32_t)(c / G_BUFS) & 1u);
            if (first && group > 0) w = mbar_wait(bar(GRAD_FREE), (uint32_t)(group - 1) & 1u) && w;
            if (!__all_sync(QMLB_FULL_MASK, w)) { ok = false; break; }
            fence_after();
            const uint32_t wh_lo = desc_lo(sbase + S::OFF_W + s * S::CHUNK, (uint32_t)KB * 128u), wl_lo = wh_lo + (S::W_HALF >> 4);
            const uint32_t gh_lo = desc_lo(sbase + S::OFF_G + gb * 2 * S::G_HALF, 2048u), gl_lo = gh_lo + (S::G_HALF >> 4);
            if (lane == 0) {
#pragma unroll
                for (int ks = 0; ks < FC / 16; ++ks) {
                    const uint32_t step = (uint32_t)ks * ((2u * KB * 128u) >> 4);
                    mma_ss(grad, gh_lo + ks * 256, ab_hi, wl_lo + step, ab_hi, idesc2, (first && ks == 0) ? 0u : 1u);
                    mma_ss(grad, gl_lo + ks * 256, ab_hi, wh_lo + step, ab_hi, idesc2, 1u);
                    mma_ss(grad, gh_lo + ks * 256, ab_hi, wh_lo + step, ab_hi, idesc2, 1u);
                }
                mma_commit(bar(W_FREE + s));
                mma_commit(bar(G_FREE + gb));
                if ((c % FLUSH_CHUNKS) == FLUSH_CHUNKS - 1 || c == nchunks - 1) mma_commit(bar(GRAD_FULL));
            }
            __syncwarp();
        }
        if (lane == 0) mma_commit(bar(ALL_DONE));
        __syncwarp();
        if (!mbar_wait(bar(ALL_DONE), 0u)) ok = false;
        if (!ok) failed = 1;
    } else if (warp == MMA_WARP + 2) {
        // ------------------------------------------------------------------ weight copies
        if (lane == 0) {
            bool ok = tmem_ok;
            int issued = 0;
            for (int c = 0; c < nchunks && ok; ++c) {
                const int s = c % NSTAGES;
                if (c >= NSTAGES && !mbar_wait(bar(W_FREE + s), (uint32_t)((c / NSTAGES) - 1) & 1u)) { ok = false; break; }
                mbar_expect_tx(bar(W_FULL + s), S::CHUNK);
                bulk_copy(sbase + S::OFF_W + s * S::CHUNK, blobs + (size_t)c * S::CHUNK, S::CHUNK, bar(W_FULL + s));
                issued = c + 1;
            }
            // no copy may still be in flight when the block leaves
            for (int c = max(0, issued - NSTAGES); c < issued; ++c)
                if (!mbar_wait(bar(W_FULL + (c % NSTAGES)), (uint32_t)(c / NSTAGES) & 1u)) ok = false;
            if (!ok) failed = 1;
        }
    }
    __syncwarp();
    fence_before();
    __syncthreads();
    fence_after();
    if (failed) {
        poison();
        if (tid == 0) {
            atomicAdd(&g_rff_tc_timeouts, 1);
            atomicExch(&g_rff_tc_failed_launch, launch_seq);
        }
    }
    if (warp == MMA_WARP) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_alloc), "r"(TMEM_COLS) : "memory");
    }
}

template <int K>
int launch_rff_tc(const float *x, const int *group_start, const int *slot_of_row, int nel, size_t rows_cap,
                  const unsigned char *packed, int fast, float *atom_energy, float *grad_x, cudaStream_t st) {
    const size_t smem = Smem<K>::TOTAL + 128;
    const unsigned grid = (unsigned)(rows_cap / BM);
    static std::atomic<unsigned> launches{0};
    const unsigned seq = ++launches;   // never 0, the initial value of the device-side marker (wraps after 2^32 launches)
    if (fast) {
        if (int rc = qmlb::ensure_smem(rff_tc_kernel<K, true>, smem, "qmlb_rff_energy_grad_tc")) return rc;
        rff_tc_kernel<K, true><<<grid, NTHREADS, smem, st>>>(x, group_start, slot_of_row, nel, packed, atom_energy, grad_x, seq);
    } else {
        if (int rc = qmlb::ensure_smem(rff_tc_kernel<K, false>, smem, "qmlb_rff_energy_grad_tc")) return rc;
        rff_tc_kernel<K, false><<<grid, NTHREADS, smem, st>>>(x, group_start, slot_of_row, nel, packed, atom_energy, grad_x, seq);
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
