// Test program for the shared-memory operand layouts of tcgen05.mma (kind::f16, M = 128, K = 16 per instruction) that the
// tensor-core kernels of this package rely on.  Part 1 fills A and B in a given layout, runs one accumulation chain and
// compares the tensor-memory result with a host product (exact: small dyadic values): the no-swizzle K-major core-matrix
// layout, the SWIZZLE_128B K-major layout and the SWIZZLE_128B MN-major layout.  Parts 2 and 3 time long chains between
// two clock64() reads: cycles per instruction against N, for A in shared or tensor memory, one or two accumulators, one
// to four issuing warps.  Every wait is bounded.  Output: one line per case; a line with "status 1" or a non-zero error
// means failure (tests/test_gpu_mma_operand_layouts.py checks them).
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <vector>

#define CK(x) do { cudaError_t e = (x); if (e != cudaSuccess) { printf("CUDA error %s at %s:%d\n", cudaGetErrorString(e), __FILE__, __LINE__); exit(1); } } while (0)

constexpr int WAIT_LIMIT = 1 << 20;
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count)); }
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (int it = 0; it < WAIT_LIMIT; ++it) {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}
__device__ __forceinline__ void mma_ss(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t bar) { asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory"); }
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&v)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];" : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]) : "r"(taddr));
}

// mode: layout of the operands
//  0: A, B K-major no swizzle (8x8 core matrices; core matrices of one 8-k block contiguous over rows: SBO = 128 B between
//     row groups, LBO = rows*16 B between k blocks)
//  1: A, B K-major SWIZZLE_128B (rows of 64 k = 128 B, 8-row atoms of 1024 B, SBO = 1024)
//  2: A K-major SW128, B MN-major SW128 (rows = k, 64 n = 128 B per row, 8-k atoms of 1024 B, SBO = 1024); N must be 64
//  3: as 2 with N = 32 (half of every 128-byte row is used)
struct Params { int mode, N, K, reps; };

__host__ __device__ inline uint32_t off_kmajor_noswz(int row, int k, int rows) { return (uint32_t)((k / 8) * rows * 16 + (row / 8) * 128 + (row % 8) * 16 + (k % 8) * 2); }
__host__ __device__ inline uint32_t off_sw128(int row, int col) {   // row-major rows of 64 elements, 128B swizzle
    return (uint32_t)((row / 8) * 1024 + (row % 8) * 128 + (((col / 8) ^ (row % 8)) * 16) + (col % 8) * 2);
}

__global__ void __launch_bounds__(128, 1) layout_check_kernel(const __half *A, const __half *B, float *D, long long *cycles, int *status, Params P) {
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t bar;
    __shared__ uint32_t tmem_slot;
    const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
    unsigned char *sp = smem_raw + (sbase - smem_u32(smem_raw));
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int M = 128, N = P.N, K = P.K;     // K = 64 for swizzled modes (one atom wide), multiple of 16
    const uint32_t offA = 0, offB = 32768;
    // fill: A[m][k] (row-major global), B[n][k] (row-major global: B as N x K)
    for (int i = tid; i < M * K; i += 128) {
        const int m = i / K, k = i % K;
        const uint32_t o = P.mode == 0 ? off_kmajor_noswz(m, k, M) : off_sw128(m, k);
        *reinterpret_cast<__half *>(sp + offA + o) = A[i];
    }
    for (int i = tid; i < N * K; i += 128) {
        const int n = i / K, k = i % K;
        uint32_t o;
        if (P.mode == 0) o = off_kmajor_noswz(n, k, N);
        else if (P.mode == 1) o = off_sw128(n, k);
        else o = off_sw128(k, n);             // MN-major: row = k, column = n
        *reinterpret_cast<__half *>(sp + offB + o) = B[i];
    }
    if (tid == 0) { mbar_init(smem_u32(&bar), 1); asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = tmem_slot;
    long long t0 = 0, t1 = 0;
    bool ok = true;
    if (warp == 0) {
        // instruction descriptor: D f32 (bit 4), A/B f16 (0), a_major bit 15, b_major bit 16 (1 = MN-major), N>>3 at 17, M>>4 at 24
        uint32_t idesc = (1u << 4) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
        if (P.mode >= 2) idesc |= (1u << 16);
        const uint64_t ver = 1ull << 46;
        if (lane == 0) {
            t0 = clock64();
            for (int r = 0; r < P.reps; ++r) {
                for (int ks = 0; ks < K / 16; ++ks) {
                    uint64_t da, db;
                    if (P.mode == 0) {
                        da = (uint64_t)(((sbase + offA) >> 4) + ks * ((2 * M * 16) >> 4)) | ((uint64_t)((M * 16) >> 4) << 16) | ((uint64_t)(128 >> 4) << 32) | ver;
                        db = (uint64_t)(((sbase + offB) >> 4) + ks * ((2 * N * 16) >> 4)) | ((uint64_t)((N * 16) >> 4) << 16) | ((uint64_t)(128 >> 4) << 32) | ver;
                    } else {
                        const uint64_t sw128 = 2ull << 61;
                        da = (uint64_t)(((sbase + offA) >> 4) + ks * 2) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | ver | sw128;
                        if (P.mode == 1) db = (uint64_t)(((sbase + offB) >> 4) + ks * 2) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | ver | sw128;
                        else db = (uint64_t)(((sbase + offB) >> 4) + ks * (2048 >> 4)) | ((uint64_t)(1024 >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) | ver | sw128;
                    }
                    mma_ss(tmem, da, db, idesc, (r > 0 || ks > 0) ? 1u : 0u);
                }
            }
            mma_commit(smem_u32(&bar));
        }
        __syncwarp();
        ok = mbar_wait(smem_u32(&bar), 0u);
        if (lane == 0) t1 = clock64();
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (tid == 0) { cycles[0] = t1 - t0; status[0] = ok ? 0 : 1; }
    // read D: thread = row (lane field), all N columns
    if (ok || warp != 0) {
        const uint32_t lane_field = (uint32_t)(warp * 32) << 16;
        for (int c = 0; c < N; c += 8) {
            uint32_t v[8];
            tmem_ld8(tmem + lane_field + (uint32_t)c, v);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            for (int q = 0; q < 8; ++q) D[(size_t)tid * N + c + q] = __uint_as_float(v[q]);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
}


__device__ __forceinline__ void mma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(tmem_d), "r"(tmem_a), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
// timing only: a_tmem 0/1, swz 0/1, nacc accumulators used in rotation, K = 64 (4 MMAs per round)
__global__ void __launch_bounds__(128, 1) time_kernel(long long *cycles, int *status, int N, int a_tmem, int swz, int nacc, int reps) {
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t bar;
    __shared__ uint32_t tmem_slot;
    const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    for (int i = tid; i < (32768 + 65536) / 4; i += 128) reinterpret_cast<uint32_t *>(smem_raw + (sbase - smem_u32(smem_raw)))[i] = 0x3c003c00u;
    const int M = 128;
    const uint32_t offA = 0, offB = 32768;
    if (tid == 0) { mbar_init(smem_u32(&bar), 1); asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = tmem_slot;
    long long t0 = 0, t1 = 0;
    bool ok = true;
    if (warp == 0) {
        const uint32_t idesc = (1u << 4) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
        const uint64_t ver = 1ull << 46, sw128 = 2ull << 61;
        if (lane == 0) {
            t0 = clock64();
            for (int r = 0; r < reps; ++r) {
                const uint32_t d = tmem + (uint32_t)((r % nacc) * N);
                for (int ks = 0; ks < 4; ++ks) {
                    uint64_t da, db;
                    if (!swz) {
                        da = (uint64_t)(((sbase + offA) >> 4) + ks * ((2 * M * 16) >> 4)) | ((uint64_t)((M * 16) >> 4) << 16) | ((uint64_t)(128 >> 4) << 32) | ver;
                        db = (uint64_t)(((sbase + offB) >> 4) + ks * ((2 * N * 16) >> 4)) | ((uint64_t)((N * 16) >> 4) << 16) | ((uint64_t)(128 >> 4) << 32) | ver;
                    } else {
                        da = (uint64_t)(((sbase + offA) >> 4) + ks * 2) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | ver | sw128;
                        db = (uint64_t)(((sbase + offB) >> 4) + ks * 2) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | ver | sw128;
                    }
                    if (a_tmem) mma_ts(d, tmem + 480u + ks * 8, db, idesc, 1u);
                    else mma_ss(d, da, db, idesc, 1u);
                }
            }
            mma_commit(smem_u32(&bar));
        }
        __syncwarp();
        ok = mbar_wait(smem_u32(&bar), 0u);
        if (lane == 0) t1 = clock64();
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (tid == 0) { cycles[0] = t1 - t0; status[0] = ok ? 0 : 1; }
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
}

// timing only: `nw` warps issue concurrently, each into its own accumulator (N columns each), A in tensor memory or shared memory
__global__ void __launch_bounds__(256, 1) time_multi_kernel(long long *cycles, int *status, int N, int a_tmem, int nw, int reps) {
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t bar[8];
    __shared__ uint32_t tmem_slot;
    __shared__ long long tstart[8], tend[8];
    const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    for (int i = tid; i < (32768 + 65536) / 4; i += 256) reinterpret_cast<uint32_t *>(smem_raw + (sbase - smem_u32(smem_raw)))[i] = 0x3c003c00u;
    const int M = 128;
    const uint32_t offA = 0, offB = 32768;
    if (tid == 0) { for (int w = 0; w < 8; ++w) mbar_init(smem_u32(&bar[w]), 1); asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = tmem_slot;
    bool ok = true;
    if (warp < nw) {
        const uint32_t idesc = (1u << 4) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
        const uint64_t ver = 1ull << 46;
        if (lane == 0) {
            const uint32_t d = tmem + (uint32_t)(warp * N);
            tstart[warp] = clock64();
            for (int r = 0; r < reps; ++r) {
#pragma unroll
                for (int ks = 0; ks < 4; ++ks) {
                    const uint64_t da = (uint64_t)(((sbase + offA) >> 4) + ks * ((2 * M * 16) >> 4)) | ((uint64_t)((M * 16) >> 4) << 16) | ((uint64_t)(128 >> 4) << 32) | ver;
                    const uint64_t db = (uint64_t)(((sbase + offB) >> 4) + ks * ((2 * N * 16) >> 4)) | ((uint64_t)((N * 16) >> 4) << 16) | ((uint64_t)(128 >> 4) << 32) | ver;
                    if (a_tmem) mma_ts(d, tmem + 480u + ks * 8, db, idesc, 1u);
                    else mma_ss(d, da, db, idesc, 1u);
                }
            }
            mma_commit(smem_u32(&bar[warp]));
        }
        __syncwarp();
        ok = mbar_wait(smem_u32(&bar[warp]), 0u);
        if (lane == 0) tend[warp] = clock64();
        if (!ok) status[0] = 1;
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (tid == 0) {
        long long a = tstart[0], b = tend[0];
        for (int w = 1; w < nw; ++w) { a = a < tstart[w] ? a : tstart[w]; b = b > tend[w] ? b : tend[w]; }
        cycles[0] = b - a;
    }
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
}

int main(int argc, char **argv) {
    const int modes[][3] = {{0, 256, 64}, {1, 256, 64}, {0, 64, 64}, {1, 64, 64}, {2, 64, 64}, {3, 32, 64}, {0, 32, 64}, {1, 32, 64}};
    for (auto &mc : modes) {
        Params P{mc[0], mc[1], mc[2], 1};
        const int M = 128, N = P.N, K = P.K;
        std::vector<__half> hA(M * K), hB(N * K);
        std::vector<float> fA(M * K), fB(N * K);
        srand(1);
        for (int i = 0; i < M * K; ++i) { fA[i] = (float)((rand() % 17) - 8) / 8.f; hA[i] = __float2half(fA[i]); }
        for (int i = 0; i < N * K; ++i) { fB[i] = (float)((rand() % 13) - 6) / 4.f; hB[i] = __float2half(fB[i]); }
        __half *dA, *dB; float *dD; long long *dc; int *ds;
        CK(cudaMalloc(&dA, M * K * 2)); CK(cudaMalloc(&dB, N * K * 2)); CK(cudaMalloc(&dD, M * N * 4)); CK(cudaMalloc(&dc, 8)); CK(cudaMalloc(&ds, 4));
        CK(cudaMemcpy(dA, hA.data(), M * K * 2, cudaMemcpyHostToDevice)); CK(cudaMemcpy(dB, hB.data(), N * K * 2, cudaMemcpyHostToDevice));
        const size_t smem = 32768 + 65536 + 1024;
        CK(cudaFuncSetAttribute(layout_check_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        layout_check_kernel<<<1, 128, smem>>>(dA, dB, dD, dc, ds, P);
        CK(cudaDeviceSynchronize());
        std::vector<float> hD(M * N);
        CK(cudaMemcpy(hD.data(), dD, M * N * 4, cudaMemcpyDeviceToHost));
        double maxerr = 0;
        for (int m = 0; m < M; ++m)
            for (int n = 0; n < N; ++n) {
                double ref = 0;
                for (int k = 0; k < K; ++k) ref += (double)fA[m * K + k] * fB[n * K + k];
                maxerr = fmax(maxerr, fabs(ref - hD[m * N + n]));
            }
        int st; CK(cudaMemcpy(&st, ds, 4, cudaMemcpyDeviceToHost));
        // timing: many repetitions
        P.reps = 256;
        layout_check_kernel<<<1, 128, smem>>>(dA, dB, dD, dc, ds, P);
        CK(cudaDeviceSynchronize());
        long long cyc; CK(cudaMemcpy(&cyc, dc, 8, cudaMemcpyDeviceToHost));
        printf("mode %d N %3d K %d: max |err| %.3g status %d, %.1f cycles per MMA (ideal math %d)\n", P.mode, N, K, maxerr, st,
               (double)cyc / (256.0 * (K / 16)), N / 2);
        cudaFree(dA); cudaFree(dB); cudaFree(dD); cudaFree(dc); cudaFree(ds);
    }

    {
        long long *dc; int *ds;
        CK(cudaMalloc(&dc, 8)); CK(cudaMalloc(&ds, 4));
        const size_t smem = 32768 + 65536 + 1024;
        CK(cudaFuncSetAttribute(time_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        const int Ns[] = {8, 16, 32, 64, 96, 128, 192, 256};
        for (int a_tmem = 0; a_tmem < 2; ++a_tmem)
            for (int swz = 0; swz < 2; ++swz)
                for (int nacc = 1; nacc <= 2; ++nacc)
                    for (int N : Ns) {
                        if (nacc * N > 448) continue;
                        const int reps = 512;
                        time_kernel<<<1, 128, smem>>>(dc, ds, N, a_tmem, swz, nacc, reps);
                        CK(cudaDeviceSynchronize());
                        long long cyc; int st;
                        CK(cudaMemcpy(&cyc, dc, 8, cudaMemcpyDeviceToHost)); CK(cudaMemcpy(&st, ds, 4, cudaMemcpyDeviceToHost));
                        printf("time: A %s, %s, accumulators %d, N %3d: %.1f cycles per MMA (math %d) status %d\n", a_tmem ? "tmem" : "smem",
                               swz ? "sw128" : "noswz", nacc, N, (double)cyc / (reps * 4.0), N / 2, st);
                    }
    }

    {
        long long *dc; int *ds;
        CK(cudaMalloc(&dc, 8)); CK(cudaMalloc(&ds, 4));
        const size_t smem = 32768 + 65536 + 1024;
        CK(cudaFuncSetAttribute(time_multi_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        const int Ns[] = {32, 64, 128, 256};
        for (int a_tmem = 0; a_tmem < 2; ++a_tmem)
            for (int nw = 1; nw <= 4; ++nw)
                for (int N : Ns) {
                    if (nw * N > 448) continue;
                    const int reps = 512;
                    CK(cudaMemset(ds, 0, 4));
                    time_multi_kernel<<<1, 256, smem>>>(dc, ds, N, a_tmem, nw, reps);
                    CK(cudaDeviceSynchronize());
                    long long cyc; int st;
                    CK(cudaMemcpy(&cyc, dc, 8, cudaMemcpyDeviceToHost)); CK(cudaMemcpy(&st, ds, 4, cudaMemcpyDeviceToHost));
                    printf("multi: A %s, issuing warps %d, N %3d: %.1f cycles per MMA overall (math %d) status %d\n", a_tmem ? "tmem" : "smem",
                           nw, N, (double)cyc / (reps * 4.0 * nw), N / 2, st);
                }
    }
    return 0;
}
