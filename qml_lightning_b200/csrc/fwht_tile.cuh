// Fast Walsh-Hadamard transform of a vector of N = 2^n floats (16 <= N <= 512) held by L = N/16 lanes of a warp with 16
// registers each: four butterfly stages in registers, a transposition of the 16 x L tile through a per-warp
// shared-memory slab (128-bit stores, conflict-free 32-bit loads, row stride 20 floats), the remaining stages in
// registers again and, for N = 512 only, one warp-shuffle stage.  A transform flips the register order between the
// natural one ("layout A": lane l holds elements 16 l .. 16 l + 15) and the transposed one ("layout B", element index
// given by layoutB_n); a warp works on V = 32/L vectors at once.  Shared by the fused prediction kernel and the
// training-row kernels.
#pragma once

#include "common.cuh"

namespace qmlb_fwht {

constexpr int ROWSTRIDE = 20;  // floats per 16-element row in the transposition slab

template <int LOG2N>
struct Cfg {
    static constexpr int N = 1 << LOG2N;
    static constexpr int LB = LOG2N - 4;              // lane bits of a vector
    static constexpr int L = 1 << LB;                 // lanes per vector
    static constexpr int V = 32 / L;                  // vectors (stacks) per warp
    static constexpr int LBT = LB > 4 ? 4 : LB;       // bits exchanged by the transposition
    static constexpr int ROWS = L;                    // rows of 16 in the slab
    static constexpr int RAW = ROWS * ROWSTRIDE + (ROWS > 16 ? 16 : 0);
    // slab stride: distinct bank ranges for the V vectors of a warp (V*L = 32 lanes read L consecutive words each)
    static constexpr int SLAB = V == 1 ? RAW : (V == 2 ? RAW + 16 : (V == 4 ? RAW + 8 : RAW + 4));
    static constexpr int WARP_FLOATS = V * SLAB;
};

// position (lane-in-vector * 16 + register) -> element index n, for the transposed layout B
__host__ __device__ inline int layoutB_n(int log2n, int pos) {
    const int LB = log2n - 4;
    const int l = pos >> 4, e = pos & 15;
    if (LB <= 4) {
        const int L = 1 << LB;
        return (e & (L - 1)) * 16 + ((e >> LB) << LB) + l;
    }
    return ((l & 16) | e) * 16 + (l & 15);
}

__device__ __forceinline__ void butterfly(float &a, float &b) {
    const float t = a;
    a = t + b;
    b = t - b;
}

// Two butterflies at once on the packed fp32x2 pipe of sm_100 (add.f32x2 / fma.f32x2): (a0,a1) and (b0,b1) are adjacent
// register pairs, which holds for every stage except the one that pairs neighbouring registers.
__device__ __forceinline__ void butterfly2(float &a0, float &a1, float &b0, float &b1) {
    const float2 a = make_float2(a0, a1), b = make_float2(b0, b1);
    const float2 s = __fadd2_rn(a, b);
    const float2 d = __ffma2_rn(b, make_float2(-1.0f, -1.0f), a);  // a - b, rounded once like a subtraction
    a0 = s.x; a1 = s.y; b0 = d.x; b1 = d.y;
}

template <int BITS>
__device__ __forceinline__ void fwht_regs(float (&u)[16]) {
#pragma unroll
    for (int h = 1; h < (1 << BITS); h <<= 1) {
        if (h >= 2) {
#pragma unroll
            for (int i = 0; i < 16; i += 2)
                if ((i & h) == 0) butterfly2(u[i], u[i + 1], u[i | h], u[(i | h) + 1]);
            continue;
        }
#pragma unroll
        for (int i = 0; i < 16; ++i)
            if ((i & h) == 0) butterfly(u[i], u[i | h]);
    }
}

template <int LOG2N>
struct Xpose {
    using C = Cfg<LOG2N>;
    // shared-memory offset of lane l's row in layout A, and of lane l's column base in layout B
    __device__ static __forceinline__ int a_base(int l) { return l * ROWSTRIDE + (l >> 4) * 16; }
    __device__ static __forceinline__ int b_base(int l) {
        if (C::LB <= 4) return l;
        return (l >> 4) * (16 * ROWSTRIDE + 16) + (l & 15);
    }
    // constant part of the layout-B address of register e
    __device__ static __forceinline__ constexpr int b_const(int e) {
        return C::LB <= 4 ? (e & (C::L - 1)) * ROWSTRIDE + ((e >> C::LB) << C::LB) : e * ROWSTRIDE;
    }
    __device__ static __forceinline__ void a_to_b(float (&u)[16], float *slab, int l) {
        float4 *w = reinterpret_cast<float4 *>(slab + a_base(l));
#pragma unroll
        for (int q = 0; q < 4; ++q) w[q] = make_float4(u[4 * q], u[4 * q + 1], u[4 * q + 2], u[4 * q + 3]);
        __syncwarp();
        const float *r = slab + b_base(l);
#pragma unroll
        for (int e = 0; e < 16; ++e) u[e] = r[b_const(e)];
        __syncwarp();
    }
    __device__ static __forceinline__ void b_to_a(float (&u)[16], float *slab, int l) {
        float *w = slab + b_base(l);
#pragma unroll
        for (int e = 0; e < 16; ++e) w[b_const(e)] = u[e];
        __syncwarp();
        const float4 *r = reinterpret_cast<const float4 *>(slab + a_base(l));
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const float4 t = r[q];
            u[4 * q] = t.x; u[4 * q + 1] = t.y; u[4 * q + 2] = t.z; u[4 * q + 3] = t.w;
        }
        __syncwarp();
    }
};

// butterfly across lanes l and l^16 (only N = 512)
__device__ __forceinline__ void lane16_stage(float (&u)[16], int lane) {
    const float sgn = (lane & 16) ? -1.0f : 1.0f;
#pragma unroll
    for (int e = 0; e < 16; ++e) {
        const float o = __shfl_xor_sync(QMLB_FULL_MASK, u[e], 16);
        u[e] = fmaf(sgn, u[e], o);
    }
}

// One unnormalised FWHT; flips the layout (A -> B when from_a, else B -> A).
template <int LOG2N>
__device__ __forceinline__ void fwht_flip(float (&u)[16], float *slab, int l, int lane, bool from_a) {
    using C = Cfg<LOG2N>;
    if (C::LB == 0) {  // N = 16: everything in registers, layouts coincide
        fwht_regs<4>(u);
        return;
    }
    if (from_a) {
        fwht_regs<4>(u);
        Xpose<LOG2N>::a_to_b(u, slab, l);
        fwht_regs<C::LBT>(u);
        if (C::LB == 5) lane16_stage(u, lane);
    } else {
        if (C::LB == 5) lane16_stage(u, lane);
        fwht_regs<C::LBT>(u);
        Xpose<LOG2N>::b_to_a(u, slab, l);
        fwht_regs<4>(u);
    }
}

}  // namespace qmlb_fwht
