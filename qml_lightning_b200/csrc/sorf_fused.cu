// Fused SORF energy + gradient kernel (sm_100a).
//
// Replaces, per atom row, the upstream chain
//   get_SORF_coefficients -> get_cos_features -> matmul(Ztest, alpha)            (models/hadamard_features.py:113-121)
// and its autograd backward (cuda/torchscript/SORF.cpp:89-101,121-133) by one pass that never writes the
// [atoms, nstacks*npcas] coefficient tensor: for every stack s
//   u = (H D_{T-1,s} ... H D_{0,s}) x ;  arg = scale*u + b_s ;  E += alpha_s . cos(arg) ;
//   g = -alpha_s sin(arg) ;  grad_x += (D_0 H ... D_{T-1} H) g            (scale applied once at the end)
// with scale = (sqrt(N)/sigma) * N^(-T/2).
//
// Data layout.  A vector of N = 2^n floats is held by L = N/16 lanes, 16 registers per lane; a warp therefore
// works on V = 32/L stacks of the same atom at once.  The fast Walsh-Hadamard transform runs 4 butterfly stages
// in registers, transposes the 16 x L tile through a per-warp shared-memory slab (128-bit stores, conflict-free
// 32-bit loads, row stride 20 floats), runs the remaining stages in registers again and, for N = 512 only, one
// warp-shuffle stage for the last bit.  The transposed register order ("layout B") is kept through the
// cos/sin step, so the backward transform starts from it and ends in the natural order ("layout A"):
// two transpositions per stack in total.  Sign diagonals, bias and weights are pre-permuted once per model by
// qmlb_sorf_pack so that every lane reads 16 consecutive floats.  The kernel is bound by instruction issue, so
// butterflies (except the stage that pairs neighbouring registers) and the element-wise steps use the packed fp32x2
// instructions of sm_100 (add.f32x2 / mul.f32x2 / fma.f32x2 through __fadd2_rn / __fmul2_rn / __ffma2_rn): same
// rounding per component, half the instructions (measured 13.3 -> 12.7 ms on 210,000 atoms x 256 stacks, N = 256).
#include <math.h>

#include "common.cuh"
#include "fwht_tile.cuh"
#include "sincos.cuh"

namespace {

using namespace qmlb_fwht;

#ifndef SORF_WARPS
#define SORF_WARPS 4
#endif
#ifndef SORF_MINB
#define SORF_MINB 4
#endif
constexpr int WARPS = SORF_WARPS;
// Several independent vectors (one per atom handled by the lane) through one pair of warp barriers.
template <int LOG2N, int ATOMS>
struct XposeN {
    using X = Xpose<LOG2N>;
    using C = Cfg<LOG2N>;
    __device__ static __forceinline__ void a_to_b(float (&u)[ATOMS][16], float *slab, int l) {
#pragma unroll
        for (int a = 0; a < ATOMS; ++a) {
            float4 *w = reinterpret_cast<float4 *>(slab + a * C::WARP_FLOATS + X::a_base(l));
#pragma unroll
            for (int q = 0; q < 4; ++q) w[q] = make_float4(u[a][4 * q], u[a][4 * q + 1], u[a][4 * q + 2], u[a][4 * q + 3]);
        }
        __syncwarp();
#pragma unroll
        for (int a = 0; a < ATOMS; ++a) {
            const float *r = slab + a * C::WARP_FLOATS + X::b_base(l);
#pragma unroll
            for (int e = 0; e < 16; ++e) u[a][e] = r[X::b_const(e)];
        }
        __syncwarp();
    }
    __device__ static __forceinline__ void b_to_a(float (&u)[ATOMS][16], float *slab, int l) {
#pragma unroll
        for (int a = 0; a < ATOMS; ++a) {
            float *w = slab + a * C::WARP_FLOATS + X::b_base(l);
#pragma unroll
            for (int e = 0; e < 16; ++e) w[X::b_const(e)] = u[a][e];
        }
        __syncwarp();
#pragma unroll
        for (int a = 0; a < ATOMS; ++a) {
            const float4 *r = reinterpret_cast<const float4 *>(slab + a * C::WARP_FLOATS + X::a_base(l));
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float4 t = r[q];
                u[a][4 * q] = t.x; u[a][4 * q + 1] = t.y; u[a][4 * q + 2] = t.z; u[a][4 * q + 3] = t.w;
            }
        }
        __syncwarp();
    }
};

// Parameter blocks (one per stack and transform) are stored interleaved: the q-th float4 of lane l sits at float
// offset (q*L + l)*4, so that one 128-bit load instruction of a vector's L lanes covers L*16 contiguous bytes
// (4 L1 wavefronts per warp-wide load instead of 16 with a lane-major order).
template <int L>
__device__ __forceinline__ void load16(float (&v)[16], const float *p) {
    const float4 *q = reinterpret_cast<const float4 *>(p);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float4 t = __ldg(q + i * L);
        v[4 * i] = t.x; v[4 * i + 1] = t.y; v[4 * i + 2] = t.z; v[4 * i + 3] = t.w;
    }
}

// natural (row) order: 16 consecutive floats per lane
template <int LOG2N, int ATOMS>
__device__ __forceinline__ void fwht_flip_n(float (&u)[ATOMS][16], float *slab, int l, int lane, bool from_a) {
    using C = Cfg<LOG2N>;
    if (C::LB == 0) {
#pragma unroll
        for (int a = 0; a < ATOMS; ++a) fwht_regs<4>(u[a]);
        return;
    }
    if (from_a) {
#pragma unroll
        for (int a = 0; a < ATOMS; ++a) fwht_regs<4>(u[a]);
        XposeN<LOG2N, ATOMS>::a_to_b(u, slab, l);
#pragma unroll
        for (int a = 0; a < ATOMS; ++a) {
            fwht_regs<C::LBT>(u[a]);
            if (C::LB == 5) lane16_stage(u[a], lane);
        }
    } else {
#pragma unroll
        for (int a = 0; a < ATOMS; ++a) {
            if (C::LB == 5) lane16_stage(u[a], lane);
            fwht_regs<C::LBT>(u[a]);
        }
        XposeN<LOG2N, ATOMS>::b_to_a(u, slab, l);
#pragma unroll
        for (int a = 0; a < ATOMS; ++a) fwht_regs<4>(u[a]);
    }
}

__device__ __forceinline__ void load16_row(float (&v)[16], const float *p) {
    const float4 *q = reinterpret_cast<const float4 *>(p);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float4 t = __ldg(q + i);
        v[4 * i] = t.x; v[4 * i + 1] = t.y; v[4 * i + 2] = t.z; v[4 * i + 3] = t.w;
    }
}

template <int LOG2N, bool FAST, int TT, int ATOMS>
__global__ void __launch_bounds__(WARPS * 32, ATOMS == 1 ? SORF_MINB : 3)
sorf_energy_grad_kernel(const float *__restrict__ x, const int *__restrict__ group_start,
                        const int *__restrict__ slot_of_row, int nel, int S, int T_rt, float scale,
                        const float *__restrict__ Dp, const float *__restrict__ bp, const float *__restrict__ ap,
                        float *__restrict__ atom_energy, float *__restrict__ grad_x) {
    using C = Cfg<LOG2N>;
    constexpr int N = C::N;
    extern __shared__ __align__(16) float smem[];
    const int T = TT > 0 ? TT : T_rt;  // compile-time trip count for the common single-transform model
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane / C::L, l = lane % C::L;  // vector within the warp, lane within the vector
    float *slab = smem + warp * (ATOMS * C::WARP_FLOATS) + g * C::SLAB;

    // A warp handles ATOMS consecutive rows (same element: groups are padded to a multiple of WARPS * ATOMS rows) and
    // shares every parameter load between them.
    const long row0 = ((long)blockIdx.x * WARPS + warp) * ATOMS;
    if (row0 >= group_start[nel]) return;
    int el = 0;
    while (el + 1 < nel && row0 >= group_start[el + 1]) ++el;

    float xr[ATOMS][16], gx[ATOMS][16];
    float2 eacc2[ATOMS];  // two interleaved partial sums of the row energy
    bool live[ATOMS];
#pragma unroll
    for (int a = 0; a < ATOMS; ++a) {
        live[a] = slot_of_row[row0 + a] >= 0;  // padding rows of an element group are computed on zeros and not stored
        if (live[a]) load16_row(xr[a], x + (size_t)(row0 + a) * N + l * 16);
        else {
#pragma unroll
            for (int e = 0; e < 16; ++e) xr[a][e] = 0.f;
        }
#pragma unroll
        for (int e = 0; e < 16; ++e) gx[a][e] = 0.f;
        eacc2[a] = make_float2(0.f, 0.f);
    }
    if (ATOMS == 1 && !live[0]) {
        if (lane == 0) atom_energy[row0] = 0.f;
        return;
    }

    const size_t pos = (size_t)l * 4;  // interleaved parameter blocks: float4 index q*L + l
    const float *Dp_e = Dp + (size_t)el * S * T * N;
    const float *bp_e = bp + (size_t)el * S * N;

    // S is the stack count padded to a multiple of V by qmlb_sorf_pack (padding stacks carry zero weights)
    for (int s0 = 0; s0 < S; s0 += C::V) {
        const int sc = s0 + g;
        const float *Ds = Dp_e + (size_t)sc * T * N + pos;
        float u[ATOMS][16], c[16];
        bool in_a = true;
        if (TT == 1) {
            // single transform: the sign diagonal stays in registers for the way back
            load16<C::L>(c, Ds);
#pragma unroll
            for (int a = 0; a < ATOMS; ++a) {
#pragma unroll
                for (int e = 0; e < 16; e += 2) {
                    const float2 t = __fmul2_rn(make_float2(xr[a][e], xr[a][e + 1]), make_float2(c[e], c[e + 1]));
                    u[a][e] = t.x; u[a][e + 1] = t.y;
                }
            }
            fwht_flip_n<LOG2N, ATOMS>(u, slab, l, lane, true);
            in_a = false;
        } else {
#pragma unroll
            for (int a = 0; a < ATOMS; ++a)
#pragma unroll
                for (int e = 0; e < 16; ++e) u[a][e] = xr[a][e];
            for (int m = 0; m < T; ++m) {
                load16<C::L>(c, Ds + (size_t)m * N);
#pragma unroll
                for (int a = 0; a < ATOMS; ++a)
#pragma unroll
                    for (int e = 0; e < 16; ++e) u[a][e] *= c[e];
                fwht_flip_n<LOG2N, ATOMS>(u, slab, l, lane, in_a);
                in_a = !in_a;
            }
        }
        {   // features: energy contribution and d/d(arg), in the layout the forward transform ended in
            const float4 *bq = reinterpret_cast<const float4 *>(bp_e + (size_t)sc * N + pos);
            const float4 *aq = reinterpret_cast<const float4 *>(ap + (size_t)sc * N + pos);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float4 b4 = __ldg(bq + q * C::L), a4 = __ldg(aq + q * C::L);
                const float bb[4] = {b4.x, b4.y, b4.z, b4.w}, aa[4] = {a4.x, a4.y, a4.z, a4.w};
#pragma unroll
                for (int a = 0; a < ATOMS; ++a)
#pragma unroll
                    for (int r = 0; r < 4; r += 2) {
                        const int e = 4 * q + r;
                        const float2 arg = __ffma2_rn(make_float2(u[a][e], u[a][e + 1]), make_float2(scale, scale),
                                                      make_float2(bb[r], bb[r + 1]));
                        float2 sn, cs;
                        if (FAST) {
                            __sincosf(arg.x, &sn.x, &cs.x);
                            __sincosf(arg.y, &sn.y, &cs.y);
                        } else {
                            qmlb_sincos::sincos_pair(arg, sn, cs);
                        }
                        eacc2[a] = __ffma2_rn(make_float2(aa[r], aa[r + 1]), cs, eacc2[a]);
                        const float2 gq = __fmul2_rn(make_float2(-aa[r], -aa[r + 1]), sn);
                        u[a][e] = gq.x; u[a][e + 1] = gq.y;
                    }
            }
        }
        if (TT == 1) {
            fwht_flip_n<LOG2N, ATOMS>(u, slab, l, lane, false);
#pragma unroll
            for (int a = 0; a < ATOMS; ++a) {
#pragma unroll
                for (int e = 0; e < 16; e += 2) {
                    const float2 t = __ffma2_rn(make_float2(u[a][e], u[a][e + 1]), make_float2(c[e], c[e + 1]),
                                                make_float2(gx[a][e], gx[a][e + 1]));
                    gx[a][e] = t.x; gx[a][e + 1] = t.y;
                }
            }
        } else {
            for (int m = T - 1; m >= 0; --m) {
                fwht_flip_n<LOG2N, ATOMS>(u, slab, l, lane, in_a);
                in_a = !in_a;
                load16<C::L>(c, Ds + (size_t)m * N);
                if (m > 0) {
#pragma unroll
                    for (int a = 0; a < ATOMS; ++a)
#pragma unroll
                        for (int e = 0; e < 16; ++e) u[a][e] *= c[e];
                } else {
#pragma unroll
                    for (int a = 0; a < ATOMS; ++a)
#pragma unroll
                        for (int e = 0; e < 16; ++e) gx[a][e] = fmaf(u[a][e], c[e], gx[a][e]);
                }
            }
        }
    }

    // sum the V stacks processed side by side, then one store per atom
#pragma unroll
    for (int a = 0; a < ATOMS; ++a) {
#pragma unroll
        for (int off = C::L; off < 32; off <<= 1)
#pragma unroll
            for (int e = 0; e < 16; ++e) gx[a][e] += __shfl_xor_sync(QMLB_FULL_MASK, gx[a][e], off);
        const float esum = warp_sum(eacc2[a].x + eacc2[a].y);
        if (g == 0 && live[a]) {
            float4 *dst = reinterpret_cast<float4 *>(grad_x + (size_t)(row0 + a) * N + l * 16);
#pragma unroll
            for (int q = 0; q < 4; ++q)
                dst[q] = make_float4(gx[a][4 * q] * scale, gx[a][4 * q + 1] * scale, gx[a][4 * q + 2] * scale,
                                     gx[a][4 * q + 3] * scale);
        }
        if (lane == 0) atom_energy[row0 + a] = live[a] ? esum : 0.f;
    }
}

// ---- two atoms per warp, interleaved in packed fp32x2 registers (single transform, 64 <= N <= 256) -------------------
// Register e of a lane holds the PAIR (atom 0, atom 1) of one element, so every butterfly stage -- including the one
// that pairs neighbouring registers, which the per-atom layout above has to run as scalar additions -- and every
// element-wise step is one packed fp32x2 instruction for both atoms, and the transposition moves the pair with one
// 64-bit load instead of two 32-bit ones.  Per (atom, stack) this needs about 30 % fewer instructions than the kernel
// above, which is what bounds it (instruction issue).  Slab: rows of 16 pairs, row stride 36 floats (nine 16-byte
// groups: the 128-bit row stores of eight consecutive lanes hit distinct groups), 64-bit loads of consecutive pairs.
template <int LOG2N>
struct PairCfg {
    using C = Cfg<LOG2N>;
    static constexpr int ROW2 = 36;
    static constexpr int RAW = C::L * ROW2;
    // vectors that share a half warp read from slabs whose bank ranges do not overlap
    static constexpr int SLAB = C::V <= 2 ? RAW : (C::V == 4 ? RAW + 16 : RAW + 8);
    static constexpr int WARP_FLOATS = C::V * SLAB;
};

__device__ __forceinline__ void butterfly_pair(float2 &a, float2 &b) {
    const float2 s = __fadd2_rn(a, b);
    b = __ffma2_rn(b, make_float2(-1.0f, -1.0f), a);   // a - b, rounded once like a subtraction
    a = s;
}

template <int BITS>
__device__ __forceinline__ void fwht_pairs(float2 (&u)[16]) {
#pragma unroll
    for (int h = 1; h < (1 << BITS); h <<= 1)
#pragma unroll
        for (int i = 0; i < 16; ++i)
            if ((i & h) == 0) butterfly_pair(u[i], u[i | h]);
}

template <int LOG2N>
struct XposePair {
    using C = Cfg<LOG2N>;
    using P = PairCfg<LOG2N>;
    __device__ static __forceinline__ int b_off(int e, int l) {
        return (e & (C::L - 1)) * P::ROW2 + 2 * (((e >> C::LB) << C::LB) + l);
    }
    __device__ static __forceinline__ void a_to_b(float2 (&u)[16], float *slab, int l) {
        float4 *w = reinterpret_cast<float4 *>(slab + l * P::ROW2);
#pragma unroll
        for (int q = 0; q < 8; ++q) w[q] = make_float4(u[2 * q].x, u[2 * q].y, u[2 * q + 1].x, u[2 * q + 1].y);
        __syncwarp();
#pragma unroll
        for (int e = 0; e < 16; ++e) u[e] = *reinterpret_cast<const float2 *>(slab + b_off(e, l));
        __syncwarp();
    }
    __device__ static __forceinline__ void b_to_a(float2 (&u)[16], float *slab, int l) {
#pragma unroll
        for (int e = 0; e < 16; ++e) *reinterpret_cast<float2 *>(slab + b_off(e, l)) = u[e];
        __syncwarp();
        const float4 *r = reinterpret_cast<const float4 *>(slab + l * P::ROW2);
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            const float4 t = r[q];
            u[2 * q] = make_float2(t.x, t.y);
            u[2 * q + 1] = make_float2(t.z, t.w);
        }
        __syncwarp();
    }
};

template <int LOG2N, bool FAST, bool SHARE>
__global__ void __launch_bounds__(WARPS * 32, 4)   // 128 registers, 22 floats spilled: 16 warps per SM beat 12 at 168 registers (12.02 against 12.23 ms on c1)
sorf_pair_kernel(const float *__restrict__ x, const int *__restrict__ group_start, const int *__restrict__ slot_of_row, int nel,
                 int S, float scale, const float *__restrict__ Dp, const float *__restrict__ bp, const float *__restrict__ ap,
                 float *__restrict__ atom_energy, float *__restrict__ grad_x) {
    using C = Cfg<LOG2N>;
    using P = PairCfg<LOG2N>;
    using X = XposePair<LOG2N>;
    constexpr int N = C::N;
    static_assert(C::LB >= 2 && C::LB <= 4, "pair kernel covers N = 64, 128, 256");
    extern __shared__ __align__(16) float smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane / C::L, l = lane % C::L;
    float *slab = smem + warp * P::WARP_FLOATS + g * P::SLAB;

    // Rows 2k and 2k+1 of an element group share the registers of a lane.  SHARE: the V lane groups of the warp take V such
    // pairs and walk the stacks together, so that a parameter load is one request for all 2 V atoms (lanes of different
    // groups read the same addresses); used when there are rows enough to fill the GPU that way.  Otherwise the V lane
    // groups take V consecutive stacks of the same pair and their partial sums are added at the end (V times as many
    // warps, each V times shorter: small batches).  Groups are padded to 128 rows, so a warp's rows belong to one element.
    constexpr int RPW = SHARE ? 2 * C::V : 2;
    const long rowb = ((long)blockIdx.x * WARPS + warp) * RPW;
    if (rowb >= group_start[nel]) return;
    int el = 0;
    while (el + 1 < nel && rowb >= group_start[el + 1]) ++el;
    const long row0 = rowb + (SHARE ? 2 * g : 0);
    const bool live0 = slot_of_row[row0] >= 0, live1 = slot_of_row[row0 + 1] >= 0;
    if (!__any_sync(QMLB_FULL_MASK, live0 || live1)) {     // padding only
        if (l == 0 && (SHARE || g == 0)) atom_energy[row0] = atom_energy[row0 + 1] = 0.f;
        return;
    }
    float2 xr[16], gx[16];
    {
        float a0[16], a1[16];
        if (live0) load16_row(a0, x + (size_t)row0 * N + l * 16);
        if (live1) load16_row(a1, x + (size_t)(row0 + 1) * N + l * 16);
#pragma unroll
        for (int e = 0; e < 16; ++e) {
            xr[e] = make_float2(live0 ? a0[e] : 0.f, live1 ? a1[e] : 0.f);   // padding rows are computed on zeros
            gx[e] = make_float2(0.f, 0.f);
        }
    }
    float2 eacc = make_float2(0.f, 0.f);
    const size_t pos = (size_t)l * 4;
    const float *Dp_e = Dp + (size_t)el * S * N;
    const float *bp_e = bp + (size_t)el * S * N;
    const float2 scale2 = make_float2(scale, scale);

    for (int s0 = 0; s0 < S; s0 += SHARE ? 1 : C::V) {
        const int sc = SHARE ? s0 : s0 + g;
        float c[16];
        float2 u[16];
        load16<C::L>(c, Dp_e + (size_t)sc * N + pos);
#pragma unroll
        for (int e = 0; e < 16; ++e) u[e] = __fmul2_rn(xr[e], make_float2(c[e], c[e]));
        fwht_pairs<4>(u);
        X::a_to_b(u, slab, l);
        fwht_pairs<C::LB>(u);
        {   // features in the transposed layout: energy contribution and d/d(arg) (its sign goes into the final scale)
            const float4 *bq = reinterpret_cast<const float4 *>(bp_e + (size_t)sc * N + pos);
            const float4 *aq = reinterpret_cast<const float4 *>(ap + (size_t)sc * N + pos);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float4 b4 = __ldg(bq + q * C::L), a4 = __ldg(aq + q * C::L);
                const float bb[4] = {b4.x, b4.y, b4.z, b4.w}, aa[4] = {a4.x, a4.y, a4.z, a4.w};
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    const int e = 4 * q + r;
                    const float2 arg = __ffma2_rn(u[e], scale2, make_float2(bb[r], bb[r]));
                    float2 sn, cs;
                    if (FAST) {
                        __sincosf(arg.x, &sn.x, &cs.x);
                        __sincosf(arg.y, &sn.y, &cs.y);
                    } else {
                        qmlb_sincos::sincos_pair(arg, sn, cs);
                    }
                    const float2 a2 = make_float2(aa[r], aa[r]);
                    eacc = __ffma2_rn(a2, cs, eacc);
                    u[e] = __fmul2_rn(a2, sn);
                }
            }
        }
        fwht_pairs<C::LB>(u);
        X::b_to_a(u, slab, l);
        fwht_pairs<4>(u);
#pragma unroll
        for (int e = 0; e < 16; ++e) gx[e] = __ffma2_rn(u[e], make_float2(c[e], c[e]), gx[e]);
    }

    // energies: sum over the lanes that hold the pair; grad = -scale * sum (alpha sin ...) (HD)^T
    if (!SHARE) {   // the V stacks processed side by side
#pragma unroll
        for (int off = C::L; off < 32; off <<= 1)
#pragma unroll
            for (int e = 0; e < 16; ++e) {
                gx[e].x += __shfl_xor_sync(QMLB_FULL_MASK, gx[e].x, off);
                gx[e].y += __shfl_xor_sync(QMLB_FULL_MASK, gx[e].y, off);
            }
    }
    float e0 = eacc.x, e1 = eacc.y;
#pragma unroll
    for (int off = (SHARE ? C::L : 32) / 2; off > 0; off >>= 1) {
        e0 += __shfl_xor_sync(QMLB_FULL_MASK, e0, off);
        e1 += __shfl_xor_sync(QMLB_FULL_MASK, e1, off);
    }
    if (SHARE || g == 0) {
        const float ns = -scale;
        if (live0) {
            float4 *dst = reinterpret_cast<float4 *>(grad_x + (size_t)row0 * N + l * 16);
#pragma unroll
            for (int q = 0; q < 4; ++q)
                dst[q] = make_float4(gx[4 * q].x * ns, gx[4 * q + 1].x * ns, gx[4 * q + 2].x * ns, gx[4 * q + 3].x * ns);
        }
        if (live1) {
            float4 *dst = reinterpret_cast<float4 *>(grad_x + (size_t)(row0 + 1) * N + l * 16);
#pragma unroll
            for (int q = 0; q < 4; ++q)
                dst[q] = make_float4(gx[4 * q].y * ns, gx[4 * q + 1].y * ns, gx[4 * q + 2].y * ns, gx[4 * q + 3].y * ns);
        }
    }
    if (l == 0 && (SHARE || g == 0)) {
        atom_energy[row0] = live0 ? e0 : 0.f;
        atom_energy[row0 + 1] = live1 ? e1 : 0.f;
    }
}

// Source element of packed float index p (0..N-1) of one block: p = (q*L + l)*4 + r holds register e = 4q + r of
// lane l, i.e. position l*16 + e of layout A, or its layout-B element when `layout_b`.
__host__ __device__ inline int packed_source(int log2n, int p, bool layout_b) {
    const int L = 1 << (log2n - 4);
    const int r = p & 3, l = (p >> 2) % L, q = (p >> 2) / L;
    const int pos = l * 16 + 4 * q + r;
    return layout_b ? layoutB_n(log2n, pos) : pos;
}

__global__ void sorf_pack_kernel(const float *__restrict__ Dmat, const float *__restrict__ bias,
                                 const float *__restrict__ alpha, int nel, int log2n, int S, int Spad, int T,
                                 float *__restrict__ Dp, float *__restrict__ bp, float *__restrict__ ap) {
    const int N = 1 << log2n;
    const size_t nD = (size_t)nel * Spad * T * N, nB = (size_t)nel * Spad * N, nA = (size_t)Spad * N;
    const float normf = sqrtf(2.0f / (float)((size_t)S * N));
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < nD + nB + nA; i += (size_t)gridDim.x * blockDim.x) {
        if (i < nD) {  // Dp[el][s][m][p] <- Dmat[el][m][s][n]
            const int p = (int)(i % N);
            const int m = (int)((i / N) % T);
            const int s = (int)((i / ((size_t)N * T)) % Spad);
            const int el = (int)(i / ((size_t)N * T * Spad));
            const int n = packed_source(log2n, p, m & 1);
            Dp[i] = s < S ? Dmat[(((size_t)el * T + m) * S + s) * N + n] : 1.0f;
        } else if (i < nD + nB) {
            const size_t k = i - nD;
            const int p = (int)(k % N);
            const int s = (int)((k / N) % Spad);
            const int el = (int)(k / ((size_t)N * Spad));
            const int n = packed_source(log2n, p, T & 1);
            bp[k] = s < S ? bias[((size_t)el * S + s) * N + n] : 0.0f;
        } else {
            const size_t k = i - nD - nB;
            const int p = (int)(k % N);
            const int s = (int)(k / N);
            const int n = packed_source(log2n, p, T & 1);
            ap[k] = s < S ? alpha[(size_t)s * N + n] * normf : 0.0f;  // padding stacks contribute nothing
        }
    }
}

inline int padded_stacks(int N, int S) {
    const int V = 512 / N;  // stacks per warp: 32 lanes / (N/16 lanes per vector)
    return (S + V - 1) / V * V;
}

int ilog2_exact(int n) {
    int l = 0;
    while ((1 << l) < n) ++l;
    return (1 << l) == n ? l : -1;
}

#ifndef SORF_ATOMS
#define SORF_ATOMS 2
#endif
#ifndef SORF_PAIR
#define SORF_PAIR 1
#endif

template <int LOG2N>
int launch_fused(const float *x, const int *group_start, const int *slot_of_row, int nel, size_t rows_cap, int S, int T,
                 float scale, const float *Dp, const float *bp, const float *ap, int fast, float *atom_energy,
                 float *grad_x, cudaStream_t st) {
    using C = Cfg<LOG2N>;
    // two atoms per warp share the parameter loads when the model has a single transform and 16 <= N... (the common case)
    constexpr int ATOMS_FAST = (LOG2N >= 6 && LOG2N <= 8) ? SORF_ATOMS : 1;
#define QMLB_LAUNCH(FASTV, TTV, AT)                                                                                    \
    do {                                                                                                              \
        const size_t smem = sizeof(float) * WARPS * AT * C::WARP_FLOATS;                                              \
        const unsigned grid = (unsigned)((rows_cap + WARPS * AT - 1) / (WARPS * AT));                                 \
        sorf_energy_grad_kernel<LOG2N, FASTV, TTV, AT><<<grid, WARPS * 32, smem, st>>>(                               \
            x, group_start, slot_of_row, nel, S, T, scale, Dp, bp, ap, atom_energy, grad_x);                           \
    } while (0)
    if (T == 1 && LOG2N >= 6 && LOG2N <= 8 && SORF_PAIR) {
        constexpr int PL = (LOG2N >= 6 && LOG2N <= 8) ? LOG2N : 8;   // keeps the other instantiations well formed
        const size_t smem = sizeof(float) * WARPS * PairCfg<PL>::WARP_FLOATS;
        // one warp per 2 V rows when that still gives every SM several waves of warps, else one warp per 2 rows
        const bool share = rows_cap / (2 * Cfg<PL>::V) >= (size_t)148 * 16 * 4;
        const int rpw = share ? 2 * Cfg<PL>::V : 2;
        const unsigned grid = (unsigned)((rows_cap + WARPS * rpw - 1) / (WARPS * rpw));
#define QMLB_PAIR(FASTV, SHAREV) \
    sorf_pair_kernel<PL, FASTV, SHAREV><<<grid, WARPS * 32, smem, st>>>(x, group_start, slot_of_row, nel, S, scale, Dp, bp, ap, atom_energy, grad_x)
        if (fast) { if (share) QMLB_PAIR(true, true); else QMLB_PAIR(true, false); }
        else { if (share) QMLB_PAIR(false, true); else QMLB_PAIR(false, false); }
#undef QMLB_PAIR
    } else if (T == 1) {
        if (fast) QMLB_LAUNCH(true, 1, ATOMS_FAST); else QMLB_LAUNCH(false, 1, 1);
    } else {
        if (fast) QMLB_LAUNCH(true, 0, 1); else QMLB_LAUNCH(false, 0, 1);
    }
#undef QMLB_LAUNCH
    return qmlb::check_launch("qmlb_sorf_energy_grad");
}

}  // namespace

extern "C" size_t qmlb_sorf_pack_bytes(int nelements, int N, int S, int T) {
    if (N < 16 || N > 512) return 0;
    const size_t Sp = padded_stacks(N, S);
    return sizeof(float) * ((size_t)nelements * Sp * T * N + (size_t)nelements * Sp * N + Sp * N);
}

extern "C" int qmlb_sorf_pack(const float *Dmat, const float *bias, const float *alpha, int nelements, int N, int S,
                              int T, void *packed, qmlb_stream_t stream) {
    QMLB_REQUIRE(Dmat && bias && alpha && packed, "qmlb_sorf_pack: null tensor");
    const int log2n = ilog2_exact(N);
    QMLB_REQUIRE(log2n >= 4 && log2n <= 9, "qmlb_sorf_pack: npcas must be a power of two in [16, 512], got %d", N);
    QMLB_REQUIRE(nelements > 0 && S > 0 && T > 0, "qmlb_sorf_pack: bad sizes");
    const size_t Sp = padded_stacks(N, S);
    float *Dp = static_cast<float *>(packed);
    float *bp = Dp + (size_t)nelements * Sp * T * N;
    float *ap = bp + (size_t)nelements * Sp * N;
    sorf_pack_kernel<<<592, 256, 0, qmlb::as_stream(stream)>>>(Dmat, bias, alpha, nelements, log2n, S, (int)Sp, T, Dp, bp, ap);
    return qmlb::check_launch("qmlb_sorf_pack");
}

extern "C" int qmlb_sorf_energy_grad(const float *x, const int *group_start, const int *slot_of_row, int nelements,
                                     size_t rows_cap, int N, int S, int T, float sigma, const void *packed,
                                     int fast_math, float *atom_energy, float *grad_x, qmlb_stream_t stream) {
    QMLB_REQUIRE(x && group_start && slot_of_row && packed && atom_energy && grad_x, "qmlb_sorf_energy_grad: null tensor");
    const int log2n = ilog2_exact(N);
    QMLB_REQUIRE(log2n >= 4 && log2n <= 9, "qmlb_sorf_energy_grad: npcas must be a power of two in [16, 512], got %d", N);
    QMLB_REQUIRE(nelements > 0 && S > 0 && T > 0 && sigma > 0.f, "qmlb_sorf_energy_grad: bad sizes");
    if (rows_cap == 0) return QMLB_OK;
    const size_t Sp = padded_stacks(N, S);
    const float *Dp = static_cast<const float *>(packed);
    const float *bp = Dp + (size_t)nelements * Sp * T * N;
    const float *ap = bp + (size_t)nelements * Sp * N;
    // coeff_normalisation sqrt(N)/sigma (models/hadamard_features.py:93) times N^(-1/2) per transform
    const float scale = (float)(sqrt((double)N) / (double)sigma * pow((double)N, -0.5 * (double)T));
    cudaStream_t st = qmlb::as_stream(stream);
    switch (log2n) {
        case 4: return launch_fused<4>(x, group_start, slot_of_row, nelements, rows_cap, (int)Sp, T, scale, Dp, bp, ap, fast_math, atom_energy, grad_x, st);
        case 5: return launch_fused<5>(x, group_start, slot_of_row, nelements, rows_cap, (int)Sp, T, scale, Dp, bp, ap, fast_math, atom_energy, grad_x, st);
        case 6: return launch_fused<6>(x, group_start, slot_of_row, nelements, rows_cap, (int)Sp, T, scale, Dp, bp, ap, fast_math, atom_energy, grad_x, st);
        case 7: return launch_fused<7>(x, group_start, slot_of_row, nelements, rows_cap, (int)Sp, T, scale, Dp, bp, ap, fast_math, atom_energy, grad_x, st);
        case 8: return launch_fused<8>(x, group_start, slot_of_row, nelements, rows_cap, (int)Sp, T, scale, Dp, bp, ap, fast_math, atom_energy, grad_x, st);
        default: return launch_fused<9>(x, group_start, slot_of_row, nelements, rows_cap, (int)Sp, T, scale, Dp, bp, ap, fast_math, atom_energy, grad_x, st);
    }
}
