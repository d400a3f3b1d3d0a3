// sin and cos with float32 accuracy (about one ulp; 7e-8 absolute against a float64 evaluation over |x| <= 9e4) without the
// library's slow path, so that the lanes of a warp and the two atoms of a packed pair never diverge: round x 2/pi to the
// nearest integer q with the 1.5 * 2^23 addition, subtract q pi/2 in three fused multiply-adds (pi/2 split into three
// floats), Taylor polynomials to r^9 (sin) and r^10 (cos) on [-pi/4, pi/4], then swap and negate by quadrant.
// Arguments beyond 1e5 in magnitude (where q would no longer fit the rounding trick) take the library function.
#pragma once

#include <math.h>

namespace qmlb_sincos {

constexpr float TWO_OVER_PI = 0.63661975f;
constexpr float MAGIC = 12582912.0f;            // 1.5 * 2^23
constexpr float PIO2_HI = 1.5707964f;           // 0x3fc90fdb
constexpr float PIO2_MID = -4.371139e-08f;      // 0xb33bbd2e
constexpr float PIO2_LO = -1.7151245e-15f;      // 0xa6f72ced
constexpr float LIMIT = 1.0e5f;
constexpr float S1 = -1.0f / 6.0f, S2 = 1.0f / 120.0f, S3 = -1.0f / 5040.0f, S4 = 1.0f / 362880.0f;
constexpr float C1 = -0.5f, C2 = 1.0f / 24.0f, C3 = -1.0f / 720.0f, C4 = 1.0f / 40320.0f, C5 = -1.0f / 3628800.0f;

__device__ __forceinline__ float2 splat(float v) { return make_float2(v, v); }

__device__ __forceinline__ void quadrant(int q, float s, float c, float &sn, float &cs) {
    const bool odd = (q & 1) != 0;
    const float a = odd ? c : s, b = odd ? s : c;
    sn = __int_as_float(__float_as_int(a) ^ ((q & 2) << 30));
    cs = __int_as_float(__float_as_int(b) ^ (((q + 1) & 2) << 30));
}

// both components at once on the packed fp32x2 pipe
__device__ __forceinline__ void sincos_pair(float2 x, float2 &sn, float2 &cs) {
    if (fmaxf(fabsf(x.x), fabsf(x.y)) > LIMIT) {
        sincosf(x.x, &sn.x, &cs.x);
        sincosf(x.y, &sn.y, &cs.y);
        return;
    }
    const float2 t = __ffma2_rn(x, splat(TWO_OVER_PI), splat(MAGIC));
    const float2 q = __fadd2_rn(t, splat(-MAGIC));
    float2 r = __ffma2_rn(q, splat(-PIO2_HI), x);
    r = __ffma2_rn(q, splat(-PIO2_MID), r);
    r = __ffma2_rn(q, splat(-PIO2_LO), r);
    const float2 r2 = __fmul2_rn(r, r);
    float2 ps = __ffma2_rn(r2, splat(S4), splat(S3));
    ps = __ffma2_rn(ps, r2, splat(S2));
    ps = __ffma2_rn(ps, r2, splat(S1));
    const float2 s = __ffma2_rn(ps, __fmul2_rn(r, r2), r);
    float2 pc = __ffma2_rn(r2, splat(C5), splat(C4));
    pc = __ffma2_rn(pc, r2, splat(C3));
    pc = __ffma2_rn(pc, r2, splat(C2));
    pc = __ffma2_rn(pc, r2, splat(C1));
    const float2 c = __ffma2_rn(pc, r2, splat(1.0f));
    quadrant(__float_as_int(t.x), s.x, c.x, sn.x, cs.x);
    quadrant(__float_as_int(t.y), s.y, c.y, sn.y, cs.y);
}

__device__ __forceinline__ void sincos_one(float x, float &sn, float &cs) {
    if (fabsf(x) > LIMIT) {
        sincosf(x, &sn, &cs);
        return;
    }
    const float t = fmaf(x, TWO_OVER_PI, MAGIC);
    const float q = t - MAGIC;
    float r = fmaf(q, -PIO2_HI, x);
    r = fmaf(q, -PIO2_MID, r);
    r = fmaf(q, -PIO2_LO, r);
    const float r2 = r * r;
    float ps = fmaf(r2, S4, S3);
    ps = fmaf(ps, r2, S2);
    ps = fmaf(ps, r2, S1);
    const float s = fmaf(ps, r * r2, r);
    float pc = fmaf(r2, C5, C4);
    pc = fmaf(pc, r2, C3);
    pc = fmaf(pc, r2, C2);
    pc = fmaf(pc, r2, C1);
    const float c = fmaf(pc, r2, 1.0f);
    quadrant(__float_as_int(t), s, c, sn, cs);
}

}  // namespace qmlb_sincos
