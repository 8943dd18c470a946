// Per-pixel arithmetic of the Huber-TV FISTA iteration and of its reverse sweep, shared by every kernel.
//
// Formulation.  The reference gathers three Huber-weighted "triangles" per pixel
// (cudaTV/cudaCode/TVInpaintFista.cu:1247-1274).  Here each triangle, anchored at pixel p with edges to p+x and
// p+y, is evaluated once and produces two fluxes
//     fx(p) = s(p) wx(p) (y[p]-y[p+x]),   fy(p) = s(p) wy(p) (y[p]-y[p+y]),   s = min(1, delta / sqrt(A)),
//     A(p) = wx(p) (y[p]-y[p+x])^2 + wy(p) (y[p]-y[p+y])^2,
// and the gradient step is the divergence  x05[p] = y[p] - fx(p) - fy(p) + fx(p-x) + fy(p-y).
// The reverse sweep has the same shape with adjoint fluxes phi1, phi2 (TVInpaintFista.cu:651-771).
// Weights are pre-multiplied by 1/8 and are zero across the image border (TVInpaintFista.cu:1204-1211, :1478).
#pragma once
#include <cuda_runtime.h>

namespace cnl {

constexpr float kDelta = 0.1f;            // __HDelta1__     TVInpaintFista.cu:44
constexpr float kClipLocal = 10000.0f;    // clipLocalGrad   :52
constexpr float kLocalGC = 0.1f;          // localGCMult     :63
constexpr float kLocalGX = 0.1f;          // localGXMult     :65
constexpr float kLocalGB = 1.0f;          // localGBMult     :67
constexpr float kGlobalG = 0.1f;          // globalGMult     :69
constexpr float kLip = 0.125f;            // 1/Lipschitz     :1478

// Fluxes of the forward-difference triangle anchored at a pixel.
__device__ __forceinline__ void tri_flux(float yc, float yr, float yd, float wx, float wy, float& fx, float& fy) {
    const float d1 = yc - yr;
    const float d2 = yc - yd;
    const float A = wx * d1 * d1 + wy * d2 * d2;
    const float T = sqrtf(A);
    const float s = (T > kDelta) ? kDelta / T : 1.0f;
    fx = s * wx * d1;
    fy = s * wy * d2;
}

// Huber data-term prox (TVInpaintFista.cu:1288-1292).
__device__ __forceinline__ float prox_huber(float x05, float b, float c) {
    float x = (c * b + x05) / (1.0f + c);
    const float lo = x05 - c;
    const float hi = x05 + c;
    if (lo > 1.0f + b) x = lo;
    if (hi < b - 1.0f) x = hi;
    return x;
}

// y^{k+1} rebuilt from two stored pre-prox iterates, exactly as the reference's reverse sweep does
// (TVInpaintFista.cu:1151-1165): the zone of iterate `it` selects the formula applied to BOTH iterates.
__device__ __forceinline__ float rederive_y(float x05, float x05m, float b, float c, float t) {
    const float diff = b - x05;
    const float sign = (diff < 0.0f) ? -1.0f : 1.0f;
    if (1.0f + c >= sign * diff) {
        const float xk = (c * b + x05) / (1.0f + c);
        const float xkm = (c * b + x05m) / (1.0f + c);
        return xk + t * (xk - xkm);
    }
    const float xk = (c <= sign * diff) ? b - diff + sign * c : b;
    const float diff2 = b - x05m;
    const float sign2 = (diff2 < 0.0f) ? -1.0f : 1.0f;
    const float xkm = (c <= sign2 * diff2) ? b - diff2 + sign2 * c : b;
    return xk + t * (xk - xkm);
}

// Adjoint fluxes of one triangle and its contribution to the edge-weight gradients.
//   e1 = g[p]-g[p+x], e2 = g[p]-g[p+y];  S = wx d1 e1 + wy d2 e2
//   phi1 = nom wx e1 - 2 den wx d1 S,  phi2 = nom wy e2 - 2 den wy d2 S
//   dwx  = -kLocalGX d1 (e1 (nom - wx d1^2 den) - e2 d1 d2 den wy)      (TVInpaintFista.cu:751-753)
//   dwy  = -kLocalGX d2 (e2 (nom - wy d2^2 den) - e1 d2 d1 den wx)      (TVInpaintFista.cu:757-759)
// with nom = delta/T, den = nom/(2 T^2) when T > delta, else nom = 1, den = 0 (:662-665, :761-769).
__device__ __forceinline__ void tri_adjoint(float yc, float yr, float yd, float gc, float gr, float gd,
                                            float wx, float wy, float& phi1, float& phi2, float& dwx, float& dwy) {
    const float d1 = yc - yr;
    const float d2 = yc - yd;
    const float e1 = gc - gr;
    const float e2 = gc - gd;
    const float A = wx * d1 * d1 + wy * d2 * d2;
    const float T = sqrtf(A);
    float nom = 1.0f, den = 0.0f;
    if (T > kDelta) {
        nom = kDelta / T;
        den = nom / (2.0f * T * T);
    }
    const float S = wx * d1 * e1 + wy * d2 * e2;
    const float k = 2.0f * den * S;
    phi1 = wx * (nom * e1 - k * d1);
    phi2 = wy * (nom * e2 - k * d2);
    dwx = -kLocalGX * d1 * (e1 * (nom - wx * d1 * d1 * den) - e2 * d1 * d2 * den * wy);
    dwy = -kLocalGX * d2 * (e2 * (nom - wy * d2 * d2 * den) - e1 * d2 * d1 * den * wx);
}

// Prox Jacobian applied to df_dxk = dL/dx^{k+1} (TVInpaintFista.cu:806-828 and the seed kernel :240-255).
// Returns dL/dx^{k+1/2}; adds the (locally scaled) confidence and rhs contributions.
__device__ __forceinline__ float prox_reverse(float df_dxk, float x05, float b, float c, float& dgc, float& dgb) {
    const float diff = b - x05;
    const float sign = (diff < 0.0f) ? -1.0f : 1.0f;
    const float opc = 1.0f + c;
    if (opc >= sign * diff) {
        dgc += df_dxk * (b / opc - (c * b + x05) / (opc * opc)) * kLocalGC;
        dgb += df_dxk * c / opc * kLocalGB;
        return df_dxk / opc;
    }
    dgc += sign * df_dxk * kLocalGC;
    return df_dxk;
}

__device__ __forceinline__ float clampf(float v, float lo, float hi) { return fminf(fmaxf(v, lo), hi); }

__device__ __forceinline__ bool finite_f(float v) { return fabsf(v) <= 3.402823466e38f; }   // false for NaN / Inf

}  // namespace cnl

// ---------------------------------------------------------------------------------------------------------------
// Fast variants used by the register-tiled kernels: MUFU reciprocal square root / reciprocal (max 2 ulp) instead of
// IEEE sqrt and divide.  rsqrtf(0) = +inf makes s = min(1, inf) = 1, the same value the exact form gives.
// ---------------------------------------------------------------------------------------------------------------
namespace cnl {

// Single-instruction MUFU approximations (flush-to-zero, max 2 ulp).  rsqrt(0) = +inf, rcp(inf) = 0.
__device__ __forceinline__ float rsqrt_approx(float x) {
    float r;
    asm("rsqrt.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}
__device__ __forceinline__ float rcp_approx(float x) {
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}

// prox with the reciprocal of (1 + c) supplied by the caller
__device__ __forceinline__ float prox_huber_fast(float x05, float b, float c, float inv1pc) {
    float x = fmaf(c, b, x05) * inv1pc;
    const float lo = x05 - c;
    const float hi = x05 + c;
    if (lo > 1.0f + b) x = lo;
    if (hi < b - 1.0f) x = hi;
    return x;
}

__device__ __forceinline__ float rederive_y_fast(float x05, float x05m, float b, float c, float inv1pc, float t) {
    const float diff = b - x05;
    const float ad = fabsf(diff);
    const float diff2 = b - x05m;
    const float ad2 = fabsf(diff2);
    // quadratic zone of iterate `it`: both iterates through the quadratic formula
    const float xq = fmaf(c, b, x05) * inv1pc;
    const float xqm = fmaf(c, b, x05m) * inv1pc;
    // otherwise: both through the soft threshold (b inside the dead zone)
    const float xl = x05 + copysignf(c, diff);          // outside the quadratic zone |diff| > 1 + c >= c always holds
    const float xlm = (c <= ad2) ? x05m + copysignf(c, diff2) : b;
    const bool quad = (1.0f + c >= ad);
    const float xk = quad ? xq : xl;
    const float xkm = quad ? xqm : xlm;
    return fmaf(t, xk - xkm, xk);
}

// prox Jacobian with the reciprocal of (1 + c) supplied by the caller (see prox_reverse)
__device__ __forceinline__ float prox_reverse_fast(float df_dxk, float x05, float b, float c, float inv1pc, float& dgc, float& dgb) {
    const float diff = b - x05;
    const float xi = df_dxk * inv1pc;
    if (1.0f + c >= fabsf(diff)) {
        dgc += xi * kLocalGC * (b - fmaf(c, b, x05) * inv1pc);
        dgb += xi * c * kLocalGB;
        return xi;
    }
    dgc += copysignf(kLocalGC, diff) * df_dxk;
    return df_dxk;
}

}  // namespace cnl

// ---------------------------------------------------------------------------------------------------------------
// Packed fp32x2 variants (Blackwell FFMA2 / FADD2 / FMUL2: one issue slot for two pixels).  The temporally blocked
// kernels are bound by instruction issue, not by FP32 throughput, so pairing the two halves of a lane's pixel quad
// roughly halves the issue slots of the add / multiply / fma part of the per-pixel math.  Differences whose operands
// are not register-pair aligned (right neighbours) are formed with scalar subtractions by the caller.
// ---------------------------------------------------------------------------------------------------------------
namespace cnl {

__device__ __forceinline__ float2 f2(float a, float b) { return make_float2(a, b); }
__device__ __forceinline__ float2 f2(float a) { return make_float2(a, a); }
__device__ __forceinline__ float2 add2(float2 a, float2 b) { return __fadd2_rn(a, b); }
__device__ __forceinline__ float2 mul2(float2 a, float2 b) { return __fmul2_rn(a, b); }
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) { return __ffma2_rn(a, b, c); }
__device__ __forceinline__ float2 sub2(float2 a, float2 b) { return __ffma2_rn(b, f2(-1.0f), a); }
__device__ __forceinline__ float2 neg2(float2 a) { return make_float2(-a.x, -a.y); }

// y_{k+1} rebuilt from two stored pre-prox iterates for two pixels (see rederive_y_fast)
__device__ __forceinline__ float2 rederive_y2(float2 x05, float2 x05m, float2 b, float2 c, float t) {
    const float2 opc = add2(c, f2(1.0f));
    const float2 inv = f2(rcp_approx(opc.x), rcp_approx(opc.y));
    const float2 cb = mul2(c, b);
    const float2 diff = sub2(b, x05);
    const float2 diff2 = sub2(b, x05m);
    const float2 xq = mul2(add2(cb, x05), inv);
    const float2 xqm = mul2(add2(cb, x05m), inv);
    float2 xk, xkm;
    {
        const bool quad = opc.x >= fabsf(diff.x);
        const float xl = x05.x + copysignf(c.x, diff.x);
        const float xlm = (c.x <= fabsf(diff2.x)) ? x05m.x + copysignf(c.x, diff2.x) : b.x;
        xk.x = quad ? xq.x : xl;
        xkm.x = quad ? xqm.x : xlm;
    }
    {
        const bool quad = opc.y >= fabsf(diff.y);
        const float xl = x05.y + copysignf(c.y, diff.y);
        const float xlm = (c.y <= fabsf(diff2.y)) ? x05m.y + copysignf(c.y, diff2.y) : b.y;
        xk.y = quad ? xq.y : xl;
        xkm.y = quad ? xqm.y : xlm;
    }
    return fma2(f2(t), sub2(xk, xkm), xk);
}

// adjoint fluxes and edge-weight gradients of two triangles given d1, d2 (y differences) and e1, e2 (g differences)
__device__ __forceinline__ void tri_adjoint2(float2 d1, float2 d2, float2 e1, float2 e2, float2 wx, float2 wy,
                                             float2& phi1, float2& phi2, float2& dwx, float2& dwy) {
    const float2 wd1 = mul2(wx, d1);
    const float2 wd2 = mul2(wy, d2);
    const float2 A = fma2(wd1, d1, mul2(wd2, d2));
    const float2 r = f2(rsqrt_approx(A.x), rsqrt_approx(A.y));
    const float2 dr = mul2(f2(kDelta), r);
    const bool bx = dr.x < 1.0f, by = dr.y < 1.0f;
    const float2 nom = f2(bx ? dr.x : 1.0f, by ? dr.y : 1.0f);
    const float2 hr = mul2(mul2(f2(0.5f), nom), mul2(r, r));
    const float2 den = f2(bx ? hr.x : 0.0f, by ? hr.y : 0.0f);
    const float2 S = fma2(wd1, e1, mul2(wd2, e2));
    const float2 dS = mul2(den, S);
    const float2 k2n = mul2(dS, f2(-2.0f));
    phi1 = mul2(wx, fma2(nom, e1, mul2(k2n, d1)));
    phi2 = mul2(wy, fma2(nom, e2, mul2(k2n, d2)));
    const float2 ndS = neg2(dS);
    dwx = mul2(mul2(f2(-kLocalGX), d1), fma2(nom, e1, mul2(ndS, d1)));
    dwy = mul2(mul2(f2(-kLocalGX), d2), fma2(nom, e2, mul2(ndS, d2)));
}

// momentum reverse + prox Jacobian for two pixels (see reverse_point in the kernels' source)
__device__ __forceinline__ float2 reverse_point2(float2 ybar, float2& acc, float2 x05, float2 b, float2 c, float t,
                                                 float2& dgc, float2& dgb, float2& xbar_out) {
    float2 xbar = fma2(f2(1.0f + t), ybar, acc);
    xbar = f2(clampf(xbar.x, -kClipLocal, kClipLocal), clampf(xbar.y, -kClipLocal, kClipLocal));
    acc = mul2(f2(-t), ybar);
    xbar_out = xbar;
    const float2 opc = add2(c, f2(1.0f));
    const float2 inv = f2(rcp_approx(opc.x), rcp_approx(opc.y));
    const float2 diff = sub2(b, x05);
    const float2 xq = mul2(fma2(c, b, x05), inv);
    const float2 xi = mul2(xbar, inv);
    // quadratic zone: d/dc = xbar (b - xq)/(1+c) * kLocalGC, d/db = xbar c/(1+c) * kLocalGB
    const float2 gc_q = mul2(mul2(xi, f2(kLocalGC)), sub2(b, xq));
    const float2 gb_q = mul2(mul2(xi, f2(kLocalGB)), c);
    float2 out;
    {
        const bool quad = opc.x >= fabsf(diff.x);
        dgc.x += quad ? gc_q.x : copysignf(kLocalGC, diff.x) * xbar.x;
        dgb.x += quad ? gb_q.x : 0.0f;
        out.x = quad ? xi.x : xbar.x;
    }
    {
        const bool quad = opc.y >= fabsf(diff.y);
        dgc.y += quad ? gc_q.y : copysignf(kLocalGC, diff.y) * xbar.y;
        dgb.y += quad ? gb_q.y : 0.0f;
        out.y = quad ? xi.y : xbar.y;
    }
    return out;
}

}  // namespace cnl

// ---------------------------------------------------------------------------------------------------------------
// Leaner forms used by the temporally blocked reverse kernels.  The reciprocal of 1 + c is the same in every fused
// step and every channel of a tile, so the caller computes it once; constant factors of the accumulated gradients
// (kLocalGC, kLocalGB, -kLocalGX) are applied once when the sums leave the CTA instead of in every step.
// ---------------------------------------------------------------------------------------------------------------
namespace cnl {

// y_{k+1} rebuilt from two stored pre-prox iterates for two pixels, 1/(1+c) supplied (see rederive_y_fast)
__device__ __forceinline__ float2 rederive_y2i(float2 x05, float2 x05m, float2 b, float2 c, float2 inv, float t) {
    const float2 opc = add2(c, f2(1.0f));
    const float2 cb = mul2(c, b);
    const float2 diff = sub2(b, x05);
    const float2 diff2 = sub2(b, x05m);
    const float2 xq = mul2(add2(cb, x05), inv);
    const float2 xqm = mul2(add2(cb, x05m), inv);
    float2 xk, xkm;
    {
        const bool quad = opc.x >= fabsf(diff.x);
        const float xl = x05.x + copysignf(c.x, diff.x);
        const float xlm = (c.x <= fabsf(diff2.x)) ? x05m.x + copysignf(c.x, diff2.x) : b.x;
        xk.x = quad ? xq.x : xl;
        xkm.x = quad ? xqm.x : xlm;
    }
    {
        const bool quad = opc.y >= fabsf(diff.y);
        const float xl = x05.y + copysignf(c.y, diff.y);
        const float xlm = (c.y <= fabsf(diff2.y)) ? x05m.y + copysignf(c.y, diff2.y) : b.y;
        xk.y = quad ? xq.y : xl;
        xkm.y = quad ? xqm.y : xlm;
    }
    return fma2(f2(t), sub2(xk, xkm), xk);
}

// Adjoint fluxes of two triangles; the edge-weight gradients are ACCUMULATED without their factor -kLocalGX:
//   awx += d1 (nom e1 - den S d1),  awy += d2 (nom e2 - den S d2)        (see tri_adjoint for the full expressions)
__device__ __forceinline__ void tri_adjoint2_acc(float2 d1, float2 d2, float2 e1, float2 e2, float2 wx, float2 wy,
                                                 float2& phi1, float2& phi2, float2& awx, float2& awy) {
    const float2 wd1 = mul2(wx, d1);
    const float2 wd2 = mul2(wy, d2);
    const float2 A = fma2(wd1, d1, mul2(wd2, d2));
    const float2 r = f2(rsqrt_approx(A.x), rsqrt_approx(A.y));
    const float2 dr = mul2(f2(kDelta), r);
    const bool bx = dr.x < 1.0f, by = dr.y < 1.0f;
    const float2 nom = f2(bx ? dr.x : 1.0f, by ? dr.y : 1.0f);
    const float2 hr = mul2(mul2(f2(-0.5f), nom), mul2(r, r));
    const float2 nden = f2(bx ? hr.x : 0.0f, by ? hr.y : 0.0f);        // -den
    const float2 S = fma2(wd1, e1, mul2(wd2, e2));
    const float2 ndS = mul2(nden, S);                                    // -den S
    const float2 r1 = mul2(ndS, d1);                                     // -den S d1
    const float2 r2 = mul2(ndS, d2);
    const float2 u1 = fma2(nom, e1, r1);                                 // nom e1 - den S d1
    const float2 u2 = fma2(nom, e2, r2);
    phi1 = mul2(wx, add2(u1, r1));                                       // wx (nom e1 - 2 den S d1)
    phi2 = mul2(wy, add2(u2, r2));
    awx = fma2(d1, u1, awx);
    awy = fma2(d2, u2, awy);
}

// Momentum reverse + prox Jacobian for two pixels with 1/(1+c) supplied.  The confidence and data-term gradients are
// ACCUMULATED without their constant factors:  agc += quad ? xi (b - xq) : sign(diff) xbar   (times kLocalGC later),
//                                              agb += quad ? xi : 0                          (times c kLocalGB later).
__device__ __forceinline__ float2 reverse_point2i(float2 ybar, float2& acc, float2 x05, float2 b, float2 c, float2 inv,
                                                  float t, float2& agc, float2& agb, float2& xbar_out) {
    float2 xbar = fma2(f2(1.0f + t), ybar, acc);
    xbar = f2(clampf(xbar.x, -kClipLocal, kClipLocal), clampf(xbar.y, -kClipLocal, kClipLocal));
    acc = mul2(f2(-t), ybar);
    xbar_out = xbar;
    const float2 opc = add2(c, f2(1.0f));
    const float2 diff = sub2(b, x05);
    const float2 xq = mul2(fma2(c, b, x05), inv);
    const float2 xi = mul2(xbar, inv);
    const float2 gq = mul2(xi, sub2(b, xq));
    float2 out;
    {
        const bool quad = opc.x >= fabsf(diff.x);
        agc.x += quad ? gq.x : copysignf(1.0f, diff.x) * xbar.x;
        agb.x += quad ? xi.x : 0.0f;
        out.x = quad ? xi.x : xbar.x;
    }
    {
        const bool quad = opc.y >= fabsf(diff.y);
        agc.y += quad ? gq.y : copysignf(1.0f, diff.y) * xbar.y;
        agb.y += quad ? xi.y : 0.0f;
        out.y = quad ? xi.y : xbar.y;
    }
    return out;
}

}  // namespace cnl
