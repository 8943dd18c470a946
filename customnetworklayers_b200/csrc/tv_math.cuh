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

__device__ __forceinline__ void tri_flux_fast(float yc, float yr, float yd, float wx, float wy, float& fx, float& fy) {
    const float wd1 = wx * (yc - yr);
    const float wd2 = wy * (yc - yd);
    const float A = fmaf(wd1, yc - yr, wd2 * (yc - yd));
    const float s = fminf(1.0f, kDelta * rsqrt_approx(A));
    fx = s * wd1;
    fy = s * wd2;
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

__device__ __forceinline__ void tri_adjoint_fast(float yc, float yr, float yd, float gc, float gr, float gd,
                                                 float wx, float wy, float& phi1, float& phi2, float& dwx, float& dwy) {
    const float d1 = yc - yr;
    const float d2 = yc - yd;
    const float e1 = gc - gr;
    const float e2 = gc - gd;
    const float wd1 = wx * d1;
    const float wd2 = wy * d2;
    const float A = fmaf(wd1, d1, wd2 * d2);
    const float r = rsqrt_approx(A);             // 1/T
    const bool big = kDelta * r < 1.0f;          // T > delta
    const float nom = big ? kDelta * r : 1.0f;
    const float den = big ? 0.5f * nom * r * r : 0.0f;
    const float S = fmaf(wd1, e1, wd2 * e2);
    const float k2 = 2.0f * den * S;
    phi1 = wx * fmaf(nom, e1, -k2 * d1);
    phi2 = wy * fmaf(nom, e2, -k2 * d2);
    // dwx = -kLocalGX d1 (nom e1 - den d1 (wx d1 e1 + wy d2 e2)) ; same for y
    const float dS = den * S;
    dwx = -kLocalGX * d1 * fmaf(nom, e1, -dS * d1);
    dwy = -kLocalGX * d2 * fmaf(nom, e2, -dS * d2);
}

}  // namespace cnl
