// Unrolled FISTA TGV-inpainting layer for sm_100a (reference: cudaTGV/cudaCode/TGVInpaintFistaBetas.cu).
//
// State per image and channel: primary plane u and auxiliary planes v1, v2, stored as [N][3][C][H][W].
// One launch per iteration.  A CTA owns a 16 x 64 pixel tile of one image and loops over the channels:
//   phase 0  the three planes of y (and of the incoming adjoint in the reverse kernel) are staged in shared memory
//            with a one-pixel frame, zero outside the image;
//   phase 1  every forward-difference triangle anchored in the tile, plus one row above and one column to the left,
//            is evaluated ONCE and its fluxes are written to shared memory (the reference evaluates three triangles
//            per pixel);
//   phase 2  every pixel combines its own fluxes with those of the triangles to its left and above (a divergence),
//            applies the prox / momentum step (forward) or the momentum reverse and prox Jacobian (reverse).
// Edge weights are multiplied by L = 1/(max(32.000001, max_p lip(p)) + 0.01), computed per image on the device.
// Per-edge gradients are accumulated by the owning pixel only, over channels in registers: no atomics.
#include <cmath>
#include <cstdlib>
#include <mutex>
#include <vector>

#include "common.h"
#include "tgv_vec.cuh"
#include "tv_math.cuh"

namespace cnl {

namespace tgv {

constexpr int TW = 64, TH = 16, NT = 256;
constexpr int YW = TW + 2, YH = TH + 2;          // staged y tile
constexpr int FW = TW + 1, FH = TH + 1;          // triangle tile (one extra column left, one extra row above)
constexpr float kDeltaU = 0.2f, kDeltaV1 = 0.2f, kDeltaV2 = 0.2f;     // __HDelta2__, __HDeltaY1__, __HDeltaY2__ (:58-60)
constexpr float kClip = 2000.0f;                 // clipLocalGrad (:78)
constexpr float kLipFloor = 32.000001f;          // max(12, 8*beta) + 1e-6 stored in a float (:2516)

struct Maps {
    const float* wx; const float* bx; const float* wy; const float* by;     // planes of dx = [wx, beta_x], dy = [wy, beta_y]
};

__device__ __forceinline__ Maps maps_of(const float* dx, const float* dy, size_t n, size_t plane) {
    Maps m;
    m.wx = dx + (n * 2 + 0) * plane; m.bx = dx + (n * 2 + 1) * plane;
    m.wy = dy + (n * 2 + 0) * plane; m.by = dy + (n * 2 + 1) * plane;
    return m;
}

// ---- Lipschitz constant (:101-148, :2513-2527) ----------------------------------------------------------------
__global__ void __launch_bounds__(NT)
tgv_lipschitz_kernel(const float* __restrict__ dx, const float* __restrict__ dy, int* __restrict__ lip_bits, int H, int W) {
    const size_t plane = (size_t)H * W;
    const size_t n = blockIdx.y;
    const Maps m = maps_of(dx, dy, n, plane);
    float best = 0.0f;
    for (size_t pix = (size_t)blockIdx.x * NT + threadIdx.x; pix < plane; pix += (size_t)gridDim.x * NT) {
        const int h = (int)(pix / W), w = (int)(pix - (size_t)h * W);
        const bool hr = w < W - 1, hd = h < H - 1, hl = w > 0, hu = h > 0;
        const float wx_0 = hl ? m.wx[pix - 1] : 0.f, wx_1 = hr ? m.wx[pix] : 0.f;
        const float wy_0 = hu ? m.wy[pix - W] : 0.f, wy_1 = hd ? m.wy[pix] : 0.f;
        // the reference reads beta at (w, h-1) under a w > 0 guard and at (w-1, h) under an h > 0 guard, relying on
        // clamp-to-edge addressing
        const size_t up = hu ? pix - W : pix, left = hl ? pix - 1 : pix;
        float wgt_x = 3.f * (wy_1 + wx_1), wgt_1 = 0.f, wgt_2 = 0.f;
        if (hu) { wgt_x += 3.f * wy_0; wgt_1 += 2.f * m.bx[left]; wgt_2 += 2.f * m.by[left]; }
        if (hl) { wgt_x += 3.f * wx_0; wgt_1 += 2.f * m.bx[up];   wgt_2 += 2.f * m.by[up]; }
        wgt_1 += 2.f * (hr ? m.bx[pix] : 0.f) + 2.f * (hd ? m.bx[pix] : 0.f) + 3.f * wx_1;
        wgt_2 += 2.f * (hr ? m.by[pix] : 0.f) + 2.f * (hd ? m.by[pix] : 0.f) + 3.f * wy_1;
        best = fmaxf(best, fmaxf(wgt_x, fmaxf(wgt_1, wgt_2)));
    }
    for (int off = 16; off > 0; off >>= 1) best = fmaxf(best, __shfl_down_sync(0xffffffffu, best, off));
    if ((threadIdx.x & 31) == 0 && best > 0.f) atomicMax(lip_bits + n, __float_as_int(best));   // positive floats order like ints
}

__global__ void tgv_lipschitz_init_kernel(int* lip_bits, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) lip_bits[i] = __float_as_int(kLipFloor);
}

__global__ void tgv_lipschitz_final_kernel(const int* __restrict__ lip_bits, float* __restrict__ L, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) L[i] = (float)(1.0 / (double)(__int_as_float(lip_bits[i]) + 0.01f));
}

// ---- shared-memory staging ------------------------------------------------------------------------------------
// Copies the (TH+2) x (TW+2) frame of one plane into shared memory; zero outside the image.
constexpr int kStagePasses = (YH * YW + NT - 1) / NT;

// Frame element handled by this thread in staging pass k: offset into the image plane, or -1 outside the image / frame.
__device__ __forceinline__ long long stage_offset(int k, int h0, int w0, int H, int W) {
    const int i = threadIdx.x + k * NT;
    const int r = i / YW, c = i - r * YW;
    const int h = h0 - 1 + r, w = w0 - 1 + c;
    return (i < YH * YW && h >= 0 && h < H && w >= 0 && w < W) ? (long long)h * W + w : -1;
}

// All loads of the three planes are issued before the first shared-memory store (15 independent loads per thread).
__device__ __forceinline__ void stage_planes3(const float* __restrict__ src, size_t plane_stride, float* __restrict__ dst,
                                              int h0, int w0, int H, int W) {
    float v[3][kStagePasses];
#pragma unroll
    for (int k = 0; k < kStagePasses; ++k) {
        const long long o = stage_offset(k, h0, w0, H, W);
#pragma unroll
        for (int q = 0; q < 3; ++q) v[q][k] = o >= 0 ? src[(size_t)q * plane_stride + o] : 0.0f;
    }
#pragma unroll
    for (int k = 0; k < kStagePasses; ++k) {
        const int i = threadIdx.x + k * NT;
        if (i < YH * YW) {
#pragma unroll
            for (int q = 0; q < 3; ++q) dst[q * YH * YW + i] = v[q][k];
        }
    }
}

struct Tri {
    float z1, z2, Hu, r_u;           // primary
    float a1[2], a2[2], H[2], r[2];  // auxiliary planes v1, v2
    float wx, wy, b[2];              // scaled, masked weights of this triangle
};

// All quantities of the triangle anchored at tile position (r, c) of the staged frame (pixel h0-1+r, w0-1+c).
__device__ __forceinline__ Tri triangle(const float* __restrict__ Y, int r, int c, int h, int w, int H, int W, const Maps& m,
                                        float L) {
    Tri t;
    const bool in = h >= 0 && w >= 0 && h < H && w < W;
    const bool mx = in && w < W - 1, my = in && h < H - 1;
    const size_t pix = in ? (size_t)h * W + w : 0;
    t.wx = mx ? __fmul_rn(L, __ldg(m.wx + pix)) : 0.f;
    t.wy = my ? __fmul_rn(L, __ldg(m.wy + pix)) : 0.f;
    t.b[0] = in ? __fmul_rn(L, __ldg(m.bx + pix)) : 0.f;
    t.b[1] = in ? __fmul_rn(L, __ldg(m.by + pix)) : 0.f;
    const float* u = Y;
    const float* v1 = Y + YH * YW;
    const float* v2 = Y + 2 * YH * YW;
    const int o = r * YW + c;
    t.z1 = mx ? (u[o + 1] - u[o] - v1[o]) : 0.f;
    t.z2 = my ? (u[o + YW] - u[o] - v2[o]) : 0.f;
    t.r_u = rsqrtf(t.wy * t.z2 * t.z2 + t.wx * t.z1 * t.z1);
    t.Hu = fminf(1.f, t.r_u * kDeltaU);
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        const float* v = j == 0 ? v1 : v2;
        t.a1[j] = mx ? (v[o + 1] - v[o]) : 0.f;
        t.a2[j] = my ? (v[o + YW] - v[o]) : 0.f;
        t.r[j] = rsqrtf(t.b[j] * (t.a1[j] * t.a1[j] + t.a2[j] * t.a2[j]));
        t.H[j] = fminf(1.f, t.r[j] * (j == 0 ? kDeltaV1 : kDeltaV2));
    }
    return t;
}

// ---- forward iteration (:1546-1776, with the history store of :2005-2236) ---------------------------------------
__global__ void __launch_bounds__(NT, 2)
tgv_fwd_kernel(const float* __restrict__ y_in, float* __restrict__ y_out, float* __restrict__ x,
               const float* __restrict__ b, const float* __restrict__ cf, const float* __restrict__ dx,
               const float* __restrict__ dy, const float* __restrict__ Lbuf, float* __restrict__ hist,
               int C, int H, int W, float t) {
    __shared__ float Y[3 * YH * YW];
    __shared__ float F[6 * FH * FW];         // Fx, Fy, G1x, G1y, G2x, G2y
    const size_t plane = (size_t)H * W;
    const size_t n = blockIdx.z;
    const int h0 = blockIdx.y * TH, w0 = blockIdx.x * TW;
    const Maps m = maps_of(dx, dy, n, plane);
    const float L = Lbuf[n];
    for (int ch = 0; ch < C; ++ch) {
        const size_t base = n * 3 * C * plane + (size_t)ch * plane;        // plane k of this channel: base + k*C*plane
        __syncthreads();
        stage_planes3(y_in + base, (size_t)C * plane, Y, h0, w0, H, W);
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < (FH * FW + NT - 1) / NT; ++kk) {
            const int i = threadIdx.x + kk * NT;
            if (i >= FH * FW) break;
            const int r = i / FW, c = i - r * FW;
            const Tri tr = triangle(Y, r, c, h0 - 1 + r, w0 - 1 + c, H, W, m, L);
            F[0 * FH * FW + i] = tr.wx * tr.z1 * tr.Hu;
            F[1 * FH * FW + i] = tr.wy * tr.z2 * tr.Hu;
            F[2 * FH * FW + i] = tr.b[0] * tr.a1[0] * tr.H[0];
            F[3 * FH * FW + i] = tr.b[0] * tr.a2[0] * tr.H[0];
            F[4 * FH * FW + i] = tr.b[1] * tr.a1[1] * tr.H[1];
            F[5 * FH * FW + i] = tr.b[1] * tr.a2[1] * tr.H[1];
        }
        __syncthreads();
        float xin[(TH * TW) / NT][3], bin[(TH * TW) / NT], cin[(TH * TW) / NT];
#pragma unroll
        for (int kk = 0; kk < (TH * TW) / NT; ++kk) {
            const int i = threadIdx.x + kk * NT;
            const int r = i / TW, c = i - r * TW;
            const int h = h0 + r, w = w0 + c;
            const bool ok = h < H && w < W;
            const size_t pix = ok ? (size_t)h * W + w : 0;
#pragma unroll
            for (int q = 0; q < 3; ++q) xin[kk][q] = ok ? x[base + (size_t)q * C * plane + pix] : 0.f;
            bin[kk] = ok ? __ldg(b + (n * C + ch) * plane + pix) : 0.f;
            cin[kk] = ok ? __ldg(cf + n * plane + pix) : 0.f;
        }
#pragma unroll
        for (int kk = 0; kk < (TH * TW) / NT; ++kk) {
            const int i = threadIdx.x + kk * NT;
            const int r = i / TW, c = i - r * TW;
            const int h = h0 + r, w = w0 + c;
            if (h >= H || w >= W) continue;
            const size_t pix = (size_t)h * W + w;
            const int fo = (r + 1) * FW + (c + 1), yo = (r + 1) * YW + (c + 1);
            const float* Fx = F; const float* Fy = F + FH * FW;
            const float u_half = Y[yo] + Fx[fo] + Fy[fo] - Fx[fo - 1] - Fy[fo - FW];
            float vnew[2];
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const float* Gx = F + (2 + 2 * j) * FH * FW;
                const float* Gy = F + (3 + 2 * j) * FH * FW;
                vnew[j] = Y[(1 + j) * YH * YW + yo] + Gx[fo] + Gy[fo] - Gx[fo - 1] - Gy[fo - FW] + (j == 0 ? Fx[fo] : Fy[fo]);
            }
            const float xu = prox_huber(u_half, bin[kk], cin[kk]);
            const float news[3] = {xu, vnew[0], vnew[1]};
            const float halfs[3] = {u_half, vnew[0], vnew[1]};
#pragma unroll
            for (int k = 0; k < 3; ++k) {
                const size_t o = base + (size_t)k * C * plane + pix;
                const float xp = xin[kk][k];
                hist[o] = halfs[k];
                x[o] = news[k];
                y_out[o] = news[k] + t * (news[k] - xp);
            }
        }
    }
}

// ---- reverse sweep ----------------------------------------------------------------------------------------------
// Seed at the last iteration (:151-218): prox Jacobian on the primary plane, auxiliary planes pass through.
__global__ void __launch_bounds__(NT)
tgv_seed_kernel(const float* __restrict__ grad, const float* __restrict__ hist_g, const float* __restrict__ b,
                const float* __restrict__ cf, float* __restrict__ g_out, float* __restrict__ g_c, float* __restrict__ g_b,
                int C, size_t plane) {
    const size_t pix = (size_t)blockIdx.x * NT + threadIdx.x;
    if (pix >= plane) return;
    const size_t n = blockIdx.y;
    const float conf = __ldg(cf + n * plane + pix);
    float dgc = 0.f;
    for (int ch = 0; ch < C; ++ch) {
        const size_t base = n * 3 * C * plane + (size_t)ch * plane + pix;
        float dgb = 0.f;
        g_out[base] = prox_reverse(grad[base], hist_g[base], __ldg(b + (n * C + ch) * plane + pix), conf, dgc, dgb);
        g_b[(n * C + ch) * plane + pix] = dgb;
        g_out[base + (size_t)C * plane] = grad[base + (size_t)C * plane];
        g_out[base + 2 * (size_t)C * plane] = grad[base + 2 * (size_t)C * plane];
    }
    g_c[n * plane + pix] = dgc;
}

constexpr int kRevSmemFloats = 6 * YH * YW + 7 * FH * FW;
constexpr int kTriPasses = (FH * FW + NT - 1) / NT;
constexpr int kPixPasses = (TH * TW) / NT;

// One reverse iteration (:224-644; with `ckpt` the segment-start variant :1061-1473).
//   hist_g, hist_gm1 : stored iterates of iteration g and g-1 ([N][3][C][H][W]); u of y_{g+1} is rebuilt from their
//                      primary planes, v1, v2 are the stored new auxiliary planes of iteration g (:1478-1541)
//   ckpt             : if non-null all three planes of y come from this checkpoint instead
//   typo             : reproduce the reference's factor W/rsqrt(A)^2 in the v2 term arriving from the triangle
//                      above (:355, :804); the reference's segment-start kernel does not have it
__global__ void __launch_bounds__(NT, 2)
tgv_rev_kernel(const float* __restrict__ hist_g, const float* __restrict__ hist_gm1, const float* __restrict__ ckpt,
               const float* __restrict__ g_in, float* __restrict__ g_out, float* __restrict__ acc,
               const float* __restrict__ b, const float* __restrict__ cf, const float* __restrict__ dx,
               const float* __restrict__ dy, const float* __restrict__ Lbuf, float* __restrict__ g_c,
               float* __restrict__ g_b, float* __restrict__ g_dx, float* __restrict__ g_dy, float* __restrict__ x1bar,
               int C, int H, int W, float t, int typo) {
    extern __shared__ float sm[];
    float* Y = sm;
    float* Gq = sm + 3 * YH * YW;
    float* A = sm + 6 * YH * YW;              // psi1, psi2, chi1x, chi1y, chi2x, chi2y, chi2y (down-going)
    const size_t plane = (size_t)H * W;
    const size_t n = blockIdx.z;
    const int h0 = blockIdx.y * TH, w0 = blockIdx.x * TW;
    const Maps m = maps_of(dx, dy, n, plane);
    const float L = Lbuf[n];
    float gw[kTriPasses][4];                  // d wx, d beta_x, d wy, d beta_y of this thread's triangles
    float gconf[kPixPasses];
#pragma unroll
    for (int k = 0; k < kTriPasses; ++k) gw[k][0] = gw[k][1] = gw[k][2] = gw[k][3] = 0.f;
#pragma unroll
    for (int k = 0; k < kPixPasses; ++k) gconf[k] = 0.f;

    for (int ch = 0; ch < C; ++ch) {
        const size_t base = n * 3 * C * plane + (size_t)ch * plane;
        const size_t bbase = (n * C + ch) * plane;
        __syncthreads();
        // phase 0: stage y and the incoming adjoint; every load of a pass is issued before the arithmetic
        {
            float hg[3][kStagePasses], hm[kStagePasses], bq[kStagePasses], cq[kStagePasses], qq[3][kStagePasses];
#pragma unroll
            for (int k = 0; k < kStagePasses; ++k) {
                const long long pix = stage_offset(k, h0, w0, H, W);
                const bool ok = pix >= 0;
                const size_t o = base + (ok ? (size_t)pix : 0);
                const float* ysrc = ckpt ? ckpt : hist_g;
#pragma unroll
                for (int q = 0; q < 3; ++q) {
                    hg[q][k] = ok ? ysrc[o + (size_t)q * C * plane] : 0.f;
                    qq[q][k] = ok ? g_in[o + (size_t)q * C * plane] : 0.f;
                }
                hm[k] = (ok && !ckpt) ? hist_gm1[o] : 0.f;
                bq[k] = (ok && !ckpt) ? __ldg(b + bbase + pix) : 0.f;
                cq[k] = (ok && !ckpt) ? __ldg(cf + n * plane + pix) : 0.f;
            }
#pragma unroll
            for (int k = 0; k < kStagePasses; ++k) {
                const int i = threadIdx.x + k * NT;
                if (i >= YH * YW) break;
                const bool ok = stage_offset(k, h0, w0, H, W) >= 0;
                float yu = hg[0][k];
                if (ok && !ckpt) yu = rederive_y(hg[0][k], hm[k], bq[k], cq[k], t);
                Y[i] = yu; Y[YH * YW + i] = hg[1][k]; Y[2 * YH * YW + i] = hg[2][k];
                Gq[i] = qq[0][k]; Gq[YH * YW + i] = qq[1][k]; Gq[2 * YH * YW + i] = qq[2][k];
            }
        }
        __syncthreads();
        // phase 1: adjoint fluxes per triangle
#pragma unroll
        for (int k = 0; k < kTriPasses; ++k) {
            const int i = threadIdx.x + k * NT;
            if (i >= FH * FW) break;
            const int r = i / FW, c = i - r * FW;
            const int h = h0 - 1 + r, w = w0 - 1 + c;
            const Tri tr = triangle(Y, r, c, h, w, H, W, m, L);
            const int o = r * YW + c;
            const float* gu = Gq; const float* g1 = Gq + YH * YW; const float* g2 = Gq + 2 * YH * YW;
            const float Ex = gu[o] - gu[o + 1] + g1[o];
            const float Ey = gu[o] - gu[o + YW] + g2[o];
            const float a1 = tr.z1 * tr.wx, a2 = tr.z2 * tr.wy;
            const float S = a1 * Ex + a2 * Ey;
            const float dW = tr.Hu < 1.f ? tr.Hu * tr.r_u * tr.r_u : 0.f;
            A[0 * FH * FW + i] = tr.wx * tr.Hu * Ex - dW * a1 * S;
            A[1 * FH * FW + i] = tr.wy * tr.Hu * Ey - dW * a2 * S;
            float gwu_x = kLocalGX * (Ex * tr.z1 * tr.Hu - 0.5f * tr.z1 * tr.z1 * dW * S);
            float gwu_y = kLocalGX * (Ey * tr.z2 * tr.Hu - 0.5f * tr.z2 * tr.z2 * dW * S);
            float gbeta[2];
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const float* gj = j == 0 ? g1 : g2;
                const bool in = h >= 0 && w >= 0 && h < H && w < W;
                const float E1 = (in && w < W - 1) ? gj[o] - gj[o + 1] : 0.f;
                const float E2 = (in && h < H - 1) ? gj[o] - gj[o + YW] : 0.f;
                const float b1 = tr.a1[j], b2 = tr.a2[j], beta = tr.b[j], Hj = tr.H[j];
                const float Sj = b1 * E1 + b2 * E2;
                const bool act = Hj < 1.f;
                const float dWj = act ? Hj * tr.r[j] * tr.r[j] : 0.f;
                const float chx = beta * (Hj * E1 - dWj * beta * b1 * Sj);
                const float chy = beta * (Hj * E2 - dWj * beta * b2 * Sj);
                A[(2 + 2 * j) * FH * FW + i] = chx;
                A[(3 + 2 * j) * FH * FW + i] = chy;
                if (j == 1) {
                    float down = chy;
                    if (typo && act) down = beta * (Hj * E2 - (Hj * beta * (b1 * b1 + b2 * b2)) * beta * b2 * Sj);
                    A[6 * FH * FW + i] = down;
                }
                gbeta[j] = kLocalGX * (Sj * Hj - 0.5f * (b1 * b1 + b2 * b2) * dWj * beta * Sj);
            }
            gw[k][0] += gwu_x; gw[k][1] += gbeta[0]; gw[k][2] += gwu_y; gw[k][3] += gbeta[1];
        }
        __syncthreads();
        // phase 2: divergence of the adjoint fluxes, momentum reverse, prox Jacobian.  The pointwise operands of all
        // passes are loaded first so that their latencies overlap.
        float accv[kPixPasses][3], hu[kPixPasses], bv[kPixPasses], cv[kPixPasses], gbv[kPixPasses];
#pragma unroll
        for (int k = 0; k < kPixPasses; ++k) {
            const int i = threadIdx.x + k * NT;
            const int r = i / TW, c = i - r * TW;
            const int h = h0 + r, w = w0 + c;
            const bool ok = h < H && w < W;
            const size_t pix = ok ? (size_t)h * W + w : 0;
#pragma unroll
            for (int q = 0; q < 3; ++q) accv[k][q] = ok ? acc[base + (size_t)q * C * plane + pix] : 0.f;
            hu[k] = ok ? hist_g[base + pix] : 0.f;
            bv[k] = ok ? __ldg(b + bbase + pix) : 0.f;
            cv[k] = ok ? __ldg(cf + n * plane + pix) : 0.f;
            gbv[k] = ok ? g_b[bbase + pix] : 0.f;
        }
#pragma unroll
        for (int k = 0; k < kPixPasses; ++k) {
            const int i = threadIdx.x + k * NT;
            const int r = i / TW, c = i - r * TW;
            const int h = h0 + r, w = w0 + c;
            if (h >= H || w >= W) continue;
            const size_t pix = (size_t)h * W + w;
            const int fo = (r + 1) * FW + (c + 1), yo = (r + 1) * YW + (c + 1);
            const float* P1 = A; const float* P2 = A + FH * FW;
            const float* C1x = A + 2 * FH * FW; const float* C1y = A + 3 * FH * FW;
            const float* C2x = A + 4 * FH * FW; const float* C2y = A + 5 * FH * FW; const float* C2d = A + 6 * FH * FW;
            float ybar[3];
            ybar[0] = Gq[yo] - P1[fo] - P2[fo] + P1[fo - 1] + P2[fo - FW];
            ybar[1] = Gq[YH * YW + yo] - P1[fo] - C1x[fo] - C1y[fo] + C1x[fo - 1] + C1y[fo - FW];
            ybar[2] = Gq[2 * YH * YW + yo] - P2[fo] - C2x[fo] - C2y[fo] + C2x[fo - 1] + C2d[fo - FW];
            float xbar[3];
#pragma unroll
            for (int q = 0; q < 3; ++q) {
                const size_t o = base + (size_t)q * C * plane + pix;
                xbar[q] = clampf(accv[k][q] + (1.0f + t) * ybar[q], -kClip, kClip);
                acc[o] = -t * ybar[q];
                if (x1bar) x1bar[o] = xbar[q];
            }
            float dgb = 0.f;
            g_out[base + pix] = prox_reverse(xbar[0], hu[k], bv[k], cv[k], gconf[k], dgb);
            g_b[bbase + pix] = gbv[k] + dgb;
            g_out[base + (size_t)C * plane + pix] = xbar[1];
            g_out[base + 2 * (size_t)C * plane + pix] = xbar[2];
        }
    }
    // per-pixel gradients shared by the channels: owner-computes, plain read-modify-write
#pragma unroll
    for (int k = 0; k < kPixPasses; ++k) {
        const int i = threadIdx.x + k * NT;
        const int r = i / TW, c = i - r * TW;
        const int h = h0 + r, w = w0 + c;
        if (h < H && w < W) g_c[n * plane + (size_t)h * W + w] += gconf[k];
    }
#pragma unroll
    for (int k = 0; k < kTriPasses; ++k) {
        const int i = threadIdx.x + k * NT;
        if (i >= FH * FW) break;
        const int r = i / FW, c = i - r * FW;
        if (r == 0 || c == 0) continue;               // frame triangles belong to the neighbouring tile
        const int h = h0 - 1 + r, w = w0 - 1 + c;
        if (h >= H || w >= W) continue;
        const size_t pix = (size_t)h * W + w;
        g_dx[(n * 2 + 0) * plane + pix] += gw[k][0];
        g_dx[(n * 2 + 1) * plane + pix] += gw[k][1];
        g_dy[(n * 2 + 0) * plane + pix] += gw[k][2];
        g_dy[(n * 2 + 1) * plane + pix] += gw[k][3];
    }
}

// ---- finalisation (TGVInpaintFistaHelp.cu:119-176, TGVInpaintFistaBetas.cu:2990-3050) ---------------------------
constexpr int kOut = 5;                 // C, X, Y, B, I
constexpr int kStatBlocks = 128;

struct FinArgs {
    float* ptr[kOut];
    unsigned long long count[kOut];
    float scale[kOut];                  // multiplied by L[n] for X and Y
    int per_image_L[kOut];
    unsigned long long per_image[kOut]; // elements per image (for the L lookup)
};

__global__ void __launch_bounds__(256)
tgv_stats_kernel(FinArgs a, double* __restrict__ partial) {
    const int o = blockIdx.y;
    const float* p = a.ptr[o];
    double s = 0.0, bad = 0.0;
    auto take = [&](float v) { if (finite_f(v)) s += fmin(fabs((double)v), 5000000.0); else bad += 1.0; };
    const unsigned long long cnt = a.count[o];
    const unsigned long long tid = (unsigned long long)blockIdx.x * 256 + threadIdx.x, nthreads = (unsigned long long)gridDim.x * 256;
    // 16-byte vectors where the plane allows it (two in flight per thread), scalars for the tail
    const unsigned long long nvec = (reinterpret_cast<size_t>(p) & 15) == 0 ? cnt / 4 : 0;
    const float4* p4 = reinterpret_cast<const float4*>(p);
    unsigned long long i = tid;
    for (; i + nthreads < nvec; i += 2 * nthreads) {
        const float4 a0 = p4[i], a1 = p4[i + nthreads];
        take(a0.x); take(a0.y); take(a0.z); take(a0.w);
        take(a1.x); take(a1.y); take(a1.z); take(a1.w);
    }
    for (; i < nvec; i += nthreads) {
        const float4 a0 = p4[i];
        take(a0.x); take(a0.y); take(a0.z); take(a0.w);
    }
    for (i = nvec * 4 + tid; i < cnt; i += nthreads) take(p[i]);
    for (int off = 16; off > 0; off >>= 1) {
        s += __shfl_down_sync(0xffffffffu, s, off);
        bad += __shfl_down_sync(0xffffffffu, bad, off);
    }
    __shared__ double sh[2][8];
    if ((threadIdx.x & 31) == 0) { sh[0][threadIdx.x >> 5] = s; sh[1][threadIdx.x >> 5] = bad; }
    __syncthreads();
    if (threadIdx.x == 0) {
        double ts = 0.0, tb = 0.0;
        for (int i = 0; i < 8; ++i) { ts += sh[0][i]; tb += sh[1][i]; }
        partial[(o * kStatBlocks + blockIdx.x) * 2] = ts;
        partial[(o * kStatBlocks + blockIdx.x) * 2 + 1] = tb;
    }
}

__global__ void __launch_bounds__(32)
tgv_conditioner_kernel(const double* __restrict__ partial, FinArgs a, double* __restrict__ state, float* __restrict__ factor,
                       int run) {
    const double run_step = fmin(0.95, (double)run / (double)(run + 1));
    for (int o = 0; o < kOut; ++o) {
        double s = 0.0, bad = 0.0;
        for (int i = threadIdx.x; i < kStatBlocks; i += 32) { s += partial[(o * kStatBlocks + i) * 2]; bad += partial[(o * kStatBlocks + i) * 2 + 1]; }
        for (int off = 16; off > 0; off >>= 1) {
            s += __shfl_down_sync(0xffffffffu, s, off);
            bad += __shfl_down_sync(0xffffffffu, bad, off);
        }
        if (threadIdx.x != 0) continue;
        double av = state[o];
        const double av_gc = (bad > 0.0) ? av * 1000.0 : (a.count[o] ? s / (double)a.count[o] : 0.0);
        float f = 1.0f;
        if (run >= 10 && av * 35.0 < av_gc) { f = 0.0f; av = av * run_step + (1.0 - run_step) * 10.0 * av; }
        else if (run >= 10 && av * 10.0 < av_gc) { const double mult = 10.0 * av / av_gc; f = (float)mult; av = av * run_step + (1.0 - run_step) * av_gc * mult; }
        else av = av * run_step + (1.0 - run_step) * av_gc;
        state[o] = av;
        factor[o] = f;
    }
}

// g = clamp(finite ? g : 0, +-5e6) * factor * scale (* L of the image for the edge-weight gradients)
__global__ void __launch_bounds__(256)
tgv_apply_kernel(FinArgs a, const float* __restrict__ factor, const float* __restrict__ Lbuf) {
    const int o = blockIdx.y;
    float* p = a.ptr[o];
    const float f = factor ? factor[o] : 1.0f;
    const float base = a.scale[o];
    const bool perL = a.per_image_L[o] != 0;
    const unsigned long long per = a.per_image[o], cnt = a.count[o];
    auto fix = [&](float v, float sc) {
        if (!finite_f(v)) v = 0.f;
        return clampf(v, -5000000.0f, 5000000.0f) * f * sc;
    };
    const unsigned long long tid = (unsigned long long)blockIdx.x * 256 + threadIdx.x, nthreads = (unsigned long long)gridDim.x * 256;
    // a 16-byte vector never straddles two images when the per-image element count is a multiple of 4
    const bool vec_ok = (reinterpret_cast<size_t>(p) & 15) == 0 && (!perL || per % 4 == 0);
    const unsigned long long nvec = vec_ok ? cnt / 4 : 0;
    float4* p4 = reinterpret_cast<float4*>(p);
    for (unsigned long long i = tid; i < nvec; i += nthreads) {
        float4 v = p4[i];
        const float sc = perL ? base * Lbuf[(i * 4) / per] : base;
        v.x = fix(v.x, sc); v.y = fix(v.y, sc); v.z = fix(v.z, sc); v.w = fix(v.w, sc);
        p4[i] = v;
    }
    for (unsigned long long i = nvec * 4 + tid; i < cnt; i += nthreads) p[i] = fix(p[i], perL ? base * Lbuf[i / per] : base);
}

// flags[0] = number of non-finite entries, flags[1] = number of non-zero entries of the upstream gradient
__global__ void __launch_bounds__(256)
tgv_upstream_check_kernel(const float* __restrict__ g, unsigned long long count, unsigned int* __restrict__ flags) {
    unsigned int bad = 0, nz = 0;
    for (unsigned long long i = (unsigned long long)blockIdx.x * 256 + threadIdx.x; i < count; i += (unsigned long long)gridDim.x * 256) {
        const float v = g[i];
        if (!finite_f(v)) bad++; else if (v != 0.f) nz++;
    }
    bad = __reduce_add_sync(0xffffffffu, bad);
    nz = __reduce_add_sync(0xffffffffu, nz);
    if ((threadIdx.x & 31) == 0) {
        if (bad) atomicAdd(flags, bad);
        if (nz) atomicAdd(flags + 1, nz > 0 ? 1u : 0u);
    }
}

// ---- per-id slots -----------------------------------------------------------------------------------------------
struct Slot {
    float* arena = nullptr;
    size_t arena_floats = 0;
    double* cond = nullptr;
    int n = 0, ch = 0, h = 0, w = 0, its = 0;
    int pitch = 0;                   // row pitch (floats) of the arena planes of the stored forward pass
    bool staged = false;             // the register-tiled kernels ran on zero-padded copies
    bool have_forward = false;
    int run = 0;
    int opt_conditioner = 1;
    std::vector<int> sched;
    std::vector<float> steps;
};

static std::mutex g_mutex;
static std::vector<Slot*> g_slots;      // [device * CNL_NUM_IDS + id]

static Slot* get_slot(int id, int* rc) {
    int dev = 0;
    const cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) { *rc = check_cuda(e, "cudaGetDevice"); return nullptr; }
    const size_t idx = (size_t)dev * CNL_NUM_IDS + id;
    if (idx >= g_slots.size()) g_slots.resize(idx + 1, nullptr);
    if (!g_slots[idx]) g_slots[idx] = new Slot();
    *rc = CNL_OK;
    return g_slots[idx];
}

static inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

struct Layout {
    size_t vol;                        // n*3*ch*h*w rounded up (w = row pitch)
    size_t map;                        // n*h*w rounded up
    size_t y0, y1, ga, gb, acc, L, lip, flags, ckpt, hist, total;
    size_t stage;                      // staged mode: 2*(2+2+1+ch) maps and 2 volumes of zero-padded copies
};

static Layout make_layout(size_t n, size_t ch, size_t h, size_t w, size_t its_eff, size_t nckpt, bool staged = false) {
    Layout l;
    l.vol = align_up(n * 3 * ch * h * w, 64);
    l.map = align_up(n * h * w, 64);
    size_t o = 0;
    l.y0 = o; o += l.vol;
    l.y1 = o; o += l.vol;
    l.ga = o; o += l.vol;
    l.gb = o; o += l.vol;
    l.acc = o; o += l.vol;
    l.L = o; o += align_up(n, 64);
    l.lip = o; o += align_up(n, 64);
    l.flags = o; o += 64;
    l.ckpt = o; o += l.vol * nckpt;
    l.hist = o; o += l.vol * its_eff;
    l.stage = o; o += staged ? 2 * (5 + ch) * l.map + 2 * l.vol : 0;
    l.total = o;
    return l;
}

static void schedule(int its, std::vector<int>& sched, std::vector<float>& steps) {
    const int n = (int)std::floor(std::sqrt((double)its));                 // :2541-2551
    sched.resize(n);
    for (int i = 0; i < n; ++i) sched[i] = (int)(std::floor(i * std::sqrt((double)its) * 0.5) * 2);
    steps.resize(its);
    double t = 1.0, t_ = 1.0;
    for (int i = 0; i < its; ++i) { t_ = t; t = (1.0 + std::sqrt(1.0 + 4.0 * t * t)) / 2.0; steps[i] = (float)std::max(0.0, (t_ - 1.0) / t); }
}

static int check_args(const void* const* ptrs, int nptr, int n, int ch, int h, int w, int its, int id) {
    if (id < 0 || id >= CNL_NUM_IDS) return fail(CNL_ERR_BAD_ID, "id %d is outside 0..%d", id, CNL_NUM_IDS - 1);
    if (n < 1 || ch < 1 || h < 1 || w < 1) return fail(CNL_ERR_BAD_SHAPE, "n, ch, h, w must be >= 1 (got %d, %d, %d, %d)", n, ch, h, w);
    if ((long long)h * w > 0x3fffffffLL || n > 65535) return fail(CNL_ERR_BAD_SHAPE, "image or batch beyond the supported range");
    if (its < 2) return fail(CNL_ERR_BAD_ITS, "its must be >= 2 (got %d)", its);
    for (int i = 0; i < nptr; ++i) if (!ptrs[i]) return fail(CNL_ERR_NULL, "null pointer argument (position %d)", i);
    return CNL_OK;
}

static int ensure_arena(Slot& s, size_t floats) {
    if (s.arena && s.arena_floats >= floats) return CNL_OK;
    const char* env = std::getenv("CNL_MAX_ARENA_GB");
    const double gb = (env && std::atof(env) > 0) ? std::atof(env) : 150.0;
    if ((double)floats * 4.0 > gb * 1024.0 * 1024.0 * 1024.0)
        return fail(CNL_ERR_ALLOC, "iterate history needs %.2f GB, above the CNL_MAX_ARENA_GB budget", floats * 4.0 / 1073741824.0);
    if (s.arena) { CNL_TRY(check_cuda(cudaDeviceSynchronize(), "cudaDeviceSynchronize")); cudaFree(s.arena); s.arena = nullptr; s.arena_floats = 0; }
    void* p = nullptr;
    if (cudaMalloc(&p, floats * sizeof(float)) != cudaSuccess) { cudaGetLastError(); return fail(CNL_ERR_ALLOC, "cudaMalloc of %.2f GB failed", floats * 4.0 / 1073741824.0); }
    s.arena = static_cast<float*>(p);
    s.arena_floats = floats;
    return CNL_OK;
}

// The register-tiled kernels serve every shape with W % 4 == 0 and 16-byte aligned planes; CNL_TGV_NO_VEC=1 forces
// the scalar shared-memory kernels.
static bool vec_enabled() {
    static int v = -1;
    if (v < 0) { const char* e = std::getenv("CNL_TGV_NO_VEC"); v = (e && e[0] == '1') ? 0 : 1; }
    return v == 1;
}

// Zero-padded copy of `rows` image rows of w floats into rows of `pitch` floats, and back.
static int pad_rows(float* dst, const float* src, size_t rows, int w, int pitch, cudaStream_t st) {
    CNL_TRY(check_cuda(cudaMemsetAsync(dst, 0, rows * pitch * sizeof(float), st), "zero staging buffer"));
    return check_cuda(cudaMemcpy2DAsync(dst, pitch * sizeof(float), src, w * sizeof(float), w * sizeof(float), rows,
                                        cudaMemcpyDeviceToDevice, st), "pad rows");
}
static int unpad_rows(float* dst, const float* src, size_t rows, int w, int pitch, cudaStream_t st) {
    return check_cuda(cudaMemcpy2DAsync(dst, w * sizeof(float), src, pitch * sizeof(float), w * sizeof(float), rows,
                                        cudaMemcpyDeviceToDevice, st), "unpad rows");
}

static int lipschitz(const float* dx, const float* dy, float* Lbuf, int* lip_bits, int n, int h, int w, cudaStream_t st) {
    tgv_lipschitz_init_kernel<<<(n + 127) / 128, 128, 0, st>>>(lip_bits, n);
    CNL_TRY(after_launch("tgv_lipschitz_init_kernel"));
    const size_t plane = (size_t)h * w;
    const unsigned gx = (unsigned)std::min<size_t>((plane + NT - 1) / NT, 592);
    tgv_lipschitz_kernel<<<dim3(gx, n), NT, 0, st>>>(dx, dy, lip_bits, h, w);
    CNL_TRY(after_launch("tgv_lipschitz_kernel"));
    tgv_lipschitz_final_kernel<<<(n + 127) / 128, 128, 0, st>>>(lip_bits, Lbuf, n);
    return after_launch("tgv_lipschitz_final_kernel");
}

static int forward_impl(const float* dx, const float* dy, const float* c, const float* b, const float* init, float* out,
                        int n, int ch, int h, int w, int its, int id, cudaStream_t st) {
    const void* ptrs[] = {dx, dy, c, b, init, out};
    CNL_TRY(check_args(ptrs, 6, n, ch, h, w, its, id));
    std::lock_guard<std::mutex> lock(g_mutex);
    int rc;
    Slot* sp = get_slot(id, &rc);
    if (!sp) return rc;
    Slot& s = *sp;
    s.have_forward = false;
    schedule(its, s.sched, s.steps);
    const int its_eff = 2 * (its / 2);
    // The register-tiled kernels read 16-byte vectors: tensors whose rows are not a multiple of 4 floats, or that are
    // not 16-byte aligned, are staged into zero-padded copies with such a pitch (pad columns stay zero through both
    // sweeps); the results are copied back row by row.
    const void* planes[] = {dx, dy, c, b, init, out};
    const bool direct = tgv_vec_supported(w, planes, 6);
    const bool vec = vec_enabled();
    const bool staged = vec && !direct;
    const int P = staged ? ((w + 3) & ~3) : w;
    const Layout l = make_layout(n, ch, h, P, its_eff, s.sched.size(), staged);
    CNL_TRY(ensure_arena(s, l.total));
    s.staged = staged;
    s.pitch = P;
    const size_t vol_bytes = (size_t)n * 3 * ch * h * P * sizeof(float);
    float* y0 = s.arena + l.y0;
    float* y1 = s.arena + l.y1;
    float* Lbuf = s.arena + l.L;
    CNL_TRY(lipschitz(dx, dy, Lbuf, reinterpret_cast<int*>(s.arena + l.lip), n, h, w, st));
    float* const user_out = out;
    if (staged) {
        float* m = s.arena + l.stage;
        float* v = m + 2 * (5 + ch) * l.map;
        CNL_TRY(pad_rows(m + 0 * l.map, dx, (size_t)n * 2 * h, w, P, st));
        CNL_TRY(pad_rows(m + 2 * l.map, dy, (size_t)n * 2 * h, w, P, st));
        CNL_TRY(pad_rows(m + 4 * l.map, c, (size_t)n * h, w, P, st));
        CNL_TRY(pad_rows(m + 5 * l.map, b, (size_t)n * ch * h, w, P, st));
        CNL_TRY(pad_rows(v, init, (size_t)n * 3 * ch * h, w, P, st));
        dx = m; dy = m + 2 * l.map; c = m + 4 * l.map; b = m + 5 * l.map; init = v;
        out = v + l.vol;
    }
    CNL_TRY(check_cuda(cudaMemcpyAsync(out, init, vol_bytes, cudaMemcpyDeviceToDevice, st), "copy init->x"));
    CNL_TRY(check_cuda(cudaMemcpyAsync(y0, init, vol_bytes, cudaMemcpyDeviceToDevice, st), "copy init->y"));
    const dim3 grid((w + TW - 1) / TW, (h + TH - 1) / TH, n);
    size_t next = 0;
    for (int g = 0; g < its_eff; ++g) {
        float* yin = (g & 1) ? y1 : y0;
        float* yout = (g & 1) ? y0 : y1;
        float* ck = nullptr;
        if (next < s.sched.size() && s.sched[next] == g) {
            ck = s.arena + l.ckpt + next * l.vol;
            ++next;
        }
        if (vec) {
            FwdVecParams q{};
            q.y_in = yin; q.y_out = yout; q.x = out; q.hist = s.arena + l.hist + (size_t)g * l.vol; q.ckpt = ck;
            q.b = b; q.c = c; q.dx = dx; q.dy = dy; q.L = Lbuf; q.N = n; q.C = ch; q.H = h; q.W = w; q.P = P; q.t = s.steps[g];
            CNL_TRY(launch_tgv_fwd_vec(q, st));
            continue;
        }
        if (ck) CNL_TRY(check_cuda(cudaMemcpyAsync(ck, yin, vol_bytes, cudaMemcpyDeviceToDevice, st), "checkpoint y"));
        tgv_fwd_kernel<<<grid, NT, 0, st>>>(yin, yout, out, b, c, dx, dy, Lbuf, s.arena + l.hist + (size_t)g * l.vol, ch, h, w, s.steps[g]);
        CNL_TRY(after_launch("tgv_fwd_kernel"));
    }
    if (staged) CNL_TRY(unpad_rows(user_out, out, (size_t)n * 3 * ch * h, w, P, st));
    s.n = n; s.ch = ch; s.h = h; s.w = w; s.its = its;
    s.have_forward = true;
    return CNL_OK;
}

static int backward_impl(const float* dx, const float* dy, const float* c, const float* b, const float* grad,
                         float* g_dx, float* g_dy, float* g_c, float* g_b, float* g_init,
                         int n, int ch, int h, int w, int its, int id, cudaStream_t st) {
    const void* ptrs[] = {dx, dy, c, b, grad, g_dx, g_dy, g_c, g_b, g_init};
    CNL_TRY(check_args(ptrs, 10, n, ch, h, w, its, id));
    std::lock_guard<std::mutex> lock(g_mutex);
    int rc;
    Slot* sp = get_slot(id, &rc);
    if (!sp) return rc;
    Slot& s = *sp;
    if (!s.have_forward || s.n != n || s.ch != ch || s.h != h || s.w != w || s.its != its)
        return fail(CNL_ERR_NO_FORWARD, "backward(id=%d) needs a preceding forward(id=%d) with the same shape and its", id, id);
    if (!s.cond) {
        void* p = nullptr;
        const size_t bytes = (kOut + (size_t)kOut * kStatBlocks * 2 + 4) * sizeof(double);
        if (cudaMalloc(&p, bytes) != cudaSuccess) { cudaGetLastError(); return fail(CNL_ERR_ALLOC, "cudaMalloc (conditioner state) failed"); }
        s.cond = static_cast<double*>(p);
        CNL_TRY(check_cuda(cudaMemset(s.cond, 0, bytes), "cudaMemset"));
    }
    const int its_eff = 2 * (its / 2);
    const bool staged = s.staged;
    const int P = s.pitch;                        // row pitch of the arena planes (w unless staged)
    const Layout l = make_layout(n, ch, h, P, its_eff, s.sched.size(), staged);
    const size_t plane = (size_t)h * w;           // plane of the caller's tensors
    const size_t vol = (size_t)n * 3 * ch * plane;
    float* Lbuf = s.arena + l.L;
    unsigned int* flags = reinterpret_cast<unsigned int*>(s.arena + l.flags);
    // the reference skips the whole pass (all-zero gradients) when the upstream gradient holds a non-finite value or is
    // identically zero (:2698-2703); the decision needs the host, as in the reference
    CNL_TRY(check_cuda(cudaMemsetAsync(flags, 0, 2 * sizeof(unsigned int), st), "zero flags"));
    tgv_upstream_check_kernel<<<296, 256, 0, st>>>(grad, vol, flags);
    CNL_TRY(after_launch("tgv_upstream_check_kernel"));
    unsigned int hflags[2] = {0, 0};
    CNL_TRY(check_cuda(cudaMemcpyAsync(hflags, flags, sizeof(hflags), cudaMemcpyDeviceToHost, st), "read flags"));
    CNL_TRY(check_cuda(cudaStreamSynchronize(st), "cudaStreamSynchronize"));
    CNL_TRY(check_cuda(cudaMemsetAsync(g_dx, 0, (size_t)n * 2 * plane * sizeof(float), st), "zero g_dx"));
    CNL_TRY(check_cuda(cudaMemsetAsync(g_dy, 0, (size_t)n * 2 * plane * sizeof(float), st), "zero g_dy"));
    if (hflags[0] != 0 || hflags[1] == 0) {
        CNL_TRY(check_cuda(cudaMemsetAsync(g_c, 0, (size_t)n * plane * sizeof(float), st), "zero g_c"));
        CNL_TRY(check_cuda(cudaMemsetAsync(g_b, 0, (size_t)n * ch * plane * sizeof(float), st), "zero g_b"));
        CNL_TRY(check_cuda(cudaMemsetAsync(g_init, 0, vol * sizeof(float), st), "zero g_init"));
        return CNL_OK;
    }
    CNL_TRY(lipschitz(dx, dy, Lbuf, reinterpret_cast<int*>(s.arena + l.lip), n, h, w, st));
    float* ga = s.arena + l.ga;
    float* gb = s.arena + l.gb;
    float* acc = s.arena + l.acc;
    const float* hist = s.arena + l.hist;
    const size_t aplane = (size_t)h * P;          // plane of the arena buffers
    CNL_TRY(check_cuda(cudaMemsetAsync(acc, 0, (size_t)n * 3 * ch * aplane * sizeof(float), st), "zero acc"));
    const dim3 grid((w + TW - 1) / TW, (h + TH - 1) / TH, n);
    const void* planes[] = {dx, dy, c, b, grad, g_dx, g_dy, g_c, g_b, g_init};
    const bool vec = vec_enabled() && (staged || tgv_vec_supported(w, planes, 10));
    if (staged && !vec) return fail(CNL_ERR_BAD_OPTION, "the forward pass of id %d ran on zero-padded staging copies; the backward pass needs the same kernels", id);
    float* const u_gdx = g_dx; float* const u_gdy = g_dy; float* const u_gc = g_c; float* const u_gb = g_b; float* const u_ginit = g_init;
    if (staged) {          // same staging as in the forward pass, plus the upstream gradient and the five outputs
        float* m = s.arena + l.stage;
        float* v = m + 2 * (5 + ch) * l.map;
        CNL_TRY(pad_rows(m + 0 * l.map, dx, (size_t)n * 2 * h, w, P, st));
        CNL_TRY(pad_rows(m + 2 * l.map, dy, (size_t)n * 2 * h, w, P, st));
        CNL_TRY(pad_rows(m + 4 * l.map, c, (size_t)n * h, w, P, st));
        CNL_TRY(pad_rows(m + 5 * l.map, b, (size_t)n * ch * h, w, P, st));
        CNL_TRY(pad_rows(v, grad, (size_t)n * 3 * ch * h, w, P, st));
        dx = m; dy = m + 2 * l.map; c = m + 4 * l.map; b = m + 5 * l.map; grad = v;
        float* o = m + (5 + ch) * l.map;
        g_dx = o; g_dy = o + 2 * l.map; g_c = o + 4 * l.map; g_b = o + 5 * l.map; g_init = v + l.vol;
        CNL_TRY(check_cuda(cudaMemsetAsync(g_dx, 0, (size_t)n * 2 * aplane * sizeof(float), st), "zero g_dx"));
        CNL_TRY(check_cuda(cudaMemsetAsync(g_dy, 0, (size_t)n * 2 * aplane * sizeof(float), st), "zero g_dy"));
    }
    CNL_TRY(ensure_dynamic_smem(tgv_rev_kernel, kRevSmemFloats * (int)sizeof(float)));
    {
        const int g = its_eff - 1;
        tgv_seed_kernel<<<dim3((unsigned)((aplane + NT - 1) / NT), n), NT, 0, st>>>(grad, hist + (size_t)g * l.vol, b, c, gb, g_c, g_b, ch, aplane);
        CNL_TRY(after_launch("tgv_seed_kernel"));
    }
    for (int g = its_eff - 2; g >= 0; --g) {
        const float* ck = nullptr;
        for (size_t i = 0; i < s.sched.size(); ++i) if (s.sched[i] == g) ck = s.arena + l.ckpt + i * l.vol;
        float* gout = (g & 1) ? gb : ga;
        const float* gin = (g & 1) ? ga : gb;
        if (vec) {
            RevVecParams q{};
            q.hist_g = hist + (size_t)g * l.vol; q.hist_gm1 = g > 0 ? hist + (size_t)(g - 1) * l.vol : nullptr; q.ckpt = ck;
            q.g_in = gin; q.g_out = gout; q.acc = acc; q.b = b; q.c = c; q.dx = dx; q.dy = dy; q.L = Lbuf;
            q.g_c = g_c; q.g_b = g_b; q.g_dx = g_dx; q.g_dy = g_dy; q.x1bar = g == 0 ? g_init : nullptr;
            q.N = n; q.C = ch; q.H = h; q.W = w; q.P = P; q.t = s.steps[g]; q.typo = ck ? 0 : 1;
            CNL_TRY(launch_tgv_rev_vec(q, st));
            continue;
        }
        tgv_rev_kernel<<<grid, NT, kRevSmemFloats * sizeof(float), st>>>(
            hist + (size_t)g * l.vol, g > 0 ? hist + (size_t)(g - 1) * l.vol : nullptr, ck, gin, gout, acc, b, c, dx, dy, Lbuf,
            g_c, g_b, g_dx, g_dy, g == 0 ? g_init : nullptr, ch, h, w, s.steps[g], ck ? 0 : 1);
        CNL_TRY(after_launch("tgv_rev_kernel"));
    }
    if (staged) {
        CNL_TRY(unpad_rows(u_gdx, g_dx, (size_t)n * 2 * h, w, P, st));
        CNL_TRY(unpad_rows(u_gdy, g_dy, (size_t)n * 2 * h, w, P, st));
        CNL_TRY(unpad_rows(u_gc, g_c, (size_t)n * h, w, P, st));
        CNL_TRY(unpad_rows(u_gb, g_b, (size_t)n * ch * h, w, P, st));
        CNL_TRY(unpad_rows(u_ginit, g_init, (size_t)n * 3 * ch * h, w, P, st));
    }
    FinArgs fa{};
    float* outs[kOut] = {u_gc, u_gdx, u_gdy, u_gb, u_ginit};
    const unsigned long long counts[kOut] = {(unsigned long long)n * plane, (unsigned long long)n * 2 * plane, (unsigned long long)n * 2 * plane,
                                             (unsigned long long)n * ch * plane, (unsigned long long)n * 3 * ch * plane};
    for (int o = 0; o < kOut; ++o) { fa.ptr[o] = outs[o]; fa.count[o] = counts[o]; fa.scale[o] = kGlobalG; fa.per_image_L[o] = 0; fa.per_image[o] = 1; }
    fa.per_image_L[1] = fa.per_image_L[2] = 1;
    fa.per_image[1] = fa.per_image[2] = 2 * plane;
    fa.scale[4] = 1.0f;
    double* state = s.cond;
    double* partial = s.cond + kOut;
    float* factor = reinterpret_cast<float*>(s.cond + kOut + (size_t)kOut * kStatBlocks * 2);
    if (n == 1) {
        // only the primary planes of the init gradient pass the sanitiser and the conditioner (:3014-3021); they are
        // the first ch planes when n == 1.  For a batch the whole tensor is treated alike.
        fa.count[4] = (unsigned long long)ch * plane;
    }
    if (s.opt_conditioner) {
        tgv_stats_kernel<<<dim3(kStatBlocks, kOut), 256, 0, st>>>(fa, partial);
        CNL_TRY(after_launch("tgv_stats_kernel"));
        tgv_conditioner_kernel<<<1, 32, 0, st>>>(partial, fa, state, factor, s.run);
        CNL_TRY(after_launch("tgv_conditioner_kernel"));
    }
    tgv_apply_kernel<<<dim3(296, kOut), 256, 0, st>>>(fa, s.opt_conditioner ? factor : nullptr, Lbuf);
    CNL_TRY(after_launch("tgv_apply_kernel"));
    s.run += 1;
    return CNL_OK;
}

}  // namespace tgv
}  // namespace cnl

using namespace cnl;

extern "C" int cnl_tgv_forward(const float* dx, const float* dy, const float* c, const float* b, const float* init,
                               float* out, int n, int ch, int h, int w, int its, int id, void* stream) {
    return tgv::forward_impl(dx, dy, c, b, init, out, n, ch, h, w, its, id, static_cast<cudaStream_t>(stream));
}

extern "C" int cnl_tgv_backward(const float* dx, const float* dy, const float* c, const float* b, const float* grad_out,
                                float* g_dx, float* g_dy, float* g_c, float* g_b, float* g_init, int n, int ch, int h,
                                int w, int its, int id, void* stream) {
    return tgv::backward_impl(dx, dy, c, b, grad_out, g_dx, g_dy, g_c, g_b, g_init, n, ch, h, w, its, id,
                              static_cast<cudaStream_t>(stream));
}

extern "C" int cnl_tgv_release(int id) {
    if (id < 0 || id >= CNL_NUM_IDS) return fail(CNL_ERR_BAD_ID, "id %d is outside 0..%d", id, CNL_NUM_IDS - 1);
    std::lock_guard<std::mutex> lock(tgv::g_mutex);
    int rc;
    tgv::Slot* sp = tgv::get_slot(id, &rc);
    if (!sp) return rc;
    CNL_TRY(check_cuda(cudaDeviceSynchronize(), "cudaDeviceSynchronize"));
    if (sp->arena) cudaFree(sp->arena);
    if (sp->cond) cudaFree(sp->cond);
    const int keep = sp->opt_conditioner;
    *sp = tgv::Slot();
    sp->opt_conditioner = keep;
    return CNL_OK;
}

extern "C" int cnl_tgv_set_option(int id, int option, int value) {
    if (id < 0 || id >= CNL_NUM_IDS) return fail(CNL_ERR_BAD_ID, "id %d is outside 0..%d", id, CNL_NUM_IDS - 1);
    std::lock_guard<std::mutex> lock(tgv::g_mutex);
    int rc;
    tgv::Slot* sp = tgv::get_slot(id, &rc);
    if (!sp) return rc;
    if (option != CNL_OPT_CONDITIONER) return fail(CNL_ERR_BAD_OPTION, "unknown option %d", option);
    sp->opt_conditioner = value ? 1 : 0;
    return CNL_OK;
}

// Copies a stored iterate of the last forward(id): kind 0 = x^{g+1/2} of iteration idx, 1 = checkpointed y number idx,
// 2 = the per-image 1/Lipschitz factors (n floats).
extern "C" int cnl_tgv_read_state(int id, int kind, int idx, float* dst, void* stream) {
    if (id < 0 || id >= CNL_NUM_IDS) return fail(CNL_ERR_BAD_ID, "id %d is outside 0..%d", id, CNL_NUM_IDS - 1);
    if (!dst) return fail(CNL_ERR_NULL, "null destination");
    std::lock_guard<std::mutex> lock(tgv::g_mutex);
    int rc;
    tgv::Slot* sp = tgv::get_slot(id, &rc);
    if (!sp) return rc;
    if (!sp->have_forward) return fail(CNL_ERR_NO_FORWARD, "slot %d holds no forward pass", id);
    const int its_eff = 2 * (sp->its / 2);
    const tgv::Layout l = tgv::make_layout(sp->n, sp->ch, sp->h, sp->pitch, its_eff, sp->sched.size(), sp->staged);
    const float* src;
    size_t bytes = (size_t)sp->n * 3 * sp->ch * sp->h * sp->w * sizeof(float);
    if (kind == 0) { if (idx < 0 || idx >= its_eff) return fail(CNL_ERR_BAD_SHAPE, "iteration %d out of range", idx); src = sp->arena + l.hist + (size_t)idx * l.vol; }
    else if (kind == 1) { if (idx < 0 || idx >= (int)sp->sched.size()) return fail(CNL_ERR_BAD_SHAPE, "checkpoint %d out of range", idx); src = sp->arena + l.ckpt + (size_t)idx * l.vol; }
    else if (kind == 2) { src = sp->arena + l.L; bytes = (size_t)sp->n * sizeof(float); }
    else return fail(CNL_ERR_BAD_OPTION, "unknown kind %d", kind);
    if (kind != 2)
        return tgv::unpad_rows(dst, src, (size_t)sp->n * 3 * sp->ch * sp->h, sp->w, sp->pitch, static_cast<cudaStream_t>(stream));
    return check_cuda(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, static_cast<cudaStream_t>(stream)), "copy stored iterate");
}

extern "C" int cnl_tgv_num_checkpoints(int id) {
    if (id < 0 || id >= CNL_NUM_IDS) return -1;
    std::lock_guard<std::mutex> lock(tgv::g_mutex);
    int rc;
    tgv::Slot* sp = tgv::get_slot(id, &rc);
    if (!sp || !sp->have_forward) return -1;
    return (int)sp->sched.size();
}
