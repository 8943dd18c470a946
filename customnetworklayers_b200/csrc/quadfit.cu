// Differentiable per-axis quadratic fit of a 5-point correlation stencil for sm_100a
// (reference: cudaQuadFit/cudaCode/quadFit.cu, kQuadFitFlow :14-136, kQuadFitFlowGrad :142-297).
//
// One thread per pixel; the feature loops are batched by eight channels so that 48 independent loads are in flight
// per thread.  The kernels are HBM/L2 bound: C reads of the first feature map (coalesced) and 5 C gathered reads of the
// second one per pixel.  The float/double promotions of the reference's expressions are kept where they decide the
// rounded integer location and the validity tests, so those are bit-identical.
#include "common.h"

namespace cnl {

struct QuadFit {
    float ax, ay, bx, by, fx, fy, score;
    bool vx, vy;
};

// quadFit.cu:74-134.  interior_* : the rounded location has both neighbours along that axis.
__device__ __forceinline__ QuadFit quad_fit(float c00, float c0p, float cp0, float c0m, float cm0, bool interior_x,
                                            bool interior_y) {
    QuadFit q;
    q.ax = (float)(0.5 * ((double)(c0p + c0m) - 2.0 * (double)c00));
    q.ay = (float)(0.5 * ((double)(cp0 + cm0) - 2.0 * (double)c00));
    q.bx = (float)(0.5 * (double)(c0p - c0m));
    q.by = (float)(0.5 * (double)(cp0 - cm0));
    q.vx = q.ax < 0.0f && (double)__fmul_rn(q.ax, q.ax) >= 0.25 * (double)q.bx * (double)q.bx && interior_x;
    q.vy = q.ay < 0.0f && (double)__fmul_rn(q.ay, q.ay) >= 0.25 * (double)q.by * (double)q.by && interior_y;
    q.fx = q.vx ? (float)(-0.5 * (double)q.bx / (double)q.ax) : 0.0f;
    q.fy = q.vy ? (float)(-0.5 * (double)q.by / (double)q.ay) : 0.0f;
    q.score = q.ax * q.fx * q.fx + q.bx * q.fx + c00 + q.ay * q.fy * q.fy + q.by * q.fy;
    return q;
}

// d loss / d (c00, c0p, c0m, cp0, cm0) given the upstream gradient of (fx, fy, score)   (quadFit.cu:245-281)
__device__ __forceinline__ void quad_fit_grad(const QuadFit& q, float gfx, float gfy, float gs, float& k00, float& k0p,
                                              float& k0m, float& kp0, float& km0) {
    if (!(q.vx || q.vy)) {          // only the score at the centre has a gradient (:290-294)
        k00 = gs; k0p = k0m = kp0 = km0 = 0.0f;
        return;
    }
    const float dfx_dbx = q.vx ? (float)(-1.0 / (2.0 * (double)q.ax)) : 0.0f;
    const float dfx_dax = q.vx ? -q.fx / q.ax : 0.0f;
    const float dfy_dby = q.vy ? (float)(-1.0 / (2.0 * (double)q.ay)) : 0.0f;
    const float dfy_day = q.vy ? -q.fy / q.ay : 0.0f;
    const double Ax = (double)gfx * dfx_dax + (double)gs * (q.vx ? q.fx * q.fx : 0.0f);
    const double Bx = (double)gfx * dfx_dbx + (double)gs * (q.vx ? q.fx : 0.0f);
    const double Ay = (double)gfy * dfy_day + (double)gs * (q.vy ? q.fy * q.fy : 0.0f);
    const double By = (double)gfy * dfy_dby + (double)gs * (q.vy ? q.fy : 0.0f);
    k00 = (float)(0.5 * (-2.0 * Ax - 2.0 * Ay + 2.0 * (double)gs));
    k0p = (float)(0.5 * (Ax + Bx));
    k0m = (float)(0.5 * (Ax - Bx));
    kp0 = (float)(0.5 * (Ay + By));
    km0 = (float)(0.5 * (Ay - By));
}

struct QfLoc {
    bool inside;
    int x, y, xm, xp, ym, yp;
};

__device__ __forceinline__ QfLoc qf_locate(const float* __restrict__ flow, size_t n, size_t plane, int pix, int h, int w,
                                           int H, int W) {
    QfLoc L;
    const float idx = (float)w + flow[(n * 2 + 0) * plane + pix];          // :31
    const float idy = (float)h + flow[(n * 2 + 1) * plane + pix];
    L.inside = !(idx > (float)(W - 1) || idx < 0.0f || idy > (float)(H - 1) || idy < 0.0f);      // :35
    L.x = L.inside ? (int)floor((double)idx + 0.5) : 0;                     // :46, rounded in double
    L.y = L.inside ? (int)floor((double)idy + 0.5) : 0;
    L.xm = max(L.x - 1, 0); L.xp = min(L.x + 1, W - 1);
    L.ym = max(L.y - 1, 0); L.yp = min(L.y + 1, H - 1);
    return L;
}

// Correlation of the pixel's feature vector with the five stencil positions in the second feature map.  The loads of
// kQfBatch channels (6 each) are all issued before the first multiply-add, so that a thread has 48 independent
// loads in flight instead of one round trip per channel.
constexpr int kQfBatch = 8;

__device__ __forceinline__ void qf_costs(const float* __restrict__ f0, const float* __restrict__ f1, size_t n, int C,
                                         size_t plane, int pix, const QfLoc& L, int W, float (&cost)[5]) {
    const int o00 = L.y * W + L.x, o0p = L.y * W + L.xp, op0 = L.yp * W + L.x, o0m = L.y * W + L.xm, om0 = L.ym * W + L.x;
    cost[0] = cost[1] = cost[2] = cost[3] = cost[4] = 0.0f;
    const float* a = f0 + n * C * plane + pix;
    const float* b = f1 + n * C * plane;
    int cc = 0;
    for (; cc + kQfBatch <= C; cc += kQfBatch) {
        float I1[kQfBatch], v[5][kQfBatch];
#pragma unroll
        for (int j = 0; j < kQfBatch; ++j) {
            const float* bc = b + (size_t)j * plane;
            I1[j] = __ldg(a + (size_t)j * plane);
            v[0][j] = __ldg(bc + o00);
            v[1][j] = __ldg(bc + o0p);
            v[2][j] = __ldg(bc + op0);
            v[3][j] = __ldg(bc + o0m);
            v[4][j] = __ldg(bc + om0);
        }
#pragma unroll
        for (int j = 0; j < kQfBatch; ++j) {            // channel order as in a plain loop: same rounding
#pragma unroll
            for (int q = 0; q < 5; ++q) cost[q] = fmaf(I1[j], v[q][j], cost[q]);
        }
        a += (size_t)kQfBatch * plane;
        b += (size_t)kQfBatch * plane;
    }
    for (; cc < C; ++cc) {
        const float I1 = __ldg(a);
        cost[0] = fmaf(I1, __ldg(b + o00), cost[0]);
        cost[1] = fmaf(I1, __ldg(b + o0p), cost[1]);
        cost[2] = fmaf(I1, __ldg(b + op0), cost[2]);
        cost[3] = fmaf(I1, __ldg(b + o0m), cost[3]);
        cost[4] = fmaf(I1, __ldg(b + om0), cost[4]);
        a += plane;
        b += plane;
    }
}

__global__ void __launch_bounds__(256, 4)
quadfit_forward_kernel(const float* __restrict__ f0, const float* __restrict__ f1, const float* __restrict__ flow,
                       int flow_ch, float* __restrict__ out, int* __restrict__ loc, int C, int H, int W) {
    const size_t plane = (size_t)H * W;
    const size_t pix_l = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (pix_l >= plane) return;
    const size_t n = blockIdx.y;
    const int pix = (int)pix_l, h = pix / W, w = pix - h * W;
    // flow may carry extra channels (the reference's layer passes three); only the first two are read
    const float* fl = flow + n * (size_t)(flow_ch - 2) * plane;
    const QfLoc L = qf_locate(fl, n, plane, pix, h, w, H, W);
    float o0 = 0.f, o1 = 0.f, o2 = 0.f;
    if (L.inside) {
        float cost[5];
        qf_costs(f0, f1, n, C, plane, pix, L, W, cost);
        const QuadFit q = quad_fit(cost[0], cost[1], cost[2], cost[3], cost[4], L.x < W - 1 && L.x > 0, L.y < H - 1 && L.y > 0);
        o0 = q.fx; o1 = q.fy; o2 = q.score;
    }
    out[(n * 3 + 0) * plane + pix] = o0;
    out[(n * 3 + 1) * plane + pix] = o1;
    out[(n * 3 + 2) * plane + pix] = o2;
    if (loc) {
        loc[(n * 2 + 0) * plane + pix] = L.inside ? L.x : -1;
        loc[(n * 2 + 1) * plane + pix] = L.inside ? L.y : -1;
    }
}

// g0 is written directly (one owner per element); g1 is a scatter with fp32 atomics like the reference's, so its
// summation order is not deterministic.
__global__ void __launch_bounds__(256, 3)
quadfit_backward_kernel(const float* __restrict__ f0, const float* __restrict__ f1, const float* __restrict__ flow,
                        int flow_ch, const float* __restrict__ grad, float* __restrict__ g0, float* __restrict__ g1,
                        int C, int H, int W) {
    const size_t plane = (size_t)H * W;
    const size_t pix_l = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (pix_l >= plane) return;
    const size_t n = blockIdx.y;
    const int pix = (int)pix_l, h = pix / W, w = pix - h * W;
    const float* fl = flow + n * (size_t)(flow_ch - 2) * plane;
    const QfLoc L = qf_locate(fl, n, plane, pix, h, w, H, W);
    if (!L.inside) {
        for (int cc = 0; cc < C; ++cc) g0[(n * C + cc) * plane + pix] = 0.0f;
        return;
    }
    float cost[5];
    qf_costs(f0, f1, n, C, plane, pix, L, W, cost);
    const QuadFit q = quad_fit(cost[0], cost[1], cost[2], cost[3], cost[4], L.x < W - 1 && L.x > 0, L.y < H - 1 && L.y > 0);
    float k00, k0p, k0m, kp0, km0;
    quad_fit_grad(q, grad[(n * 3 + 0) * plane + pix], grad[(n * 3 + 1) * plane + pix], grad[(n * 3 + 2) * plane + pix],
                  k00, k0p, k0m, kp0, km0);
    const int o00 = L.y * W + L.x, o0p = L.y * W + L.xp, op0 = L.yp * W + L.x, o0m = L.y * W + L.xm, om0 = L.ym * W + L.x;
    const bool stencil = q.vx || q.vy;
    constexpr int kB = 4;                      // channels whose loads are issued together
    int cc = 0;
    for (; cc + kB <= C; cc += kB) {
        float I1[kB], v[5][kB];
#pragma unroll
        for (int j = 0; j < kB; ++j) {
            const size_t base = (n * C + cc + j) * plane;
            I1[j] = __ldg(f0 + base + pix);
            v[0][j] = __ldg(f1 + base + o00);
            if (stencil) {
                v[1][j] = __ldg(f1 + base + o0p); v[2][j] = __ldg(f1 + base + o0m);
                v[3][j] = __ldg(f1 + base + op0); v[4][j] = __ldg(f1 + base + om0);
            }
        }
#pragma unroll
        for (int j = 0; j < kB; ++j) {
            const size_t base = (n * C + cc + j) * plane;
            float acc = k00 * v[0][j];
            atomicAdd(g1 + base + o00, I1[j] * k00);
            if (stencil) {
                acc += k0p * v[1][j] + k0m * v[2][j] + kp0 * v[3][j] + km0 * v[4][j];
                atomicAdd(g1 + base + o0p, I1[j] * k0p);
                atomicAdd(g1 + base + o0m, I1[j] * k0m);
                atomicAdd(g1 + base + op0, I1[j] * kp0);
                atomicAdd(g1 + base + om0, I1[j] * km0);
            }
            g0[base + pix] = acc;
        }
    }
    for (; cc < C; ++cc) {
        const size_t base = (n * C + cc) * plane;
        const float I1 = __ldg(f0 + base + pix);
        float acc = k00 * __ldg(f1 + base + o00);
        atomicAdd(g1 + base + o00, I1 * k00);
        if (stencil) {
            acc += k0p * __ldg(f1 + base + o0p) + k0m * __ldg(f1 + base + o0m) + kp0 * __ldg(f1 + base + op0) +
                   km0 * __ldg(f1 + base + om0);
            atomicAdd(g1 + base + o0p, I1 * k0p);
            atomicAdd(g1 + base + o0m, I1 * k0m);
            atomicAdd(g1 + base + op0, I1 * kp0);
            atomicAdd(g1 + base + om0, I1 * km0);
        }
        g0[base + pix] = acc;
    }
}

// Variant that takes the 5-point stencil directly: cost5 [N,5,H,W] = (c00, c0p, cp0, c0m, cm0).
__global__ void __launch_bounds__(256)
quadfit_cost_forward_kernel(const float* __restrict__ cost5, float* __restrict__ out, size_t plane) {
    const size_t pix = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (pix >= plane) return;
    const size_t n = blockIdx.y;
    const float* c = cost5 + n * 5 * plane + pix;
    const QuadFit q = quad_fit(c[0], c[plane], c[2 * plane], c[3 * plane], c[4 * plane], true, true);
    out[(n * 3 + 0) * plane + pix] = q.fx;
    out[(n * 3 + 1) * plane + pix] = q.fy;
    out[(n * 3 + 2) * plane + pix] = q.score;
}

__global__ void __launch_bounds__(256)
quadfit_cost_backward_kernel(const float* __restrict__ cost5, const float* __restrict__ grad, float* __restrict__ gcost,
                             size_t plane) {
    const size_t pix = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (pix >= plane) return;
    const size_t n = blockIdx.y;
    const float* c = cost5 + n * 5 * plane + pix;
    const QuadFit q = quad_fit(c[0], c[plane], c[2 * plane], c[3 * plane], c[4 * plane], true, true);
    float k00, k0p, k0m, kp0, km0;
    quad_fit_grad(q, grad[(n * 3 + 0) * plane + pix], grad[(n * 3 + 1) * plane + pix], grad[(n * 3 + 2) * plane + pix],
                  k00, k0p, k0m, kp0, km0);
    float* g = gcost + n * 5 * plane + pix;
    g[0] = k00; g[plane] = k0p; g[2 * plane] = kp0; g[3 * plane] = k0m; g[4 * plane] = km0;
}

static int qf_check(int n, int c, int h, int w) {
    if (n < 1 || c < 1 || h < 1 || w < 1) return fail(CNL_ERR_BAD_SHAPE, "n, c, h, w must be >= 1 (got %d, %d, %d, %d)", n, c, h, w);
    if ((long long)h * w > 0x3fffffffLL || n > 65535) return fail(CNL_ERR_BAD_SHAPE, "image or batch beyond the supported range");
    return CNL_OK;
}

}  // namespace cnl

using namespace cnl;

extern "C" int cnl_quadfit_forward(const float* feat0, const float* feat1, const float* flow, int flow_channels,
                                   float* out, int* loc, int n, int c, int h, int w, void* stream) {
    if (!feat0 || !feat1 || !flow || !out) return fail(CNL_ERR_NULL, "null pointer argument");
    CNL_TRY(qf_check(n, c, h, w));
    if (flow_channels < 2) return fail(CNL_ERR_BAD_SHAPE, "flow needs at least 2 channels (got %d)", flow_channels);
    const size_t plane = (size_t)h * w;
    const dim3 grid((unsigned)((plane + 255) / 256), n);
    quadfit_forward_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(feat0, feat1, flow, flow_channels, out, loc, c, h, w);
    return after_launch("quadfit_forward_kernel");
}

extern "C" int cnl_quadfit_backward(const float* feat0, const float* feat1, const float* flow, int flow_channels,
                                    const float* grad, float* g_feat0, float* g_feat1, int n, int c, int h, int w,
                                    void* stream) {
    if (!feat0 || !feat1 || !flow || !grad || !g_feat0 || !g_feat1) return fail(CNL_ERR_NULL, "null pointer argument");
    CNL_TRY(qf_check(n, c, h, w));
    if (flow_channels < 2) return fail(CNL_ERR_BAD_SHAPE, "flow needs at least 2 channels (got %d)", flow_channels);
    const size_t plane = (size_t)h * w;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    CNL_TRY(check_cuda(cudaMemsetAsync(g_feat1, 0, (size_t)n * c * plane * sizeof(float), st), "zero g_feat1"));
    const unsigned gx = (unsigned)((plane + 255) / 256);
    quadfit_backward_kernel<<<dim3(gx, n), 256, 0, st>>>(feat0, feat1, flow, flow_channels, grad, g_feat0, g_feat1, c, h, w);
    return after_launch("quadfit_backward_kernel");
}

extern "C" int cnl_quadfit_cost_forward(const float* cost5, float* out, int n, int h, int w, void* stream) {
    if (!cost5 || !out) return fail(CNL_ERR_NULL, "null pointer argument");
    CNL_TRY(qf_check(n, 1, h, w));
    const size_t plane = (size_t)h * w;
    quadfit_cost_forward_kernel<<<dim3((unsigned)((plane + 255) / 256), n), 256, 0, static_cast<cudaStream_t>(stream)>>>(cost5, out, plane);
    return after_launch("quadfit_cost_forward_kernel");
}

extern "C" int cnl_quadfit_cost_backward(const float* cost5, const float* grad, float* g_cost5, int n, int h, int w,
                                         void* stream) {
    if (!cost5 || !grad || !g_cost5) return fail(CNL_ERR_NULL, "null pointer argument");
    CNL_TRY(qf_check(n, 1, h, w));
    const size_t plane = (size_t)h * w;
    quadfit_cost_backward_kernel<<<dim3((unsigned)((plane + 255) / 256), n), 256, 0, static_cast<cudaStream_t>(stream)>>>(cost5, grad, g_cost5, plane);
    return after_launch("quadfit_cost_backward_kernel");
}
