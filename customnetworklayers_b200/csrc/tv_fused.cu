// Register-tiled, temporally blocked TV-FISTA kernels for sm_100a (geometry: see tv_fused.cuh).
#include "tv_fused.cuh"

#include "common.h"
#include "tv_math.cuh"

namespace cnl {

namespace {

constexpr int kWarps = 16;
constexpr int kRows = 2;                         // rows per warp
constexpr int kThreads = kWarps * 32;
static_assert(kWarps * kRows == kRegionH, "region height");
constexpr unsigned kFull = 0xffffffffu;

__device__ __forceinline__ float4 ld4(const float* p, bool ok) {
    return ok ? __ldg(reinterpret_cast<const float4*>(p)) : make_float4(0.f, 0.f, 0.f, 0.f);
}
__device__ __forceinline__ void st4(float* p, const float4& v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ float4 zero4() { return make_float4(0.f, 0.f, 0.f, 0.f); }
__device__ __forceinline__ void add4(float4& a, const float4& b) { a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w; }

// Fluxes of the four triangles anchored at one lane's pixels of a row.  `yd` is the row below.
__device__ __forceinline__ void flux_row(const float4& y, const float4& yd, const float4& wx, const float4& wy,
                                         float4& fx, float4& fy) {
    const float yr3 = __shfl_down_sync(kFull, y.x, 1);      // first pixel of the lane to the right
    tri_flux_fast(y.x, y.y, yd.x, wx.x, wy.x, fx.x, fy.x);
    tri_flux_fast(y.y, y.z, yd.y, wx.y, wy.y, fx.y, fy.y);
    tri_flux_fast(y.z, y.w, yd.z, wx.z, wy.z, fx.z, fy.z);
    tri_flux_fast(y.w, yr3, yd.w, wx.w, wy.w, fx.w, fy.w);
}

struct TileGeom {
    int lane, warp;
    int gx;                 // image column of the lane's first pixel (multiple of 4, may be outside the image)
    int gy[kRows];          // image rows of the warp
    bool ok[kRows];         // the lane's vector lies inside the image
    bool store[kRows];      // ... and inside the interior this CTA writes back
};

template <int K>
__device__ __forceinline__ TileGeom make_geom(int H, int W) {
    TileGeom g;
    g.lane = threadIdx.x & 31;
    g.warp = threadIdx.x >> 5;
    constexpr int TH = kRegionH - 2 * K;
    g.gx = blockIdx.x * kTileW - kHaloX + 4 * g.lane;
    const bool col_ok = g.gx >= 0 && g.gx < W;
    const bool col_int = g.lane >= 1 && g.lane <= 30;
#pragma unroll
    for (int r = 0; r < kRows; ++r) {
        const int lr = g.warp * kRows + r;
        g.gy[r] = blockIdx.y * TH - K + lr;
        g.ok[r] = col_ok && g.gy[r] >= 0 && g.gy[r] < H;
        g.store[r] = g.ok[r] && col_int && lr >= K && lr < kRegionH - K;
    }
    return g;
}

// Confidence and edge weights of a lane's pixels; the weights are scaled by 1/8 and zero on the last column (wx) /
// last row (wy) of the image.
template <typename P>
__device__ __forceinline__ void load_maps(const P& p, const TileGeom& g, size_t n, float4 (&c)[kRows],
                                          float4 (&wx)[kRows], float4 (&wy)[kRows]) {
    const size_t plane = (size_t)p.H * p.W;
#pragma unroll
    for (int r = 0; r < kRows; ++r) {
        const size_t o = n * plane + (size_t)g.gy[r] * p.W + g.gx;
        c[r] = ld4(p.c + o, g.ok[r]);
        float4 a = ld4(p.wx + o, g.ok[r]);
        float4 bq = ld4(p.wy + o, g.ok[r]);
        const int last = p.W - 1 - g.gx;               // index of the image's last column within this vector
        a.x = (last == 0) ? 0.f : kLip * a.x;
        a.y = (last == 1) ? 0.f : kLip * a.y;
        a.z = (last == 2) ? 0.f : kLip * a.z;
        a.w = (last == 3) ? 0.f : kLip * a.w;
        const float sy = (g.gy[r] == p.H - 1) ? 0.f : kLip;
        bq.x *= sy; bq.y *= sy; bq.z *= sy; bq.w *= sy;
        wx[r] = a;
        wy[r] = bq;
    }
}

}  // namespace

// ---------------------------------------------------------------------------------------------------------------
// forward: K iterations per launch
// ---------------------------------------------------------------------------------------------------------------
template <int K>
__global__ void __launch_bounds__(kThreads, 1)
tv_fwd_fused_kernel(const __grid_constant__ FwdFusedParams p) {
    __shared__ float4 sh_y[kWarps][32];     // each warp's first row of y
    __shared__ float4 sh_f[kWarps][32];     // each warp's last-row vertical flux
    const TileGeom g = make_geom<K>(p.H, p.W);
    const size_t n = blockIdx.z;
    const size_t plane = (size_t)p.H * p.W;
    float4 c[kRows], wx[kRows], wy[kRows], inv[kRows];
    load_maps(p, g, n, c, wx, wy);
#pragma unroll
    for (int r = 0; r < kRows; ++r) {
        inv[r].x = rcp_approx(1.0f + c[r].x);
        inv[r].y = rcp_approx(1.0f + c[r].y);
        inv[r].z = rcp_approx(1.0f + c[r].z);
        inv[r].w = rcp_approx(1.0f + c[r].w);
    }
    for (int ch = 0; ch < p.C; ++ch) {
        float4 y[kRows], x[kRows], b[kRows];
        size_t off[kRows];
#pragma unroll
        for (int r = 0; r < kRows; ++r) {
            off[r] = (n * p.C + ch) * plane + (size_t)g.gy[r] * p.W + g.gx;
            y[r] = ld4(p.y_in + off[r], g.ok[r]);
            x[r] = ld4(p.x_in + off[r], g.ok[r]);
            b[r] = ld4(p.b + off[r], g.ok[r]);
        }
#pragma unroll
        for (int j = 0; j < K; ++j) {
            const float t = p.t[j];
            sh_y[g.warp][g.lane] = y[0];
            __syncthreads();
            const float4 ybelow = (g.warp + 1 < kWarps) ? sh_y[g.warp + 1][g.lane] : zero4();
            if (p.ckpt[j]) {
#pragma unroll
                for (int r = 0; r < kRows; ++r)
                    if (g.store[r]) st4(p.ckpt[j] + off[r], y[r]);
            }
            float4 fxl, fyl;                                  // fluxes of the warp's last row
            flux_row(y[kRows - 1], ybelow, wx[kRows - 1], wy[kRows - 1], fxl, fyl);
            sh_f[g.warp][g.lane] = fyl;
            __syncthreads();
            float4 fyc = (g.warp > 0) ? sh_f[g.warp - 1][g.lane] : zero4();    // vertical flux arriving from above
#pragma unroll
            for (int r = 0; r < kRows; ++r) {
                float4 fx, fy;
                if (r == kRows - 1) { fx = fxl; fy = fyl; }
                else flux_row(y[r], y[r + 1], wx[r], wy[r], fx, fy);
                const float fx_left = __shfl_up_sync(kFull, fx.w, 1);          // last pixel of the lane to the left
                float4 x05;
                x05.x = y[r].x - fx.x - fy.x + fx_left + fyc.x;
                x05.y = y[r].y - fx.y - fy.y + fx.x + fyc.y;
                x05.z = y[r].z - fx.z - fy.z + fx.y + fyc.z;
                x05.w = y[r].w - fx.w - fy.w + fx.z + fyc.w;
                fyc = fy;
                if (g.store[r]) st4(p.hist[j] + off[r], x05);
                float4 xn;
                xn.x = prox_huber_fast(x05.x, b[r].x, c[r].x, inv[r].x);
                xn.y = prox_huber_fast(x05.y, b[r].y, c[r].y, inv[r].y);
                xn.z = prox_huber_fast(x05.z, b[r].z, c[r].z, inv[r].z);
                xn.w = prox_huber_fast(x05.w, b[r].w, c[r].w, inv[r].w);
                y[r].x = fmaf(t, xn.x - x[r].x, xn.x);
                y[r].y = fmaf(t, xn.y - x[r].y, xn.y);
                y[r].z = fmaf(t, xn.z - x[r].z, xn.z);
                y[r].w = fmaf(t, xn.w - x[r].w, xn.w);
                x[r] = xn;
            }
        }
#pragma unroll
        for (int r = 0; r < kRows; ++r)
            if (g.store[r]) {
                st4(p.y_out + off[r], y[r]);
                st4(p.x_out + off[r], x[r]);
            }
        __syncthreads();      // the next channel reuses the exchange rows
    }
}

bool fused_supported(int W, const void* const* ptrs, int nptr) {
    if (W % 4 != 0) return false;
    for (int i = 0; i < nptr; ++i)
        if ((reinterpret_cast<size_t>(ptrs[i]) & 15) != 0) return false;
    return true;
}

int launch_tv_fwd_fused(const FwdFusedParams& p, int K, cudaStream_t st) {
    if (K < 1 || K > kFuseMax) return fail(CNL_ERR_BAD_OPTION, "fuse factor %d is outside 1..%d", K, kFuseMax);
    const int TH = kRegionH - 2 * K;
    const dim3 grid((p.W + kTileW - 1) / kTileW, (p.H + TH - 1) / TH, p.N);
    switch (K) {
        case 1: tv_fwd_fused_kernel<1><<<grid, kThreads, 0, st>>>(p); break;
        case 2: tv_fwd_fused_kernel<2><<<grid, kThreads, 0, st>>>(p); break;
        case 3: tv_fwd_fused_kernel<3><<<grid, kThreads, 0, st>>>(p); break;
        default: tv_fwd_fused_kernel<4><<<grid, kThreads, 0, st>>>(p); break;
    }
    return after_launch("tv_fwd_fused_kernel");
}

// ---------------------------------------------------------------------------------------------------------------
// reverse: K reverse iterations per launch
// ---------------------------------------------------------------------------------------------------------------
namespace {

// Adjoint fluxes of the four triangles anchored at one lane's pixels of a row, plus their edge-weight gradients.
__device__ __forceinline__ void adjoint_row(const float4& y, const float4& yd, const float4& g, const float4& gd,
                                            const float4& wx, const float4& wy, float4& p1, float4& p2,
                                            float4& dwx, float4& dwy) {
    const float yr3 = __shfl_down_sync(kFull, y.x, 1);
    const float gr3 = __shfl_down_sync(kFull, g.x, 1);
    tri_adjoint_fast(y.x, y.y, yd.x, g.x, g.y, gd.x, wx.x, wy.x, p1.x, p2.x, dwx.x, dwy.x);
    tri_adjoint_fast(y.y, y.z, yd.y, g.y, g.z, gd.y, wx.y, wy.y, p1.y, p2.y, dwx.y, dwy.y);
    tri_adjoint_fast(y.z, y.w, yd.z, g.z, g.w, gd.z, wx.z, wy.z, p1.z, p2.z, dwx.z, dwy.z);
    tri_adjoint_fast(y.w, yr3, yd.w, g.w, gr3, gd.w, wx.w, wy.w, p1.w, p2.w, dwx.w, dwy.w);
}

// Momentum reverse + prox Jacobian for one pixel (TVInpaintFista.cu:796-828); returns dL/dx^{g+1/2}.
__device__ __forceinline__ float reverse_point(float ybar, float& acc, float x05, float b, float c, float t,
                                               float& dgc, float& dgb, float& xbar_out) {
    const float xbar = clampf(fmaf(1.0f + t, ybar, acc), -kClipLocal, kClipLocal);
    acc = -t * ybar;
    xbar_out = xbar;
    const float diff = b - x05;
    const float inv = rcp_approx(1.0f + c);
    if (1.0f + c >= fabsf(diff)) {
        // d/dc of (c b + x05)/(1+c) = (b - x)/(1+c) with x the prox output
        const float xq = fmaf(c, b, x05) * inv;
        dgc = fmaf(xbar * kLocalGC, (b - xq) * inv, dgc);
        dgb = fmaf(xbar * kLocalGB, c * inv, dgb);
        return xbar * inv;
    }
    dgc = fmaf(copysignf(kLocalGC, diff), xbar, dgc);
    return xbar;
}

}  // namespace

constexpr int kRevSmemBytes = (4 * kRows * kThreads + 3 * kWarps * 32) * (int)sizeof(float4);

template <int K>
__global__ void __launch_bounds__(kThreads, 1)
tv_rev_fused_kernel(const __grid_constant__ RevFusedParams p) {
    extern __shared__ float4 smem[];
    float4* sh_dc = smem;                                  // [kRows][kThreads] per-thread accumulators over channels
    float4* sh_dwx = sh_dc + kRows * kThreads;
    float4* sh_dwy = sh_dwx + kRows * kThreads;
    float4* sh_db = sh_dwy + kRows * kThreads;             // per channel
    float4(*sh_y)[32] = reinterpret_cast<float4(*)[32]>(sh_db + kRows * kThreads);    // first rows of y
    float4(*sh_g)[32] = sh_y + kWarps;                                               // first rows of g
    float4(*sh_p)[32] = sh_g + kWarps;                                               // last-row vertical adjoint flux
    const TileGeom g = make_geom<K>(p.H, p.W);
    const size_t n = blockIdx.z;
    const size_t plane = (size_t)p.H * p.W;
    float4 c[kRows], wx[kRows], wy[kRows];
    load_maps(p, g, n, c, wx, wy);
#pragma unroll
    for (int r = 0; r < kRows; ++r) {
        sh_dc[r * kThreads + threadIdx.x] = zero4();
        sh_dwx[r * kThreads + threadIdx.x] = zero4();
        sh_dwy[r * kThreads + threadIdx.x] = zero4();
    }
    for (int ch = 0; ch < p.C; ++ch) {
        float4 gq[kRows], acc[kRows], b[kRows], xh[kRows], xhm[kRows];
        size_t off[kRows];
#pragma unroll
        for (int r = 0; r < kRows; ++r) {
            off[r] = (n * p.C + ch) * plane + (size_t)g.gy[r] * p.W + g.gx;
            gq[r] = ld4(p.g_in + off[r], g.ok[r]);
            acc[r] = ld4(p.acc_in + off[r], g.ok[r]);
            b[r] = ld4(p.b + off[r], g.ok[r]);
            xh[r] = ld4(p.hist[0] + off[r], g.ok[r]);
            xhm[r] = ld4(p.hist[1] + off[r], g.ok[r] && p.hist[1] != nullptr);
            sh_db[r * kThreads + threadIdx.x] = zero4();
        }
#pragma unroll
        for (int j = 0; j < K; ++j) {
            const float t = p.t[j];
            // prefetch the pre-prox iterate the next fused step needs
            float4 xnext[kRows];
#pragma unroll
            for (int r = 0; r < kRows; ++r)
                xnext[r] = (j + 2 <= K) ? ld4(p.hist[j + 2 <= K ? j + 2 : K] + off[r], g.ok[r] && p.hist[j + 2 <= K ? j + 2 : K] != nullptr)
                                        : zero4();
            float4 y[kRows];
            if (p.ckpt[j]) {
#pragma unroll
                for (int r = 0; r < kRows; ++r) y[r] = ld4(p.ckpt[j] + off[r], g.ok[r]);
            } else {
#pragma unroll
                for (int r = 0; r < kRows; ++r) {
                    y[r].x = rederive_y_fast(xh[r].x, xhm[r].x, b[r].x, c[r].x, rcp_approx(1.0f + c[r].x), t);
                    y[r].y = rederive_y_fast(xh[r].y, xhm[r].y, b[r].y, c[r].y, rcp_approx(1.0f + c[r].y), t);
                    y[r].z = rederive_y_fast(xh[r].z, xhm[r].z, b[r].z, c[r].z, rcp_approx(1.0f + c[r].z), t);
                    y[r].w = rederive_y_fast(xh[r].w, xhm[r].w, b[r].w, c[r].w, rcp_approx(1.0f + c[r].w), t);
                }
            }
            sh_y[g.warp][g.lane] = y[0];
            sh_g[g.warp][g.lane] = gq[0];
            __syncthreads();
            const bool has_below = g.warp + 1 < kWarps;
            const float4 ybelow = has_below ? sh_y[g.warp + 1][g.lane] : zero4();
            const float4 gbelow = has_below ? sh_g[g.warp + 1][g.lane] : zero4();
            float4 p1l, p2l, dwxl, dwyl;
            adjoint_row(y[kRows - 1], ybelow, gq[kRows - 1], gbelow, wx[kRows - 1], wy[kRows - 1], p1l, p2l, dwxl, dwyl);
            sh_p[g.warp][g.lane] = p2l;
            add4(sh_dwx[(kRows - 1) * kThreads + threadIdx.x], dwxl);
            add4(sh_dwy[(kRows - 1) * kThreads + threadIdx.x], dwyl);
            __syncthreads();
            float4 p2c = (g.warp > 0) ? sh_p[g.warp - 1][g.lane] : zero4();
#pragma unroll
            for (int r = 0; r < kRows; ++r) {
                float4 p1, p2;
                if (r == kRows - 1) { p1 = p1l; p2 = p2l; }
                else {
                    float4 ax, ay;
                    adjoint_row(y[r], y[r + 1], gq[r], gq[r + 1], wx[r], wy[r], p1, p2, ax, ay);
                    add4(sh_dwx[r * kThreads + threadIdx.x], ax);
                    add4(sh_dwy[r * kThreads + threadIdx.x], ay);
                }
                const float p1_left = __shfl_up_sync(kFull, p1.w, 1);
                float4 ybar;
                ybar.x = gq[r].x - p1.x - p2.x + p1_left + p2c.x;
                ybar.y = gq[r].y - p1.y - p2.y + p1.x + p2c.y;
                ybar.z = gq[r].z - p1.z - p2.z + p1.y + p2c.z;
                ybar.w = gq[r].w - p1.w - p2.w + p1.z + p2c.w;
                p2c = p2;
                float4 xb;
                float4 dc = sh_dc[r * kThreads + threadIdx.x];
                float4 db = sh_db[r * kThreads + threadIdx.x];
                gq[r].x = reverse_point(ybar.x, acc[r].x, xh[r].x, b[r].x, c[r].x, t, dc.x, db.x, xb.x);
                gq[r].y = reverse_point(ybar.y, acc[r].y, xh[r].y, b[r].y, c[r].y, t, dc.y, db.y, xb.y);
                gq[r].z = reverse_point(ybar.z, acc[r].z, xh[r].z, b[r].z, c[r].z, t, dc.z, db.z, xb.z);
                gq[r].w = reverse_point(ybar.w, acc[r].w, xh[r].w, b[r].w, c[r].w, t, dc.w, db.w, xb.w);
                sh_dc[r * kThreads + threadIdx.x] = dc;
                sh_db[r * kThreads + threadIdx.x] = db;
                if (j == K - 1 && p.x1bar != nullptr && g.store[r]) st4(p.x1bar + off[r], xb);
            }
#pragma unroll
            for (int r = 0; r < kRows; ++r) {
                xh[r] = xhm[r];
                xhm[r] = xnext[r];
            }
        }
#pragma unroll
        for (int r = 0; r < kRows; ++r) {
            if (g.store[r]) {
                st4(p.g_out + off[r], gq[r]);
                st4(p.acc_out + off[r], acc[r]);
                float4 v = *reinterpret_cast<const float4*>(p.g_b + off[r]);
                add4(v, sh_db[r * kThreads + threadIdx.x]);
                st4(p.g_b + off[r], v);
            }
        }
    }
    // per-pixel gradients shared by all channels
#pragma unroll
    for (int r = 0; r < kRows; ++r) {
        if (!g.store[r]) continue;
        const size_t o = n * plane + (size_t)g.gy[r] * p.W + g.gx;
        const float4 dc = sh_dc[r * kThreads + threadIdx.x];
        float4 ax = sh_dwx[r * kThreads + threadIdx.x];
        float4 ay = sh_dwy[r * kThreads + threadIdx.x];
        const int last = p.W - 1 - g.gx;          // no edge leaves the last column / last row
        if (last == 0) ax.x = 0.f;
        if (last == 1) ax.y = 0.f;
        if (last == 2) ax.z = 0.f;
        if (last == 3) ax.w = 0.f;
        if (g.gy[r] == p.H - 1) ay = zero4();
        float4 v = *reinterpret_cast<const float4*>(p.g_c + o);
        v.x += dc.x; v.y += dc.y; v.z += dc.z; v.w += dc.w;
        st4(p.g_c + o, v);
        v = *reinterpret_cast<const float4*>(p.g_wx + o);
        v.x += ax.x; v.y += ax.y; v.z += ax.z; v.w += ax.w;
        st4(p.g_wx + o, v);
        v = *reinterpret_cast<const float4*>(p.g_wy + o);
        v.x += ay.x; v.y += ay.y; v.z += ay.z; v.w += ay.w;
        st4(p.g_wy + o, v);
    }
}

int launch_tv_rev_fused(const RevFusedParams& p, int K, cudaStream_t st) {
    if (K < 1 || K > kFuseMax) return fail(CNL_ERR_BAD_OPTION, "fuse factor %d is outside 1..%d", K, kFuseMax);
    static bool attr_set[kFuseMax + 1] = {};
    const int TH = kRegionH - 2 * K;
    const dim3 grid((p.W + kTileW - 1) / kTileW, (p.H + TH - 1) / TH, p.N);
    auto set_attr = [&](const void* fn) -> int {
        if (attr_set[K]) return CNL_OK;
        attr_set[K] = true;
        return check_cuda(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, kRevSmemBytes),
                          "cudaFuncSetAttribute");
    };
    switch (K) {
        case 1:
            CNL_TRY(set_attr(reinterpret_cast<const void*>(tv_rev_fused_kernel<1>)));
            tv_rev_fused_kernel<1><<<grid, kThreads, kRevSmemBytes, st>>>(p);
            break;
        case 2:
            CNL_TRY(set_attr(reinterpret_cast<const void*>(tv_rev_fused_kernel<2>)));
            tv_rev_fused_kernel<2><<<grid, kThreads, kRevSmemBytes, st>>>(p);
            break;
        case 3:
            CNL_TRY(set_attr(reinterpret_cast<const void*>(tv_rev_fused_kernel<3>)));
            tv_rev_fused_kernel<3><<<grid, kThreads, kRevSmemBytes, st>>>(p);
            break;
        default:
            CNL_TRY(set_attr(reinterpret_cast<const void*>(tv_rev_fused_kernel<4>)));
            tv_rev_fused_kernel<4><<<grid, kThreads, kRevSmemBytes, st>>>(p);
            break;
    }
    return after_launch("tv_rev_fused_kernel");
}

}  // namespace cnl
