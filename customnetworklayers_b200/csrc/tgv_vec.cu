// Register-tiled TGV-FISTA iteration kernels for sm_100a (geometry: see tgv_vec.cuh; math: the divergence form of
// cudaTGV/cudaCode/TGVInpaintFistaBetas.cu:1546-1776 forward and :224-644 / :1061-1473 reverse, as in tgv.cu).
#include "tgv_vec.cuh"

#include <algorithm>
#include <cstdlib>

#include "common.h"
#include "tv_math.cuh"

namespace cnl {
namespace tgv {

namespace {

constexpr int kNT = kTgvWarps * 32;
constexpr unsigned kFull = 0xffffffffu;
constexpr float kDeltaU = 0.2f, kDeltaV1 = 0.2f, kDeltaV2 = 0.2f;     // __HDelta2__, __HDeltaY1__, __HDeltaY2__ (:58-60)
constexpr float kClip = 2000.0f;                                      // clipLocalGrad (:78)

__device__ __forceinline__ float4 ld4(const float* p, bool ok) {
    return ok ? __ldg(reinterpret_cast<const float4*>(p)) : make_float4(0.f, 0.f, 0.f, 0.f);
}
__device__ __forceinline__ void st4(float* p, const float4& v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ float4 zero4() { return make_float4(0.f, 0.f, 0.f, 0.f); }
__device__ __forceinline__ void red_add4(float* p, const float4& v) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}
// 16-byte asynchronous global->shared copy; with ok == false nothing is read and the destination is zero-filled
__device__ __forceinline__ void cp_async16(float4* smem_dst, const float* gsrc, bool ok) {
    const unsigned dst = (unsigned)__cvta_generic_to_shared(smem_dst);
    const int bytes = ok ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(gsrc), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }
__device__ __forceinline__ void unpack(const float4& v, float (&a)[4]) { a[0] = v.x; a[1] = v.y; a[2] = v.z; a[3] = v.w; }
__device__ __forceinline__ float4 pack(const float (&a)[4]) { return make_float4(a[0], a[1], a[2], a[3]); }

struct Geom {
    int lane, warp, gx, gy;
    bool ok;          // the lane's vector lies inside the image
    bool okb;         // ... and so does the vector one row below
    bool store;       // inside the interior this CTA writes
    bool my;          // a vertical edge leaves this row
    bool mx[4];       // a horizontal edge leaves pixel k
    size_t pix;       // gy * pitch + gx (0 when !ok)
};

__device__ __forceinline__ Geom make_geom_at(int tx, int ty, int H, int W, int P) {
    Geom g;
    g.lane = threadIdx.x & 31;
    g.warp = threadIdx.x >> 5;
    g.gx = tx * kTgvTileW - 4 + 4 * g.lane;
    g.gy = ty * kTgvTileH - 1 + g.warp;
    const bool col = g.gx >= 0 && g.gx < W;
    g.ok = col && g.gy >= 0 && g.gy < H;
    g.okb = col && g.gy + 1 >= 0 && g.gy + 1 < H;
    g.store = g.ok && g.warp >= 1 && g.lane >= 1 && g.lane <= 30;
    g.my = g.ok && g.gy < H - 1;
#pragma unroll
    for (int k = 0; k < 4; ++k) g.mx[k] = g.ok && g.gx + k < W - 1;
    g.pix = g.ok ? (size_t)g.gy * P + g.gx : 0;
    return g;
}
__device__ __forceinline__ Geom make_geom(int H, int W, int P) { return make_geom_at(blockIdx.x, blockIdx.y, H, W, P); }

// Edge weights of the lane's four triangles, scaled by 1/Lipschitz and zero where no edge leaves the pixel.
struct Weights {
    float wx[4], wy[4], b0[4], b1[4];
};
__device__ __forceinline__ Weights scale_weights(const float4& wx, const float4& wy, const float4& bx, const float4& by,
                                                 const Geom& g, float L) {
    Weights w;
    float a[4];
    unpack(wx, a);
#pragma unroll
    for (int k = 0; k < 4; ++k) w.wx[k] = g.mx[k] ? __fmul_rn(L, a[k]) : 0.f;
    unpack(wy, a);
#pragma unroll
    for (int k = 0; k < 4; ++k) w.wy[k] = g.my ? __fmul_rn(L, a[k]) : 0.f;
    unpack(bx, a);
#pragma unroll
    for (int k = 0; k < 4; ++k) w.b0[k] = g.ok ? __fmul_rn(L, a[k]) : 0.f;
    unpack(by, a);
#pragma unroll
    for (int k = 0; k < 4; ++k) w.b1[k] = g.ok ? __fmul_rn(L, a[k]) : 0.f;
    return w;
}
__device__ __forceinline__ Weights load_weights(const float* dx, const float* dy, size_t n, size_t plane, const Geom& g, float L) {
    return scale_weights(ld4(dx + (n * 2 + 0) * plane + g.pix, g.ok), ld4(dy + (n * 2 + 0) * plane + g.pix, g.ok),
                         ld4(dx + (n * 2 + 1) * plane + g.pix, g.ok), ld4(dy + (n * 2 + 1) * plane + g.pix, g.ok), g, L);
}

// Differences and Huber factors of the triangle anchored at one pixel (c = centre, r = right, d = below).
struct TriQ {
    float z1, z2, Hu, r_u;
    float a1[2], a2[2], H[2], r[2];
};
__device__ __forceinline__ TriQ tri_quantities(float uc, float ur, float ud, float v1c, float v1r, float v1d, float v2c,
                                               float v2r, float v2d, float wx, float wy, float b0, float b1, bool mx, bool my) {
    TriQ t;
    t.z1 = mx ? (ur - uc - v1c) : 0.f;
    t.z2 = my ? (ud - uc - v2c) : 0.f;
    t.r_u = rsqrt_approx(wy * t.z2 * t.z2 + wx * t.z1 * t.z1);
    t.Hu = fminf(1.f, t.r_u * kDeltaU);
    t.a1[0] = mx ? (v1r - v1c) : 0.f;
    t.a2[0] = my ? (v1d - v1c) : 0.f;
    t.r[0] = rsqrt_approx(b0 * (t.a1[0] * t.a1[0] + t.a2[0] * t.a2[0]));
    t.H[0] = fminf(1.f, t.r[0] * kDeltaV1);
    t.a1[1] = mx ? (v2r - v2c) : 0.f;
    t.a2[1] = my ? (v2d - v2c) : 0.f;
    t.r[1] = rsqrt_approx(b1 * (t.a1[1] * t.a1[1] + t.a2[1] * t.a2[1]));
    t.H[1] = fminf(1.f, t.r[1] * kDeltaV2);
    return t;
}

}  // namespace

// ---------------------------------------------------------------------------------------------------------------
// forward iteration
// ---------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kNT, 2)
tgv_fwd_vec_kernel(const __grid_constant__ FwdVecParams p) {
    __shared__ float4 sh[2][3][kTgvWarps][32];        // per channel parity: Fy, G1y, G2y of each warp's row
    __shared__ float4 slots[5][kNT];                  // private landing slots of the pointwise operands
    float4* slot = &slots[0][threadIdx.x];
    const Geom g = make_geom(p.H, p.W, p.P);
    const size_t plane = (size_t)p.H * p.P;
    const size_t n = blockIdx.z;
    const float L = p.L[n];
    const Weights w = load_weights(p.dx, p.dy, n, plane, g, L);
    const size_t cstride = (size_t)p.C * plane;         // distance between the u, v1, v2 planes of a channel
    for (int ch = 0; ch < p.C; ++ch) {
        const size_t o = n * 3 * cstride + (size_t)ch * plane + g.pix;
        const float4 yu4 = ld4(p.y_in + o, g.ok), y14 = ld4(p.y_in + o + cstride, g.ok), y24 = ld4(p.y_in + o + 2 * cstride, g.ok);
        const float4 du4 = ld4(p.y_in + o + p.P, g.okb), d14 = ld4(p.y_in + o + cstride + p.P, g.okb),
                     d24 = ld4(p.y_in + o + 2 * cstride + p.P, g.okb);
        // pointwise operands are only needed where the CTA stores and not before the divergence: fetched
        // asynchronously so that they hold no registers meanwhile
        cp_async16(slot + 0 * kNT, p.x + o, g.store);
        cp_async16(slot + 1 * kNT, p.x + o + cstride, g.store);
        cp_async16(slot + 2 * kNT, p.x + o + 2 * cstride, g.store);
        cp_async16(slot + 3 * kNT, p.b + (n * p.C + ch) * plane + g.pix, g.store);
        cp_async16(slot + 4 * kNT, p.c + n * plane + g.pix, g.store);
        cp_async_commit();
        if (p.ckpt && g.store) {
            st4(p.ckpt + o, yu4); st4(p.ckpt + o + cstride, y14); st4(p.ckpt + o + 2 * cstride, y24);
        }
        float yu[5], y1[5], y2[5], du[4], d1[4], d2[4];
        {
            float a[4];
            unpack(yu4, a); for (int k = 0; k < 4; ++k) yu[k] = a[k];
            unpack(y14, a); for (int k = 0; k < 4; ++k) y1[k] = a[k];
            unpack(y24, a); for (int k = 0; k < 4; ++k) y2[k] = a[k];
        }
        unpack(du4, du); unpack(d14, d1); unpack(d24, d2);
        yu[4] = __shfl_down_sync(kFull, yu4.x, 1);
        y1[4] = __shfl_down_sync(kFull, y14.x, 1);
        y2[4] = __shfl_down_sync(kFull, y24.x, 1);
        float fx[4], fy[4], g1x[4], g1y[4], g2x[4], g2y[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const TriQ t = tri_quantities(yu[k], yu[k + 1], du[k], y1[k], y1[k + 1], d1[k], y2[k], y2[k + 1], d2[k],
                                          w.wx[k], w.wy[k], w.b0[k], w.b1[k], g.mx[k], g.my);
            fx[k] = w.wx[k] * t.z1 * t.Hu;
            fy[k] = w.wy[k] * t.z2 * t.Hu;
            g1x[k] = w.b0[k] * t.a1[0] * t.H[0];
            g1y[k] = w.b0[k] * t.a2[0] * t.H[0];
            g2x[k] = w.b1[k] * t.a1[1] * t.H[1];
            g2y[k] = w.b1[k] * t.a2[1] * t.H[1];
        }
        float4(*ex)[kTgvWarps][32] = sh[ch & 1];
        ex[0][g.warp][g.lane] = pack(fy);
        ex[1][g.warp][g.lane] = pack(g1y);
        ex[2][g.warp][g.lane] = pack(g2y);
        __syncthreads();
        float fya[4], g1ya[4], g2ya[4];                  // vertical fluxes of the row above
        unpack(g.warp > 0 ? ex[0][g.warp - 1][g.lane] : zero4(), fya);
        unpack(g.warp > 0 ? ex[1][g.warp - 1][g.lane] : zero4(), g1ya);
        unpack(g.warp > 0 ? ex[2][g.warp - 1][g.lane] : zero4(), g2ya);
        const float fxl = __shfl_up_sync(kFull, fx[3], 1);      // horizontal fluxes of the pixel to the left
        const float g1xl = __shfl_up_sync(kFull, g1x[3], 1);
        const float g2xl = __shfl_up_sync(kFull, g2x[3], 1);
        float xu[4], x1[4], x2[4], bq[4], cf[4];
        cp_async_wait_all();
        unpack(slot[0 * kNT], xu); unpack(slot[1 * kNT], x1); unpack(slot[2 * kNT], x2); unpack(slot[3 * kNT], bq); unpack(slot[4 * kNT], cf);
        float hu[4], h1[4], h2[4], nu[4], ou[4], o1[4], o2[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float fx_l = k == 0 ? fxl : fx[k - 1];
            const float g1x_l = k == 0 ? g1xl : g1x[k - 1];
            const float g2x_l = k == 0 ? g2xl : g2x[k - 1];
            hu[k] = yu[k] + fx[k] + fy[k] - fx_l - fya[k];
            h1[k] = y1[k] + g1x[k] + g1y[k] - g1x_l - g1ya[k] + fx[k];
            h2[k] = y2[k] + g2x[k] + g2y[k] - g2x_l - g2ya[k] + fy[k];
            nu[k] = prox_huber_fast(hu[k], bq[k], cf[k], rcp_approx(1.0f + cf[k]));
            ou[k] = nu[k] + p.t * (nu[k] - xu[k]);
            o1[k] = h1[k] + p.t * (h1[k] - x1[k]);
            o2[k] = h2[k] + p.t * (h2[k] - x2[k]);
        }
        if (g.store) {
            st4(p.hist + o, pack(hu)); st4(p.hist + o + cstride, pack(h1)); st4(p.hist + o + 2 * cstride, pack(h2));
            st4(p.x + o, pack(nu));    st4(p.x + o + cstride, pack(h1));    st4(p.x + o + 2 * cstride, pack(h2));
            st4(p.y_out + o, pack(ou)); st4(p.y_out + o + cstride, pack(o1)); st4(p.y_out + o + 2 * cstride, pack(o2));
        }
    }
}

// Persistent, software-pipelined forward iteration: two CTAs per SM walk over the (tile, channel) items.  Every operand
// of an item lands in shared memory by cp.async while the previous item is still being finished, so no warp waits
// for DRAM at the head of an item, and the row below a warp's own is read from the neighbouring warp's landing slots
// instead of being fetched twice.
constexpr int kFwdPipeSmemBytes = (2 * 3 * kNT + 8 * kNT + 4 * kNT + 3 * 32) * (int)sizeof(float4);

__global__ void __launch_bounds__(kNT, 2)
tgv_fwd_pipe_kernel(const __grid_constant__ FwdVecParams p, int tiles_x, int tiles_y) {
    extern __shared__ float4 fwd_smem[];
    float4(*ex)[3][kTgvWarps][32] = reinterpret_cast<float4(*)[3][kTgvWarps][32]>(fwd_smem);          // [2]: flux exchange
    float4(*sy)[kTgvWarps][32] = reinterpret_cast<float4(*)[kTgvWarps][32]>(fwd_smem + 6 * kNT);     // [3]: y rows of the item
    float4* sx = fwd_smem + 9 * kNT + threadIdx.x;       // [5][kNT]: x (3 planes), b, c of the lane's own pixels
    float4* sw = fwd_smem + 14 * kNT + threadIdx.x;      // [4][kNT]: wx, wy, beta_x, beta_y of the tile
    float4(*sbelow)[32] = reinterpret_cast<float4(*)[32]>(fwd_smem + 18 * kNT);                      // [3]: row under the region
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const size_t plane = (size_t)p.H * p.P;
    const size_t cstride = (size_t)p.C * plane;
    const int ntiles = tiles_x * tiles_y * p.N;

    auto tile_geom = [&](int tile, size_t& n) -> Geom {
        const int tx = tile % tiles_x, q = tile / tiles_x;
        n = (size_t)(q / tiles_y);
        return make_geom_at(tx, q % tiles_y, p.H, p.W, p.P);
    };
    // starts fetching every operand of (tile, ch); the edge weights only with the first channel of a tile
    auto issue = [&](int tile, int ch) {
        if (tile < ntiles) {
            size_t n;
            const Geom g = tile_geom(tile, n);
            const size_t o = n * 3 * cstride + (size_t)ch * plane + g.pix;
#pragma unroll
            for (int q = 0; q < 3; ++q) {
                cp_async16(&sy[q][warp][lane], p.y_in + o + q * cstride, g.ok);
                if (warp == kTgvWarps - 1) cp_async16(&sbelow[q][lane], p.y_in + o + q * cstride + (g.okb ? p.P : 0), g.okb);
                cp_async16(sx + q * kNT, p.x + o + q * cstride, g.store);
            }
            cp_async16(sx + 3 * kNT, p.b + (n * p.C + ch) * plane + g.pix, g.store);
            cp_async16(sx + 4 * kNT, p.c + n * plane + g.pix, g.store);
            if (ch == 0) {
                cp_async16(sw + 0 * kNT, p.dx + (n * 2 + 0) * plane + g.pix, g.ok);
                cp_async16(sw + 1 * kNT, p.dy + (n * 2 + 0) * plane + g.pix, g.ok);
                cp_async16(sw + 2 * kNT, p.dx + (n * 2 + 1) * plane + g.pix, g.ok);
                cp_async16(sw + 3 * kNT, p.dy + (n * 2 + 1) * plane + g.pix, g.ok);
            }
        }
        cp_async_commit();
    };

    int tile = blockIdx.x;
    if (tile >= ntiles) return;
    issue(tile, 0);
    int parity = 0;
    for (; tile < ntiles; tile += gridDim.x) {
        size_t n;
        const Geom g = tile_geom(tile, n);
        const float L = p.L[n];
        Weights w;
        for (int ch = 0; ch < p.C; ++ch, parity ^= 1) {
            const size_t o = n * 3 * cstride + (size_t)ch * plane + g.pix;
            cp_async_wait_all();
            __syncthreads();                                  // every thread's operands of this item have landed
            if (ch == 0) w = scale_weights(sw[0 * kNT], sw[1 * kNT], sw[2 * kNT], sw[3 * kNT], g, L);
            const float4 yu4 = sy[0][warp][lane], y14 = sy[1][warp][lane], y24 = sy[2][warp][lane];
            float4 du4, d14, d24;
            if (warp < kTgvWarps - 1) { du4 = sy[0][warp + 1][lane]; d14 = sy[1][warp + 1][lane]; d24 = sy[2][warp + 1][lane]; }
            else { du4 = sbelow[0][lane]; d14 = sbelow[1][lane]; d24 = sbelow[2][lane]; }
            if (p.ckpt && g.store) {
                st4(p.ckpt + o, yu4); st4(p.ckpt + o + cstride, y14); st4(p.ckpt + o + 2 * cstride, y24);
            }
            float yu[5], y1[5], y2[5], du[4], d1[4], d2[4];
            {
                float a[4];
                unpack(yu4, a); for (int k = 0; k < 4; ++k) yu[k] = a[k];
                unpack(y14, a); for (int k = 0; k < 4; ++k) y1[k] = a[k];
                unpack(y24, a); for (int k = 0; k < 4; ++k) y2[k] = a[k];
            }
            unpack(du4, du); unpack(d14, d1); unpack(d24, d2);
            yu[4] = __shfl_down_sync(kFull, yu4.x, 1);
            y1[4] = __shfl_down_sync(kFull, y14.x, 1);
            y2[4] = __shfl_down_sync(kFull, y24.x, 1);
            float fx[4], fy[4], g1x[4], g1y[4], g2x[4], g2y[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const TriQ t = tri_quantities(yu[k], yu[k + 1], du[k], y1[k], y1[k + 1], d1[k], y2[k], y2[k + 1], d2[k],
                                              w.wx[k], w.wy[k], w.b0[k], w.b1[k], g.mx[k], g.my);
                fx[k] = w.wx[k] * t.z1 * t.Hu;
                fy[k] = w.wy[k] * t.z2 * t.Hu;
                g1x[k] = w.b0[k] * t.a1[0] * t.H[0];
                g1y[k] = w.b0[k] * t.a2[0] * t.H[0];
                g2x[k] = w.b1[k] * t.a1[1] * t.H[1];
                g2y[k] = w.b1[k] * t.a2[1] * t.H[1];
            }
            ex[parity][0][warp][lane] = pack(fy);
            ex[parity][1][warp][lane] = pack(g1y);
            ex[parity][2][warp][lane] = pack(g2y);
            __syncthreads();                                  // fluxes published; all reads of the y rows are done
            float xu[4], x1[4], x2[4], bq[4], cf[4];
            unpack(sx[0 * kNT], xu); unpack(sx[1 * kNT], x1); unpack(sx[2 * kNT], x2); unpack(sx[3 * kNT], bq); unpack(sx[4 * kNT], cf);
            // every landing slot is free again: start fetching the next item
            if (ch + 1 < p.C) issue(tile, ch + 1);
            else issue(tile + gridDim.x, 0);
            float fya[4], g1ya[4], g2ya[4];
            unpack(warp > 0 ? ex[parity][0][warp - 1][lane] : zero4(), fya);
            unpack(warp > 0 ? ex[parity][1][warp - 1][lane] : zero4(), g1ya);
            unpack(warp > 0 ? ex[parity][2][warp - 1][lane] : zero4(), g2ya);
            const float fxl = __shfl_up_sync(kFull, fx[3], 1);
            const float g1xl = __shfl_up_sync(kFull, g1x[3], 1);
            const float g2xl = __shfl_up_sync(kFull, g2x[3], 1);
            float hu[4], h1[4], h2[4], nu[4], ou[4], o1[4], o2[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float fx_l = k == 0 ? fxl : fx[k - 1];
                const float g1x_l = k == 0 ? g1xl : g1x[k - 1];
                const float g2x_l = k == 0 ? g2xl : g2x[k - 1];
                hu[k] = yu[k] + fx[k] + fy[k] - fx_l - fya[k];
                h1[k] = y1[k] + g1x[k] + g1y[k] - g1x_l - g1ya[k] + fx[k];
                h2[k] = y2[k] + g2x[k] + g2y[k] - g2x_l - g2ya[k] + fy[k];
                nu[k] = prox_huber_fast(hu[k], bq[k], cf[k], rcp_approx(1.0f + cf[k]));
                ou[k] = nu[k] + p.t * (nu[k] - xu[k]);
                o1[k] = h1[k] + p.t * (h1[k] - x1[k]);
                o2[k] = h2[k] + p.t * (h2[k] - x2[k]);
            }
            if (g.store) {
                st4(p.hist + o, pack(hu)); st4(p.hist + o + cstride, pack(h1)); st4(p.hist + o + 2 * cstride, pack(h2));
                st4(p.x + o, pack(nu));    st4(p.x + o + cstride, pack(h1));    st4(p.x + o + 2 * cstride, pack(h2));
                st4(p.y_out + o, pack(ou)); st4(p.y_out + o + cstride, pack(o1)); st4(p.y_out + o + 2 * cstride, pack(o2));
            }
        }
    }
    cp_async_wait_all();
}

// ---------------------------------------------------------------------------------------------------------------
// reverse iteration
// ---------------------------------------------------------------------------------------------------------------
namespace {

// y (momentum variable) and incoming adjoint of one row of the lane's pixels.  u of y is rebuilt from the stored
// pre-prox iterates of iterations g and g-1 unless a checkpoint supplies all three planes (:1478-1541).
struct RowState {
    float4 yu, y1, y2, gu, g1, g2;
};
__device__ __forceinline__ RowState load_row(const RevVecParams& p, size_t o, size_t ob, size_t oc, size_t cstride, bool ok) {
    RowState r;
    const float* ysrc = p.ckpt ? p.ckpt : p.hist_g;
    r.yu = ld4(ysrc + o, ok);
    r.y1 = ld4(ysrc + o + cstride, ok);
    r.y2 = ld4(ysrc + o + 2 * cstride, ok);
    r.gu = ld4(p.g_in + o, ok);
    r.g1 = ld4(p.g_in + o + cstride, ok);
    r.g2 = ld4(p.g_in + o + 2 * cstride, ok);
    if (!p.ckpt) {
        const float4 hm = ld4(p.hist_gm1 + o, ok && p.hist_gm1 != nullptr);
        const float4 b = ld4(p.b + ob, ok);
        const float4 c = ld4(p.c + oc, ok);
        if (ok) {
            r.yu.x = rederive_y_fast(r.yu.x, hm.x, b.x, c.x, rcp_approx(1.0f + c.x), p.t);
            r.yu.y = rederive_y_fast(r.yu.y, hm.y, b.y, c.y, rcp_approx(1.0f + c.y), p.t);
            r.yu.z = rederive_y_fast(r.yu.z, hm.z, b.z, c.z, rcp_approx(1.0f + c.z), p.t);
            r.yu.w = rederive_y_fast(r.yu.w, hm.w, b.w, c.w, rcp_approx(1.0f + c.w), p.t);
        }
    }
    return r;
}


// Adjoint fluxes of the lane's four triangles (kept for the divergence) and their edge-weight gradients.
struct RevFlux {
    float P1[4], P2[4], C1x[4], C1y[4], C2x[4], C2y[4], C2d[4];      // psi1, psi2, chi1x, chi1y, chi2x, chi2y, down-going chi2y
    float gu[4], g1[4], g2[4];                                        // incoming adjoint of the lane's own pixels
};
__device__ __forceinline__ void rev_adjoint_fluxes(const RowState& own, const RowState& below, const Weights& w, const Geom& g,
                                                   int typo, RevFlux& f, float4 (&gw_out)[4]) {
    float yu[5], y1[5], y2[5], gu[5], g1[5], g2[5], du[4], d1[4], d2[4], eu[4], e1[4], e2[4];
    {
        float a[4];
        unpack(own.yu, a); for (int k = 0; k < 4; ++k) yu[k] = a[k];
        unpack(own.y1, a); for (int k = 0; k < 4; ++k) y1[k] = a[k];
        unpack(own.y2, a); for (int k = 0; k < 4; ++k) y2[k] = a[k];
        unpack(own.gu, a); for (int k = 0; k < 4; ++k) gu[k] = a[k];
        unpack(own.g1, a); for (int k = 0; k < 4; ++k) g1[k] = a[k];
        unpack(own.g2, a); for (int k = 0; k < 4; ++k) g2[k] = a[k];
    }
    unpack(below.yu, du); unpack(below.y1, d1); unpack(below.y2, d2);
    unpack(below.gu, eu); unpack(below.g1, e1); unpack(below.g2, e2);
    yu[4] = __shfl_down_sync(kFull, own.yu.x, 1); y1[4] = __shfl_down_sync(kFull, own.y1.x, 1); y2[4] = __shfl_down_sync(kFull, own.y2.x, 1);
    gu[4] = __shfl_down_sync(kFull, own.gu.x, 1); g1[4] = __shfl_down_sync(kFull, own.g1.x, 1); g2[4] = __shfl_down_sync(kFull, own.g2.x, 1);
    float gw0[4], gw1[4], gw2[4], gw3[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const TriQ tr = tri_quantities(yu[k], yu[k + 1], du[k], y1[k], y1[k + 1], d1[k], y2[k], y2[k + 1], d2[k],
                                       w.wx[k], w.wy[k], w.b0[k], w.b1[k], g.mx[k], g.my);
        const float Ex = gu[k] - gu[k + 1] + g1[k];
        const float Ey = gu[k] - eu[k] + g2[k];
        const float a1 = tr.z1 * w.wx[k], a2 = tr.z2 * w.wy[k];
        const float S = a1 * Ex + a2 * Ey;
        const float dW = tr.Hu < 1.f ? tr.Hu * tr.r_u * tr.r_u : 0.f;
        f.P1[k] = w.wx[k] * tr.Hu * Ex - dW * a1 * S;
        f.P2[k] = w.wy[k] * tr.Hu * Ey - dW * a2 * S;
        gw0[k] = kLocalGX * (Ex * tr.z1 * tr.Hu - 0.5f * tr.z1 * tr.z1 * dW * S);
        gw2[k] = kLocalGX * (Ey * tr.z2 * tr.Hu - 0.5f * tr.z2 * tr.z2 * dW * S);
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const float gc = j == 0 ? g1[k] : g2[k], gr = j == 0 ? g1[k + 1] : g2[k + 1], gd = j == 0 ? e1[k] : e2[k];
            const float E1 = g.mx[k] ? gc - gr : 0.f;
            const float E2 = g.my ? gc - gd : 0.f;
            const float b1 = tr.a1[j], b2 = tr.a2[j], beta = j == 0 ? w.b0[k] : w.b1[k], Hj = tr.H[j];
            const float Sj = b1 * E1 + b2 * E2;
            const bool act = Hj < 1.f;
            const float dWj = act ? Hj * tr.r[j] * tr.r[j] : 0.f;
            const float chx = beta * (Hj * E1 - dWj * beta * b1 * Sj);
            const float chy = beta * (Hj * E2 - dWj * beta * b2 * Sj);
            const float gbeta = kLocalGX * (Sj * Hj - 0.5f * (b1 * b1 + b2 * b2) * dWj * beta * Sj);
            if (j == 0) { f.C1x[k] = chx; f.C1y[k] = chy; gw1[k] = gbeta; }
            else {
                f.C2x[k] = chx; f.C2y[k] = chy; gw3[k] = gbeta;
                float down = chy;
                if (typo && act) down = beta * (Hj * E2 - (Hj * beta * (b1 * b1 + b2 * b2)) * beta * b2 * Sj);
                f.C2d[k] = down;
            }
        }
        f.gu[k] = gu[k]; f.g1[k] = g1[k]; f.g2[k] = g2[k];
    }
    gw_out[0] = pack(gw0); gw_out[1] = pack(gw1); gw_out[2] = pack(gw2); gw_out[3] = pack(gw3);
}

// Divergence of the adjoint fluxes, momentum reverse and prox Jacobian for the lane's four pixels.
struct RevOut {
    float4 xb0, xb1, xb2;      // dL/dx of this iteration (u, v1, v2)
    float4 na0, na1, na2;      // new pending momentum terms
    float4 go;                 // dL/dx^{g-1/2}, primary plane
    float4 dgc, dgb;           // confidence and data-term gradient contributions
};
__device__ __forceinline__ void rev_divergence_and_prox(const RevFlux& f, const float4& P2a4, const float4& C1ya4, const float4& C2da4,
                                                        const float4& au4, const float4& a14, const float4& a24, const float4& hu4,
                                                        const float4& b4, const float4& c4, float t, RevOut& r) {
    float P2a[4], C1ya[4], C2da[4], au[4], a1v[4], a2v[4], hu[4], bq[4], cq[4];
    unpack(P2a4, P2a); unpack(C1ya4, C1ya); unpack(C2da4, C2da);
    unpack(au4, au); unpack(a14, a1v); unpack(a24, a2v); unpack(hu4, hu); unpack(b4, bq); unpack(c4, cq);
    const float P1l = __shfl_up_sync(kFull, f.P1[3], 1);
    const float C1xl = __shfl_up_sync(kFull, f.C1x[3], 1);
    const float C2xl = __shfl_up_sync(kFull, f.C2x[3], 1);
    float xb0[4], xb1[4], xb2[4], na0[4], na1[4], na2[4], go[4], dgc[4], dgb[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const float P1_l = k == 0 ? P1l : f.P1[k - 1];
        const float C1x_l = k == 0 ? C1xl : f.C1x[k - 1];
        const float C2x_l = k == 0 ? C2xl : f.C2x[k - 1];
        const float yb0 = f.gu[k] - f.P1[k] - f.P2[k] + P1_l + P2a[k];
        const float yb1 = f.g1[k] - f.P1[k] - f.C1x[k] - f.C1y[k] + C1x_l + C1ya[k];
        const float yb2 = f.g2[k] - f.P2[k] - f.C2x[k] - f.C2y[k] + C2x_l + C2da[k];
        xb0[k] = clampf(au[k] + (1.0f + t) * yb0, -kClip, kClip);
        xb1[k] = clampf(a1v[k] + (1.0f + t) * yb1, -kClip, kClip);
        xb2[k] = clampf(a2v[k] + (1.0f + t) * yb2, -kClip, kClip);
        na0[k] = -t * yb0; na1[k] = -t * yb1; na2[k] = -t * yb2;
        dgc[k] = 0.f; dgb[k] = 0.f;
        go[k] = prox_reverse_fast(xb0[k], hu[k], bq[k], cq[k], rcp_approx(1.0f + cq[k]), dgc[k], dgb[k]);
    }
    r.xb0 = pack(xb0); r.xb1 = pack(xb1); r.xb2 = pack(xb2);
    r.na0 = pack(na0); r.na1 = pack(na1); r.na2 = pack(na2);
    r.go = pack(go); r.dgc = pack(dgc); r.dgb = pack(dgb);
}

}  // namespace

__global__ void __launch_bounds__(kNT, 2)
tgv_rev_vec_kernel(const __grid_constant__ RevVecParams p) {
    extern __shared__ float4 rev_smem[];
    float4(*sh_row)[kTgvWarps][32] = reinterpret_cast<float4(*)[kTgvWarps][32]>(rev_smem);             // [6]: y and g planes of each warp's row
    float4(*sh_flux)[kTgvWarps][32] = reinterpret_cast<float4(*)[kTgvWarps][32]>(rev_smem + 6 * kNT);  // [3]: psi2, chi1y, down-going chi2y
    float4* slot = rev_smem + 9 * kNT + threadIdx.x;   // [6][kNT] private landing slots of the pointwise operands
    const Geom g = make_geom(p.H, p.W, p.P);
    const size_t plane = (size_t)p.H * p.P;
    const size_t n = blockIdx.z;
    const float L = p.L[n];
    const Weights w = load_weights(p.dx, p.dy, n, plane, g, L);
    const size_t cstride = (size_t)p.C * plane;
    const size_t oc = n * plane + g.pix;
    for (int ch = 0; ch < p.C; ++ch) {
        const size_t o = n * 3 * cstride + (size_t)ch * plane + g.pix;
        const size_t ob = (n * p.C + ch) * plane + g.pix;
        const RowState own = load_row(p, o, ob, oc, cstride, g.ok);
        // pointwise operands of the lane's own pixels (only where the CTA stores)
        // they are not needed before the divergence: fetched asynchronously so that they hold no registers meanwhile
        cp_async16(slot + 0 * kNT, p.hist_g + o, g.store);                    // x^{g+1/2}, primary plane
        cp_async16(slot + 1 * kNT, p.b + ob, g.store);
        cp_async16(slot + 2 * kNT, p.c + oc, g.store);
        cp_async16(slot + 3 * kNT, p.acc + o, g.store);
        cp_async16(slot + 4 * kNT, p.acc + o + cstride, g.store);
        cp_async16(slot + 5 * kNT, p.acc + o + 2 * cstride, g.store);
        cp_async_commit();
        sh_row[0][g.warp][g.lane] = own.yu; sh_row[1][g.warp][g.lane] = own.y1; sh_row[2][g.warp][g.lane] = own.y2;
        sh_row[3][g.warp][g.lane] = own.gu; sh_row[4][g.warp][g.lane] = own.g1; sh_row[5][g.warp][g.lane] = own.g2;
        RowState below;
        if (g.warp == kTgvWarps - 1) below = load_row(p, o + p.P, ob + p.P, oc + p.P, cstride, g.okb);   // row under the region
        __syncthreads();
        if (g.warp < kTgvWarps - 1) {
            below.yu = sh_row[0][g.warp + 1][g.lane]; below.y1 = sh_row[1][g.warp + 1][g.lane]; below.y2 = sh_row[2][g.warp + 1][g.lane];
            below.gu = sh_row[3][g.warp + 1][g.lane]; below.g1 = sh_row[4][g.warp + 1][g.lane]; below.g2 = sh_row[5][g.warp + 1][g.lane];
        }
        RevFlux f;
        float4 gw[4];
        rev_adjoint_fluxes(own, below, w, g, p.typo, f, gw);
        sh_flux[0][g.warp][g.lane] = pack(f.P2);
        sh_flux[1][g.warp][g.lane] = pack(f.C1y);
        sh_flux[2][g.warp][g.lane] = pack(f.C2d);
        if (g.store) {      // every triangle's weight gradient is accumulated by the pixel that anchors it
            red_add4(p.g_dx + (n * 2 + 0) * plane + g.pix, gw[0]);
            red_add4(p.g_dx + (n * 2 + 1) * plane + g.pix, gw[1]);
            red_add4(p.g_dy + (n * 2 + 0) * plane + g.pix, gw[2]);
            red_add4(p.g_dy + (n * 2 + 1) * plane + g.pix, gw[3]);
        }
        __syncthreads();
        const float4 P2a = g.warp > 0 ? sh_flux[0][g.warp - 1][g.lane] : zero4();
        const float4 C1ya = g.warp > 0 ? sh_flux[1][g.warp - 1][g.lane] : zero4();
        const float4 C2da = g.warp > 0 ? sh_flux[2][g.warp - 1][g.lane] : zero4();
        cp_async_wait_all();
        RevOut r;
        rev_divergence_and_prox(f, P2a, C1ya, C2da, slot[3 * kNT], slot[4 * kNT], slot[5 * kNT], slot[0 * kNT], slot[1 * kNT],
                                slot[2 * kNT], p.t, r);
        if (g.store) {
            st4(p.acc + o, r.na0); st4(p.acc + o + cstride, r.na1); st4(p.acc + o + 2 * cstride, r.na2);
            if (p.x1bar) { st4(p.x1bar + o, r.xb0); st4(p.x1bar + o + cstride, r.xb1); st4(p.x1bar + o + 2 * cstride, r.xb2); }
            st4(p.g_out + o, r.go); st4(p.g_out + o + cstride, r.xb1); st4(p.g_out + o + 2 * cstride, r.xb2);
            red_add4(p.g_b + ob, r.dgb);
            red_add4(p.g_c + oc, r.dgc);
        }
    }
}

// Tiles a launch must have before the persistent kernel is used; CNL_TGV_PIPELINE_MIN_TILES overrides the default
// (read at every call so that tests can force either kernel; a negative value disables the persistent kernel).
static long long pipeline_min_tiles(int sms) {
    const char* e = std::getenv("CNL_TGV_PIPELINE_MIN_TILES");
    if (e && e[0]) { const long long v = std::atoll(e); return v < 0 ? (1ll << 40) : v; }
    return 16LL * sms;
}

// Same for the reverse kernel (CNL_TGV_REV_PIPELINE_MIN_TILES).
static long long rev_pipeline_min_tiles(int sms) {
    const char* e = std::getenv("CNL_TGV_REV_PIPELINE_MIN_TILES");
    if (e && e[0]) { const long long v = std::atoll(e); return v < 0 ? (1ll << 40) : v; }
    return 16LL * sms;
}

// Persistent, software-pipelined reverse iteration (same scheme as tgv_fwd_pipe_kernel): every operand plane of the
// next (tile, channel) item lands in shared memory while the current item is finished.  The rows of y and of the
// incoming adjoint arrive raw; each warp rebuilds u of y for its own row and for the row below it from the raw
// iterates (a few redundant flops instead of a second exchange and barrier).
constexpr int kRevPipeSmemBytes = (23 * kNT + 9 * 32) * (int)sizeof(float4);

__global__ void __launch_bounds__(kNT, 2)
tgv_rev_pipe_kernel(const __grid_constant__ RevVecParams p, int tiles_x, int tiles_y) {
    extern __shared__ float4 rp_smem[];
    typedef float4 (*Rows)[kTgvWarps][32];
    float4(*ex)[3][kTgvWarps][32] = reinterpret_cast<float4(*)[3][kTgvWarps][32]>(rp_smem);     // [2]: flux exchange
    Rows sy = reinterpret_cast<Rows>(rp_smem + 6 * kNT);       // [3] raw y source rows (checkpoint or stored iterate g)
    Rows sg = reinterpret_cast<Rows>(rp_smem + 9 * kNT);       // [3] incoming adjoint rows
    Rows sq = reinterpret_cast<Rows>(rp_smem + 12 * kNT);      // [3] stored iterate g-1 (u), b, c rows
    float4* sacc = rp_smem + 15 * kNT + threadIdx.x;           // [3][kNT] pending momentum of the lane's own pixels
    float4* shu = rp_smem + 18 * kNT + threadIdx.x;            // [kNT] x^{g+1/2} (u) when y comes from a checkpoint
    float4* sw = rp_smem + 19 * kNT + threadIdx.x;             // [4][kNT] edge weights of the tile
    float4(*sbelow)[32] = reinterpret_cast<float4(*)[32]>(rp_smem + 23 * kNT);                   // [9] row under the region
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const size_t plane = (size_t)p.H * p.P;
    const size_t cstride = (size_t)p.C * plane;
    const int ntiles = tiles_x * tiles_y * p.N;
    const float* ysrc = p.ckpt ? p.ckpt : p.hist_g;
    const bool rebuild = p.ckpt == nullptr;

    auto tile_geom = [&](int tile, size_t& n) -> Geom {
        const int tx = tile % tiles_x, q = tile / tiles_x;
        n = (size_t)(q / tiles_y);
        return make_geom_at(tx, q % tiles_y, p.H, p.W, p.P);
    };
    auto issue = [&](int tile, int ch) {
        if (tile < ntiles) {
            size_t n;
            const Geom g = tile_geom(tile, n);
            const size_t o = n * 3 * cstride + (size_t)ch * plane + g.pix;
            const size_t ob = (n * p.C + ch) * plane + g.pix, oc = n * plane + g.pix;
            const bool last = warp == kTgvWarps - 1;
            const size_t dn = g.okb ? (size_t)p.P : 0;         // one image row further down
#pragma unroll
            for (int q = 0; q < 3; ++q) {
                cp_async16(&sy[q][warp][lane], ysrc + o + q * cstride, g.ok);
                cp_async16(&sg[q][warp][lane], p.g_in + o + q * cstride, g.ok);
                cp_async16(sacc + q * kNT, p.acc + o + q * cstride, g.store);
                if (last) {
                    cp_async16(&sbelow[q][lane], ysrc + o + q * cstride + dn, g.okb);
                    cp_async16(&sbelow[3 + q][lane], p.g_in + o + q * cstride + dn, g.okb);
                }
            }
            const bool hm_ok = rebuild && p.hist_gm1 != nullptr;
            cp_async16(&sq[0][warp][lane], hm_ok ? p.hist_gm1 + o : p.b, g.ok && hm_ok);
            cp_async16(&sq[1][warp][lane], p.b + ob, g.ok);
            cp_async16(&sq[2][warp][lane], p.c + oc, g.ok);
            if (last) {
                cp_async16(&sbelow[6][lane], hm_ok ? p.hist_gm1 + o + dn : p.b, g.okb && hm_ok);
                cp_async16(&sbelow[7][lane], p.b + ob + dn, g.okb);
                cp_async16(&sbelow[8][lane], p.c + oc + dn, g.okb);
            }
            if (!rebuild) cp_async16(shu, p.hist_g + o, g.store);
            if (ch == 0) {
                cp_async16(sw + 0 * kNT, p.dx + (n * 2 + 0) * plane + g.pix, g.ok);
                cp_async16(sw + 1 * kNT, p.dy + (n * 2 + 0) * plane + g.pix, g.ok);
                cp_async16(sw + 2 * kNT, p.dx + (n * 2 + 1) * plane + g.pix, g.ok);
                cp_async16(sw + 3 * kNT, p.dy + (n * 2 + 1) * plane + g.pix, g.ok);
            }
        }
        cp_async_commit();
    };
    // y and adjoint of one row from its raw planes
    auto make_row = [&](const float4& ru, const float4& r1, const float4& r2, const float4& qu, const float4& q1, const float4& q2,
                        const float4& hm, const float4& b, const float4& c, bool ok) -> RowState {
        RowState r;
        r.yu = ru; r.y1 = r1; r.y2 = r2; r.gu = qu; r.g1 = q1; r.g2 = q2;
        if (rebuild && ok) {
            r.yu.x = rederive_y_fast(ru.x, hm.x, b.x, c.x, rcp_approx(1.0f + c.x), p.t);
            r.yu.y = rederive_y_fast(ru.y, hm.y, b.y, c.y, rcp_approx(1.0f + c.y), p.t);
            r.yu.z = rederive_y_fast(ru.z, hm.z, b.z, c.z, rcp_approx(1.0f + c.z), p.t);
            r.yu.w = rederive_y_fast(ru.w, hm.w, b.w, c.w, rcp_approx(1.0f + c.w), p.t);
        }
        return r;
    };

    int tile = blockIdx.x;
    if (tile >= ntiles) return;
    issue(tile, 0);
    int parity = 0;
    for (; tile < ntiles; tile += gridDim.x) {
        size_t n;
        const Geom g = tile_geom(tile, n);
        const float L = p.L[n];
        const size_t oc = n * plane + g.pix;
        Weights w;
        for (int ch = 0; ch < p.C; ++ch, parity ^= 1) {
            const size_t o = n * 3 * cstride + (size_t)ch * plane + g.pix;
            const size_t ob = (n * p.C + ch) * plane + g.pix;
            cp_async_wait_all();
            __syncthreads();                                  // every thread's operands of this item have landed
            if (ch == 0) w = scale_weights(sw[0 * kNT], sw[1 * kNT], sw[2 * kNT], sw[3 * kNT], g, L);
            const RowState own = make_row(sy[0][warp][lane], sy[1][warp][lane], sy[2][warp][lane], sg[0][warp][lane], sg[1][warp][lane],
                                          sg[2][warp][lane], sq[0][warp][lane], sq[1][warp][lane], sq[2][warp][lane], g.ok);
            RowState below;
            if (warp < kTgvWarps - 1)
                below = make_row(sy[0][warp + 1][lane], sy[1][warp + 1][lane], sy[2][warp + 1][lane], sg[0][warp + 1][lane],
                                 sg[1][warp + 1][lane], sg[2][warp + 1][lane], sq[0][warp + 1][lane], sq[1][warp + 1][lane],
                                 sq[2][warp + 1][lane], g.okb);
            else
                below = make_row(sbelow[0][lane], sbelow[1][lane], sbelow[2][lane], sbelow[3][lane], sbelow[4][lane], sbelow[5][lane],
                                 sbelow[6][lane], sbelow[7][lane], sbelow[8][lane], g.okb);
            RevFlux f;
            float4 gw[4];
            rev_adjoint_fluxes(own, below, w, g, p.typo, f, gw);
            ex[parity][0][warp][lane] = pack(f.P2);
            ex[parity][1][warp][lane] = pack(f.C1y);
            ex[parity][2][warp][lane] = pack(f.C2d);
            if (g.store) {
                red_add4(p.g_dx + (n * 2 + 0) * plane + g.pix, gw[0]);
                red_add4(p.g_dx + (n * 2 + 1) * plane + g.pix, gw[1]);
                red_add4(p.g_dy + (n * 2 + 0) * plane + g.pix, gw[2]);
                red_add4(p.g_dy + (n * 2 + 1) * plane + g.pix, gw[3]);
            }
            __syncthreads();                                  // fluxes published; all reads of the raw rows are done
            const float4 au4 = sacc[0 * kNT], a14 = sacc[1 * kNT], a24 = sacc[2 * kNT];
            const float4 hu4 = rebuild ? sy[0][warp][lane] : shu[0];
            const float4 b4 = sq[1][warp][lane], c4 = sq[2][warp][lane];
            // every landing slot is free again: start fetching the next item
            if (ch + 1 < p.C) issue(tile, ch + 1);
            else issue(tile + gridDim.x, 0);
            const float4 P2a = warp > 0 ? ex[parity][0][warp - 1][lane] : zero4();
            const float4 C1ya = warp > 0 ? ex[parity][1][warp - 1][lane] : zero4();
            const float4 C2da = warp > 0 ? ex[parity][2][warp - 1][lane] : zero4();
            RevOut r;
            rev_divergence_and_prox(f, P2a, C1ya, C2da, au4, a14, a24, hu4, b4, c4, p.t, r);
            if (g.store) {
                st4(p.acc + o, r.na0); st4(p.acc + o + cstride, r.na1); st4(p.acc + o + 2 * cstride, r.na2);
                if (p.x1bar) { st4(p.x1bar + o, r.xb0); st4(p.x1bar + o + cstride, r.xb1); st4(p.x1bar + o + 2 * cstride, r.xb2); }
                st4(p.g_out + o, r.go); st4(p.g_out + o + cstride, r.xb1); st4(p.g_out + o + 2 * cstride, r.xb2);
                red_add4(p.g_b + ob, r.dgb);
                red_add4(p.g_c + oc, r.dgc);
            }
        }
    }
    cp_async_wait_all();
}


int launch_tgv_rev_vec(const RevVecParams& p, cudaStream_t st) {
    const dim3 grid((p.W + kTgvTileW - 1) / kTgvTileW, (p.H + kTgvTileH - 1) / kTgvTileH, p.N);
    const long long ntiles = (long long)grid.x * grid.y * grid.z;
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
    if (ntiles >= rev_pipeline_min_tiles(sms) && ntiles < (1ll << 30)) {
        CNL_TRY(ensure_dynamic_smem(tgv_rev_pipe_kernel, kRevPipeSmemBytes));
        const unsigned ctas = (unsigned)std::min<long long>(ntiles, 2LL * sms);
        tgv_rev_pipe_kernel<<<ctas, kNT, kRevPipeSmemBytes, st>>>(p, (int)grid.x, (int)grid.y);
        return after_launch("tgv_rev_pipe_kernel");
    }
    constexpr int smem_bytes = 15 * kNT * (int)sizeof(float4);
    CNL_TRY(ensure_dynamic_smem(tgv_rev_vec_kernel, smem_bytes));
    tgv_rev_vec_kernel<<<grid, kNT, smem_bytes, st>>>(p);
    return after_launch("tgv_rev_vec_kernel");
}

bool tgv_vec_supported(int W, const void* const* ptrs, int nptr) {
    if (W % 4 != 0) return false;
    for (int i = 0; i < nptr; ++i)
        if ((reinterpret_cast<size_t>(ptrs[i]) & 15) != 0) return false;
    return true;
}

int launch_tgv_fwd_vec(const FwdVecParams& p, cudaStream_t st) {
    const dim3 grid((p.W + kTgvTileW - 1) / kTgvTileW, (p.H + kTgvTileH - 1) / kTgvTileH, p.N);
    const long long ntiles = (long long)grid.x * grid.y * grid.z;
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
    // the persistent kernel pays off once every CTA has a queue of tiles to overlap (measured: 3 % faster at 15 tiles
    // per CTA, 10 % slower at 4)
    if (ntiles >= pipeline_min_tiles(sms) && ntiles < (1ll << 30)) {
        CNL_TRY(ensure_dynamic_smem(tgv_fwd_pipe_kernel, kFwdPipeSmemBytes));
        const unsigned ctas = (unsigned)std::min<long long>(ntiles, 2LL * sms);
        tgv_fwd_pipe_kernel<<<ctas, kNT, kFwdPipeSmemBytes, st>>>(p, (int)grid.x, (int)grid.y);
        return after_launch("tgv_fwd_pipe_kernel");
    }
    tgv_fwd_vec_kernel<<<grid, kNT, 0, st>>>(p);
    return after_launch("tgv_fwd_vec_kernel");
}

}  // namespace tgv
}  // namespace cnl
