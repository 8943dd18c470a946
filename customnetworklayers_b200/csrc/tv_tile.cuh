// Device-side building blocks of the register-tiled TV-FISTA kernels: tile geometry, vector loads and stores,
// cp.async slots, and the per-row arithmetic of the forward and the reverse iteration.  Included by the kernels'
// translation units only; everything is force-inlined or constexpr.
#pragma once
#include "tv_fused.cuh"
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

// 16-byte asynchronous global->shared copy; with ok == false nothing is read and the destination is zero-filled.
__device__ __forceinline__ void cp_async16(float4* smem_dst, const float* gsrc, bool ok) {
    const unsigned dst = (unsigned)__cvta_generic_to_shared(smem_dst);
    const int bytes = ok ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(gsrc), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// Fire-and-forget vector accumulation into global memory: the addition happens in L2, so no load round trip is
// exposed to the SM.  Each address is touched by exactly one thread per launch, which keeps the sum order fixed.
__device__ __forceinline__ void red_add4(float* p, const float4& v) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}

__device__ __forceinline__ float2 lo2(const float4& v) { return make_float2(v.x, v.y); }
__device__ __forceinline__ float2 hi2(const float4& v) { return make_float2(v.z, v.w); }
__device__ __forceinline__ float4 join4(float2 a, float2 b) { return make_float4(a.x, a.y, b.x, b.y); }

// v - f1 - f2 + f1[left neighbour] + f2[row above] in packed fp32x2 arithmetic (reverse sweep)
__device__ __forceinline__ float4 divergence_row(const float4& v, const float4& f1, const float4& f2v, float f1_left,
                                                 const float4& f2_above) {
    float2 a = add2(sub2(sub2(lo2(v), lo2(f1)), lo2(f2v)), lo2(f2_above));
    float2 b = add2(sub2(sub2(hi2(v), hi2(f1)), hi2(f2v)), hi2(f2_above));
    a.x += f1_left; a.y += f1.x;
    b.x += f1.y;    b.y += f1.z;
    return join4(a, b);
}

// Forward-sweep helpers.  Plain fp32 here: the packed fp32x2 forms that the reverse sweep uses measured 3 % slower
// in the forward kernel.
// Fluxes of the forward-difference triangle anchored at a pixel (c = centre, r = right, d = below).
__device__ __forceinline__ void tri_flux_fast(float yc, float yr, float yd, float wx, float wy, float& fx, float& fy) {
    const float wd1 = wx * (yc - yr);
    const float wd2 = wy * (yc - yd);
    const float A = fmaf(wd1, yc - yr, wd2 * (yc - yd));
    const float s = fminf(1.0f, kDelta * rsqrt_approx(A));
    fx = s * wd1;
    fy = s * wd2;
}
// Fluxes of the four triangles anchored at one lane's pixels of a row; `yd` is the row below.
__device__ __forceinline__ void flux_row(const float4& y, const float4& yd, const float4& wx, const float4& wy,
                                         float4& fx, float4& fy) {
    const float yr3 = __shfl_down_sync(kFull, y.x, 1);
    tri_flux_fast(y.x, y.y, yd.x, wx.x, wy.x, fx.x, fy.x);
    tri_flux_fast(y.y, y.z, yd.y, wx.y, wy.y, fx.y, fy.y);
    tri_flux_fast(y.z, y.w, yd.z, wx.z, wy.z, fx.z, fy.z);
    tri_flux_fast(y.w, yr3, yd.w, wx.w, wy.w, fx.w, fy.w);
}
// v - f1 - f2 + f1[left neighbour] + f2[row above]
__device__ __forceinline__ float4 divergence_row_fwd(const float4& v, const float4& f1, const float4& f2v, float f1_left,
                                                     const float4& f2_above) {
    float4 o;
    o.x = v.x - f1.x - f2v.x + f1_left + f2_above.x;
    o.y = v.y - f1.y - f2v.y + f1.x + f2_above.y;
    o.z = v.z - f1.z - f2v.z + f1.y + f2_above.z;
    o.w = v.w - f1.w - f2v.w + f1.z + f2_above.w;
    return o;
}
// Huber data prox of one pixel
__device__ __forceinline__ float prox_point(float x05, float b, float c) {
    float x = fmaf(c, b, x05) * rcp_approx(1.0f + c);
    const float lo = x05 - c, hi = x05 + c;
    if (lo > 1.0f + b) x = lo;
    if (hi < b - 1.0f) x = hi;
    return x;
}
// the same with 1/(1+c) supplied (it is the same in every iteration of a tile)
__device__ __forceinline__ float prox_point_inv(float x05, float b, float c, float inv) {
    float x = fmaf(c, b, x05) * inv;
    const float lo = x05 - c, hi = x05 + c;
    if (lo > 1.0f + b) x = lo;
    if (hi < b - 1.0f) x = hi;
    return x;
}
__device__ __forceinline__ void prox_extrapolate_row_inv(const float4& x05, const float4& b, const float4& c, const float4& inv,
                                                         float t, float4& x, float4& y) {
    float4 xn;
    xn.x = prox_point_inv(x05.x, b.x, c.x, inv.x);
    xn.y = prox_point_inv(x05.y, b.y, c.y, inv.y);
    xn.z = prox_point_inv(x05.z, b.z, c.z, inv.z);
    xn.w = prox_point_inv(x05.w, b.w, c.w, inv.w);
    y.x = fmaf(t, xn.x - x.x, xn.x);
    y.y = fmaf(t, xn.y - x.y, xn.y);
    y.z = fmaf(t, xn.z - x.z, xn.z);
    y.w = fmaf(t, xn.w - x.w, xn.w);
    x = xn;
}
// prox + momentum extrapolation of one row: updates x (primal) and y (momentum variable)
__device__ __forceinline__ void prox_extrapolate_row(const float4& x05, const float4& b, const float4& c, float t,
                                                     float4& x, float4& y) {
    float4 xn;
    xn.x = prox_point(x05.x, b.x, c.x);
    xn.y = prox_point(x05.y, b.y, c.y);
    xn.z = prox_point(x05.z, b.z, c.z);
    xn.w = prox_point(x05.w, b.w, c.w);
    y.x = fmaf(t, xn.x - x.x, xn.x);
    y.y = fmaf(t, xn.y - x.y, xn.y);
    y.z = fmaf(t, xn.z - x.z, xn.z);
    y.w = fmaf(t, xn.w - x.w, xn.w);
    x = xn;
}

struct TileGeom {
    int lane, warp;
    int gx;                 // image column of the lane's first pixel (multiple of 4, may be outside the image)
    int gy[kRows];          // image rows of the warp
    bool ok[kRows];         // the lane's vector lies inside the image
    bool store[kRows];      // ... and inside the interior this CTA writes back
};

template <int K>
__device__ __forceinline__ TileGeom make_geom_at(int tx, int ty, int H, int W);

template <int K>
__device__ __forceinline__ TileGeom make_geom(int H, int W) {
    return make_geom_at<K>(blockIdx.x, blockIdx.y, H, W);
}

template <int K>
__device__ __forceinline__ TileGeom make_geom_at(int tx, int ty, int H, int W) {
    TileGeom g;
    g.lane = threadIdx.x & 31;
    g.warp = threadIdx.x >> 5;
    constexpr int TH = kRegionH - 2 * K;
    g.gx = tx * kTileW - kHaloX + 4 * g.lane;
    const bool col_ok = g.gx >= 0 && g.gx < W;
    const bool col_int = g.lane >= 1 && g.lane <= 30;
#pragma unroll
    for (int r = 0; r < kRows; ++r) {
        const int lr = g.warp * kRows + r;
        g.gy[r] = ty * TH - K + lr;
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
    const size_t plane = (size_t)p.H * p.P;
#pragma unroll
    for (int r = 0; r < kRows; ++r) {
        const size_t o = n * plane + (size_t)g.gy[r] * p.P + g.gx;
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

// Scales / masks edge weights that were fetched raw (see load_maps).
__device__ __forceinline__ void finish_maps(const TileGeom& g, int H, int W, float4 (&wx)[kRows], float4 (&wy)[kRows]) {
#pragma unroll
    for (int r = 0; r < kRows; ++r) {
        const int last = W - 1 - g.gx;
        wx[r].x = (last == 0) ? 0.f : kLip * wx[r].x;
        wx[r].y = (last == 1) ? 0.f : kLip * wx[r].y;
        wx[r].z = (last == 2) ? 0.f : kLip * wx[r].z;
        wx[r].w = (last == 3) ? 0.f : kLip * wx[r].w;
        const float sy = (g.gy[r] == H - 1) ? 0.f : kLip;
        wy[r].x *= sy; wy[r].y *= sy; wy[r].z *= sy; wy[r].w *= sy;
    }
}

struct TileCoord {
    int tx, ty;
    size_t n;
};
__device__ __forceinline__ TileCoord tile_coord(int tile, int tiles_x, int tiles_y) {
    TileCoord t;
    t.tx = tile % tiles_x;
    const int q = tile / tiles_x;
    t.ty = q % tiles_y;
    t.n = (size_t)(q / tiles_y);
    return t;
}

// ---- reverse sweep ---------------------------------------------------------------------------------------------

__device__ __forceinline__ float xor_sign(float v, float s) {          // v with its sign flipped where s is negative
    return __int_as_float(__float_as_int(v) ^ (__float_as_int(s) & 0x80000000));
}

// Adjoint fluxes of the four triangles anchored at one lane's pixels of a row; their edge-weight gradients are added
// (without the factor -kLocalGX) to awx, awy.
__device__ __forceinline__ void adjoint_row(const float4& y, const float4& yd, const float4& g, const float4& gd,
                                            const float4& wx, const float4& wy, float4& p1, float4& p2,
                                            float4& awx, float4& awy) {
    const float yr3 = __shfl_down_sync(kFull, y.x, 1);
    const float gr3 = __shfl_down_sync(kFull, g.x, 1);
    const float2 d1a = make_float2(y.x - y.y, y.y - y.z), d1b = make_float2(y.z - y.w, y.w - yr3);
    const float2 e1a = make_float2(g.x - g.y, g.y - g.z), e1b = make_float2(g.z - g.w, g.w - gr3);
    const float2 d2a = sub2(lo2(y), lo2(yd)), d2b = sub2(hi2(y), hi2(yd));
    const float2 e2a = sub2(lo2(g), lo2(gd)), e2b = sub2(hi2(g), hi2(gd));
    float2 p1a, p2a, p1b, p2b, ax = lo2(awx), ay = lo2(awy), bx = hi2(awx), by = hi2(awy);
    tri_adjoint2_acc(d1a, d2a, e1a, e2a, lo2(wx), lo2(wy), p1a, p2a, ax, ay);
    tri_adjoint2_acc(d1b, d2b, e1b, e2b, hi2(wx), hi2(wy), p1b, p2b, bx, by);
    p1 = join4(p1a, p1b);
    p2 = join4(p2a, p2b);
    awx = join4(ax, bx);
    awy = join4(ay, by);
}

// y_{g+1} of one row rebuilt from two stored pre-prox iterates
__device__ __forceinline__ float4 rederive_row(const float4& xh, const float4& xhm, const float4& b, const float4& c,
                                               const float4& inv, float t) {
    return join4(rederive_y2i(lo2(xh), lo2(xhm), lo2(b), lo2(c), lo2(inv), t),
                 rederive_y2i(hi2(xh), hi2(xhm), hi2(b), hi2(c), hi2(inv), t));
}

// momentum reverse + prox Jacobian of one row; returns dL/dx^{g+1/2}; agc, agb accumulate without constant factors
__device__ __forceinline__ float4 reverse_row(const float4& ybar, float4& acc, const float4& xh, const float4& b,
                                              const float4& c, const float4& inv, float t, float4& agc, float4& agb,
                                              float4& xbar) {
    float2 acca = lo2(acc), accb = hi2(acc), dca = lo2(agc), dcb = hi2(agc), dba = lo2(agb), dbb = hi2(agb), xa, xb;
    const float2 ga = reverse_point2i(lo2(ybar), acca, lo2(xh), lo2(b), lo2(c), lo2(inv), t, dca, dba, xa);
    const float2 gb = reverse_point2i(hi2(ybar), accb, hi2(xh), hi2(b), hi2(c), hi2(inv), t, dcb, dbb, xb);
    acc = join4(acca, accb);
    agc = join4(dca, dcb);
    agb = join4(dba, dbb);
    xbar = join4(xa, xb);
    return join4(ga, gb);
}

// Shared-memory layout of a reverse CTA: per-thread slots (one float4 per thread and row) for the gradient
// accumulators, the prefetched iterate and 1/(1+c), then the rows the warps exchange.
constexpr int kRevSlots = 6;
constexpr int kRevSmemBytes = (kRevSlots * kRows * kThreads + 3 * kWarps * 32) * (int)sizeof(float4);
struct RevSmem {
    float4* dc;       // accumulated over steps and channels (factor kLocalGC pending)
    float4* dwx;      // ... (factor -kLocalGX pending)
    float4* dwy;
    float4* db;       // accumulated over the steps of one channel (factor c kLocalGB pending)
    float4* xn;       // landing slots of the prefetched pre-prox iterate
    float4* inv;      // 1 / (1 + c)
    float4 (*y)[32];  // first rows of y
    float4 (*g)[32];  // first rows of g
    float4 (*p)[32];  // last-row vertical adjoint flux
};
__device__ __forceinline__ RevSmem rev_smem(float4* base) {
    RevSmem s;
    s.dc = base;
    s.dwx = s.dc + kRows * kThreads;
    s.dwy = s.dwx + kRows * kThreads;
    s.db = s.dwy + kRows * kThreads;
    s.xn = s.db + kRows * kThreads;
    s.inv = s.xn + kRows * kThreads;
    s.y = reinterpret_cast<float4(*)[32]>(s.inv + kRows * kThreads);
    s.g = s.y + kWarps;
    s.p = s.g + kWarps;
    return s;
}

// Start of a tile: clears the accumulators shared by its channels and stores 1/(1+c).
__device__ __forceinline__ void rev_tile_begin(const RevSmem& sh, const float4 (&c)[kRows]) {
#pragma unroll
    for (int r = 0; r < kRows; ++r) {
        const int s = r * kThreads + threadIdx.x;
        sh.dc[s] = zero4();
        sh.dwx[s] = zero4();
        sh.dwy[s] = zero4();
        sh.inv[s] = make_float4(rcp_approx(1.0f + c[r].x), rcp_approx(1.0f + c[r].y), rcp_approx(1.0f + c[r].z),
                                rcp_approx(1.0f + c[r].w));
    }
}

// End of a tile: the per-pixel gradients shared by all channels leave through reductions in L2.
template <typename P>
__device__ __forceinline__ void rev_tile_end(const RevSmem& sh, const P& p, const TileGeom& g, size_t n) {
    const size_t plane = (size_t)p.H * p.P;
#pragma unroll
    for (int r = 0; r < kRows; ++r) {
        if (!g.store[r]) continue;
        const int s = r * kThreads + threadIdx.x;
        const size_t o = n * plane + (size_t)g.gy[r] * p.P + g.gx;
        float4 dc = sh.dc[s], ax = sh.dwx[s], ay = sh.dwy[s];
        dc.x *= kLocalGC; dc.y *= kLocalGC; dc.z *= kLocalGC; dc.w *= kLocalGC;
        const int last = p.W - 1 - g.gx;          // no edge leaves the last column / last row
        ax.x = (last == 0) ? 0.f : -kLocalGX * ax.x;
        ax.y = (last == 1) ? 0.f : -kLocalGX * ax.y;
        ax.z = (last == 2) ? 0.f : -kLocalGX * ax.z;
        ax.w = (last == 3) ? 0.f : -kLocalGX * ax.w;
        const float sy = (g.gy[r] == p.H - 1) ? 0.f : -kLocalGX;
        ay.x *= sy; ay.y *= sy; ay.z *= sy; ay.w *= sy;
        red_add4(p.g_c + o, dc);
        red_add4(p.g_wx + o, ax);
        red_add4(p.g_wy + o, ay);
    }
}

// K reverse steps of one channel of one tile.  `st` supplies, per fused step j, the stored iterate hist(j) (j = 0..K;
// null where there is none), the checkpointed y ckpt(j) (null: y is rebuilt), the momentum factor t(j), whether the step
// exists at all (active(j): the last time block of a sweep may be shorter than K) and whether it is the sweep's last
// one (last(j): dL/dx of that step is the init gradient).
// kCoherent: g_in / acc_in are written by other CTAs of the same launch and must come from L2.
// `hook(j)` runs in every thread right after the first barrier of step j (the single-launch sweep publishes there).
template <int K, bool kCoherent, typename Steps, typename Hook>
__device__ __forceinline__ void rev_channel(const RevSmem& sh, const TileGeom& g, const size_t (&off)[kRows],
                                            const float* g_in, const float* acc_in, const float* b_in, float* g_out,
                                            float* acc_out, float* g_b, float* x1bar, const float4 (&c)[kRows],
                                            const float4 (&wx)[kRows], const float4 (&wy)[kRows], const Steps& st,
                                            Hook hook) {
    const int tid = threadIdx.x;
    float4 gq[kRows], acc[kRows], b[kRows], xh[kRows], xhm[kRows];
    {
        const float* h0 = st.hist(0);
        const float* h1 = st.hist(1);
#pragma unroll
        for (int r = 0; r < kRows; ++r) {
            if (kCoherent) {
                gq[r] = g.ok[r] ? __ldcg(reinterpret_cast<const float4*>(g_in + off[r])) : zero4();
                acc[r] = g.ok[r] ? __ldcg(reinterpret_cast<const float4*>(acc_in + off[r])) : zero4();
            } else {
                gq[r] = ld4(g_in + off[r], g.ok[r]);
                acc[r] = ld4(acc_in + off[r], g.ok[r]);
            }
            b[r] = ld4(b_in + off[r], g.ok[r]);
            xh[r] = ld4(h0 + off[r], g.ok[r]);
            xhm[r] = ld4(h1 + off[r], g.ok[r] && h1 != nullptr);
            sh.db[r * kThreads + tid] = zero4();
        }
    }
#pragma unroll
    for (int j = 0; j < K; ++j) {
        if (!st.active(j)) continue;         // uniform over the CTA: the barriers below are skipped by all or none
        const float t = st.t(j);
        // prefetch the pre-prox iterate the next fused step needs
        if (j + 2 <= K) {
            const float* src = st.hist(j + 2);
#pragma unroll
            for (int r = 0; r < kRows; ++r) {
                const bool okr = g.ok[r] && src != nullptr;
                cp_async16(sh.xn + r * kThreads + tid, okr ? src + off[r] : b_in, okr);
            }
            cp_async_commit();
        }
        float4 y[kRows];
        const float* ck = st.ckpt(j);
        if (ck != nullptr) {
#pragma unroll
            for (int r = 0; r < kRows; ++r) y[r] = ld4(ck + off[r], g.ok[r]);
        } else {
#pragma unroll
            for (int r = 0; r < kRows; ++r) y[r] = rederive_row(xh[r], xhm[r], b[r], c[r], sh.inv[r * kThreads + tid], t);
        }
        sh.y[g.warp][g.lane] = y[0];
        sh.g[g.warp][g.lane] = gq[0];
        __syncthreads();
        hook(j);
        const bool has_below = g.warp + 1 < kWarps;
        const float4 ybelow = has_below ? sh.y[g.warp + 1][g.lane] : zero4();
        const float4 gbelow = has_below ? sh.g[g.warp + 1][g.lane] : zero4();
        float4 p1l, p2l;
        {
            float4 ax = sh.dwx[(kRows - 1) * kThreads + tid], ay = sh.dwy[(kRows - 1) * kThreads + tid];
            adjoint_row(y[kRows - 1], ybelow, gq[kRows - 1], gbelow, wx[kRows - 1], wy[kRows - 1], p1l, p2l, ax, ay);
            sh.dwx[(kRows - 1) * kThreads + tid] = ax;
            sh.dwy[(kRows - 1) * kThreads + tid] = ay;
        }
        sh.p[g.warp][g.lane] = p2l;
        __syncthreads();
        float4 p2c = (g.warp > 0) ? sh.p[g.warp - 1][g.lane] : zero4();
#pragma unroll
        for (int r = 0; r < kRows; ++r) {
            float4 p1, p2;
            if (r == kRows - 1) { p1 = p1l; p2 = p2l; }
            else {
                float4 ax = sh.dwx[r * kThreads + tid], ay = sh.dwy[r * kThreads + tid];
                adjoint_row(y[r], y[r + 1], gq[r], gq[r + 1], wx[r], wy[r], p1, p2, ax, ay);
                sh.dwx[r * kThreads + tid] = ax;
                sh.dwy[r * kThreads + tid] = ay;
            }
            const float p1_left = __shfl_up_sync(kFull, p1.w, 1);
            const float4 ybar = divergence_row(gq[r], p1, p2, p1_left, p2c);
            p2c = p2;
            float4 xb;
            float4 dc = sh.dc[r * kThreads + tid];
            float4 db = sh.db[r * kThreads + tid];
            gq[r] = reverse_row(ybar, acc[r], xh[r], b[r], c[r], sh.inv[r * kThreads + tid], t, dc, db, xb);
            sh.dc[r * kThreads + tid] = dc;
            sh.db[r * kThreads + tid] = db;
            if (st.last(j) && x1bar != nullptr && g.store[r]) st4(x1bar + off[r], xb);
        }
        cp_async_wait_all();
#pragma unroll
        for (int r = 0; r < kRows; ++r) {
            xh[r] = xhm[r];
            xhm[r] = (j + 2 <= K) ? sh.xn[r * kThreads + tid] : zero4();
        }
    }
#pragma unroll
    for (int r = 0; r < kRows; ++r) {
        if (g.store[r]) {
            st4(g_out + off[r], gq[r]);
            st4(acc_out + off[r], acc[r]);
            float4 db = sh.db[r * kThreads + tid];          // sum of xi over the quadratic-zone steps: times c kLocalGB
            db.x *= c[r].x * kLocalGB; db.y *= c[r].y * kLocalGB; db.z *= c[r].z * kLocalGB; db.w *= c[r].w * kLocalGB;
            red_add4(g_b + off[r], db);
        }
    }
}

}  // namespace
}  // namespace cnl
