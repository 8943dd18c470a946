// Register-tiled, temporally blocked TV-FISTA kernels for sm_100a (geometry: see tv_fused.cuh).
#include "tv_fused.cuh"

#include <algorithm>
#include <cstdlib>

#include "common.h"
#include "tv_tile.cuh"

namespace cnl {


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
    const size_t plane = (size_t)p.H * p.P;
    float4 c[kRows], wx[kRows], wy[kRows];
    load_maps(p, g, n, c, wx, wy);
    for (int ch = 0; ch < p.C; ++ch) {
        float4 y[kRows], x[kRows], b[kRows];
        size_t off[kRows];
#pragma unroll
        for (int r = 0; r < kRows; ++r) {
            off[r] = (n * p.C + ch) * plane + (size_t)g.gy[r] * p.P + g.gx;
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
                const float4 x05 = divergence_row_fwd(y[r], fx, fy, fx_left, fyc);
                fyc = fy;
                if (g.store[r] && p.hist[j]) st4(p.hist[j] + off[r], x05);
                prox_extrapolate_row(x05, b[r], c[r], t, x[r], y[r]);
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

// Persistent, software-pipelined variant: one CTA per SM walks over the tiles; while it iterates on one (tile, channel)
// item, the operands of the next item are already on their way into shared memory (cp.async, one private 16-byte
// slot per thread, plane and row), so the load phase of every item overlaps the arithmetic of the previous one.
constexpr int kFwdPipeSmemBytes = (2 * kWarps * 32 + 6 * kRows * kThreads) * (int)sizeof(float4);

template <int K>
__global__ void __launch_bounds__(kThreads, 1)
tv_fwd_pipe_kernel(const __grid_constant__ FwdFusedParams p, int tiles_x, int tiles_y) {
    extern __shared__ float4 smem4[];
    float4(*sh_y)[32] = reinterpret_cast<float4(*)[32]>(smem4);
    float4(*sh_f)[32] = sh_y + kWarps;
    float4* buf_item = smem4 + 2 * kWarps * 32;                 // y, x, b of the next item
    float4* buf_maps = buf_item + 3 * kRows * kThreads;         // c, wx, wy of the next tile
    const int tid = threadIdx.x;
    const int ntiles = tiles_x * tiles_y * p.N;
    const size_t plane = (size_t)p.H * p.P;

    auto issue = [&](int tile, int ch) {
        const TileCoord tc = tile_coord(tile, tiles_x, tiles_y);
        const TileGeom gg = make_geom_at<K>(tc.tx, tc.ty, p.H, p.W);
#pragma unroll
        for (int r = 0; r < kRows; ++r) {
            const size_t pix = gg.ok[r] ? (size_t)gg.gy[r] * p.P + gg.gx : 0;
            const size_t o = gg.ok[r] ? (tc.n * p.C + ch) * plane + pix : 0;
            cp_async16(buf_item + (0 * kRows + r) * kThreads + tid, p.y_in + o, gg.ok[r]);
            cp_async16(buf_item + (1 * kRows + r) * kThreads + tid, p.x_in + o, gg.ok[r]);
            cp_async16(buf_item + (2 * kRows + r) * kThreads + tid, p.b + o, gg.ok[r]);
            if (ch == 0) {
                const size_t o2 = gg.ok[r] ? tc.n * plane + pix : 0;
                cp_async16(buf_maps + (0 * kRows + r) * kThreads + tid, p.c + o2, gg.ok[r]);
                cp_async16(buf_maps + (1 * kRows + r) * kThreads + tid, p.wx + o2, gg.ok[r]);
                cp_async16(buf_maps + (2 * kRows + r) * kThreads + tid, p.wy + o2, gg.ok[r]);
            }
        }
        cp_async_commit();
    };

    int tile = blockIdx.x;
    if (tile >= ntiles) return;
    issue(tile, 0);
    for (; tile < ntiles; tile += gridDim.x) {
        const TileCoord tc = tile_coord(tile, tiles_x, tiles_y);
        const TileGeom g = make_geom_at<K>(tc.tx, tc.ty, p.H, p.W);
        float4 c[kRows], wx[kRows], wy[kRows];
        for (int ch = 0; ch < p.C; ++ch) {
            cp_async_wait_all();
            if (ch == 0) {
#pragma unroll
                for (int r = 0; r < kRows; ++r) {
                    c[r] = buf_maps[(0 * kRows + r) * kThreads + tid];
                    wx[r] = buf_maps[(1 * kRows + r) * kThreads + tid];
                    wy[r] = buf_maps[(2 * kRows + r) * kThreads + tid];
                }
                finish_maps(g, p.H, p.W, wx, wy);
            }
            float4 y[kRows], x[kRows], b[kRows];
            size_t off[kRows];
#pragma unroll
            for (int r = 0; r < kRows; ++r) {
                off[r] = (tc.n * p.C + ch) * plane + (size_t)g.gy[r] * p.P + g.gx;
                y[r] = buf_item[(0 * kRows + r) * kThreads + tid];
                x[r] = buf_item[(1 * kRows + r) * kThreads + tid];
                b[r] = buf_item[(2 * kRows + r) * kThreads + tid];
            }
            // the private slots are free again: start fetching the next item
            if (ch + 1 < p.C) issue(tile, ch + 1);
            else if (tile + gridDim.x < ntiles) issue(tile + gridDim.x, 0);
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
                float4 fxl, fyl;
                flux_row(y[kRows - 1], ybelow, wx[kRows - 1], wy[kRows - 1], fxl, fyl);
                sh_f[g.warp][g.lane] = fyl;
                __syncthreads();
                float4 fyc = (g.warp > 0) ? sh_f[g.warp - 1][g.lane] : zero4();
#pragma unroll
                for (int r = 0; r < kRows; ++r) {
                    float4 fx, fy;
                    if (r == kRows - 1) { fx = fxl; fy = fyl; }
                    else flux_row(y[r], y[r + 1], wx[r], wy[r], fx, fy);
                    const float fx_left = __shfl_up_sync(kFull, fx.w, 1);
                    const float4 x05 = divergence_row_fwd(y[r], fx, fy, fx_left, fyc);
                    fyc = fy;
                    if (g.store[r] && p.hist[j]) st4(p.hist[j] + off[r], x05);
                    prox_extrapolate_row(x05, b[r], c[r], t, x[r], y[r]);
                }
            }
#pragma unroll
            for (int r = 0; r < kRows; ++r)
                if (g.store[r]) {
                    st4(p.y_out + off[r], y[r]);
                    st4(p.x_out + off[r], x[r]);
                }
        }
    }
}

static int sm_count() {
    static int n = 0;
    if (n == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    }
    return n;
}

static bool pipeline_enabled() {
    static int v = -1;
    if (v < 0) { const char* e = std::getenv("CNL_TV_NO_PIPELINE"); v = (e && e[0] == '1') ? 0 : 1; }
    return v == 1;
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
    if (pipeline_enabled() && (long long)grid.x * grid.y * grid.z < (1ll << 30)) {
        const long long ntiles = (long long)grid.x * grid.y * grid.z;
        const unsigned ctas = (unsigned)std::min<long long>(ntiles, sm_count());
        auto go = [&](auto kern) -> int {
            CNL_TRY(ensure_dynamic_smem(kern, kFwdPipeSmemBytes));
            kern<<<ctas, kThreads, kFwdPipeSmemBytes, st>>>(p, (int)grid.x, (int)grid.y);
            return after_launch("tv_fwd_pipe_kernel");
        };
        switch (K) {
            case 1: return go(tv_fwd_pipe_kernel<1>);
            case 2: return go(tv_fwd_pipe_kernel<2>);
            case 3: return go(tv_fwd_pipe_kernel<3>);
            default: return go(tv_fwd_pipe_kernel<4>);
        }
    }
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

constexpr int kRevSmemBytes = (5 * kRows * kThreads + 3 * kWarps * 32) * (int)sizeof(float4);

template <int K>
__global__ void __launch_bounds__(kThreads, 1)
tv_rev_fused_kernel(const __grid_constant__ RevFusedParams p) {
    extern __shared__ float4 smem[];
    float4* sh_dc = smem;                                  // [kRows][kThreads] per-thread accumulators over channels
    float4* sh_dwx = sh_dc + kRows * kThreads;
    float4* sh_dwy = sh_dwx + kRows * kThreads;
    float4* sh_db = sh_dwy + kRows * kThreads;             // per channel
    float4* sh_xn = sh_db + kRows * kThreads;              // private landing slots of the prefetched pre-prox iterate
    float4(*sh_y)[32] = reinterpret_cast<float4(*)[32]>(sh_xn + kRows * kThreads);    // first rows of y
    float4(*sh_g)[32] = sh_y + kWarps;                                               // first rows of g
    float4(*sh_p)[32] = sh_g + kWarps;                                               // last-row vertical adjoint flux
    const TileGeom g = make_geom<K>(p.H, p.W);
    const size_t n = blockIdx.z;
    const size_t plane = (size_t)p.H * p.P;
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
            off[r] = (n * p.C + ch) * plane + (size_t)g.gy[r] * p.P + g.gx;
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
            if (j + 2 <= K) {
                const float* src = p.hist[j + 2 <= K ? j + 2 : K];
#pragma unroll
                for (int r = 0; r < kRows; ++r) {
                    const bool okr = g.ok[r] && src != nullptr;
                    cp_async16(sh_xn + r * kThreads + threadIdx.x, okr ? src + off[r] : p.b, okr);
                }
                cp_async_commit();
            }
            float4 y[kRows];
            if (p.ckpt[j]) {
#pragma unroll
                for (int r = 0; r < kRows; ++r) y[r] = ld4(p.ckpt[j] + off[r], g.ok[r]);
            } else {
#pragma unroll
                for (int r = 0; r < kRows; ++r) y[r] = rederive_row(xh[r], xhm[r], b[r], c[r], t);
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
                const float4 ybar = divergence_row(gq[r], p1, p2, p1_left, p2c);
                p2c = p2;
                float4 xb;
                float4 dc = sh_dc[r * kThreads + threadIdx.x];
                float4 db = sh_db[r * kThreads + threadIdx.x];
                gq[r] = reverse_row(ybar, acc[r], xh[r], b[r], c[r], t, dc, db, xb);
                sh_dc[r * kThreads + threadIdx.x] = dc;
                sh_db[r * kThreads + threadIdx.x] = db;
                if (j == K - 1 && p.x1bar != nullptr && g.store[r]) st4(p.x1bar + off[r], xb);
            }
            cp_async_wait_all();
#pragma unroll
            for (int r = 0; r < kRows; ++r) {
                xh[r] = xhm[r];
                xhm[r] = (j + 2 <= K) ? sh_xn[r * kThreads + threadIdx.x] : zero4();
            }
        }
#pragma unroll
        for (int r = 0; r < kRows; ++r) {
            if (g.store[r]) {
                st4(p.g_out + off[r], gq[r]);
                st4(p.acc_out + off[r], acc[r]);
                red_add4(p.g_b + off[r], sh_db[r * kThreads + threadIdx.x]);
            }
        }
    }
    // per-pixel gradients shared by all channels
#pragma unroll
    for (int r = 0; r < kRows; ++r) {
        if (!g.store[r]) continue;
        const size_t o = n * plane + (size_t)g.gy[r] * p.P + g.gx;
        const float4 dc = sh_dc[r * kThreads + threadIdx.x];
        float4 ax = sh_dwx[r * kThreads + threadIdx.x];
        float4 ay = sh_dwy[r * kThreads + threadIdx.x];
        const int last = p.W - 1 - g.gx;          // no edge leaves the last column / last row
        if (last == 0) ax.x = 0.f;
        if (last == 1) ax.y = 0.f;
        if (last == 2) ax.z = 0.f;
        if (last == 3) ax.w = 0.f;
        if (g.gy[r] == p.H - 1) ay = zero4();
        red_add4(p.g_c + o, dc);
        red_add4(p.g_wx + o, ax);
        red_add4(p.g_wy + o, ay);
    }
}


int launch_tv_rev_fused(const RevFusedParams& p, int K, cudaStream_t st) {
    if (K < 1 || K > kFuseMax) return fail(CNL_ERR_BAD_OPTION, "fuse factor %d is outside 1..%d", K, kFuseMax);
    const int TH = kRegionH - 2 * K;
    const dim3 grid((p.W + kTileW - 1) / kTileW, (p.H + TH - 1) / TH, p.N);
    auto go = [&](auto kern) -> int {
        CNL_TRY(ensure_dynamic_smem(kern, kRevSmemBytes));
        kern<<<grid, kThreads, kRevSmemBytes, st>>>(p);
        return CNL_OK;
    };
    switch (K) {
        case 1: CNL_TRY(go(tv_rev_fused_kernel<1>)); break;
        case 2: CNL_TRY(go(tv_rev_fused_kernel<2>)); break;
        case 3: CNL_TRY(go(tv_rev_fused_kernel<3>)); break;
        default: CNL_TRY(go(tv_rev_fused_kernel<4>)); break;
    }
    return after_launch("tv_rev_fused_kernel");
}

}  // namespace cnl
