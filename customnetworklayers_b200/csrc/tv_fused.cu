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

// Per-step inputs of a launch that fuses K reverse iterations: straight from the launch parameters.
template <int K>
struct FusedSteps {
    const RevFusedParams& p;
    __device__ __forceinline__ const float* hist(int j) const { return p.hist[j]; }
    __device__ __forceinline__ const float* ckpt(int j) const { return p.ckpt[j]; }
    __device__ __forceinline__ float t(int j) const { return p.t[j]; }
    __device__ __forceinline__ constexpr bool active(int) const { return true; }
    __device__ __forceinline__ constexpr bool last(int j) const { return j == K - 1; }     // the driver passes x1bar only in the sweep's last launch
};

template <int K>
__global__ void __launch_bounds__(kThreads, 1)
tv_rev_fused_kernel(const __grid_constant__ RevFusedParams p) {
    extern __shared__ float4 smem[];
    const RevSmem sh = rev_smem(smem);
    const TileGeom g = make_geom<K>(p.H, p.W);
    const size_t n = blockIdx.z;
    const size_t plane = (size_t)p.H * p.P;
    float4 c[kRows], wx[kRows], wy[kRows];
    load_maps(p, g, n, c, wx, wy);
    rev_tile_begin(sh, c);
    const FusedSteps<K> steps{p};
    for (int ch = 0; ch < p.C; ++ch) {
        size_t off[kRows];
#pragma unroll
        for (int r = 0; r < kRows; ++r) off[r] = (n * p.C + ch) * plane + (size_t)g.gy[r] * p.P + g.gx;
        rev_channel<K, false>(sh, g, off, p.g_in, p.acc_in, p.b, p.g_out, p.acc_out, p.g_b, p.x1bar, c, wx, wy, steps, [](int) {});
    }
    rev_tile_end(sh, p, g, n);
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
