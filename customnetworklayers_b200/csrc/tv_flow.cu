// Single-launch sweeps of the temporally blocked TV-FISTA kernels: tile-level dataflow instead of one launch per K
// iterations.
//
// One persistent CTA per SM walks over work units in time-block-major order (unit index = time block * units per
// block + position).  A unit of time block kb needs the 3 x 3 neighbourhood of its tile to have finished time block
// kb - 1; each tile has a counter in global memory that its units bump when their results are visible, and a unit
// starts (or is prefetched) once the nine counters around it have reached kb.  Nothing else orders the CTAs: no
// grid-wide barrier, no launch boundary between time blocks, no tail of idle SMs at the end of every block.  Units are
// dealt round-robin, every CTA takes its units in increasing order and a unit only ever waits for units with smaller
// indices, so the unit with the smallest unfinished index can always run; the launch is cooperative, which makes the
// driver refuse it rather than run it if the CTAs could not all be resident.  Every wait is bounded: after
// kSpinLimit polls a CTA raises the abort word, the other CTAs leave at their next poll, and the host finds the reason
// in a status word in pinned host memory at its next call.
//
// Buffers that change during the launch (the ping-pong iterates) are read with cp.async.cg / ld.global.cg, i.e. from
// L2, never through the non-coherent path.
#include <algorithm>
#include <climits>
#include <cstdlib>
#include <mutex>

#include "common.h"
#include "tv_tile.cuh"

namespace cnl {

namespace {

constexpr long long kSpinLimit = 1ll << 21;       // polls of ~0.5 us or more each: about a second before a wait gives up

struct FlowSync {
    int* progress;      // per tile: time blocks completed so far
    int* abort;         // device word: non-zero tells every CTA to leave
    int* status;        // host-mapped word the host reads at its next call
};

__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ int ld_relaxed_gpu(const int* p) {
    int v;
    asm volatile("ld.relaxed.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// Publishes a finished unit: called by ONE thread after a CTA barrier that follows every thread's stores.  The release
// at device scope is cumulative over that barrier, so all of the CTA's writes are visible to whoever acquires the counter.
__device__ __forceinline__ void red_release_gpu(int* p, int v) {
    asm volatile("red.release.gpu.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Address of the progress counter this lane watches: lanes 0..8 take the 3 x 3 tiles around (tx, ty) of image n;
// `valid` is false for lanes beyond 8 and for neighbours outside the image.
__device__ __forceinline__ const int* neighbour_counter(const int* progress, const TileCoord& tc, int tiles_x, int tiles_y,
                                                        bool& valid) {
    const int lane = threadIdx.x & 31;
    const int nx = tc.tx + lane % 3 - 1, ny = tc.ty + (lane / 3) % 3 - 1;
    valid = lane < 9 && nx >= 0 && nx < tiles_x && ny >= 0 && ny < tiles_y;
    return progress + ((size_t)tc.n * tiles_y + (valid ? ny : tc.ty)) * tiles_x + (valid ? nx : tc.tx);
}

// Whole warp: waits until the tiles around `tc` have each completed `need` time blocks.  Returns 1 when they have,
// 0 when the wait was given up (abort word set by this or another CTA).
__device__ __forceinline__ int flow_wait(const FlowSync& s, const TileCoord& tc, int tiles_x, int tiles_y, int need) {
    if (need <= 0) return 1;
    bool valid;
    const int* addr = neighbour_counter(s.progress, tc, tiles_x, tiles_y, valid);
    for (long long spin = 0;; ++spin) {
        const bool ok = !valid || ld_acquire_gpu(addr) >= need;
        if (__all_sync(kFull, ok)) return 1;
        if ((spin & 63) == 63) {
            int ab = ld_relaxed_gpu(s.abort);
            ab = __shfl_sync(kFull, ab, 0);
            if (ab != 0 || spin >= kSpinLimit) {
                if ((threadIdx.x & 31) == 0) {
                    atomicExch(s.abort, 1);
                    if (ab == 0) {                       // this CTA is the one whose wait ran out
                        *reinterpret_cast<volatile int*>(s.status) = 1;
                        __threadfence_system();
                    }
                }
                return 0;
            }
        }
        __nanosleep(64);
    }
}

// A work unit: one tile (all its channels, in turn) in one time block.
struct Unit {
    int kb, tile;
    TileCoord tc;
};
__device__ __forceinline__ Unit decode_unit(int u, int ntiles, int tiles_x, int tiles_y) {
    Unit q;
    q.kb = u / ntiles;
    q.tile = u - q.kb * ntiles;
    q.tc = tile_coord(q.tile, tiles_x, tiles_y);
    return q;
}

}  // namespace

// ---------------------------------------------------------------------------------------------------------------
// forward sweep: p.nblocks time blocks of K iterations in one launch
// ---------------------------------------------------------------------------------------------------------------
constexpr int kFwdFlowSmemBytes = (2 * kWarps * 32 + 7 * kRows * kThreads) * (int)sizeof(float4);

// kShort: the sweep's last time block has fewer than K iterations (the iteration count is not a multiple of K).
template <int K, bool kShort>
__global__ void __launch_bounds__(kThreads, 1)
tv_fwd_flow_kernel(const __grid_constant__ FwdFlowParams p, int tiles_x, int tiles_y) {
    extern __shared__ float4 smem4[];
    __shared__ int sh_ctl[2];
    float4(*sh_y)[32] = reinterpret_cast<float4(*)[32]>(smem4);
    float4(*sh_f)[32] = sh_y + kWarps;
    float4* buf_item = smem4 + 2 * kWarps * 32;                 // y, x, b of the next (unit, channel)
    float4* buf_maps = buf_item + 3 * kRows * kThreads;         // c, wx, wy of the next unit
    float4* sh_inv = buf_maps + 3 * kRows * kThreads;           // 1 / (1 + c) of the current unit, one slot per thread and row
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int ntiles = tiles_x * tiles_y * p.N;
    const int total = ntiles * p.nblocks;
    const size_t plane = (size_t)p.H * p.P;
    const FlowSync sync{p.progress, p.abort, p.status};

    auto issue = [&](const Unit& q, int ch, bool maps) {
        const TileGeom gg = make_geom_at<K>(q.tc.tx, q.tc.ty, p.H, p.W);
        const float* y_in = q.kb == 0 ? p.init : p.ybuf[(q.kb - 1) & 1];
        const float* x_in = q.kb == 0 ? p.init : p.xbuf[(q.kb - 1) & 1];
#pragma unroll
        for (int r = 0; r < kRows; ++r) {
            const size_t pix = gg.ok[r] ? (size_t)gg.gy[r] * p.P + gg.gx : 0;
            const size_t o = gg.ok[r] ? (q.tc.n * p.C + ch) * plane + pix : 0;
            cp_async16(buf_item + (0 * kRows + r) * kThreads + tid, y_in + o, gg.ok[r]);
            cp_async16(buf_item + (1 * kRows + r) * kThreads + tid, x_in + o, gg.ok[r]);
            cp_async16(buf_item + (2 * kRows + r) * kThreads + tid, p.b + o, gg.ok[r]);
            if (maps) {
                const size_t o2 = gg.ok[r] ? q.tc.n * plane + pix : 0;
                cp_async16(buf_maps + (0 * kRows + r) * kThreads + tid, p.c + o2, gg.ok[r]);
                cp_async16(buf_maps + (1 * kRows + r) * kThreads + tid, p.wx + o2, gg.ok[r]);
                cp_async16(buf_maps + (2 * kRows + r) * kThreads + tid, p.wy + o2, gg.ok[r]);
            }
        }
        cp_async_commit();
    };

    int u = blockIdx.x;
    if (u >= total) return;
    Unit cur = decode_unit(u, ntiles, tiles_x, tiles_y);
    if (warp == 0) {
        const int ok = flow_wait(sync, cur.tc, tiles_x, tiles_y, cur.kb);
        if (lane == 0) sh_ctl[0] = ok;
    }
    __syncthreads();
    if (!sh_ctl[0]) return;
    issue(cur, 0, true);
    for (;;) {
        const int un = u + (int)gridDim.x;
        const bool has_next = un < total;
        const Unit nxt = has_next ? decode_unit(un, ntiles, tiles_x, tiles_y) : cur;
        const TileGeom g = make_geom_at<K>(cur.tc.tx, cur.tc.ty, p.H, p.W);
        float* const y_out = p.ybuf[cur.kb & 1];
        float* const x_out = p.xbuf[cur.kb & 1];
        const int g0 = cur.kb * K;
        float4 c[kRows], wx[kRows], wy[kRows];
        // Is the CTA's next unit ready?  Warp 0 fetches the counters of its neighbourhood (acquire loads) at the start of
        // the unit's last channel and looks at them before the second barrier of the first fused step, so that the round
        // trip to L2 hides behind the arithmetic in between.  (A relaxed load followed by a fence costs 6 % of the sweep:
        // the fence waits for the stores the whole CTA has in flight.)
        bool next_issued = false;
        for (int ch = 0; ch < p.C; ++ch) {
            const bool last_ch = ch + 1 == p.C;
            int seen = INT_MAX;
            if (last_ch && has_next && warp == 0 && nxt.kb > 0) {
                bool valid;
                const int* addr = neighbour_counter(sync.progress, nxt.tc, tiles_x, tiles_y, valid);
                if (valid) seen = ld_acquire_gpu(addr);
            }
            cp_async_wait_all();
            if (ch == 0) {
#pragma unroll
                for (int r = 0; r < kRows; ++r) {
                    c[r] = buf_maps[(0 * kRows + r) * kThreads + tid];
                    wx[r] = buf_maps[(1 * kRows + r) * kThreads + tid];
                    wy[r] = buf_maps[(2 * kRows + r) * kThreads + tid];
                }
                finish_maps(g, p.H, p.W, wx, wy);
#pragma unroll
                for (int r = 0; r < kRows; ++r)
                    sh_inv[r * kThreads + tid] = make_float4(rcp_approx(1.0f + c[r].x), rcp_approx(1.0f + c[r].y),
                                                             rcp_approx(1.0f + c[r].z), rcp_approx(1.0f + c[r].w));
            }
            float4 y[kRows], x[kRows], b[kRows];
            size_t off[kRows];
#pragma unroll
            for (int r = 0; r < kRows; ++r) {
                off[r] = (cur.tc.n * p.C + ch) * plane + (size_t)g.gy[r] * p.P + g.gx;
                y[r] = buf_item[(0 * kRows + r) * kThreads + tid];
                x[r] = buf_item[(1 * kRows + r) * kThreads + tid];
                b[r] = buf_item[(2 * kRows + r) * kThreads + tid];
            }
            // the private slots are free again: the next channel of this unit can be fetched right away
            if (!last_ch) issue(cur, ch + 1, false);
#pragma unroll
            for (int j = 0; j < K; ++j) {
                if (kShort && g0 + j >= p.its) continue;       // a shorter last time block; uniform over the CTA
                const float t = p.tab.t[g0 + j];
                const int slot = p.tab.ckpt_slot[g0 + j];
                sh_y[g.warp][g.lane] = y[0];
                __syncthreads();
                const float4 ybelow = (g.warp + 1 < kWarps) ? sh_y[g.warp + 1][g.lane] : zero4();
                if (slot >= 0) {
                    float* ck = p.ckpt + (size_t)slot * p.vol;
#pragma unroll
                    for (int r = 0; r < kRows; ++r)
                        if (g.store[r]) st4(ck + off[r], y[r]);
                }
                float4 fxl, fyl;
                flux_row(y[kRows - 1], ybelow, wx[kRows - 1], wy[kRows - 1], fxl, fyl);
                sh_f[g.warp][g.lane] = fyl;
                if (j == 0 && last_ch && has_next && warp == 0) {
                    const int ok = __all_sync(kFull, seen >= nxt.kb);
                    if (lane == 0) sh_ctl[1] = ok;
                }
                __syncthreads();
                if (j == 0 && last_ch && has_next && sh_ctl[1]) {
                    issue(nxt, 0, true);
                    next_issued = true;
                }
                float4 fyc = (g.warp > 0) ? sh_f[g.warp - 1][g.lane] : zero4();
                float* const hj = p.hist + (size_t)(g0 + j) * p.vol;
#pragma unroll
                for (int r = 0; r < kRows; ++r) {
                    float4 fx, fy;
                    if (r == kRows - 1) { fx = fxl; fy = fyl; }
                    else flux_row(y[r], y[r + 1], wx[r], wy[r], fx, fy);
                    const float fx_left = __shfl_up_sync(kFull, fx.w, 1);
                    const float4 x05 = divergence_row_fwd(y[r], fx, fy, fx_left, fyc);
                    fyc = fy;
                    if (g.store[r]) st4(hj + off[r], x05);
                    prox_extrapolate_row_inv(x05, b[r], c[r], sh_inv[r * kThreads + tid], t, x[r], y[r]);
                }
            }
#pragma unroll
            for (int r = 0; r < kRows; ++r)
                if (g.store[r]) {
                    st4(y_out + off[r], y[r]);
                    st4(x_out + off[r], x[r]);
                }
        }
        // publish: the barrier orders every thread's stores before the release that moves the counter
        __syncthreads();
        if (tid == 0) red_release_gpu(p.progress + cur.tile, 1);
        if (!has_next) break;
        if (!next_issued) {
            if (warp == 0) {
                const int ok = flow_wait(sync, nxt.tc, tiles_x, tiles_y, nxt.kb);
                if (lane == 0) sh_ctl[0] = ok;
            }
            __syncthreads();
            if (!sh_ctl[0]) return;               // no copy of this thread is in flight here
            issue(nxt, 0, true);
        }
        u = un;
        cur = nxt;
    }
}

// ---------------------------------------------------------------------------------------------------------------
// reverse sweep: p.nblocks time blocks of K reverse iterations in one launch; a unit is one tile with all its channels
// ---------------------------------------------------------------------------------------------------------------
// Per-step inputs of one time block: addresses and factors follow from the iteration number.
struct FlowSteps {
    const RevFlowParams& p;
    int gfirst;                 // iteration of the block's first reverse step
    __device__ __forceinline__ const float* hist(int j) const {
        return gfirst - j >= 0 ? p.hist + (size_t)(gfirst - j) * p.vol : nullptr;
    }
    __device__ __forceinline__ const float* ckpt(int j) const {
        const int slot = p.tab.ckpt_slot[gfirst - j];
        return slot >= 0 ? p.ckpt + (size_t)slot * p.vol : nullptr;
    }
    __device__ __forceinline__ float t(int j) const { return p.tab.t[gfirst - j]; }
    __device__ __forceinline__ bool active(int j) const { return gfirst - j >= 0; }      // the last time block may be short
    __device__ __forceinline__ bool last(int j) const { return gfirst - j == 0; }
};

template <int K>
__global__ void __launch_bounds__(kThreads, 1)
tv_rev_flow_kernel(const __grid_constant__ RevFlowParams p, int tiles_x, int tiles_y) {
    extern __shared__ float4 smem[];
    __shared__ int sh_ctl[2];
    const RevSmem sh = rev_smem(smem);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ntiles = tiles_x * tiles_y * p.N;
    const int total = ntiles * p.nblocks;
    const size_t plane = (size_t)p.H * p.P;
    const FlowSync sync{p.progress, p.abort, p.status};

    // Unit-level values (time block, tile, buffer parity, ...) are recomputed from the unit index where they are needed
    // instead of being kept in registers across the fused steps, which have none to spare: `opaque` hides the index from
    // the optimiser so that it cannot hoist those computations back out.
    auto opaque = [](int v) { asm volatile("" : "+r"(v)); return v; };
    int next_ready = 0;          // the unit about to start was found ready while the previous one was still running
    for (int u = blockIdx.x; u < total; u += gridDim.x) {
        if (!next_ready) {
            if (warp == 0) {
                const int kb = u / ntiles;
                const int ok = flow_wait(sync, tile_coord(u - kb * ntiles, tiles_x, tiles_y), tiles_x, tiles_y, kb);
                if (lane == 0) sh_ctl[0] = ok;
            }
            __syncthreads();
            if (!sh_ctl[0]) return;
        }
        float4 c[kRows], wx[kRows], wy[kRows];
        {
            const int kb = u / ntiles;
            const TileCoord tc = tile_coord(u - kb * ntiles, tiles_x, tiles_y);
            const TileGeom g = make_geom_at<K>(tc.tx, tc.ty, p.H, p.W);
            load_maps(p, g, (size_t)tc.n, c, wx, wy);
        }
        rev_tile_begin(sh, c);
        int seen = INT_MAX;
        for (int ch = 0; ch < p.C; ++ch) {
            const int uo = opaque(u);
            const int kb = uo / ntiles;
            const TileCoord tc = tile_coord(uo - kb * ntiles, tiles_x, tiles_y);
            const TileGeom g = make_geom_at<K>(tc.tx, tc.ty, p.H, p.W);
            // Readiness of this CTA's next unit: its neighbours' counters are fetched at the start of the last channel and
            // looked at when the unit ends, so that the round trip to L2 costs nothing.
            if (ch + 1 == p.C && warp == 0) {
                const int un = uo + (int)gridDim.x;
                const int kb_next = un / ntiles;
                if (un < total && kb_next > 0) {
                    bool valid;
                    const int* addr = neighbour_counter(sync.progress, tile_coord(un - kb_next * ntiles, tiles_x, tiles_y),
                                                        tiles_x, tiles_y, valid);
                    if (valid) seen = ld_acquire_gpu(addr);
                }
            }
            const FlowSteps steps{p, p.g_first - K * kb};
            size_t off[kRows];
#pragma unroll
            for (int r = 0; r < kRows; ++r) off[r] = ((size_t)tc.n * p.C + ch) * plane + (size_t)g.gy[r] * p.P + g.gx;
            rev_channel<K, true>(sh, g, off, p.gbuf[(kb + 1) & 1], p.abuf[(kb + 1) & 1], p.b, p.gbuf[kb & 1], p.abuf[kb & 1],
                                 p.g_b, p.x1bar, c, wx, wy, steps, [](int) {});
        }
        const int ue = opaque(u);
        const int kbe = ue / ntiles;
        const int tile = ue - kbe * ntiles;
        {
            const TileCoord tc = tile_coord(tile, tiles_x, tiles_y);
            rev_tile_end(sh, p, make_geom_at<K>(tc.tx, tc.ty, p.H, p.W), (size_t)tc.n);
        }
        if (warp == 0) {
            const int un = ue + (int)gridDim.x;
            const int ok = un < total ? __all_sync(kFull, seen >= un / ntiles) : 0;
            if (lane == 0) sh_ctl[1] = ok;
        }
        // publish: the barrier orders every thread's stores and reductions before the release that moves the counter
        __syncthreads();
        next_ready = sh_ctl[1];
        if (threadIdx.x == 0) red_release_gpu(p.progress + tile, 1);
    }
}

// ---------------------------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------------------------
namespace {

struct FlowHost {
    int* status_host = nullptr;       // pinned, mapped
    int* status_dev = nullptr;
    int coop = -1;                    // cooperative launch supported
    int sms = 0;
};
std::mutex g_flow_mu;
FlowHost g_flow[64];

int flow_host(FlowHost** out) {
    int dev = 0;
    CNL_TRY(check_cuda(cudaGetDevice(&dev), "cudaGetDevice"));
    if (dev < 0 || dev >= 64) return fail(CNL_ERR_BAD_SHAPE, "device ordinal %d is beyond 63", dev);
    std::lock_guard<std::mutex> lock(g_flow_mu);
    FlowHost& f = g_flow[dev];
    if (f.coop < 0) {
        int coop = 0, sms = 0;
        CNL_TRY(check_cuda(cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev), "cudaDeviceGetAttribute"));
        CNL_TRY(check_cuda(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev), "cudaDeviceGetAttribute"));
        void* h = nullptr;
        CNL_TRY(check_cuda(cudaHostAlloc(&h, 64, cudaHostAllocMapped), "cudaHostAlloc (status word)"));
        void* d = nullptr;
        CNL_TRY(check_cuda(cudaHostGetDevicePointer(&d, h, 0), "cudaHostGetDevicePointer"));
        f.status_host = static_cast<int*>(h);
        f.status_dev = static_cast<int*>(d);
        *f.status_host = 0;
        f.sms = sms;
        f.coop = coop;
    }
    *out = &f;
    return CNL_OK;
}

template <typename Kern, typename Params>
int launch_flow(Kern kern, const Params& p, int smem, long long units, int tiles_x, int tiles_y, cudaStream_t st,
                const char* name) {
    FlowHost* f;
    CNL_TRY(flow_host(&f));
    CNL_TRY(ensure_dynamic_smem(kern, smem));
    const unsigned ctas = (unsigned)std::min<long long>(units, f->sms);
    void* args[] = {const_cast<Params*>(&p), &tiles_x, &tiles_y};
    CNL_TRY(check_cuda(cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(kern), dim3(ctas), dim3(kThreads), args,
                                                   (size_t)smem, st), name));
    return after_launch(name);
}

}  // namespace

bool flow_enabled() {
    static int v = -1;
    if (v < 0) {
        const char* e = std::getenv("CNL_TV_NO_FLOW");
        v = (e && e[0] == '1') ? 0 : 1;
    }
    if (v != 1) return false;
    FlowHost* f;
    if (flow_host(&f) != CNL_OK) return false;
    return f->coop == 1;
}

int flow_status_take() {
    FlowHost* f;
    CNL_TRY(flow_host(&f));
    const int v = *reinterpret_cast<volatile int*>(f->status_host);
    if (v == 0) return CNL_OK;
    *f->status_host = 0;
    return fail(CNL_ERR_CUDA, "a single-launch sweep gave up waiting for a neighbouring tile (status %d): the results of that "
                "call are invalid; set CNL_TV_NO_FLOW=1 to run one launch per time block instead", v);
}

int* flow_status_device_ptr() {
    FlowHost* f;
    if (flow_host(&f) != CNL_OK) return nullptr;
    return f->status_dev;
}

int launch_tv_fwd_flow(const FwdFlowParams& p, cudaStream_t st) {
    constexpr int K = kFuseMax;
    const int TH = kRegionH - 2 * K;
    const int tiles_x = (p.W + kTileW - 1) / kTileW, tiles_y = (p.H + TH - 1) / TH;
    const long long units = (long long)tiles_x * tiles_y * p.N * p.nblocks;
    if (units <= 0 || units >= (1ll << 30)) return fail(CNL_ERR_BAD_SHAPE, "too many work units for a single-launch sweep");
    if (p.its % K != 0)
        return launch_flow(tv_fwd_flow_kernel<K, true>, p, kFwdFlowSmemBytes, units, tiles_x, tiles_y, st, "tv_fwd_flow_kernel");
    return launch_flow(tv_fwd_flow_kernel<K, false>, p, kFwdFlowSmemBytes, units, tiles_x, tiles_y, st, "tv_fwd_flow_kernel");
}

int launch_tv_rev_flow(const RevFlowParams& p, cudaStream_t st) {
    constexpr int K = kFuseMax;
    const int TH = kRegionH - 2 * K;
    const int tiles_x = (p.W + kTileW - 1) / kTileW, tiles_y = (p.H + TH - 1) / TH;
    const long long units = (long long)tiles_x * tiles_y * p.N * p.nblocks;
    if (units <= 0 || units >= (1ll << 30)) return fail(CNL_ERR_BAD_SHAPE, "too many work units for a single-launch sweep");
    return launch_flow(tv_rev_flow_kernel<K>, p, kRevSmemBytes, units, tiles_x, tiles_y, st, "tv_rev_flow_kernel");
}

int flow_tiles(int H, int W, int N) {
    const int TH = kRegionH - 2 * kFuseMax;
    return ((W + kTileW - 1) / kTileW) * ((H + TH - 1) / TH) * N;
}

}  // namespace cnl
