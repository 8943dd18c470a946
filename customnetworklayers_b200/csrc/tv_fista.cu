// Unrolled FISTA TV-inpainting layer for sm_100a: kernels, per-id device arenas, host drivers and C entry points.
//
// Data flow (all device resident, nothing is copied to the host):
//   forward : y (ping-pong), x (= the caller's output buffer), history hist[g] = x^{g+1/2} for every iteration g,
//             and the momentum variable y_g at the reference's checkpoint iterations (needed to reproduce the
//             reference's segment-start evaluation point, cudaTV/cudaCode/TVInpaintFista.cu:1724-1727).
//   backward: walks g = last .. 0; y_{g+1} is rebuilt from hist[g], hist[g-1] like the reference does (:1130-1189);
//             per-pixel gradient accumulators live in the caller's output buffers.
#include <cooperative_groups.h>

#include <cmath>
#include <cstdlib>
#include <mutex>
#include <vector>

#include "common.h"
#include "tv_fused.cuh"
#include "tv_math.cuh"

namespace cnl {

// ---------------------------------------------------------------------------------------------------------------
// one-iteration kernels (one thread per pixel, channels looped in-thread, neighbours through L1)
// ---------------------------------------------------------------------------------------------------------------
constexpr int kBX = 32;
constexpr int kBY = 8;

struct PixelWeights {
    float wx_c, wy_c;   // triangle anchored at (h, w)
    float wx_l, wy_l;   // triangle anchored at (h, w-1)
    float wx_u, wy_u;   // triangle anchored at (h-1, w)
};

__device__ __forceinline__ PixelWeights load_weights(const float* __restrict__ wx, const float* __restrict__ wy,
                                                     int h, int w, int H, int W) {
    PixelWeights p;
    const int pix = h * W + w;
    const bool inx = w < W - 1, iny = h < H - 1;
    p.wx_c = inx ? kLip * __ldg(wx + pix) : 0.0f;
    p.wy_c = iny ? kLip * __ldg(wy + pix) : 0.0f;
    p.wx_l = (w > 0) ? kLip * __ldg(wx + pix - 1) : 0.0f;
    p.wy_l = (w > 0 && iny) ? kLip * __ldg(wy + pix - 1) : 0.0f;
    p.wx_u = (h > 0 && inx) ? kLip * __ldg(wx + pix - W) : 0.0f;
    p.wy_u = (h > 0) ? kLip * __ldg(wy + pix - W) : 0.0f;
    return p;
}

struct Stencil7 {
    float c, r, d, l, u, dl, ur;   // centre, right, down, left, up, down-left, up-right; 0 outside the image
};

__device__ __forceinline__ Stencil7 load_stencil(const float* __restrict__ a, int h, int w, int H, int W) {
    Stencil7 s;
    const int pix = h * W + w;
    const bool hr = w < W - 1, hd = h < H - 1, hl = w > 0, hu = h > 0;
    s.c = a[pix];
    s.r = hr ? a[pix + 1] : 0.0f;
    s.d = hd ? a[pix + W] : 0.0f;
    s.l = hl ? a[pix - 1] : 0.0f;
    s.u = hu ? a[pix - W] : 0.0f;
    s.dl = (hd && hl) ? a[pix + W - 1] : 0.0f;
    s.ur = (hu && hr) ? a[pix - W + 1] : 0.0f;
    return s;
}

// One FISTA iteration: gradient step on y, Huber prox, momentum extrapolation; stores x^{g+1/2}.
__global__ void __launch_bounds__(kBX* kBY)
tv_fwd_iter_kernel(const float* __restrict__ y_in, float* __restrict__ y_out, float* __restrict__ x,
                   const float* __restrict__ b, const float* __restrict__ c, const float* __restrict__ wx,
                   const float* __restrict__ wy, float* __restrict__ hist, int C, int H, int W, float t) {
    const int w = blockIdx.x * kBX + threadIdx.x;
    const int h = blockIdx.y * kBY + threadIdx.y;
    if (w >= W || h >= H) return;
    const size_t plane = (size_t)H * W;
    const size_t n = blockIdx.z;
    const int pix = h * W + w;
    const PixelWeights pw = load_weights(wx + n * plane, wy + n * plane, h, w, H, W);
    const float conf = __ldg(c + n * plane + pix);
    for (int ch = 0; ch < C; ++ch) {
        const size_t off = (n * C + ch) * plane;
        const Stencil7 y = load_stencil(y_in + off, h, w, H, W);
        float fx, fy, fxl, fyu, unused;
        tri_flux(y.c, y.r, y.d, pw.wx_c, pw.wy_c, fx, fy);
        tri_flux(y.l, y.c, y.dl, pw.wx_l, pw.wy_l, fxl, unused);
        tri_flux(y.u, y.ur, y.c, pw.wx_u, pw.wy_u, unused, fyu);
        const float x05 = y.c - fx - fy + fxl + fyu;
        const float bb = __ldg(b + off + pix);
        const float xn = prox_huber(x05, bb, conf);
        const float xp = x[off + pix];
        hist[off + pix] = x05;
        x[off + pix] = xn;
        y_out[off + pix] = xn + t * (xn - xp);
    }
}

// Seeds the reverse sweep at the last iteration (TVInpaintFista.cu:222-287): prox Jacobian on the upstream gradient.
// Also clears what the sweep accumulates into (the pending momentum term, the two edge-weight gradients) and the
// progress counters of the single-launch reverse sweep.
__global__ void __launch_bounds__(256)
tv_rev_seed_kernel(const float* __restrict__ grad_out, const float* __restrict__ hist_g, const float* __restrict__ b,
                   const float* __restrict__ c, float* __restrict__ g_out, float* __restrict__ g_c,
                   float* __restrict__ g_b, float* __restrict__ acc, float* __restrict__ g_wx, float* __restrict__ g_wy,
                   int C, size_t plane, int* __restrict__ sync, int sync_words) {
    const size_t pix = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    // the progress counters of the reverse sweep that follows start at zero
    if (sync != nullptr && blockIdx.y == 0)
        for (size_t i = pix; i < (size_t)sync_words; i += (size_t)gridDim.x * blockDim.x) sync[i] = 0;
    if (pix >= plane) return;
    const size_t n = blockIdx.y;
    const float conf = __ldg(c + n * plane + pix);
    float dgc = 0.0f;
    for (int ch = 0; ch < C; ++ch) {
        const size_t i = (n * C + ch) * plane + pix;
        float up = grad_out[i];
        if (!finite_f(up)) up = 0.0f;                       // TVInpaintFista.cu:1616
        float dgb = 0.0f;
        g_out[i] = prox_reverse(up, hist_g[i], __ldg(b + i), conf, dgc, dgb);
        g_b[i] = dgb;
        acc[i] = 0.0f;
    }
    g_c[n * plane + pix] = dgc;
    g_wx[n * plane + pix] = 0.0f;
    g_wy[n * plane + pix] = 0.0f;
}

// y_{g+1} from hist[g], hist[g-1] (TVInpaintFista.cu:1130-1189).
__global__ void __launch_bounds__(256)
tv_rederive_y_kernel(const float* __restrict__ hist_g, const float* __restrict__ hist_gm1, const float* __restrict__ b,
                     const float* __restrict__ c, float* __restrict__ y, int C, size_t plane, float t) {
    const size_t pix = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (pix >= plane) return;
    const size_t n = blockIdx.y;
    const float conf = __ldg(c + n * plane + pix);
    for (int ch = 0; ch < C; ++ch) {
        const size_t i = (n * C + ch) * plane + pix;
        y[i] = rederive_y(hist_g[i], hist_gm1[i], __ldg(b + i), conf, t);
    }
}

// One reverse iteration (TVInpaintFista.cu:586-859): Laplacian-transpose at y, momentum reverse, prox Jacobian,
// accumulation of the per-pixel gradients.  `x1bar` (optional) receives dL/dx^{g+1}, the value the reference
// returns as the init gradient after the last reverse step (:1816).
__global__ void __launch_bounds__(kBX* kBY)
tv_rev_iter_kernel(const float* __restrict__ y, const float* __restrict__ g_in, float* __restrict__ g_out,
                   float* __restrict__ acc, const float* __restrict__ hist_g, const float* __restrict__ b,
                   const float* __restrict__ c, const float* __restrict__ wx, const float* __restrict__ wy,
                   float* __restrict__ g_c, float* __restrict__ g_b, float* __restrict__ g_wx,
                   float* __restrict__ g_wy, float* __restrict__ x1bar, int C, int H, int W, float t) {
    const int w = blockIdx.x * kBX + threadIdx.x;
    const int h = blockIdx.y * kBY + threadIdx.y;
    if (w >= W || h >= H) return;
    const size_t plane = (size_t)H * W;
    const size_t n = blockIdx.z;
    const int pix = h * W + w;
    const PixelWeights pw = load_weights(wx + n * plane, wy + n * plane, h, w, H, W);
    const float conf = __ldg(c + n * plane + pix);
    float dgc = 0.0f, dgwx = 0.0f, dgwy = 0.0f;
    for (int ch = 0; ch < C; ++ch) {
        const size_t off = (n * C + ch) * plane;
        const Stencil7 yy = load_stencil(y + off, h, w, H, W);
        const Stencil7 gg = load_stencil(g_in + off, h, w, H, W);
        float p1, p2, p1l, p2u, dwx, dwy, u0, u1, u2;
        tri_adjoint(yy.c, yy.r, yy.d, gg.c, gg.r, gg.d, pw.wx_c, pw.wy_c, p1, p2, dwx, dwy);
        tri_adjoint(yy.l, yy.c, yy.dl, gg.l, gg.c, gg.dl, pw.wx_l, pw.wy_l, p1l, u0, u1, u2);
        tri_adjoint(yy.u, yy.ur, yy.c, gg.u, gg.ur, gg.c, pw.wx_u, pw.wy_u, u0, p2u, u1, u2);
        dgwx += dwx;
        dgwy += dwy;
        const float ybar = gg.c - p1 - p2 + p1l + p2u;
        const float xbar = clampf(acc[off + pix] + (1.0f + t) * ybar, -kClipLocal, kClipLocal);
        acc[off + pix] = -t * ybar;
        float dgb = 0.0f;
        g_out[off + pix] = prox_reverse(xbar, hist_g[off + pix], __ldg(b + off + pix), conf, dgc, dgb);
        g_b[off + pix] += dgb;
        if (x1bar) x1bar[off + pix] = xbar;
    }
    g_c[n * plane + pix] += dgc;
    if (w < W - 1) g_wx[n * plane + pix] += dgwx;
    if (h < H - 1) g_wy[n * plane + pix] += dgwy;
}

// ---------------------------------------------------------------------------------------------------------------
// finalisation: sanitise, running-mean conditioner, output scalings (TVInpaintFista.cu:128-175, :1760-1818)
// ---------------------------------------------------------------------------------------------------------------
constexpr int kStatBlocks = 128;     // partial sums per output
constexpr int kNumOutputs = 5;       // C, X, Y, B, I in the reference's order

struct FinalizeArgs {
    float* ptr[kNumOutputs];
    unsigned long long count[kNumOutputs];
    float scale[kNumOutputs];
};

// partial[o][blk] = (sum of |g| over finite entries, number of non-finite entries)
__device__ __forceinline__ void grad_stats_block(const FinalizeArgs& a, double* __restrict__ partial) {
    const int o = blockIdx.y;
    const float* p = a.ptr[o];
    const unsigned long long cnt = a.count[o];
    double s = 0.0, bad = 0.0;
    auto take = [&](float v) { if (finite_f(v)) s += fabs((double)v); else bad += 1.0; };
    const unsigned long long tid = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x;
    const unsigned long long nthreads = (unsigned long long)gridDim.x * blockDim.x;
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
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    if (lane == 0) { sh[0][wid] = s; sh[1][wid] = bad; }
    __syncthreads();
    if (threadIdx.x == 0) {
        double ts = 0.0, tb = 0.0;
        for (int i = 0; i < 8; ++i) { ts += sh[0][i]; tb += sh[1][i]; }
        partial[(o * kStatBlocks + blockIdx.x) * 2 + 0] = ts;
        partial[(o * kStatBlocks + blockIdx.x) * 2 + 1] = tb;
    }
}

__global__ void __launch_bounds__(256)
tv_grad_stats_kernel(FinalizeArgs a, double* __restrict__ partial) { grad_stats_block(a, partial); }

// One warp: combines the partials of output o in a fixed order (lane-strided sums + shuffle tree, so the result does not
// depend on timing) and applies the running-mean rules.  Returns (in lane 0) the factor of this call and the new mean.
__device__ __forceinline__ float conditioner_warp(const double* __restrict__ partial, const FinalizeArgs& a, int o, double av,
                                                  int run, double& av_out) {
    const double run_step = fmin(0.975, (double)run / (double)(run + 1));       // :1761
    const int lane = threadIdx.x & 31;
    double s = 0.0, bad = 0.0;
    for (int i = lane; i < kStatBlocks; i += 32) {
        s += partial[(o * kStatBlocks + i) * 2];
        bad += partial[(o * kStatBlocks + i) * 2 + 1];
    }
    for (int off = 16; off > 0; off >>= 1) {
        s += __shfl_down_sync(0xffffffffu, s, off);
        bad += __shfl_down_sync(0xffffffffu, bad, off);
    }
    // mean |g|; a non-finite entry makes the reference restart its mean from 1000 x the running mean (:171)
    const double av_gc = (bad > 0.0) ? av * 1000.0 : (a.count[o] ? s / (double)a.count[o] : 0.0);
    float f = 1.0f;
    if (run >= 10 && av * 50.0 < av_gc) {                 // kill (:132-140)
        f = 0.0f;
        av = av * run_step + (1.0 - run_step) * 10.0 * av;
    } else if (run >= 10 && av * 10.0 < av_gc) {          // rescale (:142-150)
        const double mult = 10.0 * av / av_gc;
        f = (float)mult;
        av = av * run_step + (1.0 - run_step) * av_gc * mult;
    } else {
        av = av * run_step + (1.0 - run_step) * av_gc;
    }
    av_out = av;
    return f;
}

// One warp per output.  state[0..4] = running means (av_GC, av_GX, av_GY, av_GB, av_GI), factor[0..4] = multiplier for
// this call.
__global__ void __launch_bounds__(32 * kNumOutputs)
tv_conditioner_kernel(const double* __restrict__ partial, FinalizeArgs a, double* __restrict__ state,
                      float* __restrict__ factor, int run) {
    const int o = threadIdx.x >> 5;
    double av_new;
    const float f = conditioner_warp(partial, a, o, state[o], run, av_new);
    if ((threadIdx.x & 31) != 0) return;
    state[o] = av_new;
    factor[o] = f;
}

// g = (finite and |g| <= 1e7 ? g : 0) * factor * scale      (:160-171, :1795-1818)
__device__ __forceinline__ void grad_apply_block(const FinalizeArgs& a, float f) {
    const int o = blockIdx.y;
    float* p = a.ptr[o];
    const unsigned long long cnt = a.count[o];
    const float sc = a.scale[o];
    auto fix = [&](float v) { return (!finite_f(v) || fabsf(v) > 10000000.0f) ? 0.0f : v * f * sc; };
    const unsigned long long tid = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x;
    const unsigned long long nthreads = (unsigned long long)gridDim.x * blockDim.x;
    const unsigned long long nvec = (reinterpret_cast<size_t>(p) & 15) == 0 ? cnt / 4 : 0;
    float4* p4 = reinterpret_cast<float4*>(p);
    unsigned long long i = tid;
    for (; i + nthreads < nvec; i += 2 * nthreads) {
        float4 a0 = p4[i], a1 = p4[i + nthreads];
        a0.x = fix(a0.x); a0.y = fix(a0.y); a0.z = fix(a0.z); a0.w = fix(a0.w);
        a1.x = fix(a1.x); a1.y = fix(a1.y); a1.z = fix(a1.z); a1.w = fix(a1.w);
        p4[i] = a0; p4[i + nthreads] = a1;
    }
    for (; i < nvec; i += nthreads) {
        float4 a0 = p4[i];
        a0.x = fix(a0.x); a0.y = fix(a0.y); a0.z = fix(a0.z); a0.w = fix(a0.w);
        p4[i] = a0;
    }
    for (i = nvec * 4 + tid; i < cnt; i += nthreads) p[i] = fix(p[i]);
}

__global__ void __launch_bounds__(256)
tv_grad_apply_kernel(FinalizeArgs a, const float* __restrict__ factor) {
    grad_apply_block(a, factor ? factor[blockIdx.y] : 1.0f);
}

// Statistics, conditioner and scaling in one cooperative launch (grid kStatBlocks x kNumOutputs): the partials of every
// block, a grid-wide barrier, then every block derives the factor of its output from the same partials in the same order
// (block 0 of each output also stores the new running mean) and applies it.  The running means are double-buffered:
// read from state_in, written to state_out, so that no block reads a mean another block has already replaced.
__global__ void __launch_bounds__(256, 5)          // 640 blocks must be resident together: at least five per SM
tv_finalize_kernel(FinalizeArgs a, double* __restrict__ partial, const double* __restrict__ state_in,
                   double* __restrict__ state_out, float* __restrict__ factor, int run, int* __restrict__ sync, int sync_words) {
    if (blockIdx.x == 0 && blockIdx.y == 0)          // the sweeps are over: the next one finds its progress counters at zero
        for (int i = threadIdx.x; i < sync_words; i += blockDim.x) sync[i] = 0;
    grad_stats_block(a, partial);
    __threadfence();
    cooperative_groups::this_grid().sync();
    __shared__ float sh_f;
    const int o = blockIdx.y;
    if (threadIdx.x < 32) {
        double av_new;
        const float f = conditioner_warp(partial, a, o, state_in[o], run, av_new);
        if (threadIdx.x == 0) {
            sh_f = f;
            if (blockIdx.x == 0) {
                state_out[o] = av_new;
                factor[o] = f;
            }
        }
    }
    __syncthreads();
    grad_apply_block(a, sh_f);
}

// ---------------------------------------------------------------------------------------------------------------
// lambda gradient: out = sum g_c * c_raw, one launch (launch_tv_dot); its grid and the doubles of scratch it needs
// ---------------------------------------------------------------------------------------------------------------
constexpr int kDotBlocks = 592;      // 4 x 148 SMs

// ---------------------------------------------------------------------------------------------------------------
// per-id slots
// ---------------------------------------------------------------------------------------------------------------
struct Slot {
    float* arena = nullptr;
    size_t arena_floats = 0;
    double* cond = nullptr;          // 5 running means + stats partials + 5 float factors (separate small allocation)
    int n = 0, ch = 0, h = 0, w = 0, its = 0;
    bool have_forward = false;
    int run = 0;
    int cond_flip = 0;               // which of the two copies of the running means is current
    bool sync_clean = false;         // the arena's progress counters are known to be zero
    int generation = 0;              // forward passes stored on this slot so far; survives release
    int opt_conditioner = 1;
    int opt_fuse = 0;
    int opt_timing = 0;
    int opt_recompute = 0;           // 1: keep only checkpoints and rebuild each segment's history in the backward pass
    int opt_flow = 1;                // 1: all full time blocks of a sweep in one cooperative launch (tv_flow.cu)
    int pitch = 0;                   // row pitch (floats) of the arena planes of the stored forward pass
    bool staged = false;             // the temporally blocked kernels ran on zero-padded copies (pitch > w or unaligned tensors)
    bool recompute = false;          // mode the stored forward pass was run in
    bool window_valid = false;       // recompute mode: the history window holds the LAST segment (left by the forward)
    // timing ring: per recorded call one (start, stop) event pair around the iteration loop and its launch count
    static constexpr int kRing = 64;
    cudaEvent_t ev_fwd[kRing][2] = {}, ev_rev[kRing][2] = {};
    int launches_fwd[kRing] = {}, launches_rev[kRing] = {};
    int iters_fwd[kRing] = {}, iters_rev[kRing] = {};       // iterations the timed launches cover
    int n_fwd = 0, n_rev = 0;
    bool events_ready = false;
    std::vector<int> sched;
    std::vector<float> steps;
};

struct DeviceSlots {
    Slot slot[CNL_NUM_IDS];
};

static std::mutex g_mutex;
static std::vector<DeviceSlots*> g_devices;      // indexed by CUDA device ordinal

static Slot* get_slot(int id, int* rc) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) { *rc = check_cuda(e, "cudaGetDevice"); return nullptr; }
    if ((size_t)dev >= g_devices.size()) g_devices.resize(dev + 1, nullptr);
    if (!g_devices[dev]) g_devices[dev] = new DeviceSlots();
    *rc = CNL_OK;
    return &g_devices[dev]->slot[id];
}

static int ensure_events(Slot& s) {
    if (s.events_ready) return CNL_OK;
    for (int i = 0; i < Slot::kRing; ++i)
        for (int j = 0; j < 2; ++j) {
            CNL_TRY(check_cuda(cudaEventCreate(&s.ev_fwd[i][j]), "cudaEventCreate"));
            CNL_TRY(check_cuda(cudaEventCreate(&s.ev_rev[i][j]), "cudaEventCreate"));
        }
    s.events_ready = true;
    return CNL_OK;
}

static size_t arena_budget_floats() {
    const char* env = std::getenv("CNL_MAX_ARENA_GB");
    double gb = env ? std::atof(env) : 150.0;
    if (gb <= 0) gb = 150.0;
    return (size_t)(gb * 1024.0 * 1024.0 * 1024.0 / 4.0);
}

static inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Layout of a slot's arena, in floats.  Every sub-buffer starts on a 256-byte boundary.
struct ArenaLayout {
    size_t vol;       // n*ch*h*w rounded up to 64 floats
    size_t y0, y1, xbuf, hist, ckpt, xck, ga, gb, acc, acc2, ybuf, sync, sync_words, total;
    size_t map;       // n*h*w rounded up to 64 floats (w = row pitch)
    size_t stage_map, stage_vol;     // 6 map-sized and 4 volume-sized staging buffers (staged mode only)
};

// hist_planes: its_eff when every iterate is kept, the longest segment in recompute mode; xck_planes: primal iterate
// at every checkpoint (recompute mode only, needed to restart the iteration there).
static ArenaLayout make_layout(size_t n, size_t ch, size_t h, size_t w, size_t hist_planes, size_t nckpt, size_t xck_planes = 0,
                               bool staged = false) {
    ArenaLayout L;
    L.vol = align_up(n * ch * h * w, 64);
    L.map = align_up(n * h * w, 64);
    size_t o = 0;
    L.y0 = o; o += L.vol;
    L.y1 = o; o += L.vol;
    L.ga = o; o += L.vol;
    L.gb = o; o += L.vol;
    L.acc = o; o += L.vol;
    L.acc2 = o; o += L.vol;
    L.xbuf = o; o += L.vol;
    L.ybuf = o; o += L.vol;
    // progress counters of the single-launch sweeps: one per tile, then the abort word and the ticket counter
    L.sync_words = align_up((size_t)flow_tiles((int)h, (int)std::min<size_t>(w, 0x3fffffff), (int)n) + 2, 64);
    L.sync = o; o += L.sync_words;
    L.ckpt = o; o += L.vol * nckpt;
    L.xck = o; o += L.vol * xck_planes;
    L.hist = o; o += L.vol * hist_planes;
    L.stage_map = o; o += staged ? 6 * L.map : 0;
    L.stage_vol = o; o += staged ? 4 * L.vol : 0;
    L.total = o;
    return L;
}

static void compute_schedule(int its, std::vector<int>& sched, std::vector<float>& steps) {
    // checkpoint iterations and momentum table, same double arithmetic as TVInpaintFista.cu:1499-1504, :1525-1532
    const int n = (int)std::floor(std::sqrt((double)its));
    sched.resize(n);
    for (int i = 0; i < n; ++i) sched[i] = (int)(std::floor(i * std::sqrt((double)its) * 0.5) * 2);
    steps.resize(its);
    double t = 1.0, t_ = 1.0;
    for (int i = 0; i < its; ++i) {
        t_ = t;
        t = (1.0 + std::sqrt(1.0 + 4.0 * t * t)) / 2.0;
        steps[i] = (float)std::max(0.0, (t_ - 1.0) / t);
    }
}

// Segment i of the iteration runs from checkpoint iteration sched[i] up to (excluding) the next checkpoint.
static inline int seg_begin(const std::vector<int>& sched, int i) { return sched[i]; }
static inline int seg_end(const std::vector<int>& sched, int i, int its_eff) {
    return i + 1 < (int)sched.size() ? sched[i + 1] : its_eff;
}
static int longest_segment(const std::vector<int>& sched, int its_eff) {
    int m = 0;
    for (int i = 0; i < (int)sched.size(); ++i) m = std::max(m, seg_end(sched, i, its_eff) - seg_begin(sched, i));
    return m;
}
// `pitch` is the row pitch of every arena plane in floats (w, or w rounded up to 4 in staged mode).
static ArenaLayout slot_layout(size_t n, size_t ch, size_t h, size_t pitch, int its_eff, const std::vector<int>& sched, bool recompute,
                               bool staged = false) {
    if (recompute) return make_layout(n, ch, h, pitch, (size_t)longest_segment(sched, its_eff), sched.size(), sched.size(), staged);
    return make_layout(n, ch, h, pitch, (size_t)its_eff, sched.size(), 0, staged);
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

static int check_common(const void* const* ptrs, int nptr, int n, int ch, int h, int w, int its, int id) {
    if (id < 0 || id >= CNL_NUM_IDS)
        return fail(CNL_ERR_BAD_ID, "id %d is outside 0..%d", id, CNL_NUM_IDS - 1);
    if (n < 1 || ch < 1 || h < 1 || w < 1)
        return fail(CNL_ERR_BAD_SHAPE, "n, ch, h, w must be >= 1 (got %d, %d, %d, %d)", n, ch, h, w);
    if ((long long)h * w > 0x3fffffffLL || n > 65535)
        return fail(CNL_ERR_BAD_SHAPE, "image of %d x %d pixels or batch %d is beyond the supported range", h, w, n);
    if (its < 2) return fail(CNL_ERR_BAD_ITS, "its must be >= 2 (got %d)", its);
    for (int i = 0; i < nptr; ++i)
        if (!ptrs[i]) return fail(CNL_ERR_NULL, "null pointer argument (position %d)", i);
    return CNL_OK;
}

static int ensure_arena(Slot& s, size_t floats) {
    if (s.arena && s.arena_floats >= floats) return CNL_OK;
    if (floats > arena_budget_floats())
        return fail(CNL_ERR_ALLOC, "iterate history needs %.2f GB, above the CNL_MAX_ARENA_GB budget",
                    floats * 4.0 / (1024.0 * 1024.0 * 1024.0));
    if (s.arena) {
        CNL_TRY(check_cuda(cudaDeviceSynchronize(), "cudaDeviceSynchronize"));
        cudaFree(s.arena);
        s.arena = nullptr;
        s.arena_floats = 0;
    }
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, floats * sizeof(float));
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(CNL_ERR_ALLOC, "cudaMalloc of %.2f GB failed: %s", floats * 4.0 / (1024.0 * 1024.0 * 1024.0),
                    cudaGetErrorString(e));
    }
    s.arena = static_cast<float*>(p);
    s.arena_floats = floats;
    s.sync_clean = false;
    return CNL_OK;
}

constexpr size_t kCondDoubles = 2 * kNumOutputs + (size_t)kNumOutputs * kStatBlocks * 2 + 4;   // means (two copies), partials, factors

static int ensure_cond(Slot& s) {
    if (s.cond) return CNL_OK;
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, kCondDoubles * sizeof(double));
    if (e != cudaSuccess) { cudaGetLastError(); return fail(CNL_ERR_ALLOC, "cudaMalloc (conditioner state) failed"); }
    s.cond = static_cast<double*>(p);
    return check_cuda(cudaMemset(s.cond, 0, kCondDoubles * sizeof(double)), "cudaMemset");
}

// Per-iteration tables of the single-launch sweeps: momentum factors and, per iteration, the checkpoint taken before it.
static void fill_flow_tables(const Slot& s, int its_eff, FlowTables& tab) {
    for (int g = 0; g < kFlowMaxIts; ++g) {
        tab.t[g] = g < its_eff ? s.steps[g] : 0.0f;
        tab.ckpt_slot[g] = -1;
    }
    for (size_t i = 0; i < s.sched.size(); ++i)
        if (s.sched[i] < its_eff && s.sched[i] < kFlowMaxIts) tab.ckpt_slot[s.sched[i]] = (signed char)i;
}

// The fused finalisation is a cooperative launch of kStatBlocks x kNumOutputs blocks: usable where they are all resident.
static bool finalize_grid_fits() {
    static int fits[64] = {};          // per device: 0 unknown, 1 yes, -1 no
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return false;
    if (fits[dev] == 0) {
        int per_sm = 0, sms = 0;
        const bool ok = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, tv_finalize_kernel, 256, 0) == cudaSuccess &&
                        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess;
        fits[dev] = (ok && per_sm * sms >= kStatBlocks * kNumOutputs) ? 1 : -1;
    }
    return fits[dev] == 1;
}

// ---------------------------------------------------------------------------------------------------------------
// host drivers
// ---------------------------------------------------------------------------------------------------------------
static int tv_forward_impl(const float* wx, const float* wy, const float* c, const float* b, const float* init,
                           float* out, int n, int ch, int h, int w, int its, int id, cudaStream_t st) {
    const void* ptrs[] = {wx, wy, c, b, init, out};
    CNL_TRY(check_common(ptrs, 6, n, ch, h, w, its, id));
    std::lock_guard<std::mutex> lock(g_mutex);
    int rc;
    Slot* sp = get_slot(id, &rc);
    if (!sp) return rc;
    Slot& s = *sp;
    s.have_forward = false;
    CNL_TRY(flow_status_take());
    compute_schedule(its, s.sched, s.steps);
    const int its_eff = 2 * (its / 2);
    const void* aligned[] = {wx, wy, c, b, init, out};          // the arena itself is 256-byte aligned
    const int fuse = s.opt_fuse == 0 ? kFuseMax : s.opt_fuse;
    const bool fused = fuse > 1;
    // The temporally blocked kernels read 16-byte vectors: tensors whose rows are not a multiple of 4 floats, or that
    // are not 16-byte aligned, are staged into zero-padded copies with such a pitch; everything the kernels touch
    // then lives in the arena and the results are copied back row by row.
    const bool staged = fused && !fused_supported(w, aligned, 6);
    const int P = staged ? ((w + 3) & ~3) : w;
    ArenaLayout L = slot_layout(n, ch, h, P, its_eff, s.sched, false, staged);
    // Keeping every iterate costs its_eff volumes.  When that exceeds the budget (or on request) only the checkpoints
    // are kept and the backward pass rebuilds the history segment by segment, like the reference does
    // (TVInpaintFista.cu:1690-1760); the temporally blocked kernels are needed for that.
    const bool recompute = fused && (s.opt_recompute || L.total > arena_budget_floats());
    if (recompute) L = slot_layout(n, ch, h, P, its_eff, s.sched, true, staged);
    CNL_TRY(ensure_arena(s, L.total));
    // a different problem lays the arena out differently: the counters of the single-launch sweeps sit elsewhere
    if (s.n != n || s.ch != ch || s.h != h || s.w != w || s.its != its || s.pitch != P || s.staged != staged || s.recompute != recompute)
        s.sync_clean = false;
    s.recompute = recompute;
    s.staged = staged;
    s.pitch = P;
    s.window_valid = false;
    const size_t vol_bytes = (size_t)n * ch * h * P * sizeof(float);
    if (staged) {
        float* m = s.arena + L.stage_map;
        float* v = s.arena + L.stage_vol;
        CNL_TRY(pad_rows(m + 0 * L.map, wx, (size_t)n * h, w, P, st));
        CNL_TRY(pad_rows(m + 1 * L.map, wy, (size_t)n * h, w, P, st));
        CNL_TRY(pad_rows(m + 2 * L.map, c, (size_t)n * h, w, P, st));
        CNL_TRY(pad_rows(v + 0 * L.vol, b, (size_t)n * ch * h, w, P, st));
        CNL_TRY(pad_rows(v + 1 * L.vol, init, (size_t)n * ch * h, w, P, st));
        wx = m + 0 * L.map; wy = m + 1 * L.map; c = m + 2 * L.map;
        b = v + 0 * L.vol; init = v + 1 * L.vol;
    }
    float* const user_out = out;
    if (staged) out = s.arena + L.stage_vol + 2 * L.vol;
    float* y0 = s.arena + L.y0;
    float* y1 = s.arena + L.y1;
    if (fused) {
        // temporally blocked path: up to `fuse` iterations per launch; x and y ping-pong between launches so that no
        // CTA reads a halo another CTA is writing, and the last launch writes x into the caller's buffer.  In
        // recompute mode launches do not straddle checkpoints, the primal iterate is saved beside every checkpoint
        // and only the last segment's history is written (the backward pass starts there).
        bool timing = s.opt_timing && s.n_fwd < Slot::kRing;
        const unsigned long long launches0 = g_launches.load();
        if (timing) {
            CNL_TRY(ensure_events(s));
            CNL_TRY(check_cuda(cudaEventRecord(s.ev_fwd[s.n_fwd][0], st), "cudaEventRecord"));
        }
        struct Launch { int g0, K; };
        std::vector<Launch> plan;
        if (recompute) {
            for (int i = 0; i < (int)s.sched.size(); ++i)
                for (int g0 = seg_begin(s.sched, i), e = seg_end(s.sched, i, its_eff); g0 < e; g0 += fuse)
                    plan.push_back({g0, std::min(fuse, e - g0)});
        } else {
            for (int g0 = 0; g0 < its_eff; g0 += fuse) plan.push_back({g0, std::min(fuse, its_eff - g0)});
        }
        const int nlaunch = (int)plan.size();
        const int last_seg = (int)s.sched.size() - 1;
        float* xbuf = s.arena + L.xbuf;
        const float* y_in = init;
        const float* x_in = init;
        size_t next_ckpt = 0;
        int first_launch = 0;
        // Single-launch sweep: every full time block of kFuseMax iterations in one cooperative launch whose tiles are
        // ordered by progress counters; a shorter last block, if any, follows as an ordinary launch.
        const int nfull = (its_eff + kFuseMax - 1) / kFuseMax;       // the last time block may be shorter
        if (!recompute && fuse == kFuseMax && s.opt_flow && its_eff <= kFlowMaxIts && flow_enabled()) {
            const bool rem = false;
            FwdFlowParams fp{};
            fp.init = init;
            fp.ybuf[0] = y0; fp.ybuf[1] = y1;
            // the primal iterate of the sweep's last launch has to land in the caller's buffer
            fp.xbuf[(nfull - 1) & 1] = rem ? xbuf : out;
            fp.xbuf[nfull & 1] = rem ? out : xbuf;
            fp.b = b; fp.c = c; fp.wx = wx; fp.wy = wy;
            fp.hist = s.arena + L.hist; fp.ckpt = s.arena + L.ckpt; fp.vol = L.vol;
            int* sync = reinterpret_cast<int*>(s.arena + L.sync);
            const int ntiles = flow_tiles(h, w, n);
            fp.progress = sync; fp.abort = sync + ntiles; fp.status = flow_status_device_ptr();
            fp.nblocks = nfull;
            fp.its = its_eff;
            fp.N = n; fp.C = ch; fp.H = h; fp.W = w; fp.P = P;
            fill_flow_tables(s, its_eff, fp.tab);
            if (!s.sync_clean || s.opt_flow == 2)
                CNL_TRY(check_cuda(cudaMemsetAsync(sync, 0, L.sync_words * sizeof(int), st), "zero progress counters"));
            s.sync_clean = false;
            if (s.opt_flow == 2)      // self-test of the bounded waits: counters that no unit can ever bring up to what its neighbours need
                CNL_TRY(check_cuda(cudaMemsetAsync(sync, 0x80, (size_t)ntiles * sizeof(int), st), "poison progress counters"));
            if (timing) CNL_TRY(check_cuda(cudaEventRecord(s.ev_fwd[s.n_fwd][0], st), "cudaEventRecord"));
            CNL_TRY(launch_tv_fwd_flow(fp, st));
            if (timing) {          // the record covers the single-launch sweep alone
                CNL_TRY(check_cuda(cudaEventRecord(s.ev_fwd[s.n_fwd][1], st), "cudaEventRecord"));
                s.launches_fwd[s.n_fwd] = 1;
                s.iters_fwd[s.n_fwd] = its_eff;
                s.n_fwd += 1;
                timing = false;
            }
            first_launch = nlaunch;          // nothing is left for the per-time-block launches
        }
        for (int i = first_launch; i < nlaunch; ++i) {
            const int g0 = plan[i].g0, K = plan[i].K;
            FwdFusedParams fp{};
            fp.y_in = y_in; fp.x_in = x_in;
            fp.y_out = (i & 1) ? y1 : y0;
            fp.x_out = ((nlaunch - 1 - i) & 1) ? xbuf : out;
            fp.b = b; fp.c = c; fp.wx = wx; fp.wy = wy;
            fp.N = n; fp.C = ch; fp.H = h; fp.W = w; fp.P = P;
            for (int j = 0; j < K; ++j) {
                const int g = g0 + j;
                fp.t[j] = s.steps[g];
                fp.ckpt[j] = nullptr;
                if (next_ckpt < s.sched.size() && s.sched[next_ckpt] == g) {
                    fp.ckpt[j] = s.arena + L.ckpt + next_ckpt * L.vol;
                    if (recompute)      // j == 0 here: x at the checkpoint is this launch's input
                        CNL_TRY(check_cuda(cudaMemcpyAsync(s.arena + L.xck + next_ckpt * L.vol, x_in, vol_bytes,
                                                           cudaMemcpyDeviceToDevice, st), "checkpoint x"));
                    ++next_ckpt;
                }
                if (!recompute) fp.hist[j] = s.arena + L.hist + (size_t)g * L.vol;
                else fp.hist[j] = g >= s.sched[last_seg] ? s.arena + L.hist + (size_t)(g - s.sched[last_seg]) * L.vol : nullptr;
            }
            CNL_TRY(launch_tv_fwd_fused(fp, K, st));
            y_in = fp.y_out;
            x_in = fp.x_out;
        }
        if (timing) {
            CNL_TRY(check_cuda(cudaEventRecord(s.ev_fwd[s.n_fwd][1], st), "cudaEventRecord"));
            s.launches_fwd[s.n_fwd] = (int)(g_launches.load() - launches0);
            s.iters_fwd[s.n_fwd] = its_eff;
            s.n_fwd += 1;
        }
        if (staged) CNL_TRY(unpad_rows(user_out, out, (size_t)n * ch * h, w, P, st));
        s.n = n; s.ch = ch; s.h = h; s.w = w; s.its = its;
        s.window_valid = recompute;
        s.have_forward = true;
        s.generation += 1;
        return CNL_OK;
    }
    CNL_TRY(check_cuda(cudaMemcpyAsync(out, init, vol_bytes, cudaMemcpyDeviceToDevice, st), "copy init->x"));
    CNL_TRY(check_cuda(cudaMemcpyAsync(y0, init, vol_bytes, cudaMemcpyDeviceToDevice, st), "copy init->y"));
    const dim3 block(kBX, kBY);
    const dim3 grid((w + kBX - 1) / kBX, (h + kBY - 1) / kBY, n);
    size_t next_ckpt = 0;
    const bool timing = s.opt_timing && s.n_fwd < Slot::kRing;
    const unsigned long long launches0 = g_launches.load();
    if (timing) {
        CNL_TRY(ensure_events(s));
        CNL_TRY(check_cuda(cudaEventRecord(s.ev_fwd[s.n_fwd][0], st), "cudaEventRecord"));
    }
    for (int g = 0; g < its_eff; ++g) {
        float* yin = (g & 1) ? y1 : y0;
        float* yout = (g & 1) ? y0 : y1;
        if (next_ckpt < s.sched.size() && s.sched[next_ckpt] == g) {
            CNL_TRY(check_cuda(cudaMemcpyAsync(s.arena + L.ckpt + next_ckpt * L.vol, yin, vol_bytes,
                                               cudaMemcpyDeviceToDevice, st), "checkpoint y"));
            ++next_ckpt;
        }
        tv_fwd_iter_kernel<<<grid, block, 0, st>>>(yin, yout, out, b, c, wx, wy, s.arena + L.hist + (size_t)g * L.vol,
                                                   ch, h, w, s.steps[g]);
        CNL_TRY(after_launch("tv_fwd_iter_kernel"));
    }
    if (timing) {
        CNL_TRY(check_cuda(cudaEventRecord(s.ev_fwd[s.n_fwd][1], st), "cudaEventRecord"));
        s.launches_fwd[s.n_fwd] = (int)(g_launches.load() - launches0);
        s.iters_fwd[s.n_fwd] = its_eff;
        s.n_fwd += 1;
    }
    s.n = n; s.ch = ch; s.h = h; s.w = w; s.its = its;
    s.have_forward = true;
    s.generation += 1;
    return CNL_OK;
}

static int tv_backward_impl(const float* wx, const float* wy, const float* c, const float* b, const float* grad_out,
                            float* g_wx, float* g_wy, float* g_c, float* g_b, float* g_init,
                            int n, int ch, int h, int w, int its, int id, cudaStream_t st) {
    const void* ptrs[] = {wx, wy, c, b, grad_out, g_wx, g_wy, g_c, g_b, g_init};
    CNL_TRY(check_common(ptrs, 10, n, ch, h, w, its, id));
    std::lock_guard<std::mutex> lock(g_mutex);
    int rc;
    Slot* sp = get_slot(id, &rc);
    if (!sp) return rc;
    Slot& s = *sp;
    if (!s.have_forward || s.n != n || s.ch != ch || s.h != h || s.w != w || s.its != its)
        return fail(CNL_ERR_NO_FORWARD, "backward(id=%d) needs a preceding forward(id=%d) with the same shape and its",
                    id, id);
    CNL_TRY(ensure_cond(s));
    CNL_TRY(flow_status_take());
    const int its_eff = 2 * (its / 2);
    const bool staged = s.staged;
    const int P = s.pitch;                        // row pitch of the arena planes (w unless staged)
    const ArenaLayout L = slot_layout(n, ch, h, P, its_eff, s.sched, s.recompute, staged);
    const size_t plane = (size_t)h * P;
    const size_t uplane = (size_t)h * w;          // plane of the caller's tensors
    const void* aligned[] = {wx, wy, c, b, grad_out, g_wx, g_wy, g_c, g_b, g_init};
    const int fuse = s.opt_fuse == 0 ? kFuseMax : s.opt_fuse;
    const bool fused = fuse > 1 && (staged || fused_supported(w, aligned, 10));
    if ((s.recompute || staged) && !fused)
        return fail(CNL_ERR_BAD_OPTION, "the forward pass of id %d ran on the temporally blocked kernels (%s); the backward pass "
                    "needs them too: keep the fuse option and pass 16-byte aligned tensors", id,
                    staged ? "zero-padded staging" : "checkpoints only");
    float* const u_gwx = g_wx; float* const u_gwy = g_wy; float* const u_gc = g_c; float* const u_gb = g_b; float* const u_ginit = g_init;
    if (staged) {          // same staging as in the forward pass, plus the upstream gradient and the five outputs
        float* m = s.arena + L.stage_map;
        float* v = s.arena + L.stage_vol;
        CNL_TRY(pad_rows(m + 0 * L.map, wx, (size_t)n * h, w, P, st));
        CNL_TRY(pad_rows(m + 1 * L.map, wy, (size_t)n * h, w, P, st));
        CNL_TRY(pad_rows(m + 2 * L.map, c, (size_t)n * h, w, P, st));
        CNL_TRY(pad_rows(v + 0 * L.vol, b, (size_t)n * ch * h, w, P, st));
        CNL_TRY(pad_rows(v + 1 * L.vol, grad_out, (size_t)n * ch * h, w, P, st));
        wx = m + 0 * L.map; wy = m + 1 * L.map; c = m + 2 * L.map;
        b = v + 0 * L.vol; grad_out = v + 1 * L.vol;
        g_wx = m + 3 * L.map; g_wy = m + 4 * L.map; g_c = m + 5 * L.map;
        g_b = v + 2 * L.vol; g_init = v + 3 * L.vol;
    }
    float* ga = s.arena + L.ga;      // d_gxk05_0_temp
    float* gb = s.arena + L.gb;      // d_gxk05_1_temp
    float* acc = s.arena + L.acc;
    float* ybuf = s.arena + L.ybuf;
    const float* hist = s.arena + L.hist;

    const dim3 block(kBX, kBY);
    const dim3 grid((w + kBX - 1) / kBX, (h + kBY - 1) / kBY, n);
    const dim3 pgrid((unsigned)((plane + 255) / 256), n);
    bool timing = s.opt_timing && s.n_rev < Slot::kRing;
    unsigned long long launches0 = g_launches.load();
    if (timing) CNL_TRY(ensure_events(s));
    bool sync_dirty = false;           // the reverse sweep has used the progress counters
    auto ckpt_of = [&](int g) -> const float* {
        for (size_t i = 0; i < s.sched.size(); ++i)
            if (s.sched[i] == g) return s.arena + L.ckpt + i * L.vol;      // segment start: the checkpointed y_g (:1724-1727)
        return nullptr;
    };
    const int nseg = (int)s.sched.size();
    // Recompute mode: rebuilds the history window of segment i from the y and x saved at its checkpoint.
    auto rebuild_segment = [&](int i) -> int {
        const int g_begin = seg_begin(s.sched, i), g_end = seg_end(s.sched, i, its_eff);
        const float* y_in = s.arena + L.ckpt + (size_t)i * L.vol;
        const float* x_in = s.arena + L.xck + (size_t)i * L.vol;
        int k = 0;
        for (int g0 = g_begin; g0 < g_end; g0 += fuse, ++k) {
            const int K = std::min(fuse, g_end - g0);
            FwdFusedParams fp{};
            fp.y_in = y_in; fp.x_in = x_in;
            fp.y_out = s.arena + ((k & 1) ? L.y1 : L.y0);        // iterates beyond the window are scratch
            fp.x_out = s.arena + ((k & 1) ? L.ybuf : L.xbuf);
            fp.b = b; fp.c = c; fp.wx = wx; fp.wy = wy;
            fp.N = n; fp.C = ch; fp.H = h; fp.W = w; fp.P = P;
            for (int j = 0; j < K; ++j) {
                fp.t[j] = s.steps[g0 + j];
                fp.ckpt[j] = nullptr;
                fp.hist[j] = s.arena + L.hist + (size_t)(g0 + j - g_begin) * L.vol;
            }
            CNL_TRY(launch_tv_fwd_fused(fp, K, st));
            y_in = fp.y_out;
            x_in = fp.x_out;
        }
        return CNL_OK;
    };
    // x^{g+1/2} of iteration g inside the segment whose history is resident (every iteration without recomputation)
    const float* hist_base = hist;
    int hist_first = 0;
    auto hist_of = [&](int g) -> const float* { return g >= hist_first ? hist_base + (size_t)(g - hist_first) * L.vol : nullptr; };
    if (s.recompute) {
        hist_first = s.sched[nseg - 1];
        if (!s.window_valid) CNL_TRY(rebuild_segment(nseg - 1));
        s.window_valid = false;
    }
    // seed at the last iteration (its_eff - 1 is odd, so the seed lands in the "odd" buffer like the reference's)
    {
        const int g = its_eff - 1;
        tv_rev_seed_kernel<<<pgrid, 256, 0, st>>>(grad_out, hist_of(g), b, c, gb, g_c, g_b, acc, g_wx, g_wy, ch, plane,
                                                  reinterpret_cast<int*>(s.arena + L.sync), (int)L.sync_words);
        CNL_TRY(after_launch("tv_rev_seed_kernel"));
    }
    if (timing) {          // after the seed: the record covers the iteration kernels
        launches0 = g_launches.load();
        CNL_TRY(check_cuda(cudaEventRecord(s.ev_rev[s.n_rev][0], st), "cudaEventRecord"));
    }
    if (fused) {
        float* acc2 = s.arena + L.acc2;
        const float* g_cur = gb;
        const float* acc_cur = acc;
        int flip = 0;
        int seg = nseg - 1;                       // segment the sweep is in (recompute mode)
        int g_start = its_eff - 2;
        const int nfull = (its_eff - 1 + kFuseMax - 1) / kFuseMax;      // time blocks of the reverse sweep, the last one may be shorter
        if (!s.recompute && fuse == kFuseMax && s.opt_flow && nfull >= 1 && its_eff <= kFlowMaxIts && flow_enabled()) {
            RevFlowParams rp{};
            rp.gbuf[0] = ga; rp.gbuf[1] = gb;                  // block 0 reads the seed in gb and writes ga
            rp.abuf[0] = acc2; rp.abuf[1] = acc;
            rp.b = b; rp.c = c; rp.wx = wx; rp.wy = wy;
            rp.hist = hist; rp.ckpt = s.arena + L.ckpt; rp.vol = L.vol;
            rp.g_c = g_c; rp.g_b = g_b; rp.g_wx = g_wx; rp.g_wy = g_wy;
            rp.x1bar = g_init;
            int* sync = reinterpret_cast<int*>(s.arena + L.sync);
            const int ntiles = flow_tiles(h, w, n);
            rp.progress = sync; rp.abort = sync + ntiles; rp.status = flow_status_device_ptr();
            rp.g_first = its_eff - 2;
            rp.nblocks = nfull;
            rp.N = n; rp.C = ch; rp.H = h; rp.W = w; rp.P = P;
            fill_flow_tables(s, its_eff, rp.tab);          // (the seed kernel has zeroed the progress counters)
            if (timing) CNL_TRY(check_cuda(cudaEventRecord(s.ev_rev[s.n_rev][0], st), "cudaEventRecord"));
            CNL_TRY(launch_tv_rev_flow(rp, st));
            sync_dirty = true;
            if (timing) {          // the record covers the single-launch sweep alone
                CNL_TRY(check_cuda(cudaEventRecord(s.ev_rev[s.n_rev][1], st), "cudaEventRecord"));
                s.launches_rev[s.n_rev] = 1;
                s.iters_rev[s.n_rev] = its_eff - 1;
                s.n_rev += 1;
                timing = false;
            }
            g_start = -1;                    // nothing is left for the per-time-block launches
        }
        for (int g0 = g_start; g0 >= 0;) {
            int K = std::min(fuse, g0 + 1);
            if (s.recompute) {
                if (g0 < seg_begin(s.sched, seg)) {          // entering the next older segment: rebuild its history
                    --seg;
                    hist_first = seg_begin(s.sched, seg);
                    CNL_TRY(rebuild_segment(seg));
                }
                K = std::min(K, g0 - seg_begin(s.sched, seg) + 1);      // launches do not straddle checkpoints
            }
            RevFusedParams rp{};
            rp.g_in = g_cur; rp.acc_in = acc_cur;
            rp.g_out = flip ? gb : ga;
            rp.acc_out = flip ? acc : acc2;
            rp.b = b; rp.c = c; rp.wx = wx; rp.wy = wy;
            rp.g_c = g_c; rp.g_b = g_b; rp.g_wx = g_wx; rp.g_wy = g_wy;
            rp.N = n; rp.C = ch; rp.H = h; rp.W = w; rp.P = P;
            for (int j = 0; j <= K; ++j) {
                const int g = g0 - j;
                rp.hist[j] = g >= 0 ? hist_of(g) : nullptr;
                if (j < K) {
                    rp.t[j] = s.steps[g];
                    rp.ckpt[j] = ckpt_of(g);
                }
            }
            rp.x1bar = (g0 - K + 1 == 0) ? g_init : nullptr;
            CNL_TRY(launch_tv_rev_fused(rp, K, st));
            g_cur = rp.g_out;
            acc_cur = rp.acc_out;
            flip ^= 1;
            g0 -= K;
        }
    } else {
        for (int g = its_eff - 2; g >= 0; --g) {
            const float t = s.steps[g];
            const float* hg = hist + (size_t)g * L.vol;
            float* gout = (g & 1) ? gb : ga;
            const float* gin = (g & 1) ? ga : gb;
            const float* yk = ckpt_of(g);
            if (!yk) {
                tv_rederive_y_kernel<<<pgrid, 256, 0, st>>>(hg, hg - L.vol, b, c, ybuf, ch, plane, t);
                CNL_TRY(after_launch("tv_rederive_y_kernel"));
                yk = ybuf;
            }
            tv_rev_iter_kernel<<<grid, block, 0, st>>>(yk, gin, gout, acc, hg, b, c, wx, wy, g_c, g_b, g_wx, g_wy,
                                                       g == 0 ? g_init : nullptr, ch, h, w, t);
            CNL_TRY(after_launch("tv_rev_iter_kernel"));
        }
    }
    if (timing) {
        CNL_TRY(check_cuda(cudaEventRecord(s.ev_rev[s.n_rev][1], st), "cudaEventRecord"));
        s.launches_rev[s.n_rev] = (int)(g_launches.load() - launches0);
        s.iters_rev[s.n_rev] = its_eff - 1;
        s.n_rev += 1;
    }

    if (staged) {
        CNL_TRY(unpad_rows(u_gwx, g_wx, (size_t)n * h, w, P, st));
        CNL_TRY(unpad_rows(u_gwy, g_wy, (size_t)n * h, w, P, st));
        CNL_TRY(unpad_rows(u_gc, g_c, (size_t)n * h, w, P, st));
        CNL_TRY(unpad_rows(u_gb, g_b, (size_t)n * ch * h, w, P, st));
        CNL_TRY(unpad_rows(u_ginit, g_init, (size_t)n * ch * h, w, P, st));
    }
    FinalizeArgs fa;
    fa.ptr[0] = u_gc;  fa.count[0] = (unsigned long long)n * uplane;      fa.scale[0] = kGlobalG;
    fa.ptr[1] = u_gwx; fa.count[1] = (unsigned long long)n * uplane;      fa.scale[1] = kGlobalG * kLip;
    fa.ptr[2] = u_gwy; fa.count[2] = (unsigned long long)n * uplane;      fa.scale[2] = kGlobalG * kLip;
    fa.ptr[3] = u_gb;  fa.count[3] = (unsigned long long)n * ch * uplane; fa.scale[3] = kGlobalG;
    fa.ptr[4] = u_ginit; fa.count[4] = (unsigned long long)n * ch * uplane; fa.scale[4] = 1.0f;
    double* state = s.cond + (size_t)s.cond_flip * kNumOutputs;
    double* state_next = s.cond + (size_t)(s.cond_flip ^ 1) * kNumOutputs;
    double* partial = s.cond + 2 * kNumOutputs;
    float* factor = reinterpret_cast<float*>(s.cond + 2 * kNumOutputs + (size_t)kNumOutputs * kStatBlocks * 2);
    if (s.opt_conditioner && flow_enabled() && finalize_grid_fits()) {
        // one cooperative launch: statistics, grid barrier, conditioner, scaling
        const double* state_in = state;
        int run = s.run;
        int* sync = reinterpret_cast<int*>(s.arena + L.sync);        // left at zero for the next forward sweep
        int sync_words = (int)L.sync_words;
        void* args[] = {&fa, &partial, &state_in, &state_next, &factor, &run, &sync, &sync_words};
        CNL_TRY(check_cuda(cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(tv_finalize_kernel),
                                                       dim3(kStatBlocks, kNumOutputs), dim3(256), args, 0, st), "tv_finalize_kernel"));
        CNL_TRY(after_launch("tv_finalize_kernel"));
        s.cond_flip ^= 1;
        s.sync_clean = true;
        sync_dirty = false;
    } else {
        if (s.opt_conditioner) {
            tv_grad_stats_kernel<<<dim3(kStatBlocks, kNumOutputs), 256, 0, st>>>(fa, partial);
            CNL_TRY(after_launch("tv_grad_stats_kernel"));
            tv_conditioner_kernel<<<1, 32 * kNumOutputs, 0, st>>>(partial, fa, state, factor, s.run);
            CNL_TRY(after_launch("tv_conditioner_kernel"));
        }
        tv_grad_apply_kernel<<<dim3(296, kNumOutputs), 256, 0, st>>>(fa, s.opt_conditioner ? factor : nullptr);
        CNL_TRY(after_launch("tv_grad_apply_kernel"));
    }
    if (sync_dirty) s.sync_clean = false;
    s.run += 1;
    return CNL_OK;
}

}  // namespace cnl

// ---------------------------------------------------------------------------------------------------------------
// C entry points
// ---------------------------------------------------------------------------------------------------------------
using namespace cnl;

extern "C" int cnl_tv_forward(const float* wx, const float* wy, const float* c, const float* b, const float* init,
                              float* out, int n, int ch, int h, int w, int its, int id, void* stream) {
    return tv_forward_impl(wx, wy, c, b, init, out, n, ch, h, w, its, id, static_cast<cudaStream_t>(stream));
}

extern "C" int cnl_tv_backward(const float* wx, const float* wy, const float* c, const float* b,
                               const float* grad_out, float* g_wx, float* g_wy, float* g_c, float* g_b,
                               float* g_init, int n, int ch, int h, int w, int its, int id, void* stream) {
    return tv_backward_impl(wx, wy, c, b, grad_out, g_wx, g_wy, g_c, g_b, g_init, n, ch, h, w, its, id,
                            static_cast<cudaStream_t>(stream));
}

extern "C" int cnl_tv_release(int id) {
    if (id < 0 || id >= CNL_NUM_IDS) return fail(CNL_ERR_BAD_ID, "id %d is outside 0..%d", id, CNL_NUM_IDS - 1);
    std::lock_guard<std::mutex> lock(g_mutex);
    int rc;
    Slot* sp = get_slot(id, &rc);
    if (!sp) return rc;
    CNL_TRY(check_cuda(cudaDeviceSynchronize(), "cudaDeviceSynchronize"));
    if (sp->arena) cudaFree(sp->arena);
    if (sp->cond) cudaFree(sp->cond);
    if (sp->events_ready)
        for (int i = 0; i < Slot::kRing; ++i)
            for (int j = 0; j < 2; ++j) { cudaEventDestroy(sp->ev_fwd[i][j]); cudaEventDestroy(sp->ev_rev[i][j]); }
    const int keep_cond = sp->opt_conditioner, keep_fuse = sp->opt_fuse, keep_rec = sp->opt_recompute, keep_gen = sp->generation;
    const int keep_flow = sp->opt_flow;
    *sp = Slot();
    sp->generation = keep_gen;
    sp->opt_flow = keep_flow;
    sp->opt_conditioner = keep_cond;
    sp->opt_fuse = keep_fuse;
    sp->opt_recompute = keep_rec;
    return CNL_OK;
}

static int read_iterate(int id, int idx, bool checkpoint, float* dst, void* stream) {
    if (id < 0 || id >= CNL_NUM_IDS) return fail(CNL_ERR_BAD_ID, "id %d is outside 0..%d", id, CNL_NUM_IDS - 1);
    if (!dst) return fail(CNL_ERR_NULL, "null destination");
    std::lock_guard<std::mutex> lock(g_mutex);
    int rc;
    Slot* sp = get_slot(id, &rc);
    if (!sp) return rc;
    if (!sp->have_forward) return fail(CNL_ERR_NO_FORWARD, "slot %d holds no forward pass", id);
    const int its_eff = 2 * (sp->its / 2);
    const int limit = checkpoint ? (int)sp->sched.size() : its_eff;
    if (idx < 0 || idx >= limit) return fail(CNL_ERR_BAD_SHAPE, "index %d is outside 0..%d", idx, limit - 1);
    const ArenaLayout L = slot_layout(sp->n, sp->ch, sp->h, sp->pitch, its_eff, sp->sched, sp->recompute, sp->staged);
    if (!checkpoint && sp->recompute) {
        const int first = sp->sched.back();
        if (!sp->window_valid || idx < first)
            return fail(CNL_ERR_NO_FORWARD, "iteration %d is not resident: this forward pass kept checkpoints only", idx);
        idx -= first;
    }
    const float* src = sp->arena + (checkpoint ? L.ckpt : L.hist) + (size_t)idx * L.vol;
    return unpad_rows(dst, src, (size_t)sp->n * sp->ch * sp->h, sp->w, sp->pitch, static_cast<cudaStream_t>(stream));
}

extern "C" int cnl_tv_read_history(int id, int g, float* dst, void* stream) {
    return read_iterate(id, g, false, dst, stream);
}

extern "C" int cnl_tv_read_checkpoint(int id, int k, float* dst, void* stream) {
    return read_iterate(id, k, true, dst, stream);
}

extern "C" int cnl_tv_num_checkpoints(int id) {
    if (id < 0 || id >= CNL_NUM_IDS) { fail(CNL_ERR_BAD_ID, "id %d is outside 0..%d", id, CNL_NUM_IDS - 1); return -1; }
    std::lock_guard<std::mutex> lock(g_mutex);
    int rc;
    Slot* sp = get_slot(id, &rc);
    if (!sp || !sp->have_forward) return -1;
    return (int)sp->sched.size();
}

extern "C" int cnl_tv_set_option(int id, int option, int value) {
    if (id < 0 || id >= CNL_NUM_IDS) return fail(CNL_ERR_BAD_ID, "id %d is outside 0..%d", id, CNL_NUM_IDS - 1);
    if (option < CNL_OPT_CONDITIONER || option > CNL_OPT_FLOW)      // rejected before anything touches the device
        return fail(CNL_ERR_BAD_OPTION, "unknown option %d", option);
    std::lock_guard<std::mutex> lock(g_mutex);
    int rc;
    Slot* sp = get_slot(id, &rc);
    if (!sp) return rc;
    switch (option) {
        case CNL_OPT_CONDITIONER: sp->opt_conditioner = value ? 1 : 0; return CNL_OK;
        case CNL_OPT_TIMING:
            sp->opt_timing = value ? 1 : 0;
            sp->n_fwd = sp->n_rev = 0;
            return CNL_OK;
        case CNL_OPT_RECOMPUTE: sp->opt_recompute = value ? 1 : 0; return CNL_OK;
        case CNL_OPT_FLOW: sp->opt_flow = (value == 2) ? 2 : (value ? 1 : 0); return CNL_OK;
        case CNL_OPT_FUSE:
            if (value < 0 || value > 4) return fail(CNL_ERR_BAD_OPTION, "fuse factor %d is outside 0..4", value);
            sp->opt_fuse = value;
            return CNL_OK;
        default: return fail(CNL_ERR_BAD_OPTION, "unknown option %d", option);
    }
}

extern "C" int cnl_tv_get_timing(int id, double* out_host) {
    if (id < 0 || id >= CNL_NUM_IDS) return fail(CNL_ERR_BAD_ID, "id %d is outside 0..%d", id, CNL_NUM_IDS - 1);
    if (!out_host) return fail(CNL_ERR_NULL, "null output");
    std::lock_guard<std::mutex> lock(g_mutex);
    int rc;
    Slot* sp = get_slot(id, &rc);
    if (!sp) return rc;
    double ms_f = 0, ms_r = 0, lf = 0, lr = 0, itf = 0, itr = 0;
    for (int i = 0; i < sp->n_fwd; ++i) {
        float ms = 0;
        CNL_TRY(check_cuda(cudaEventSynchronize(sp->ev_fwd[i][1]), "cudaEventSynchronize"));
        CNL_TRY(check_cuda(cudaEventElapsedTime(&ms, sp->ev_fwd[i][0], sp->ev_fwd[i][1]), "cudaEventElapsedTime"));
        ms_f += ms; lf += sp->launches_fwd[i]; itf += sp->iters_fwd[i];
    }
    for (int i = 0; i < sp->n_rev; ++i) {
        float ms = 0;
        CNL_TRY(check_cuda(cudaEventSynchronize(sp->ev_rev[i][1]), "cudaEventSynchronize"));
        CNL_TRY(check_cuda(cudaEventElapsedTime(&ms, sp->ev_rev[i][0], sp->ev_rev[i][1]), "cudaEventElapsedTime"));
        ms_r += ms; lr += sp->launches_rev[i]; itr += sp->iters_rev[i];
    }
    out_host[0] = ms_f; out_host[1] = lf; out_host[2] = sp->n_fwd;
    out_host[3] = ms_r; out_host[4] = lr; out_host[5] = sp->n_rev;
    out_host[6] = itf; out_host[7] = itr;
    sp->n_fwd = sp->n_rev = 0;
    return CNL_OK;
}

extern "C" int cnl_tv_run_count(int id) {
    if (id < 0 || id >= CNL_NUM_IDS) { fail(CNL_ERR_BAD_ID, "id %d is outside 0..%d", id, CNL_NUM_IDS - 1); return -1; }
    std::lock_guard<std::mutex> lock(g_mutex);
    int rc;
    Slot* sp = get_slot(id, &rc);
    return sp ? sp->run : -1;
}

extern "C" int cnl_tv_forward_count(int id) {
    if (id < 0 || id >= CNL_NUM_IDS) { fail(CNL_ERR_BAD_ID, "id %d is outside 0..%d", id, CNL_NUM_IDS - 1); return -1; }
    std::lock_guard<std::mutex> lock(g_mutex);
    int rc;
    Slot* sp = get_slot(id, &rc);
    return sp ? sp->generation : -1;
}

extern "C" int cnl_dot_scratch_floats(void) { return 2 * kDotBlocks; }

extern "C" int cnl_tv_lambda_grad(const float* g_c, const float* c_raw, long long count, float* out, float* scratch,
                                  void* stream) {
    if (!g_c || !c_raw || !out || !scratch) return fail(CNL_ERR_NULL, "null pointer argument");
    if (count < 0) return fail(CNL_ERR_BAD_SHAPE, "negative element count");
    if ((reinterpret_cast<size_t>(scratch) & 7) != 0) return fail(CNL_ERR_BAD_SHAPE, "scratch must be 8-byte aligned");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return launch_tv_dot(g_c, c_raw, count, out, scratch, kDotBlocks, nullptr, 0, 1, 0, st);
}

extern "C" int cnl_tv_lambda_grad_allreduce(const float* g_c, const float* c_raw, long long count, float* out, float* scratch,
                                            void* const* peer_bufs, int rank, int world, unsigned long long seq, void* stream) {
    if (!g_c || !c_raw || !out || !scratch) return fail(CNL_ERR_NULL, "null pointer argument");
    if (count < 0) return fail(CNL_ERR_BAD_SHAPE, "negative element count");
    if ((reinterpret_cast<size_t>(scratch) & 7) != 0) return fail(CNL_ERR_BAD_SHAPE, "scratch must be 8-byte aligned");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (!peer_bufs) return fail(CNL_ERR_NULL, "null pointer argument");
    return launch_tv_dot(g_c, c_raw, count, out, scratch, kDotBlocks, peer_bufs, rank, world, seq, st);
}
