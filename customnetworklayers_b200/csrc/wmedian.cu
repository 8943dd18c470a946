// Learnable weighted-median filter for sm_100a, built around the reference's selection rule
// (cudaMedian/cudaCode/medimax.cu:17-100): k x k window (replicate border), taps sorted by value (stable), the k*k
// normalised weights permuted alike, sequential fp32 running sum, first rank with score < 0.5 <= score + p selected.
// Output = value of the selected tap; the window, the sort and the pass-through input gradient have no counterpart in
// the reference.
//
// The K = k*k window values live in registers; the rank of every tap in the stable ascending order (found by
// comparing it with all others at the start of a run of pixels, then updated incrementally as the window slides)
// places its weight at its sorted position in a thread-private column of shared memory; the scan then runs over
// that column in rank order, i.e. in exactly the order the selection rule prescribes, so the selected index is
// bit-identical to the CPU restatement.  The [N,H,W,K] weight volume of the reference layout is never materialised: HBM traffic is one
// read and one write per pixel, the kernel is bound by the compares.
#include <algorithm>
#include <cstdlib>

#include "common.h"

namespace cnl {
namespace wmed {

constexpr int NT = 128;

// The k*k normalised weights (device memory) are copied to shared memory once per block; every thread then reads them
// with compile-time indices (broadcast).
template <int K>
__device__ __forceinline__ void stage_weights(const float* __restrict__ weights, float* sp) {
    if (threadIdx.x < K) sp[threadIdx.x] = weights[threadIdx.x];
    __syncthreads();
}

template <int KS>
__device__ __forceinline__ void load_window(const float* __restrict__ img, int h, int w, int H, int W, float (&v)[KS * KS]) {
    constexpr int R = KS / 2;
#pragma unroll
    for (int dy = 0; dy < KS; ++dy) {
        const int yy = min(max(h + dy - R, 0), H - 1);
#pragma unroll
        for (int dx = 0; dx < KS; ++dx) {
            const int xx = min(max(w + dx - R, 0), W - 1);
            v[dy * KS + dx] = __ldg(img + (size_t)yy * W + xx);
        }
    }
}

// rank of tap i in the stable ascending order
template <int K>
__device__ __forceinline__ int rank_of(const float (&v)[K], int i_static, float vi) {
    int r = 0;
#pragma unroll
    for (int j = 0; j < K; ++j) {
        if (j < i_static) r += (v[j] <= vi) ? 1 : 0;
        else if (j > i_static) r += (v[j] < vi) ? 1 : 0;
    }
    return r;
}

struct Crossing {
    int rank;          // -1: the weights never reach 0.5
    float pmid, alpha;
};

template <int K>
__device__ __forceinline__ Crossing scan_sorted(const float* __restrict__ sw) {
    Crossing c;
    c.rank = -1; c.pmid = 1.0f; c.alpha = 0.0f;
    float score = 0.0f;
    for (int r = 0; r < K; ++r) {
        const float p = sw[r * NT];
        const float nxt = score + p;
        if (score < 0.5f && nxt >= 0.5f) {                       // medimax.cu:30
            c.rank = r;
            c.pmid = p;
            c.alpha = (float)((1.0 - 2.0 * (double)score - (double)p) / (2.0 * (double)p));     // :33
            break;
        }
        score = nxt;
    }
    return c;
}

template <int KS>
__global__ void __launch_bounds__(NT)
wmedian_forward_kernel(const float* __restrict__ flow, const float* __restrict__ weights, float* __restrict__ out,
                       int* __restrict__ tap, float* __restrict__ alpha, long long total, int H, int W) {
    constexpr int K = KS * KS;
    extern __shared__ unsigned char smem_raw[];
    __shared__ float sp[K];
    stage_weights<K>(weights, sp);
    float* sw = reinterpret_cast<float*>(smem_raw) + threadIdx.x;                      // sw[r * NT]
    unsigned char* sidx = smem_raw + (size_t)K * NT * sizeof(float) + threadIdx.x;     // sidx[r * NT]
    const long long plane = (long long)H * W;
    for (long long idx = (long long)blockIdx.x * NT + threadIdx.x; idx < total; idx += (long long)gridDim.x * NT) {
        const long long img = idx / plane;
        const int pix = (int)(idx - img * plane), h = pix / W, w = pix - h * W;
        const float* src = flow + img * plane;
        float v[K];
        load_window<KS>(src, h, w, H, W, v);
#pragma unroll
        for (int i = 0; i < K; ++i) {
            const int r = rank_of<K>(v, i, v[i]);
            sw[r * NT] = sp[i];
            sidx[r * NT] = (unsigned char)i;
        }
        const Crossing c = scan_sorted<K>(sw);
        int t = -1;
        float o = v[K / 2];                                      // no crossing: the centre value passes through
        if (c.rank >= 0) {
            t = sidx[c.rank * NT];
            const int dy = t / KS - KS / 2, dx = t % KS - KS / 2;
            o = __ldg(src + (size_t)min(max(h + dy, 0), H - 1) * W + min(max(w + dx, 0), W - 1));
        }
        out[idx] = o;
        if (tap) tap[idx] = t;
        if (alpha) alpha[idx] = c.alpha;
    }
}

// Sliding-window variant of the forward kernel.  A thread walks DOWN a run of consecutive pixels of one image column
// (the lanes of a warp take consecutive columns, so every load and store is coalesced) and keeps, per window tap, its
// value and ONE packed word: bits 0-5 the tap's rank in the stable ascending order of the window, then one 3-bit field
// per older window row holding how many taps of that row precede it.  Moving one pixel down
//   * removes the top row: a kept tap's rank drops by its field for that row, and its fields move down one place
//     (five integer instructions per tap, no compares: the counts were found when the tap entered the window);
//   * inserts the new bottom row: one float compare per (kept, new) pair decides which of the two precedes the other
//     and adds either 1 to the kept tap's rank or (1 + one count in the kept tap's row field) to the new tap's word.
// The stable order breaks ties by window index (row-major), which is invariant under the shift; a new tap sits in the
// last row, so an equal kept tap always precedes it, and among equal new taps the left one comes first.  A run starts
// from a window of equal sentinel values, whose ranks and counts are compile-time constants, and slides the k real rows
// in before the first output: the start-up shares the code of the steady state, which keeps the unrolled body inside
// the instruction caches.
constexpr int kRun = 32;                  // pixels per thread of the weight-gradient walk
constexpr int kAhead = 4;                 // rows by which that walk prefetches into L2

__device__ __forceinline__ void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }
constexpr int kRkBits = 6, kCntBits = 3;
constexpr int kFwdThreads = 64, kFwdBlocksPerSm = 8;     // sliding forward kernel: 128 registers, 16 warps per SM
constexpr unsigned kRkMask = (1u << kRkBits) - 1u;

struct WeightTap {        // staged per block: the normalised weight of a tap and the tap's window index
    float p;
    int index;
};

// The sequential scan of the selection rule over the weights in rank order, G entries per round: the loads of a round are
// issued together, the running sum still takes them one by one in rank order.  With weights that are all >= 0
// (`monotone`) the running sum never falls, so the first crossing lies in the first round that ends at or above 0.5:
// the rounds then only add, and the round of the crossing is walked a second time to find the entry.
template <int K, int G, int TPB>
__device__ __forceinline__ Crossing scan_sorted_pairs(const WeightTap* __restrict__ sw, bool monotone, int& index) {
    static_assert(K % G == 0, "the scan takes whole rounds");
    Crossing c;
    c.rank = -1; c.pmid = 1.0f; c.alpha = 0.0f;
    index = -1;
    float before = 0.0f;                                          // the sum in front of the crossing
    if (monotone) {
        int round = -1;
        float score = 0.0f;
#pragma unroll 1
        for (int r0 = 0; r0 < K; r0 += G) {
            float p[G];
#pragma unroll
            for (int i = 0; i < G; ++i) p[i] = sw[(r0 + i) * TPB].p;
            float s = score;
#pragma unroll
            for (int i = 0; i < G; ++i) s += p[i];
            if (s >= 0.5f) {
                round = r0;
                break;
            }
            score = s;
        }
        if (round >= 0) {
            float p[G];
#pragma unroll
            for (int i = 0; i < G; ++i) p[i] = sw[(round + i) * TPB].p;
#pragma unroll
            for (int i = 0; i < G; ++i) {
                const float nxt = score + p[i];
                if (c.rank < 0 && nxt >= 0.5f) {                  // score < 0.5 holds up to the crossing (medimax.cu:30)
                    c.rank = round + i;
                    c.pmid = p[i];
                    before = score;
                }
                score = nxt;
            }
        }
    } else {
        float score = 0.0f;
#pragma unroll 1
        for (int r0 = 0; r0 < K && c.rank < 0; r0 += G) {
            float p[G];
#pragma unroll
            for (int i = 0; i < G; ++i) p[i] = sw[(r0 + i) * TPB].p;
#pragma unroll
            for (int i = 0; i < G; ++i) {
                const float nxt = score + p[i];
                if (c.rank < 0 && score < 0.5f && nxt >= 0.5f) {  // medimax.cu:30
                    c.rank = r0 + i;
                    c.pmid = p[i];
                    before = score;
                }
                score = nxt;
            }
        }
    }
    if (c.rank >= 0) {
        c.alpha = (float)((1.0 - 2.0 * (double)before - (double)c.pmid) / (2.0 * (double)c.pmid));      // :33
        index = sw[c.rank * TPB].index;
    }
    return c;
}

template <int KS>
__global__ void __launch_bounds__(kFwdThreads, kFwdBlocksPerSm)
wmedian_forward_slide_kernel(const float* __restrict__ flow, const float* __restrict__ weights, float* __restrict__ out,
                             int* __restrict__ tap, float* __restrict__ alpha, long long nthreads, int H, int W, int runs,
                             int run_len) {
    constexpr int K = KS * KS, R = KS / 2;
    static_assert(K <= (1 << kRkBits) && KS < (1 << kCntBits) && kRkBits + kCntBits * (KS - 1) <= 32, "packed word too small");
    extern __shared__ unsigned char smem_raw[];
    __shared__ WeightTap sp[K];
    float mine = 0.0f;
    if (threadIdx.x < K) {
        mine = weights[threadIdx.x];
        sp[threadIdx.x].p = mine;
        sp[threadIdx.x].index = threadIdx.x;
    }
    const bool monotone = __syncthreads_and(mine >= 0.0f) != 0;      // no negative (or NaN) weight: the running sum never falls
    WeightTap* sw = reinterpret_cast<WeightTap*>(smem_raw) + threadIdx.x;             // sw[r * kFwdThreads]
    const long long plane = (long long)H * W;
    for (long long tix = (long long)blockIdx.x * kFwdThreads + threadIdx.x; tix < nthreads; tix += (long long)gridDim.x * kFwdThreads) {
        const int w = (int)(tix % W);
        const long long q = tix / W;
        const int run = (int)(q % runs);
        const long long img = q / runs;
        const float* src = flow + img * plane;
        const int h0 = run * run_len;
        const int len = min(run_len, H - h0);
        int coloff[KS];
#pragma unroll
        for (int dx = 0; dx < KS; ++dx) coloff[dx] = min(max(w + dx - R, 0), W - 1);
        // the sentinel window: equal values, so a tap is preceded by the taps of smaller window index
        float v[K];
        unsigned wd[K];
#pragma unroll
        for (int dy = 0; dy < KS; ++dy)
#pragma unroll
            for (int dx = 0; dx < KS; ++dx) {
                unsigned word = (unsigned)(dy * KS + dx);
#pragma unroll
                for (int a = 0; a < dy; ++a) word |= (unsigned)KS << (kRkBits + kCntBits * a);
                v[dy * KS + dx] = 0.0f;
                wd[dy * KS + dx] = word;
            }
        float nxt[KS];                                       // the row that enters with the next slide
        {
            const float* row = src + max(h0 - R, 0) * W;
#pragma unroll
            for (int dx = 0; dx < KS; ++dx) nxt[dx] = __ldg(row + coloff[dx]);
        }
        const long long base = img * plane + w;
        // step s: the window is centred on row h0 - KS + s; the first KS steps only slide the real rows in
#pragma unroll 1
        for (int s = 0; s < KS + len; ++s) {
            const int h = h0 - KS + s;
            if (s >= KS) {
#pragma unroll
                for (int i = 0; i < K; ++i) sw[(wd[i] & kRkMask) * kFwdThreads] = sp[i];
                int t;
                const Crossing c = scan_sorted_pairs<K, KS, kFwdThreads>(sw, monotone, t);
                float o = v[K / 2];                              // no crossing: the centre value passes through
                if (t >= 0) {
                    const int dy = t / KS - R, dx = t % KS - R;
                    o = __ldg(src + min(max(h + dy, 0), H - 1) * W + min(max(w + dx, 0), W - 1));
                }
                const long long at = base + (long long)h * W;
                out[at] = o;
                if (tap) tap[at] = t;
                if (alpha) alpha[at] = c.alpha;
                if (s + 1 >= KS + len) break;
            }
            // --- slide the window one pixel down ---
            // 1. the top row leaves, the others move up one place
#pragma unroll
            for (int dy = 0; dy + 1 < KS; ++dy)
#pragma unroll
                for (int dx = 0; dx < KS; ++dx) {
                    const unsigned old = wd[(dy + 1) * KS + dx];
                    const unsigned below = (old >> kRkBits) & ((1u << kCntBits) - 1u);   // taps of the leaving row below it
                    wd[dy * KS + dx] = ((old >> kCntBits) & ~kRkMask) | ((old - below) & kRkMask);
                    v[dy * KS + dx] = v[(dy + 1) * KS + dx];
                }
            // 2. the new bottom row enters
            unsigned wnew[KS];
#pragma unroll
            for (int nx = 0; nx < KS; ++nx) wnew[nx] = 0u;
#pragma unroll
            for (int nx = 0; nx < KS; ++nx) {
                const float x = nxt[nx];
#pragma unroll
                for (int dy = 0; dy + 1 < KS; ++dy)
#pragma unroll
                    for (int dx = 0; dx < KS; ++dx) {
                        // an equal kept tap has the smaller window index and comes first
                        if (v[dy * KS + dx] <= x) wnew[nx] += (1u << (kRkBits + kCntBits * dy)) + 1u;
                        else wd[dy * KS + dx] += 1u;
                    }
#pragma unroll
                for (int mx = 0; mx < nx; ++mx) {               // among the new taps the left one wins ties
                    if (nxt[mx] <= x) wnew[nx] += 1u;
                    else wnew[mx] += 1u;
                }
            }
#pragma unroll
            for (int nx = 0; nx < KS; ++nx) {
                v[(KS - 1) * KS + nx] = nxt[nx];
                wd[(KS - 1) * KS + nx] = wnew[nx];
            }
            {
                const float* row = src + min(max(h + 2 + R, 0), H - 1) * W;
#pragma unroll
                for (int dx = 0; dx < KS; ++dx) nxt[dx] = __ldg(row + coloff[dx]);
            }
        }
    }
}

// Weight gradient: per problem d/dp in sorted order (medimax.cu:73, :91-95 with the output gradient as g0, g1 = 0),
// scattered back to the taps and accumulated per thread in shared memory, reduced per block in a fixed order.
// The sort is not repeated: a tap precedes the selected one in the stable ascending order exactly when its value is
// smaller, or equal with a smaller window index; the selected tap and the interpolation factor alpha come from the
// forward pass, the weight at the crossing is the selected tap's own weight.
template <int KS>
__global__ void __launch_bounds__(NT)
wmedian_weight_grad_kernel(const float* __restrict__ flow, const float* __restrict__ weights, const int* __restrict__ tap,
                           const float* __restrict__ alpha, const float* __restrict__ grad, double* __restrict__ partial,
                           long long total, int H, int W) {
    constexpr int K = KS * KS;
    extern __shared__ unsigned char smem_raw[];
    __shared__ float sp[K];
    stage_weights<K>(weights, sp);
    float* sacc = reinterpret_cast<float*>(smem_raw) + threadIdx.x;            // sacc[i * NT]
    const long long plane = (long long)H * W;
#pragma unroll
    for (int i = 0; i < K; ++i) sacc[i * NT] = 0.0f;
    for (long long idx = (long long)blockIdx.x * NT + threadIdx.x; idx < total; idx += (long long)gridDim.x * NT) {
        const long long img = idx / plane;
        const int pix = (int)(idx - img * plane), h = pix / W, w = pix - h * W;
        float v[K];
        load_window<KS>(flow + img * plane, h, w, H, W, v);
        const int t = tap[idx];
        const float g0 = grad[idx];
        const float pmid = t >= 0 ? sp[t] : 1.0f;
        const float half = (float)((double)g0 / (2.0 * (double)pmid));
        const float mid = __fdiv_rn(__fmul_rn(g0, alpha[idx]), -pmid);
        float vsel = 0.0f;
#pragma unroll
        for (int i = 0; i < K; ++i) vsel = (i == t) ? v[i] : vsel;
#pragma unroll
        for (int i = 0; i < K; ++i) {
            // no crossing (t < 0): every bin counts as "before"
            const bool before = t < 0 || v[i] < vsel || (v[i] == vsel && i < t);
            sacc[i * NT] += before ? -half : ((i == t) ? mid : half);
        }
    }
    __syncthreads();
    if (threadIdx.x < K) {
        const float* row = reinterpret_cast<float*>(smem_raw) + (size_t)threadIdx.x * NT;
        double s = 0.0;
        for (int t = 0; t < NT; ++t) s += (double)row[t];
        partial[(size_t)blockIdx.x * K + threadIdx.x] = s;
    }
}

// Sliding-window variant of the weight-gradient kernel: a thread walks DOWN kRun pixels of an image column and keeps
// the window in registers (one new window row per pixel instead of K loads) and its per-tap sums in registers too; the
// lanes of a warp take consecutive columns, so every load is coalesced.  Every tap is
// first counted as lying before (-half) or after (+half) the selected one, the selected tap itself as "after"; the
// difference (mid - half) owed to the selected tap goes to a thread-private column of shared memory, because the tap
// index is only known at run time.  The selected tap's value is read back from the image (the forward pass put
// exactly that value out) instead of being picked from the registers with K compares.
template <int KS>
__global__ void __launch_bounds__(NT, 3)
wmedian_weight_grad_slide_kernel(const float* __restrict__ flow, const float* __restrict__ weights, const int* __restrict__ tap,
                                 const float* __restrict__ alpha, const float* __restrict__ grad, double* __restrict__ partial,
                                 long long nthreads, int H, int W, int runs) {
    constexpr int K = KS * KS, R = KS / 2;
    extern __shared__ unsigned char smem_raw[];
    __shared__ float sp[K];
    stage_weights<K>(weights, sp);
    float* sacc = reinterpret_cast<float*>(smem_raw) + threadIdx.x;            // sacc[i * NT]
    const long long plane = (long long)H * W;
    float acc[K];
#pragma unroll
    for (int i = 0; i < K; ++i) {
        acc[i] = 0.0f;
        sacc[i * NT] = 0.0f;
    }
    for (long long tix = (long long)blockIdx.x * NT + threadIdx.x; tix < nthreads; tix += (long long)gridDim.x * NT) {
        const int w = (int)(tix % W);
        const long long q = tix / W;
        const int run = (int)(q % runs);
        const long long img = q / runs;
        const float* src = flow + img * plane;
        const int h0 = run * kRun;
        int coloff[KS];
#pragma unroll
        for (int dx = 0; dx < KS; ++dx) coloff[dx] = min(max(w + dx - R, 0), W - 1);
        float v[K];
#pragma unroll
        for (int dy = 0; dy < KS; ++dy) {
            const float* row = src + min(max(h0 + dy - R, 0), H - 1) * W;
#pragma unroll
            for (int dx = 0; dx < KS; ++dx) v[dy * KS + dx] = __ldg(row + coloff[dx]);
        }
        const int hend = min(h0 + kRun, H);
        const long long base = img * plane + w;
        // value of the tap that the window centred on (h, w) selected; the centre when there was no crossing
        auto selected_value = [&](int t, int h) {
            const int tt = t < 0 ? K / 2 : t;
            return __ldg(src + min(max(h + tt / KS - R, 0), H - 1) * W + min(max(w + tt % KS - R, 0), W - 1));
        };
        // per-pixel operands are fetched ahead (the tap two pixels, the rest one) so that no load latency sits between two pixels
        int t_n = tap[base + (long long)h0 * W];
        int t_nn = h0 + 1 < hend ? tap[base + (long long)(h0 + 1) * W] : -1;
        float g_n = grad[base + (long long)h0 * W], a_n = alpha[base + (long long)h0 * W], vs_n = selected_value(t_n, h0);
#pragma unroll 1
        for (int h = h0; h < hend; ++h) {
            const int t = t_n;
            const float g0 = g_n, al = a_n, vsel = vs_n;
            float nxt[KS];                                   // bottom row of the next pixel's window
            {
                const float* row = src + min(h + 1 + R, H - 1) * W;
#pragma unroll
                for (int dx = 0; dx < KS; ++dx) nxt[dx] = __ldg(row + coloff[dx]);
            }
            {   // rows further down are pulled into L2 ahead of the loads below
                const long long ahead = base + (long long)min(h + kAhead, H - 1) * W;
                prefetch_l2(src + (long long)min(h + kAhead + R, H - 1) * W + w);
                prefetch_l2(tap + ahead);
                prefetch_l2(grad + ahead);
                prefetch_l2(alpha + ahead);
            }
            if (h + 1 < hend) {
                const long long at = base + (long long)(h + 1) * W;
                t_n = t_nn;
                g_n = grad[at];
                a_n = alpha[at];
                vs_n = selected_value(t_n, h + 1);
                if (h + 2 < hend) t_nn = tap[at + W];
            }
            if (t >= 0) {
                const float pmid = sp[t];
                // g0 / (2 pmid) rounded once; the reference divides in double and rounds the quotient to float, which gives
                // the same bits (a quotient of two floats rounded to 53 bits and then to 24 rounds like one rounding)
                const float half = __fdiv_rn(g0, __fmul_rn(2.0f, pmid));
                const float mid = __fdiv_rn(__fmul_rn(g0, al), -pmid);
                sacc[t * NT] += mid - half;
#pragma unroll
                for (int i = 0; i < K; ++i) {
                    const bool before = v[i] < vsel || (v[i] == vsel && i < t);
                    acc[i] += before ? -half : half;
                }
            } else {                                         // no crossing: every bin counts as "before" (weight 1)
                const float half = 0.5f * g0;
#pragma unroll
                for (int i = 0; i < K; ++i) acc[i] -= half;
            }
#pragma unroll
            for (int dx = 0; dx < KS; ++dx) {
#pragma unroll
                for (int dy = 0; dy + 1 < KS; ++dy) v[dy * KS + dx] = v[(dy + 1) * KS + dx];
                v[(KS - 1) * KS + dx] = nxt[dx];
            }
        }
    }
#pragma unroll
    for (int i = 0; i < K; ++i) sacc[i * NT] += acc[i];
    __syncthreads();
    if (threadIdx.x < K) {
        const float* row = reinterpret_cast<float*>(smem_raw) + (size_t)threadIdx.x * NT;
        double s = 0.0;
        for (int t = 0; t < NT; ++t) s += (double)row[t];
        partial[(size_t)blockIdx.x * K + threadIdx.x] = s;
    }
}

// Sum over the per-block partial sums in a fixed order: sixteen interleaved slices of the blocks, then the slices.
__global__ void __launch_bounds__(1024)
wmedian_weight_grad_final_kernel(const double* __restrict__ partial, int nblocks, int K, float* __restrict__ g_p) {
    __shared__ double slice[16][64];
    const int i = threadIdx.x & 63, part = threadIdx.x >> 6;
    double s = 0.0;
    if (i < K)
        for (int b = part; b < nblocks; b += 16) s += partial[(size_t)b * K + i];
    slice[part][i] = s;
    __syncthreads();
    if (part == 0 && i < K) {
        double t = 0.0;
        for (int q = 0; q < 16; ++q) t += slice[q][i];
        g_p[i] = (float)t;
    }
}

// Input gradient, gather form: pixel q collects the upstream gradient of every pixel p in its neighbourhood whose
// selected tap lands on q (after the replicate-border clamp).  Fixed summation order, no atomics.
template <int KS>
__global__ void __launch_bounds__(256)
wmedian_input_grad_kernel(const int* __restrict__ tap, const float* __restrict__ grad, float* __restrict__ g_flow,
                          long long total, int H, int W) {
    constexpr int R = KS / 2;
    const long long plane = (long long)H * W;
    const long long idx = (long long)blockIdx.x * 256 + threadIdx.x;
    if (idx >= total) return;
    const long long img = idx / plane;
    const int pix = (int)(idx - img * plane), qh = pix / W, qw = pix - qh * W;
    const int* tp = tap + img * plane;
    const float* gp = grad + img * plane;
    float s = 0.0f;
    for (int ph = max(qh - R, 0); ph <= min(qh + R, H - 1); ++ph)
        for (int pw = max(qw - R, 0); pw <= min(qw + R, W - 1); ++pw) {
            int t = __ldg(tp + (size_t)ph * W + pw);
            if (t < 0) t = (KS * KS - 1) / 2;                       // no crossing: the centre passed through
            const int th = min(max(ph + t / KS - R, 0), H - 1), tw = min(max(pw + t % KS - R, 0), W - 1);
            if (th == qh && tw == qw) s += __ldg(gp + (size_t)ph * W + pw);
        }
    g_flow[idx] = s;
}

// The same sum from a shared-memory tile of 32 x 32 pixels.  Every window centre of the tile and its halo first marks,
// in a 49-bit mask of the pixel it selected, which of that pixel's K surrounding centres it is (an integer atomic OR, so
// the marks do not depend on timing); every pixel then walks the set bits of its own mask in rising order, which is the
// order in which the kernel above scans the K centres, so the two give the same bits.  A pixel is selected by one
// centre on average, so it adds about one value instead of comparing K; a thread serves four pixels, so that a block
// has enough loads in flight to cover their latency.
template <int KS>
__global__ void __launch_bounds__(256)
wmedian_input_grad_tiled_kernel(const int* __restrict__ tap, const float* __restrict__ grad, float* __restrict__ g_flow,
                                int H, int W) {
    constexpr int R = KS / 2, BW = 32, BH = 32, TW = BW + 2 * R, TH = BH + 2 * R;
    __shared__ unsigned int s_mask[BH][BW][2];
    __shared__ float s_grad[TH][TW];
    const size_t plane = (size_t)H * W;
    const int* tp = tap + (size_t)blockIdx.z * plane;
    const float* gp = grad + (size_t)blockIdx.z * plane;
    const int h0 = blockIdx.y * BH, w0 = blockIdx.x * BW;
    const int tx = threadIdx.x & (BW - 1), ty0 = threadIdx.x / BW;
#pragma unroll
    for (int ty = ty0; ty < BH; ty += 256 / BW) {
        s_mask[ty][tx][0] = 0u;
        s_mask[ty][tx][1] = 0u;
    }
    __syncthreads();
    // all of a thread's centres are fetched before the first is worked on, so that a block waits for memory once
    constexpr int kPer = (TH * TW + 255) / 256;
    int taps[kPer];
    float grads[kPer];
#pragma unroll
    for (int j = 0; j < kPer; ++j) {
        const int i = threadIdx.x + j * 256;
        const int r = i / TW, c = i - r * TW;
        const int ph = h0 - R + r, pw = w0 - R + c;
        const bool inside = i < TH * TW && ph >= 0 && ph < H && pw >= 0 && pw < W;
        taps[j] = inside ? __ldg(tp + (size_t)ph * W + pw) : 0;
        grads[j] = inside ? __ldg(gp + (size_t)ph * W + pw) : 0.0f;
    }
#pragma unroll
    for (int j = 0; j < kPer; ++j) {
        const int i = threadIdx.x + j * 256;
        if (i >= TH * TW) break;
        const int r = i / TW, c = i - r * TW;
        const int ph = h0 - R + r, pw = w0 - R + c;
        if (ph >= 0 && ph < H && pw >= 0 && pw < W) {
            int t = taps[j];
            if (t < 0) t = (KS * KS - 1) / 2;                       // no crossing: the centre passed through
            const int th = min(max(ph + t / KS - R, 0), H - 1), tw = min(max(pw + t % KS - R, 0), W - 1);
            const int qy = th - h0, qx = tw - w0;
            if (qy >= 0 && qy < BH && qx >= 0 && qx < BW) {
                const int bit = (ph - th + R) * KS + (pw - tw + R);     // this centre's place among the K around (th, tw)
                atomicOr(&s_mask[qy][qx][bit >> 5], 1u << (bit & 31));
            }
        }
        s_grad[r][c] = grads[j];
    }
    __syncthreads();
    const int qw = w0 + tx;
    if (qw >= W) return;
#pragma unroll
    for (int ty = ty0; ty < BH; ty += 256 / BW) {
        const int qh = h0 + ty;
        if (qh >= H) break;
        float s = 0.0f;
#pragma unroll
        for (int word = 0; word < 2; ++word) {
            unsigned int m = s_mask[ty][tx][word];
            while (m) {
                const int bit = word * 32 + __ffs(m) - 1;
                m &= m - 1u;
                const int dy = bit / KS, dx = bit - dy * KS;
                s += s_grad[ty + dy][tx + dx];
            }
        }
        g_flow[(size_t)blockIdx.z * plane + (size_t)qh * W + qw] = s;
    }
}

constexpr int kGradBlocks = 592;

// CNL_WMEDIAN_NO_SLIDE=1 selects the one-thread-per-pixel forward kernel (read at every call)
static bool slide_enabled() {
    const char* e = std::getenv("CNL_WMEDIAN_NO_SLIDE");
    return !(e && e[0] == '1');
}

template <int KS>
static int run_forward(const float* flow, const float* wts, float* out, int* tap, float* alpha, long long total, int H, int W,
                       cudaStream_t st) {
    constexpr int K = KS * KS;
    const int smem = K * NT * (int)sizeof(float) + K * NT;
    CNL_TRY(ensure_dynamic_smem(wmedian_forward_kernel<KS>, smem));
    if (slide_enabled()) {
        const int smem_slide = K * kFwdThreads * (int)sizeof(WeightTap);
        CNL_TRY(ensure_dynamic_smem(wmedian_forward_slide_kernel<KS>, smem_slide));
        // Long runs amortise the KS start-up slides; short ones keep every SM busy on small inputs.
        const long long cols = total / H, resident = 148LL * kFwdBlocksPerSm;
        int run_len = 16;
        if ((cols * ((H + 63) / 64) + kFwdThreads - 1) / kFwdThreads >= 4 * resident) run_len = 64;
        else if ((cols * ((H + 31) / 32) + kFwdThreads - 1) / kFwdThreads >= resident) run_len = 32;
        const int runs = (H + run_len - 1) / run_len;
        const long long nthreads = cols * runs;                      // one thread per (image-channel, column, run of rows)
        const unsigned sblocks = (unsigned)std::min<long long>((nthreads + kFwdThreads - 1) / kFwdThreads, 148LL * 128);
        wmedian_forward_slide_kernel<KS><<<sblocks, kFwdThreads, smem_slide, st>>>(flow, wts, out, tap, alpha, nthreads, H, W, runs, run_len);
        return after_launch("wmedian_forward_slide_kernel");
    }
    const unsigned blocks = (unsigned)std::min<long long>((total + NT - 1) / NT, 148LL * 64);
    wmedian_forward_kernel<KS><<<blocks, NT, smem, st>>>(flow, wts, out, tap, alpha, total, H, W);
    return after_launch("wmedian_forward_kernel");
}

template <int KS>
static int run_backward(const float* flow, const float* wts, const int* tap, const float* alpha, const float* grad,
                        float* g_flow, float* g_p, double* scratch, long long total, int H, int W, cudaStream_t st) {
    constexpr int K = KS * KS;
    const int smem = K * NT * (int)sizeof(float);
    CNL_TRY(ensure_dynamic_smem(wmedian_weight_grad_kernel<KS>, smem));
    int blocks;
    if (slide_enabled()) {
        CNL_TRY(ensure_dynamic_smem(wmedian_weight_grad_slide_kernel<KS>, smem));
        const int runs = (H + kRun - 1) / kRun;
        const long long nthreads = total / H * runs;                 // one thread per (image-channel, column, run of rows)
        // every block walks the same number of runs, so the grid is what one wave of the device holds
        static int wave = 0;                                // the GPUs of one process are alike
        if (wave == 0) {
            int per_sm = 0, dev = 0, sms = 0;
            CNL_TRY(check_cuda(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, wmedian_weight_grad_slide_kernel<KS>, NT, smem), "occupancy of the weight-gradient kernel"));
            CNL_TRY(check_cuda(cudaGetDevice(&dev), "cudaGetDevice"));
            CNL_TRY(check_cuda(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev), "SM count"));
            wave = std::max(1, per_sm * sms);
        }
        blocks = (int)std::min<long long>((nthreads + NT - 1) / NT, std::min(kGradBlocks, wave));
        wmedian_weight_grad_slide_kernel<KS><<<blocks, NT, smem, st>>>(flow, wts, tap, alpha, grad, scratch, nthreads, H, W, runs);
        CNL_TRY(after_launch("wmedian_weight_grad_slide_kernel"));
    } else {
        blocks = (int)std::min<long long>((total + NT - 1) / NT, kGradBlocks);
        wmedian_weight_grad_kernel<KS><<<blocks, NT, smem, st>>>(flow, wts, tap, alpha, grad, scratch, total, H, W);
        CNL_TRY(after_launch("wmedian_weight_grad_kernel"));
    }
    wmedian_weight_grad_final_kernel<<<1, 1024, 0, st>>>(scratch, blocks, K, g_p);
    CNL_TRY(after_launch("wmedian_weight_grad_final_kernel"));
    const long long images = total / ((long long)H * W);
    if (images <= 65535) {
        const dim3 grid((W + 31) / 32, (H + 31) / 32, (unsigned)images);
        wmedian_input_grad_tiled_kernel<KS><<<grid, 256, 0, st>>>(tap, grad, g_flow, H, W);
        return after_launch("wmedian_input_grad_tiled_kernel");
    }
    wmedian_input_grad_kernel<KS><<<(unsigned)((total + 255) / 256), 256, 0, st>>>(tap, grad, g_flow, total, H, W);
    return after_launch("wmedian_input_grad_kernel");
}

static int check(int n, int c, int h, int w, int k) {
    if (n < 1 || c < 1 || h < 1 || w < 1) return fail(CNL_ERR_BAD_SHAPE, "n, c, h, w must be >= 1 (got %d, %d, %d, %d)", n, c, h, w);
    if ((long long)h * w > 0x3fffffffLL) return fail(CNL_ERR_BAD_SHAPE, "image beyond the supported range");
    if (k != 3 && k != 5 && k != 7) return fail(CNL_ERR_BAD_SHAPE, "window size must be 3, 5 or 7 (got %d)", k);
    return CNL_OK;
}

}  // namespace wmed
}  // namespace cnl

using namespace cnl;

extern "C" long long cnl_wmedian_scratch_bytes(int k) { return (long long)wmed::kGradBlocks * k * k * (long long)sizeof(double); }

extern "C" int cnl_wmedian_forward(const float* flow, const float* weights, float* out, int* tap, float* alpha, int n,
                                   int c, int h, int w, int k, void* stream) {
    if (!flow || !weights || !out) return fail(CNL_ERR_NULL, "null pointer argument");
    CNL_TRY(wmed::check(n, c, h, w, k));
    const float* wts = weights;
    const long long total = (long long)n * c * h * w;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    switch (k) {
        case 3: return wmed::run_forward<3>(flow, wts, out, tap, alpha, total, h, w, st);
        case 5: return wmed::run_forward<5>(flow, wts, out, tap, alpha, total, h, w, st);
        default: return wmed::run_forward<7>(flow, wts, out, tap, alpha, total, h, w, st);
    }
}

extern "C" int cnl_wmedian_backward(const float* flow, const float* weights, const int* tap, const float* alpha,
                                    const float* grad, float* g_flow, float* g_weights, void* scratch, int n, int c, int h,
                                    int w, int k, void* stream) {
    if (!flow || !weights || !tap || !alpha || !grad || !g_flow || !g_weights || !scratch) return fail(CNL_ERR_NULL, "null pointer argument");
    CNL_TRY(wmed::check(n, c, h, w, k));
    const float* wts = weights;
    const long long total = (long long)n * c * h * w;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    double* sc = static_cast<double*>(scratch);
    switch (k) {
        case 3: return wmed::run_backward<3>(flow, wts, tap, alpha, grad, g_flow, g_weights, sc, total, h, w, st);
        case 5: return wmed::run_backward<5>(flow, wts, tap, alpha, grad, g_flow, g_weights, sc, total, h, w, st);
        default: return wmed::run_backward<7>(flow, wts, tap, alpha, grad, g_flow, g_weights, sc, total, h, w, st);
    }
}
