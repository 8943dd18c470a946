// Weighted-median selection layer for sm_100a: forward and gradient over a channel-last weight volume
// [N, H, W, K] (reference: cudaMedian/cudaCode/medimax.cu, kMedianScore :17-42 and kMedianScoreGrad :44-100).
//
// Both kernels are HBM bound (K floats in, 2 out / K floats in, K out per pixel).  A warp stages the K weights of
// its 32 pixels, which are contiguous in memory, with coalesced loads into shared memory (row stride K|1, odd, so
// the per-thread sequential scans are bank-conflict free), then every thread scans its own row.  With an odd K the
// staged rows have the layout they have in memory, so staging is a straight 16-byte asynchronous copy and the
// write-back a straight 16-byte copy out; an even K goes through a scatter that pads every row by one float.  The
// running sum is the same sequential fp32 sum in bin order as the reference's (the loads of eight bins are issued
// together, the sum still takes them one by one), so the crossing index is bit-identical.
#include "common.h"

namespace cnl {

constexpr int kMedWarps = 4;
constexpr int kMedThreads = kMedWarps * 32;
constexpr int kMedMaxBins = 453;          // 128 staged rows of (k | 1) floats fill the 227 KB of shared memory a block may use

__device__ __forceinline__ int med_stride(int k) { return k | 1; }

// Division of a small index by the number of bins: q = floor(i / k) for 0 <= i < 2^15, 1 <= k <= 1024, with the
// multiplier m = floor(2^32 / k) + 1 (exact because i * k < 2^32); k = 1 has no 32-bit multiplier and is marked by 0.
__device__ __forceinline__ unsigned med_magic(int k) { return k == 1 ? 0u : (unsigned)(0x100000000ULL / (unsigned)k) + 1u; }
__device__ __forceinline__ int med_div(int i, unsigned magic) { return magic ? (int)__umulhi((unsigned)i, magic) : i; }

// Cooperative, coalesced copy of the rows of this warp's 32 pixels (contiguous in memory) into shared memory:
// 16-byte vector loads where the chunk is aligned, scalars otherwise and for the tail.
__device__ __forceinline__ void stage_rows(const float* __restrict__ src, float* __restrict__ dst, long long first_pixel,
                                           long long total_pixels, int k, int lane) {
    const int stride = med_stride(k);
    const unsigned magic = med_magic(k);
    const long long left = total_pixels - first_pixel;
    const int count = (int)(left > 32 ? 32 : left) * k;
    const float* base = src + first_pixel * k;
    const int nvec = (reinterpret_cast<size_t>(base) & 15) == 0 ? count >> 2 : 0;
    if (stride == k) {                                       // odd k: same layout on both sides
        for (int v = lane; v < nvec; v += 32) {
            const unsigned to = (unsigned)__cvta_generic_to_shared(reinterpret_cast<float4*>(dst) + v);
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(to), "l"(reinterpret_cast<const float4*>(base) + v) : "memory");
        }
        for (int i = 4 * nvec + lane; i < count; i += 32) dst[i] = __ldg(base + i);
        asm volatile("cp.async.commit_group;\ncp.async.wait_all;" ::: "memory");
        return;
    }
    for (int v = lane; v < nvec; v += 32) {
        const float4 q = __ldg(reinterpret_cast<const float4*>(base) + v);
        int p = med_div(4 * v, magic), c = 4 * v - p * k;
        dst[p * stride + c] = q.x; if (++c == k) { c = 0; ++p; }
        dst[p * stride + c] = q.y; if (++c == k) { c = 0; ++p; }
        dst[p * stride + c] = q.z; if (++c == k) { c = 0; ++p; }
        dst[p * stride + c] = q.w;
    }
    for (int i = 4 * nvec + lane; i < count; i += 32) {
        const int p = med_div(i, magic);
        dst[p * stride + (i - p * k)] = __ldg(base + i);
    }
}

// The reverse: coalesced write-back of the warp's rows from shared memory.
__device__ __forceinline__ void unstage_rows(const float* __restrict__ rows, float* __restrict__ dst, long long first_pixel,
                                             long long total_pixels, int k, int lane) {
    const int stride = med_stride(k);
    const unsigned magic = med_magic(k);
    const long long left = total_pixels - first_pixel;
    const int count = (int)(left > 32 ? 32 : left) * k;
    float* base = dst + first_pixel * k;
    const int nvec = (reinterpret_cast<size_t>(base) & 15) == 0 ? count >> 2 : 0;
    if (stride == k) {                                       // odd k: same layout on both sides
        for (int v = lane; v < nvec; v += 32) reinterpret_cast<float4*>(base)[v] = reinterpret_cast<const float4*>(rows)[v];
        for (int i = 4 * nvec + lane; i < count; i += 32) base[i] = rows[i];
        return;
    }
    for (int v = lane; v < nvec; v += 32) {
        int p = med_div(4 * v, magic), c = 4 * v - p * k;
        float4 q;
        q.x = rows[p * stride + c]; if (++c == k) { c = 0; ++p; }
        q.y = rows[p * stride + c]; if (++c == k) { c = 0; ++p; }
        q.z = rows[p * stride + c]; if (++c == k) { c = 0; ++p; }
        q.w = rows[p * stride + c];
        reinterpret_cast<float4*>(base)[v] = q;
    }
    for (int i = 4 * nvec + lane; i < count; i += 32) {
        const int p = med_div(i, magic);
        base[i] = rows[p * stride + (i - p * k)];
    }
}

// First bin c with score < 0.5 <= score + p[c] (medimax.cu:30) for the sequential fp32 running sum over the row;
// returns -1 if there is none.  Eight loads per round are issued together.
__device__ __forceinline__ int med_crossing(const float* __restrict__ row, int k, float& p_at, float& score_before) {
    constexpr int G = 8;
    int hit = -1;
    float score = 0.0f;
    p_at = 1.0f;
    score_before = 0.0f;
    for (int c0 = 0; c0 < k && hit < 0; c0 += G) {
        float p[G];
#pragma unroll
        for (int i = 0; i < G; ++i) p[i] = c0 + i < k ? row[c0 + i] : 0.0f;
#pragma unroll
        for (int i = 0; i < G; ++i) {
            const float nxt = score + p[i];
            if (hit < 0 && c0 + i < k && score < 0.5f && nxt >= 0.5f) {
                hit = c0 + i;
                p_at = p[i];
                score_before = score;
            }
            score = nxt;
        }
    }
    return hit;
}

// The same for a row without negative weights, whose running sum never falls: the rounds only add (and look at the
// signs), the first round that ends at or above 0.5 holds the crossing and is walked again for the bin.  `negative`
// reports a weight below zero (or NaN) anywhere in the row; the result is then not to be used.
__device__ __forceinline__ int med_crossing_rising(const float* __restrict__ row, int k, float& p_at, float& score_before,
                                                   bool& negative) {
    constexpr int G = 8;
    int round = -1;
    float score = 0.0f, at_round = 0.0f;
    negative = false;
    for (int c0 = 0; c0 < k; c0 += G) {
        float p[G];
#pragma unroll
        for (int i = 0; i < G; ++i) p[i] = c0 + i < k ? row[c0 + i] : 0.0f;
        float s = score;
#pragma unroll
        for (int i = 0; i < G; ++i) {
            negative |= !(p[i] >= 0.0f);
            s += p[i];
        }
        if (round < 0 && s >= 0.5f) {
            round = c0;
            at_round = score;
        }
        score = s;
    }
    p_at = 1.0f;
    score_before = 0.0f;
    if (round < 0) return -1;
    int hit = -1;
    score = at_round;
#pragma unroll
    for (int i = 0; i < G; ++i) {
        const float p = round + i < k ? row[round + i] : 0.0f;
        const float nxt = score + p;
        if (hit < 0 && round + i < k && nxt >= 0.5f) {          // score < 0.5 holds up to the crossing
            hit = round + i;
            p_at = p;
            score_before = score;
        }
        score = nxt;
    }
    return hit;
}

__global__ void __launch_bounds__(kMedThreads)
median_forward_kernel(const float* __restrict__ vol, float* __restrict__ out, int* __restrict__ index,
                      long long plane, int n_images, int k) {
    extern __shared__ float sh[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const long long total = plane * n_images;
    const long long first = ((long long)blockIdx.x * kMedWarps + warp) * 32;
    if (first >= total) return;
    float* rows = sh + (size_t)warp * 32 * med_stride(k);
    stage_rows(vol, rows, first, total, k, lane);
    __syncwarp();
    const long long pix = first + lane;
    if (pix >= total) return;
    const float* row = rows + lane * med_stride(k);
    float o0 = 0.0f, o1 = 0.0f, p, score;
    bool negative;
    int hit = med_crossing_rising(row, k, p, score, negative);
    if (negative) hit = med_crossing(row, k, p, score);
    if (hit >= 0) {
        const double alpha = (1.0 - 2.0 * (double)score - (double)p) / (2.0 * (double)p);         // :33
        o0 = (float)((double)hit + alpha);                           // :34
        o1 = p;                                                      // :35
    }
    const long long img = pix / plane, off = pix - img * plane;
    out[(img * 2 + 0) * plane + off] = o0;
    out[(img * 2 + 1) * plane + off] = o1;
    if (index) index[pix] = hit;
}

__global__ void __launch_bounds__(kMedThreads)
median_backward_kernel(const float* __restrict__ vol, const float* __restrict__ grad, float* __restrict__ gvol,
                       long long plane, int n_images, int k) {
    extern __shared__ float sh[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const long long total = plane * n_images;
    const long long first = ((long long)blockIdx.x * kMedWarps + warp) * 32;
    if (first >= total) return;
    const int stride = med_stride(k);
    float* rows = sh + (size_t)warp * 32 * stride;
    stage_rows(vol, rows, first, total, k, lane);
    __syncwarp();
    const long long pix = first + lane;
    if (pix < total) {
        float* row = rows + lane * stride;
        const long long img = pix / plane, off = pix - img * plane;
        const float g0 = grad[(img * 2 + 0) * plane + off];
        const float g1 = grad[(img * 2 + 1) * plane + off];
        // pass 1: crossing bin (medimax.cu:55-80)
        float score, pmid, gmid = 0.0f;
        bool negative;
        int hit = med_crossing_rising(row, k, pmid, score, negative);
        if (negative) hit = med_crossing(row, k, pmid, score);
        if (hit >= 0) {
            const float alpha = (float)((1.0 - 2.0 * (double)score - (double)pmid) / (2.0 * (double)pmid));
            gmid = __fadd_rn(__fdiv_rn(__fmul_rn(g0, alpha), -pmid), g1);        // :73, fp32, no contraction
        }
        // pass 2: bins before / after the crossing (:82-99); the row in shared memory is overwritten by its gradient
        const float half = (float)((double)g0 / (2.0 * (double)pmid));
        if (!negative) {
            // the running sum never falls: bins in front of the crossing are the ones the tests below call "before"
            // (nxt < 0.5), bins behind it the ones they call "after" (score >= 0.5); no crossing: all "before"
            const int at = hit < 0 ? k : hit;
            for (int c = 0; c < k; ++c) row[c] = c < at ? -half : (c == at ? gmid : half);
        } else {
            score = 0.0f;
            for (int c0 = 0; c0 < k; c0 += 8) {
                float p[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) p[i] = c0 + i < k ? row[c0 + i] : 0.0f;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float nxt = score + p[i];
                    float g = 0.0f;
                    if (nxt < 0.5f) g = -half;
                    else if (score >= 0.5f) g = half;
                    if (c0 + i == hit) g = gmid;
                    if (c0 + i < k) row[c0 + i] = g;
                    score = nxt;
                }
            }
        }
    }
    __syncwarp();
    unstage_rows(rows, gvol, first, total, k, lane);
}

static int median_check(const void* a, const void* b, int n, int h, int w, int k) {
    if (!a || !b) return fail(CNL_ERR_NULL, "null pointer argument");
    if (n < 1 || h < 1 || w < 1 || k < 1) return fail(CNL_ERR_BAD_SHAPE, "n, h, w, k must be >= 1 (got %d, %d, %d, %d)", n, h, w, k);
    if (k > kMedMaxBins)
        return fail(CNL_ERR_BAD_SHAPE, "at most %d bins are supported (got %d): a block stages %d rows of k floats in shared memory",
                    kMedMaxBins, k, kMedWarps * 32);
    return CNL_OK;
}

static int median_smem(int k) { return kMedWarps * 32 * (k | 1) * (int)sizeof(float); }
static_assert(kMedWarps * 32 * (kMedMaxBins | 1) * (int)sizeof(float) <= 227 * 1024, "staging rows must fit the shared memory of one block");

template <typename Kern>
static int median_prepare(Kern kern, int k) {
    const int bytes = median_smem(k);
    if (bytes > 48 * 1024) return ensure_dynamic_smem(kern, bytes);
    return CNL_OK;
}

}  // namespace cnl

using namespace cnl;

extern "C" int cnl_median_forward(const float* vol, float* out, int* index, int n, int h, int w, int k, void* stream) {
    CNL_TRY(median_check(vol, out, n, h, w, k));
    CNL_TRY(median_prepare(median_forward_kernel, k));
    const long long plane = (long long)h * w;
    const long long warps = (plane * n + 31) / 32;
    const unsigned blocks = (unsigned)((warps + kMedWarps - 1) / kMedWarps);
    median_forward_kernel<<<blocks, kMedThreads, median_smem(k), static_cast<cudaStream_t>(stream)>>>(vol, out, index, plane, n, k);
    return after_launch("median_forward_kernel");
}

extern "C" int cnl_median_backward(const float* vol, const float* grad, float* gvol, int n, int h, int w, int k,
                                   void* stream) {
    CNL_TRY(median_check(vol, gvol, n, h, w, k));
    if (!grad) return fail(CNL_ERR_NULL, "null pointer argument");
    CNL_TRY(median_prepare(median_backward_kernel, k));
    const long long plane = (long long)h * w;
    const long long warps = (plane * n + 31) / 32;
    const unsigned blocks = (unsigned)((warps + kMedWarps - 1) / kMedWarps);
    median_backward_kernel<<<blocks, kMedThreads, median_smem(k), static_cast<cudaStream_t>(stream)>>>(vol, grad, gvol, plane, n, k);
    return after_launch("median_backward_kernel");
}
