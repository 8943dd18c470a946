// Register-tiled, temporally blocked TV-FISTA kernels: interface between the host driver and tv_fused.cu.
//
// Geometry shared by the forward and the reverse kernel.  A CTA of 16 warps owns a region of 32 rows x 128 columns
// of one image; warp w owns rows 2w, 2w+1 and lane l owns columns 4l..4l+3 of them, so every global access is one
// aligned 16-byte vector per lane and 512 contiguous bytes per warp.  K iterations are fused per launch: the
// region's outer K rows (4 columns) are a halo that is recomputed redundantly and never written back, so the
// interior that a CTA stores is (32-2K) x 120 pixels.  Horizontal neighbours travel by warp shuffle, vertical
// neighbours across warps through two 512-byte rows of shared memory per warp; all pointwise state of the
// iteration lives in registers.
#pragma once
#include <cuda_runtime.h>

namespace cnl {

constexpr int kFuseMax = 4;          // iterations fused per launch at most (= column halo)
constexpr int kRegionH = 32;
constexpr int kRegionW = 128;
constexpr int kHaloX = 4;
constexpr int kTileW = kRegionW - 2 * kHaloX;     // 120

struct FwdFusedParams {
    const float* y_in;
    const float* x_in;
    float* y_out;
    float* x_out;
    const float* b;
    const float* c;
    const float* wx;
    const float* wy;
    float* hist[kFuseMax];      // destination of x^{g+1/2} for each fused iteration (null: not stored)
    float* ckpt[kFuseMax];      // if non-null: y before fused iteration j is stored here (checkpoint)
    float t[kFuseMax];          // momentum factors
    int N, C, H, W;
    int P;                      // row pitch of every plane in floats (multiple of 4, >= W; pad columns hold zeros)
};

struct RevFusedParams {
    const float* g_in;          // dL/dx^{g+3/2} entering the first fused reverse iteration
    float* g_out;
    const float* acc_in;        // pending momentum term
    float* acc_out;
    const float* b;
    const float* c;
    const float* wx;
    const float* wy;
    const float* hist[kFuseMax + 1];   // hist[j] = x^{g_j+1/2} of fused reverse step j (g_j = g_first - j); hist[K] = one older
    const float* ckpt[kFuseMax];       // if non-null: y is read from here instead of being rebuilt (segment start)
    float t[kFuseMax];
    float* g_c;
    float* g_b;
    float* g_wx;
    float* g_wy;
    float* x1bar;               // if non-null: dL/dx of the last fused step is stored here (init gradient)
    int N, C, H, W;
    int P;                      // row pitch in floats, as in FwdFusedParams
};

// ---- single-launch sweeps (tv_flow.cu) -------------------------------------------------------------------------------
// All time blocks of kFuseMax iterations run in one cooperative launch; tiles of consecutive time blocks are ordered
// through per-tile progress counters in global memory instead of launch boundaries.
constexpr int kFlowMaxIts = 512;     // the per-iteration tables travel as kernel parameters

struct FlowTables {
    float t[kFlowMaxIts];                 // momentum factor of iteration g
    signed char ckpt_slot[kFlowMaxIts];   // index of the checkpoint taken before iteration g, or -1
};

struct FwdFlowParams {
    const float* init;          // y and x entering time block 0
    float* ybuf[2];             // time block kb writes ybuf[kb & 1] and reads ybuf[(kb - 1) & 1]
    float* xbuf[2];
    const float* b;
    const float* c;
    const float* wx;
    const float* wy;
    float* hist;                // x^{g+1/2} of iteration g goes to hist + g * vol
    float* ckpt;                // checkpoint k goes to ckpt + k * vol
    size_t vol;                 // floats between consecutive stored iterates
    int* progress;              // one counter per tile, zero at launch
    int* abort;                 // device word, zero at launch; set when a wait gave up
    int* status;                // host-mapped word that receives the reason
    int nblocks;                // time blocks of kFuseMax iterations (the last one may be shorter)
    int its;                    // iterations of the sweep
    int N, C, H, W;
    int P;                      // row pitch in floats, as in FwdFusedParams
    FlowTables tab;
};

struct RevFlowParams {
    float* gbuf[2];             // time block kb reads gbuf[(kb + 1) & 1] (block 0: the seed) and writes gbuf[kb & 1]
    float* abuf[2];             // same for the pending momentum term
    const float* b;
    const float* c;
    const float* wx;
    const float* wy;
    const float* hist;
    const float* ckpt;
    size_t vol;
    float* g_c;
    float* g_b;
    float* g_wx;
    float* g_wy;
    float* x1bar;               // written by the time block that ends at iteration 0, if this launch reaches it
    int* progress;
    int* abort;
    int* status;
    int g_first;                // iteration of the first reverse step of time block 0
    int nblocks;                // time blocks of kFuseMax reverse steps; the last one ends at iteration 0 and may be shorter
    int N, C, H, W;
    int P;
    FlowTables tab;
};

bool flow_enabled();                       // cooperative launch available and CNL_TV_NO_FLOW not set
int flow_status_take();                    // CNL_OK, or an error if an earlier single-launch sweep gave up a wait
int* flow_status_device_ptr();             // device view of the host-mapped status word of the current device
int flow_tiles(int H, int W, int N);       // tiles (= progress counters) of a launch
int launch_tv_fwd_flow(const FwdFlowParams& p, cudaStream_t st);
int launch_tv_rev_flow(const RevFlowParams& p, cudaStream_t st);

// True if the fused kernels can run directly on these tensors: 16-byte vectors need a row pitch divisible by 4 and
// aligned base pointers.  Otherwise the driver stages zero-padded copies with such a pitch.
bool fused_supported(int W, const void* const* ptrs, int nptr);

// Enqueue K (1..kFuseMax) fused iterations.  Return 0 or a CNL_ERR_* code.
int launch_tv_fwd_fused(const FwdFusedParams& p, int K, cudaStream_t st);
int launch_tv_rev_fused(const RevFusedParams& p, int K, cudaStream_t st);

}  // namespace cnl
