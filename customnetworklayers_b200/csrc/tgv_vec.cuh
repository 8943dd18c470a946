// Register-tiled TGV-FISTA iteration kernels (one iteration per launch): launch interface.
//
// Geometry.  A CTA of kTgvWarps warps works on a region of kTgvWarps rows x 128 columns of one image: every warp owns
// one row, every lane four consecutive pixels of it (one 16-byte vector per plane).  The first row and the first /
// last lane of the region are halo: they only supply fluxes / neighbour values, so the CTA stores an interior of
// (kTgvWarps - 1) x 120 pixels.  Horizontal neighbours travel by warp shuffle, vertical ones through one
// shared-memory row per warp and plane.  Needs a row pitch divisible by 4 and 16-byte aligned planes; the driver
// stages zero-padded copies of tensors that do not have them.
#pragma once
#include <cuda_runtime.h>

namespace cnl {
namespace tgv {

constexpr int kTgvWarps = 8;
constexpr int kTgvTileW = 120;
constexpr int kTgvTileH = kTgvWarps - 1;

struct FwdVecParams {
    const float* y_in;      // [N][3][C][H][W] momentum variable
    float* y_out;
    float* x;               // primal iterate, updated in place
    float* hist;            // pre-prox iterate of this iteration
    float* ckpt;            // if non-null: y_in is copied here (checkpoint)
    const float* b;         // [N][C][H][W]
    const float* c;         // [N][H][W]
    const float* dx;        // [N][2][H][W] = wx, beta_x
    const float* dy;        // [N][2][H][W] = wy, beta_y
    const float* L;         // [N] 1/Lipschitz per image
    int N, C, H, W;
    int P;                  // row pitch of every plane in floats (multiple of 4, >= W; pad columns hold zeros)
    float t;
};

struct RevVecParams {
    const float* hist_g;    // stored iterate of iteration g
    const float* hist_gm1;  // ... of iteration g-1 (null at g == 0)
    const float* ckpt;      // if non-null: y of iteration g comes from this checkpoint
    const float* g_in;
    float* g_out;
    float* acc;             // pending momentum term, updated in place
    const float* b;
    const float* c;
    const float* dx;
    const float* dy;
    const float* L;
    float* g_c;             // accumulated gradients (added to)
    float* g_b;
    float* g_dx;
    float* g_dy;
    float* x1bar;           // if non-null: dL/dx of this iteration is stored here (last reverse step)
    int N, C, H, W;
    int P;                  // row pitch in floats, as in FwdVecParams
    float t;
    int typo;               // reproduce the reference's factor in the v2 term arriving from the triangle above
};

bool tgv_vec_supported(int W, const void* const* ptrs, int nptr);
int launch_tgv_fwd_vec(const FwdVecParams& p, cudaStream_t st);
int launch_tgv_rev_vec(const RevVecParams& p, cudaStream_t st);

}  // namespace tgv
}  // namespace cnl
