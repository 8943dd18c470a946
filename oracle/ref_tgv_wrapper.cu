// Builds the reference's cudaTGV translation unit unmodified (#included from where it lies) and exports its two
// static entry points with C linkage.  TEST INFRASTRUCTURE ONLY.
// Buffers: d_x = [wx, beta_x] and d_y = [wy, beta_y] hold two planes each; init / solution / upstream gradient /
// init gradient hold 3*ic planes (u, v1, v2), as the kernels index them (TGVInpaintFistaBetas.cu:2492-2499, :2650).
// Sizes are restricted to heights % 16 == 0 and widths % 32 == 0 (full thread blocks only).
#include "TGVInpaintFistaBetas.cu"

static bool ref_tgv_shape_ok(int ih, int iw) { return ih > 0 && iw > 0 && ih % 16 == 0 && iw % 32 == 0 && ih < 32768 && iw < 32768; }

extern "C" int ref_tgv_forward(float* d_x, float* d_y, float* d_c, float* d_b, float* d_i, float* d_out, int ic, int ih,
                               int iw, int its, int id) {
    if (!ref_tgv_shape_ok(ih, iw) || its < 2) return -1;
    cudaGetLastError();
    const int rc = FistaTGVHuberB2_id::forward(d_x, d_y, d_c, d_b, d_i, d_out, ic, ih, iw, its, id);
    if (cudaDeviceSynchronize() != cudaSuccess) return -2;
    const cudaError_t pending = cudaGetLastError();      // the reference checks no launch; report what it left behind
    if (pending != cudaSuccess) { std::fprintf(stderr, "reference TGV forward left: %s\n", cudaGetErrorString(pending)); return -3; }
    return rc;
}

extern "C" int ref_tgv_backward(float* d_x, float* d_y, float* d_c, float* d_b, float* d_in_grad, float* g_x, float* g_y,
                                float* g_c, float* g_b, float* g_i, int ic, int ih, int iw, int its, int id) {
    if (!ref_tgv_shape_ok(ih, iw) || its < 2) return -1;
    cudaGetLastError();
    const int rc = FistaTGVHuberB2_id::backward(d_x, d_y, d_c, d_b, d_in_grad, g_x, g_y, g_c, g_b, g_i, ic, ih, iw, its, id);
    if (cudaDeviceSynchronize() != cudaSuccess) return -2;
    const cudaError_t pending = cudaGetLastError();
    if (pending != cudaSuccess) { std::fprintf(stderr, "reference TGV backward left: %s\n", cudaGetErrorString(pending)); return -3; }
    return rc;
}
