// Builds the reference's cudaTV translation unit unmodified (it is #included from where it lies, never copied) and
// exports its two static entry points with C linkage.  TEST INFRASTRUCTURE ONLY.
//
// The reference's pybind binding calls a class `TVInpaint` that is never defined
// (cudaTV/TVInpaintFista_cuda.cpp:10-20); the class the sources define is `TVInpaintFista`
// (cudaTV/cudaCode/TVInpaintFista.cu:1463, :1570), which is what is called here.
//
// The reference kernels read `d_y(n, ch, h, w)` before their bounds check (TVInpaintFista.cu:615, :888), so they
// are only safe when the image height is a multiple of 16 and the width a multiple of 32; ref_tv_* refuse other
// sizes (return -1) instead of launching.
#include "TVInpaintFista.cu"

static bool ref_shape_ok(int ih, int iw) { return ih > 0 && iw > 0 && ih % 16 == 0 && iw % 32 == 0 && ih < 32768 && iw < 32768; }

extern "C" int ref_tv_forward(float* d_x, float* d_y, float* d_c, float* d_b, float* d_i, float* d_out, int ic, int ih,
                              int iw, int its, int id) {
    if (!ref_shape_ok(ih, iw) || its < 2) return -1;
    const int rc = TVInpaintFista::forward(d_x, d_y, d_c, d_b, d_i, d_out, ic, ih, iw, its, id);
    const cudaError_t e = cudaDeviceSynchronize();
    return e == cudaSuccess ? rc : -2;
}

extern "C" int ref_tv_backward(float* d_x, float* d_y, float* d_c, float* d_b, float* d_in_grad, float* g_x, float* g_y,
                               float* g_c, float* g_b, float* g_i, int ic, int ih, int iw, int its, int id) {
    if (!ref_shape_ok(ih, iw) || its < 2) return -1;
    const int rc = TVInpaintFista::backward(d_x, d_y, d_c, d_b, d_in_grad, g_x, g_y, g_c, g_b, g_i, ic, ih, iw, its, id);
    const cudaError_t e = cudaDeviceSynchronize();
    return e == cudaSuccess ? rc : -2;
}
