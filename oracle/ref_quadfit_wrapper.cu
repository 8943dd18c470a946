// Builds the reference's cudaQuadFit translation unit unmodified (#included from where it lies) and exports its
// two static entry points with C linkage.  TEST INFRASTRUCTURE ONLY.  The output buffer must hold THREE planes per
// image (the reference kernel writes fx, fy and the score, cudaQuadFit/cudaCode/quadFit.cu:123-134).
#include "quadFit.cu"

extern "C" int ref_quadfit_forward(float* f0, float* f1, float* flow, float* out, int in, int ic, int ih, int iw) {
    if (in < 1 || ic < 1 || ih < 1 || iw < 1) return -1;
    const int rc = FlowQuadFitting::forward(f0, f1, flow, out, in, ic, ih, iw);
    return cudaDeviceSynchronize() == cudaSuccess ? rc : -2;
}

extern "C" int ref_quadfit_backward(float* f0, float* f1, float* flow, float* grad, float* g0, float* g1, int in, int ic,
                                    int ih, int iw) {
    if (in < 1 || ic < 1 || ih < 1 || iw < 1) return -1;
    const int rc = FlowQuadFitting::backward(f0, f1, flow, grad, g0, g1, in, ic, ih, iw);
    return cudaDeviceSynchronize() == cudaSuccess ? rc : -2;
}
