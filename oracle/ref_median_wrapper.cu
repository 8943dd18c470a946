// Builds the reference's cudaMedian translation unit unmodified (#included from where it lies) and exports its two
// static entry points with C linkage.  TEST INFRASTRUCTURE ONLY.
// The reference decodes pixel indices correctly only for a batch of one (cudaMedian/cudaCode/medimax.cu:18-22), so
// the wrapper refuses other batch sizes.
#include "medimax.cu"

extern "C" int ref_median_forward(float* d_vol, float* d_out, int in, int ih, int iw, int k) {
    if (in != 1 || ih < 1 || iw < 1 || k < 1) return -1;
    const int rc = MediMax::forward(d_vol, d_out, in, ih, iw, k);
    return cudaDeviceSynchronize() == cudaSuccess ? rc : -2;
}

extern "C" int ref_median_backward(float* d_vol, float* d_in_grad, float* d_out_grad, int in, int ih, int iw, int k) {
    if (in != 1 || ih < 1 || iw < 1 || k < 1) return -1;
    const int rc = MediMax::backward(d_vol, d_in_grad, d_out_grad, in, ih, iw, k);
    return cudaDeviceSynchronize() == cudaSuccess ? rc : -2;
}
