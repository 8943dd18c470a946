// Minimal stand-in for the ImageUtilities headers, written from the call sites in the reference's CUDA sources
// (not from ImageUtilities itself), so that the UNMODIFIED reference translation unit compiles with nvcc.
// TEST INFRASTRUCTURE ONLY: used by oracle/build_ref.py to build oracle/_ref/libtvref.so, the reference's own CUDA
// kernels, as a second checker on a GPU box.
//
// Surface provided (what cudaTV/cudaCode/TVInpaintFista.cu uses):
//   iu::TensorGpu_32f(ptr, N, C, H, W, ext, NCHW)   wrap caller memory
//   iu::TensorGpu_32f(N, C, H, W, NCHW)             own allocation
//   .data(), .begin(), .end(), .width(), .height(), .samples(), .channels()
//   conversion to TensorKernelData with operator()(n, c, h, w), coords(idx, &n, &c, &h, &w), fields N, C, H, W, length_
//   iu::ImageGpu_32f_C1(ptr, w, h, pitch, ext=false)   COPIES the data; .begin(), .end(), .getTexture()
//   texture: unnormalised coordinates, clamp addressing, point filtering, element reads
#pragma once
#include <cuda_runtime.h>
#include <thrust/device_ptr.h>
#include <thrust/fill.h>
#include <thrust/functional.h>
#include <thrust/transform.h>

#include <cmath>
#include <cstddef>
#include <cstdio>
#include <cstdlib>
#include <iostream>
#include <vector>

namespace iu {

inline void shim_check(cudaError_t e, const char* what) {
    if (e != cudaSuccess) {
        std::fprintf(stderr, "iu shim: %s: %s\n", what, cudaGetErrorString(e));
        std::abort();
    }
}

class TensorGpu_32f {
public:
    enum MemoryLayout { NCHW, NHWC };

    struct TensorKernelData {
        float* data_;
        unsigned int length_;
        int N, C, H, W;
        __device__ float& operator()(int n, int c, int h, int w) {
            return data_[((static_cast<size_t>(n) * C + c) * H + h) * W + w];
        }
        // linear index -> (n, c, h, w) of the row-major 4-D layout
        template <typename I>
        __device__ void coords(unsigned int idx, I* n, I* c, I* h, I* w) const {
            *w = static_cast<I>(idx % W);
            *h = static_cast<I>((idx / W) % H);
            *c = static_cast<I>((idx / (static_cast<unsigned int>(W) * H)) % C);
            *n = static_cast<I>(idx / (static_cast<unsigned int>(W) * H * C));
        }
    };

    TensorGpu_32f(float* ptr, unsigned int n, unsigned int c, unsigned int h, unsigned int w, bool ext_data_pointer,
                  MemoryLayout)
        : data_(ptr), n_(n), c_(c), h_(h), w_(w), owned_(false) {
        if (!ext_data_pointer) {
            const size_t bytes = static_cast<size_t>(n) * c * h * w * sizeof(float);
            shim_check(cudaMalloc(reinterpret_cast<void**>(&data_), bytes), "cudaMalloc");
            shim_check(cudaMemcpy(data_, ptr, bytes, cudaMemcpyDeviceToDevice), "cudaMemcpy");
            owned_ = true;
        }
    }
    TensorGpu_32f(unsigned int n, unsigned int c, unsigned int h, unsigned int w, MemoryLayout)
        : data_(nullptr), n_(n), c_(c), h_(h), w_(w), owned_(true) {
        shim_check(cudaMalloc(reinterpret_cast<void**>(&data_), static_cast<size_t>(n) * c * h * w * sizeof(float)),
                   "cudaMalloc");
    }
    ~TensorGpu_32f() {
        if (owned_ && data_) cudaFree(data_);
    }
    TensorGpu_32f(const TensorGpu_32f&) = delete;
    TensorGpu_32f& operator=(const TensorGpu_32f&) = delete;

    float* data(int offset = 0) { return data_ + offset; }
    thrust::device_ptr<float> begin() { return thrust::device_pointer_cast(data_); }
    thrust::device_ptr<float> end() { return thrust::device_pointer_cast(data_ + numel()); }
    unsigned int samples() const { return n_; }
    unsigned int channels() const { return c_; }
    unsigned int height() const { return h_; }
    unsigned int width() const { return w_; }
    size_t numel() const { return static_cast<size_t>(n_) * c_ * h_ * w_; }

    operator TensorKernelData() {
        TensorKernelData k;
        k.data_ = data_;
        k.length_ = static_cast<unsigned int>(numel());
        k.N = static_cast<int>(n_);
        k.C = static_cast<int>(c_);
        k.H = static_cast<int>(h_);
        k.W = static_cast<int>(w_);
        return k;
    }

private:
    float* data_;
    unsigned int n_, c_, h_, w_;
    bool owned_;
};

// Single-channel image that always holds a private dense copy of the caller's data and exposes it as a texture.
class ImageGpu_32f_C1 {
public:
    ImageGpu_32f_C1(float* ptr, unsigned int width, unsigned int height, size_t pitch, bool /*ext_data_pointer*/ = false)
        : data_(nullptr), w_(width), h_(height), tex_(0) {
        const size_t row = static_cast<size_t>(width) * sizeof(float);
        shim_check(cudaMalloc(reinterpret_cast<void**>(&data_), row * height), "cudaMalloc");
        shim_check(cudaMemcpy2D(data_, row, ptr, pitch, row, height, cudaMemcpyDeviceToDevice), "cudaMemcpy2D");
    }
    ~ImageGpu_32f_C1() {
        if (tex_) cudaDestroyTextureObject(tex_);
        if (data_) cudaFree(data_);
    }
    ImageGpu_32f_C1(const ImageGpu_32f_C1&) = delete;
    ImageGpu_32f_C1& operator=(const ImageGpu_32f_C1&) = delete;

    thrust::device_ptr<float> begin() { return thrust::device_pointer_cast(data_); }
    thrust::device_ptr<float> end() { return thrust::device_pointer_cast(data_ + static_cast<size_t>(w_) * h_); }

    cudaTextureObject_t getTexture() {
        if (tex_) return tex_;
        cudaResourceDesc res{};
        res.resType = cudaResourceTypePitch2D;
        res.res.pitch2D.devPtr = data_;
        res.res.pitch2D.desc = cudaCreateChannelDesc<float>();
        res.res.pitch2D.width = w_;
        res.res.pitch2D.height = h_;
        res.res.pitch2D.pitchInBytes = static_cast<size_t>(w_) * sizeof(float);
        cudaTextureDesc td{};
        td.addressMode[0] = cudaAddressModeClamp;
        td.addressMode[1] = cudaAddressModeClamp;
        td.filterMode = cudaFilterModePoint;
        td.readMode = cudaReadModeElementType;
        td.normalizedCoords = 0;
        shim_check(cudaCreateTextureObject(&tex_, &res, &td, nullptr), "cudaCreateTextureObject");
        return tex_;
    }

private:
    float* data_;
    unsigned int w_, h_;
    cudaTextureObject_t tex_;
};

}  // namespace iu
