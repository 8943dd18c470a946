// Allocation-free variant of the lambda-gradient reduction  out = sum_i g_c[i] * c_raw[i].
//
// Who needs it: code that runs where device allocation is not allowed or not possible -- a real-time inference
// loop that must not hit the allocator's implicit synchronisation, a host process that hands this library a fixed
// memory carve-out and forbids cudaMalloc, or a plugin loaded into an engine that owns all device memory.  Such a
// caller passes its inputs and its one-float output; the block partials that the two-stage reduction needs live in
// a fixed array inside this library instead of in a caller-provided scratch buffer.
//
// Costs and rules:
//  * every GPU that loads the library holds the array (kStaticSlots doubles = 32 KiB) until the process exits;
//  * at most kStaticMaxCount elements per call (one slot per chunk of kChunk elements); larger inputs are refused;
//  * all calls on a device share the array.  Nothing in it has to start at zero -- each call overwrites exactly
//    the slots it later reads -- but two calls that overlap on the GPU (different streams, or different host
//    threads without ordering) race on it and give wrong sums.  Calls on one stream are safe;
//  * the first call on each device looks the array's device address up (cudaGetSymbolAddress); make that first
//    call outside any stream capture.
#include "common.h"

namespace cnl {

constexpr int kChunk = 4096;                       // elements reduced by one block
constexpr int kStaticSlots = 4096;                 // block partials available
constexpr long long kStaticMaxCount = (long long)kChunk * kStaticSlots;      // 16,777,216 elements
constexpr int kMaxDevices = 64;

// In host code this name is only a handle for the runtime; the device address is fetched once per device below.
static __device__ __align__(256) double g_static_partials[kStaticSlots];

__global__ void __launch_bounds__(256)
tv_dot_chunk_kernel(const float* __restrict__ a, const float* __restrict__ b, long long count,
                    double* __restrict__ partial) {
    const long long base = (long long)blockIdx.x * kChunk;
    double s = 0.0;
#pragma unroll 4
    for (int k = threadIdx.x; k < kChunk; k += 256) {
        const long long i = base + k;
        if (i < count) s += (double)a[i] * (double)b[i];
    }
    for (int off = 16; off > 0; off >>= 1) s += __shfl_down_sync(0xffffffffu, s, off);
    __shared__ double sh[8];
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        double ts = 0.0;
        for (int i = 0; i < 8; ++i) ts += sh[i];
        partial[blockIdx.x] = ts;
    }
}

__global__ void __launch_bounds__(256)
tv_dot_chunk_final_kernel(const double* __restrict__ partial, int nblocks, float* __restrict__ out) {
    double s = 0.0;
    for (int i = threadIdx.x; i < nblocks; i += 256) s += partial[i];
    for (int off = 16; off > 0; off >>= 1) s += __shfl_down_sync(0xffffffffu, s, off);
    __shared__ double sh[8];
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        double ts = 0.0;
        for (int i = 0; i < 8; ++i) ts += sh[i];
        out[0] = (float)ts;
    }
}

static double* g_partials_addr[kMaxDevices] = {};      // device address of g_static_partials, per device ordinal
static std::atomic<int> g_setup_lock{0};

// One-time set-up for the current device: resolves the device address of the static array.
static int static_partials(double** out) {
    int dev = 0;
    CNL_TRY(check_cuda(cudaGetDevice(&dev), "cudaGetDevice"));
    if (dev < 0 || dev >= kMaxDevices) return fail(CNL_ERR_BAD_SHAPE, "device ordinal %d is beyond %d", dev, kMaxDevices - 1);
    while (g_setup_lock.exchange(1, std::memory_order_acquire)) {}
    int rc = CNL_OK;
    if (!g_partials_addr[dev]) {
        void* ptr = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_partials);
        if (e != cudaSuccess || !ptr) rc = fail(CNL_ERR_CUDA, "cudaGetSymbolAddress(static scratch): %s", cudaGetErrorString(e));
        else g_partials_addr[dev] = static_cast<double*>(ptr);
    }
    *out = g_partials_addr[dev];
    g_setup_lock.store(0, std::memory_order_release);
    return rc;
}

}  // namespace cnl

using namespace cnl;

extern "C" long long cnl_tv_lambda_grad_static_max_count(void) { return kStaticMaxCount; }

extern "C" int cnl_tv_lambda_grad_static(const float* g_c, const float* c_raw, long long count, float* out,
                                         void* stream) {
    if (!g_c || !c_raw || !out) return fail(CNL_ERR_NULL, "null pointer argument");
    if (count < 0) return fail(CNL_ERR_BAD_SHAPE, "negative element count");
    if (count > kStaticMaxCount)
        return fail(CNL_ERR_BAD_SHAPE,
                    "cnl_tv_lambda_grad_static handles at most %lld elements (got %lld): use cnl_tv_lambda_grad with "
                    "caller-provided scratch for larger inputs", kStaticMaxCount, count);
    double* partials = nullptr;
    CNL_TRY(static_partials(&partials));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int nblocks = (int)((count + kChunk - 1) / kChunk);
    if (nblocks > 0) {
        tv_dot_chunk_kernel<<<nblocks, 256, 0, st>>>(g_c, c_raw, count, partials);
        CNL_TRY(after_launch("tv_dot_chunk_kernel"));
    }
    tv_dot_chunk_final_kernel<<<1, 256, 0, st>>>(partials, nblocks, out);
    return after_launch("tv_dot_chunk_final_kernel");
}
