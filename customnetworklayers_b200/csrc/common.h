// Host-side helpers shared by the translation units of the C-ABI library: error reporting and launch accounting.
#pragma once
#include <cuda_runtime.h>

#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <string>

#include "../../include/cnl_b200.h"

namespace cnl {

std::string& last_error_ref();                       // thread-local message storage
int fail(int code, const char* fmt, ...);            // records the message, returns code
extern std::atomic<unsigned long long> g_launches;   // kernels enqueued since load

inline int check_cuda(cudaError_t e, const char* what) {
    if (e == cudaSuccess) return CNL_OK;
    return fail(CNL_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

// Opts a kernel in to `bytes` of dynamic shared memory once per (kernel, device); the attribute belongs to the device's
// context, so a process that drives several GPUs needs it on each.
int ensure_dynamic_smem(const void* kernel, int bytes);
template <typename K>
inline int ensure_dynamic_smem(K* kernel, int bytes) { return ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), bytes); }

// Counts a launch and turns a launch-configuration error into an error code.
inline int after_launch(const char* kernel) {
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return check_cuda(cudaGetLastError(), kernel);
}

// peer_allreduce.cu: the lambda-gradient reduction out = sum a * b in one launch (scratch: nblocks doubles); with
// peer_bufs non-null the sum over all ranks, exchanged over peer memory inside the same kernel
int launch_tv_dot(const float* a, const float* b, long long count, float* out, float* scratch, int nblocks,
                  void* const* peer_bufs, int rank, int world, unsigned long long seq, cudaStream_t st);

#define CNL_TRY(expr)                 \
    do {                              \
        int _rc = (expr);             \
        if (_rc != CNL_OK) return _rc; \
    } while (0)

}  // namespace cnl
