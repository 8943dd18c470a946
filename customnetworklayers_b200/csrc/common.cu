// Error reporting and launch accounting of the C-ABI library.
#include "common.h"

#include <map>
#include <mutex>
#include <utility>

namespace cnl {

std::atomic<unsigned long long> g_launches{0};

std::string& last_error_ref() {
    static thread_local std::string msg;
    return msg;
}

int fail(int code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    last_error_ref() = buf;
    return code;
}

int ensure_dynamic_smem(const void* kernel, int bytes) {
    static std::mutex mu;
    static std::map<std::pair<const void*, int>, int> done;      // (kernel, device) -> bytes granted
    int dev = 0;
    CNL_TRY(check_cuda(cudaGetDevice(&dev), "cudaGetDevice"));
    std::lock_guard<std::mutex> lock(mu);
    int& granted = done[{kernel, dev}];
    if (granted >= bytes) return CNL_OK;
    CNL_TRY(check_cuda(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes), "cudaFuncSetAttribute"));
    granted = bytes;
    return CNL_OK;
}

}  // namespace cnl

extern "C" const char* cnl_last_error(void) { return cnl::last_error_ref().c_str(); }
extern "C" const char* cnl_version(void) { return "customnetworklayers_b200 0.1 (sm_100a)"; }
extern "C" unsigned long long cnl_launch_count(void) { return cnl::g_launches.load(); }
