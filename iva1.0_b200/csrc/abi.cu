// Host-side plumbing shared by every entry point of libivab.so: thread-local error text,
// CUDA error translation, cached device properties, launch counter.
#include <atomic>
#include <cstdarg>
#include <cstdio>

#include "common.cuh"

namespace ivab {

static thread_local char g_err[512] = "";
std::atomic<long long> g_launches{0};

int set_error(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

int check_cuda(cudaError_t e, const char* what) {
    if (e == cudaSuccess) return IVAB_OK;
    return set_error(IVAB_ERR_CUDA, "%s: %s (%s)", what, cudaGetErrorName(e), cudaGetErrorString(e));
}

int sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

size_t dtype_size(int dtype) {
    switch (dtype) {
        case IVAB_F32: return 4;
        case IVAB_F16: return 2;
        case IVAB_BF16: return 2;
        case IVAB_F8E4M3: return 1;
        default: return 0;
    }
}

}  // namespace ivab

extern "C" {

const char* ivab_last_error(void) { return ivab::g_err; }

int ivab_version(void) { return 111; }   // 111: peer exchange buffers carry a staging area instead of arrival counters

int64_t ivab_launch_count(void) { return ivab::g_launches.load(); }

}  // extern "C"
