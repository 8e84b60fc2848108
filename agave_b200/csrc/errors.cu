// Error message storage for the exported C functions.
#include "common.cuh"
#include <string.h>

static thread_local char g_msg[1024] = "";

int g_agv_pdl = 1;

// Turns programmatic dependent launch of this library's kernels on (1) or off (0);
// returns the previous setting.
AGV_API int agv_set_dependent_launch(int on) {
    const int old = g_agv_pdl;
    g_agv_pdl = on ? 1 : 0;
    return old;
}

int agv_fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_msg, sizeof(g_msg), fmt, ap);
    va_end(ap);
    return code;
}

// The message of the last failed call on this thread.
AGV_API const char* agv_last_error() { return g_msg; }

// Compute capability of the current device as major * 10 + minor, or a
// negative code.
AGV_API int agv_device_arch() {
    int dev = 0, major = 0, minor = 0;
    AGV_CUDA_OK(cudaGetDevice(&dev));
    AGV_CUDA_OK(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
    AGV_CUDA_OK(cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev));
    return major * 10 + minor;
}
