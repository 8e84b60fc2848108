// Shared helpers of the sm_100a kernels: error reporting to the host caller,
// element types, warp and block reductions.
//
// Every exported function returns 0 or a negative code and leaves a message
// that agv_last_error() returns; nothing here aborts or traps.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>
#include <utility>

#define AGV_API extern "C" __attribute__((visibility("default")))

enum AgvDtype { AGV_F32 = 0, AGV_BF16 = 1 };

// Sets the calling thread's error message and returns code (host only).
int agv_fail(int code, const char* fmt, ...);

#define AGV_REQUIRE(cond, ...)                         \
    do {                                               \
        if (!(cond)) return agv_fail(-1, __VA_ARGS__); \
    } while (0)

#define AGV_CUDA_OK(expr)                                                              \
    do {                                                                               \
        cudaError_t e_ = (expr);                                                       \
        if (e_ != cudaSuccess)                                                         \
            return agv_fail(-2, "%s failed: %s", #expr, cudaGetErrorString(e_));       \
    } while (0)

#define AGV_LAUNCH_OK(name)                                                            \
    do {                                                                               \
        cudaError_t e_ = cudaGetLastError();                                           \
        if (e_ != cudaSuccess)                                                         \
            return agv_fail(-3, "launch of %s failed: %s", name, cudaGetErrorString(e_)); \
    } while (0)

static inline bool agv_aligned(const void* p, size_t a) { return ((uintptr_t)p % a) == 0; }

// ------------------------------------------------- programmatic dependent launch
// Every kernel is launched so that it may start while the kernel before it on
// the stream is still draining: its CTAs are scheduled and run whatever does not
// depend on earlier results, then pdl_wait() blocks until the earlier kernel has
// finished and its writes are visible.  Before its pdl_wait() a kernel reads only what
// no kernel of the step writes (weights, what the host copied in at the start of the
// step, cache rows of earlier steps) and writes nothing to global memory.
// pdl_launch_next() lets the kernel after this one be scheduled.
__device__ __forceinline__ void pdl_wait() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
}
// Every kernel lets its successor in as soon as it runs: the successor's CTAs set up,
// read what does not depend on this kernel (weights, step metadata) and then wait.
__device__ __forceinline__ void pdl_launch_next() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

extern int g_agv_pdl;      // 1: launches carry the programmatic-serialization attribute

template <typename... KArgs, typename... Args>
inline void agv_launch(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem,
                       cudaStream_t stream, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = g_agv_pdl ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    (void)cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);   // error: cudaGetLastError
}

// The same with the CTAs grouped into thread-block clusters.
template <typename... KArgs, typename... Args>
inline void agv_launch_cluster(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem,
                               cudaStream_t stream, dim3 cluster, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = g_agv_pdl ? 1 : 0;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = cluster.x;
    attr[1].val.clusterDim.y = cluster.y;
    attr[1].val.clusterDim.z = cluster.z;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    (void)cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

// ---------------------------------------------------------------- element types
__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
    return __float2bfloat16_rn(v);
}

// ------------------------------------------------------------------ reductions
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.
// `scratch` holds 33 floats of shared memory; safe to call repeatedly.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarps ? scratch[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarps ? scratch[lane] : -INFINITY;
        t = warp_max(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}
