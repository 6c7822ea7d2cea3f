// Shared device helpers of the sm_100a kernels.  Header only; every .cu file of this
// folder is built into a shared library of its own and exports plain C functions that
// take device pointers and a stream and return 0 or an error code.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define NI_DTYPE_F32 0
#define NI_DTYPE_BF16 1

// Error codes of the exported functions: positive = a cudaError_t, negative = ours.
#define NI_OK 0
#define NI_ERR_BAD_ARGUMENT (-1)
#define NI_ERR_UNSUPPORTED_SIZE (-2)
#define NI_ERR_DEVICE_TIMEOUT (-3)

#define NI_EXPORT extern "C" __attribute__((visibility("default")))

#define NI_RETURN_LAUNCH_STATUS()                      \
    do {                                               \
        cudaError_t e__ = cudaGetLastError();          \
        return e__ == cudaSuccess ? NI_OK : (int)e__;  \
    } while (0)

// Streaming multiprocessors of the current device (asked once per device; 148 on a B200).
// Grid sizes and work splits are derived from it, never from a literal.
static inline int ni_sm_count() {
    static int cached[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
    if (cached[dev] <= 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 1;
        cached[dev] = n;
    }
    return cached[dev];
}

template <typename T> __device__ __forceinline__ float ni_to_float(T v);
template <> __device__ __forceinline__ float ni_to_float<float>(float v) { return v; }
template <> __device__ __forceinline__ float ni_to_float<__nv_bfloat16>(__nv_bfloat16 v) {
    return __bfloat162float(v);
}
template <typename T> __device__ __forceinline__ T ni_from_float(float v);
template <> __device__ __forceinline__ float ni_from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 ni_from_float<__nv_bfloat16>(float v) {
    return __float2bfloat16_rn(v);
}

__device__ __forceinline__ float ni_warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float ni_warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads, same value in every thread, fixed order.
// `scratch` holds 32 floats of shared memory.
__device__ __forceinline__ float ni_block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = ni_warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float t = 0.f;
    for (int w = 0; w < nwarps; ++w) t += scratch[w];
    return t;
}
__device__ __forceinline__ float ni_block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = ni_warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float t = scratch[0];
    for (int w = 1; w < nwarps; ++w) t = fmaxf(t, scratch[w]);
    return t;
}
