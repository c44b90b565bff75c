// Shared helpers of the sm_100a kernels: element types, fp32 conversions,
// warp and block reductions, and the status word that kernels write instead of
// trapping when they meet a bad index.
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

#define TW_EXPORT extern "C" __attribute__((visibility("default")))

// Element type codes shared with the Python side.
enum : int { TW_F32 = 0, TW_BF16 = 1 };

// Error bits in the status word (device memory, one int32, read by the host
// after a step).  A kernel that finds a bad index records it and skips the
// access; it never traps.
enum : int {
    TW_ERR_TOKEN_ID = 1,    // token id outside the vocabulary
    TW_ERR_PAGE = 2,        // block table holds no page where one is needed
    TW_ERR_WAIT = 4,        // a bounded wait ran out
};

__device__ __forceinline__ float tw_to_float(float v) { return v; }
__device__ __forceinline__ float tw_to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T tw_from_float(float v);
template <> __device__ __forceinline__ float tw_from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 tw_from_float<__nv_bfloat16>(float v) {
    return __float2bfloat16_rn(v);
}

__device__ __forceinline__ float tw_warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float tw_warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Block-wide sum; every thread gets the result.  `scratch` holds 33 floats.
__device__ __forceinline__ float tw_block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = tw_warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarps ? scratch[lane] : 0.f;
        t = tw_warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

__device__ __forceinline__ float tw_block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = tw_warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarps ? scratch[lane] : -INFINITY;
        t = tw_warp_max(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

#define TW_LAUNCH_CHECK() (int)cudaGetLastError()
