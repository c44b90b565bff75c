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

// ---------------------------------------------------------------------------------------
// Programmatic dependent launch.  Every kernel of this engine starts with tw_grid_wait():
// nothing it reads that an earlier kernel wrote, and nothing it writes, is touched before.
// Kernels are launched with the programmatic-serialization attribute, so inside a CUDA graph
// the next kernel's launch overlaps the tail of the one before (measured on B200: 2 % off a
// decode step).  Letting the next kernel become resident even earlier with an explicit
// griddepcontrol.launch_dependents -- at the top of short kernels or after the main loop of long
// ones -- made the step slower (up to 8 %), so tw_grid_launch_dependents() compiles to nothing
// unless TW_PDL_TRIGGERS is defined.  TESSWEAVE_PDL=0 in the environment launches every kernel
// the ordinary way.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void tw_grid_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void tw_grid_launch_dependents() {
#ifdef TW_PDL_TRIGGERS
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
#endif
}
__device__ __forceinline__ void tw_grid_launch_dependents_late() { tw_grid_launch_dependents(); }
// The exception, measured to pay: kernels whose successor is small (or whose own blocks are few) let it
// become resident at once.  Used by the clustered norm and, on request, by the small-M product.
__device__ __forceinline__ void tw_launch_dependents_now() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

#ifndef __CUDA_ARCH__
#include <stdlib.h>
static inline bool tw_pdl_enabled() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("TESSWEAVE_PDL");
        v = (e && e[0] == '0') ? 0 : 1;
    }
    return v != 0;
}
#endif

// Launch `kernel` on `stream`, allowing it to be scheduled before its predecessor has finished
// (the kernel itself waits where it must), optionally as clusters of `cluster_x` blocks.
template <typename... KArgs, typename... Args>
static inline int tw_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                            int cluster_x, Args... args) {
#ifndef __CUDA_ARCH__
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attrs[2];
    int n = 0;
    // only while the stream is being captured into a graph: on plain launches the attribute costs time
    cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
    if (tw_pdl_enabled() && cudaStreamIsCapturing(stream, &capturing) == cudaSuccess &&
        capturing == cudaStreamCaptureStatusActive) {
        attrs[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attrs[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    if (cluster_x > 1) {
        attrs[n].id = cudaLaunchAttributeClusterDimension;
        attrs[n].val.clusterDim.x = cluster_x;
        attrs[n].val.clusterDim.y = 1;
        attrs[n].val.clusterDim.z = 1;
        ++n;
    }
    cfg.attrs = attrs;
    cfg.numAttrs = n;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
    return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
#else
    return 0;
#endif
}
