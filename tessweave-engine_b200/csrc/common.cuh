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
// Device-side timeline (-DTW_TIMELINE, off in the product): every block of an instrumented kernel appends
// {kernel id | blocks of its grid << 16, its linear index, start, time after its wait for the kernel before,
// end} to a buffer the host hands over with tw_timeline_set (global timer, ns).  Sorted by time this shows
// how the kernels of a step overlap, where SMs stand idle between them and how long the tails are.
// ---------------------------------------------------------------------------------------
enum : int {
    TW_K_EMBED = 1, TW_K_NORM = 2, TW_K_NORM_CLUSTER = 3, TW_K_ROPE = 4, TW_K_GEMM_SMALLM = 5, TW_K_ATTN_DECODE = 6,
    TW_K_ATTN_PREFILL = 7, TW_K_SAMPLE = 8, TW_K_SILU_MUL = 9, TW_K_REDUCE_PARTIAL = 10, TW_K_OTHER = 11,
};
#ifdef TW_TIMELINE
__device__ unsigned long long* g_tw_timeline = nullptr;      // [0] entries so far, [1] capacity, then 5 words per entry
__device__ __forceinline__ unsigned long long tw_global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
struct TwTimelineScope {
    unsigned long long t0, t1;
    int id;
    __device__ __forceinline__ explicit TwTimelineScope(int id_) : t0(tw_global_ns()), t1(0), id(id_) {}
    __device__ __forceinline__ void mark() { t1 = tw_global_ns(); }
    __device__ __forceinline__ ~TwTimelineScope() {
        if (threadIdx.x == 0 && threadIdx.y == 0 && g_tw_timeline) {
            const unsigned long long i = atomicAdd(g_tw_timeline, 1ull);
            if (i < g_tw_timeline[1]) {
                unsigned long long* e = g_tw_timeline + 2 + 5 * i;
                const unsigned long long nblocks = (unsigned long long)gridDim.x * gridDim.y * gridDim.z;
                e[0] = (unsigned long long)id | (nblocks << 16);
                e[1] = blockIdx.x + (unsigned long long)gridDim.x * (blockIdx.y + (unsigned long long)gridDim.y * blockIdx.z);
                e[2] = t0; e[3] = t1; e[4] = tw_global_ns();
            }
        }
    }
};
#define TW_TIMELINE_SCOPE(id) TwTimelineScope tw_timeline_scope_(id)
#define TW_TIMELINE_MARK() tw_timeline_scope_.mark()
TW_EXPORT int tw_timeline_set(void* buffer) {
    return (int)cudaMemcpyToSymbol(g_tw_timeline, &buffer, sizeof(buffer));
}
#else
#define TW_TIMELINE_SCOPE(id) ((void)0)
#define TW_TIMELINE_MARK() ((void)0)
#endif

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

// A hint to bring this block's share of [ptr, ptr + bytes) into L2: what the next kernel will stream (its
// weights), asked for while this kernel's last blocks finish and the memory system has little to do.  One
// thread issues bulk prefetches of up to 16 KB; `ptr` is 16-byte aligned.  Nothing waits for them.
__device__ __forceinline__ void tw_prefetch_l2_share(const void* ptr, long long bytes) {
    if (!ptr || bytes <= 0) return;
    const long long nblk = (long long)gridDim.x * gridDim.y * gridDim.z;
    const long long b = blockIdx.x + (long long)gridDim.x * (blockIdx.y + (long long)gridDim.y * blockIdx.z);
    const long long share = (((bytes + nblk - 1) / nblk) + 127) & ~127ll;
    const long long beg = b * share;
    long long end = beg + share < bytes ? beg + share : bytes;
    end &= ~15ll;
    for (long long o = beg; o < end; o += 16384) {
        const unsigned size = (unsigned)(end - o < 16384 ? end - o : 16384);
        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"((const char*)ptr + o), "r"(size) : "memory");
    }
}

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
