// Matrix products with few rows (decode steps): out[m, n] = sum_k x[m, k] * w[n, k] for
// m <= 64, bf16 operands, fp32 accumulation.  The product is bound by reading w once, so
// the kernel streams w straight from global memory into tensor-core fragments.
//
// The weights are the 16-row operand of mma.m16n8k16, the (up to 8) tokens of an n-tile the
// other one ("swap-AB").  A thread reads 16 contiguous bytes (8 values of k) of its two
// weight rows and of its token row per 32 values of k; since a dot product does not care
// about the order of k, each group of 4 values feeds one MMA without any shuffle or shared
// memory: k-slot (2c + j) is element j of the group and slot (2c + 8 + j) is element 2 + j, for
// the weights and for the tokens alike.  (The kernel reads 32 bytes per row and step, so that
// the four threads of a row cover a whole 128-byte line, and keeps two steps in flight.)
//
// When a matrix has too few rows to fill the GPU, k is split over blockIdx.y and each slice
// writes fp32 partial sums to scratch memory [slice][token][n]; the kernels that consume the
// result (residual add + norm, bias + rotary + cache write) add the slices in a fixed order.
//
// A caller may name the weights that the kernel after this one streams (`next_weights`): every block asks for
// its share of them to be brought into L2 when its own stream is over, so that the memory system has work
// while the last blocks finish and the next kernel starts (gate/up before down, 7B-size layer: 0.7 % of a step).
//
// The reference runs these products through a library (nn.Linear: flow_engine/model.py:54,
// 76-80,201,204).
#include "common.cuh"

namespace {

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// streaming 16-byte load: the weights are read once, keep them out of L1
__device__ __forceinline__ uint4 ld_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

#ifndef TW_GEMM_WARPS
#define TW_GEMM_WARPS 4
#endif
constexpr int WARPS = TW_GEMM_WARPS;
constexpr int ROWS_PER_BLOCK = WARPS * 16;
constexpr int CHUNK = 64;      // values of k per step: a thread reads 32 contiguous bytes of each of its rows

enum : int { OUT_BF16 = 0, OUT_F32 = 1, OUT_PARTIAL = 2, OUT_SILU_MUL = 3, OUT_EARLY_DEPENDENTS = 16 /* flag, or-ed in */ };

struct Frag {          // 16 consecutive values of k of one row
    uint4 lo, hi;
};

// KS = 1: the block's four warps take four 16-row tiles.  KS = 2: two tiles, each by two warps that
// share its values of k and add their sums through shared memory: twice the warps for a matrix with few
// row tiles whose k cannot be split over blocks (the SiLU.mul output needs whole sums): 27,648 x 5,120
// at 8 rows 52 -> 45 us.
template <int NT, int KS>
__global__ void __launch_bounds__(WARPS * 32, (NT == 1 ? 5 : 0))
gemm_smallm_kernel(const bf16* __restrict__ w, const bf16* __restrict__ x, int M, int N, int K, int kper,
                   void* __restrict__ out, int out_mode, int out_stride, const void* next_weights, long long next_bytes) {
    constexpr int TILES = WARPS / KS;                  // 16-row tiles of a block
    __shared__ float s_part[KS > 1 ? TILES * 32 * NT * 4 : 1];
    TW_TIMELINE_SCOPE(TW_K_GEMM_SMALLM);
    tw_grid_wait();
    TW_TIMELINE_MARK();
    // With OUT_EARLY_DEPENDENTS the kernel launched after this one may become resident right away (it waits
    // for this kernel's results itself).  That pays when the next kernel is small, like the residual add +
    // norm after the o_proj and down products (measured: 0.5 % of a decode step); before the attention or
    // another large product it costs more than it gives, so the caller decides.
    if (out_mode & OUT_EARLY_DEPENDENTS) tw_launch_dependents_now();
    out_mode &= ~OUT_EARLY_DEPENDENTS;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, c = lane & 3;
    const int tile = warp % TILES, khalf = warp / TILES;
    const int r0 = blockIdx.x * (TILES * 16) + tile * 16;
    if (KS == 1 && r0 >= N) return;
    const int kbeg0 = blockIdx.y * kper, kend0 = min(K, kbeg0 + kper);
    // with KS > 1: this warp's share of the block's values of k, in whole steps
    const int span = KS > 1 ? ((kend0 - kbeg0 + KS - 1) / KS + CHUNK - 1) / CHUNK * CHUNK : 0;
    const int kbeg = KS > 1 ? kbeg0 + khalf * span : kbeg0;
    const int kend = KS > 1 ? min(kend0, kbeg + span) : kend0;
    const int ra = r0 + g, rb = r0 + g + 8;
    const bool va = ra < N && (KS == 1 || kbeg < kend), vb = rb < N && (KS == 1 || kbeg < kend);
    const bf16* wa = w + (size_t)(va ? ra : 0) * K;
    const bf16* wb = w + (size_t)(vb ? rb : 0) * K;
    const bf16* xr[NT];
    bool vx[NT];
#pragma unroll
    for (int t = 0; t < NT; ++t) {
        vx[t] = t * 8 + g < M;
        xr[t] = x + (size_t)(vx[t] ? t * 8 + g : 0) * K;
    }
    float acc[NT][4];
#pragma unroll
    for (int t = 0; t < NT; ++t) { acc[t][0] = acc[t][1] = acc[t][2] = acc[t][3] = 0.f; }
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);

    // kk .. kk + 15 are this thread's values of k in the step that starts at k0
    auto load_w = [&](const bf16* row, bool valid, int k0) -> Frag {
        const int kk = k0 + 16 * c;
        Frag f;
        f.lo = (valid && kk < kend) ? ld_stream(row + kk) : zero;
        f.hi = (valid && kk + 8 < kend) ? ld_stream(row + kk + 8) : zero;
        return f;
    };
    auto load_x = [&](const bf16* row, bool valid, int k0) -> Frag {
        const int kk = k0 + 16 * c;
        Frag f;
        f.lo = (valid && kk < kend) ? *reinterpret_cast<const uint4*>(row + kk) : zero;
        f.hi = (valid && kk + 8 < kend) ? *reinterpret_cast<const uint4*>(row + kk + 8) : zero;
        return f;
    };

    Frag a_cur = load_w(wa, va, kbeg), b_cur = load_w(wb, vb, kbeg);
    Frag a_nxt = load_w(wa, va, kbeg + CHUNK), b_nxt = load_w(wb, vb, kbeg + CHUNK);
    if constexpr (NT == 1) {
        // Up to 8 tokens: their values come one step ahead as well.  They are shared by all blocks and sit in L1
        // or L2, but a matrix with few values of k per warp (o_proj and q/k/v at batch 8: six steps) would
        // otherwise wait one L2 round trip in every step.
        Frag x_nxt = load_x(xr[0], vx[0], kbeg);
        for (int k = kbeg; k < kend; k += CHUNK) {
            const Frag a_far = load_w(wa, va, k + 2 * CHUNK), b_far = load_w(wb, vb, k + 2 * CHUNK);
            const Frag xf = x_nxt;
            x_nxt = load_x(xr[0], vx[0], k + CHUNK);
            mma_bf16(acc[0], a_cur.lo.x, b_cur.lo.x, a_cur.lo.y, b_cur.lo.y, xf.lo.x, xf.lo.y);
            mma_bf16(acc[0], a_cur.lo.z, b_cur.lo.z, a_cur.lo.w, b_cur.lo.w, xf.lo.z, xf.lo.w);
            mma_bf16(acc[0], a_cur.hi.x, b_cur.hi.x, a_cur.hi.y, b_cur.hi.y, xf.hi.x, xf.hi.y);
            mma_bf16(acc[0], a_cur.hi.z, b_cur.hi.z, a_cur.hi.w, b_cur.hi.w, xf.hi.z, xf.hi.w);
            a_cur = a_nxt; b_cur = b_nxt;
            a_nxt = a_far; b_nxt = b_far;
        }
    } else {
        for (int k = kbeg; k < kend; k += CHUNK) {
            // two steps ahead: the loads of step k + 2 CHUNK are in flight while step k is multiplied
            const Frag a_far = load_w(wa, va, k + 2 * CHUNK), b_far = load_w(wb, vb, k + 2 * CHUNK);
#pragma unroll
            for (int t = 0; t < NT; ++t) {
                const Frag xf = load_x(xr[t], vx[t], k);
                mma_bf16(acc[t], a_cur.lo.x, b_cur.lo.x, a_cur.lo.y, b_cur.lo.y, xf.lo.x, xf.lo.y);
                mma_bf16(acc[t], a_cur.lo.z, b_cur.lo.z, a_cur.lo.w, b_cur.lo.w, xf.lo.z, xf.lo.w);
                mma_bf16(acc[t], a_cur.hi.x, b_cur.hi.x, a_cur.hi.y, b_cur.hi.y, xf.hi.x, xf.hi.y);
                mma_bf16(acc[t], a_cur.hi.z, b_cur.hi.z, a_cur.hi.w, b_cur.hi.w, xf.hi.z, xf.hi.w);
            }
            a_cur = a_nxt; b_cur = b_nxt;
            a_nxt = a_far; b_nxt = b_far;
        }
    }
    tw_grid_launch_dependents_late();     // the stream of weights is over: the next kernel may be scheduled
    if (threadIdx.x == WARPS * 32 - 1) tw_prefetch_l2_share(next_weights, next_bytes);
    if (KS > 1) {
        // the warps of the later values of k hand their sums to the first warp of their tile
        float* mine = s_part + (tile * 32 + lane) * NT * 4;
        if (khalf > 0) {
#pragma unroll
            for (int t = 0; t < NT; ++t) { mine[4 * t] = acc[t][0]; mine[4 * t + 1] = acc[t][1]; mine[4 * t + 2] = acc[t][2]; mine[4 * t + 3] = acc[t][3]; }
        }
        __syncthreads();
        if (khalf > 0) return;
#pragma unroll
        for (int t = 0; t < NT; ++t) { acc[t][0] += mine[4 * t]; acc[t][1] += mine[4 * t + 1]; acc[t][2] += mine[4 * t + 2]; acc[t][3] += mine[4 * t + 3]; }
    }
    const bool wa_ok = ra < N, wb_ok = rb < N;        // rows of the matrix (va / vb also say whether this warp had values of k)
    // acc[t][0..1]: weight row ra, tokens t*8 + 2c, +1;  acc[t][2..3]: weight row rb
#pragma unroll
    for (int t = 0; t < NT; ++t) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int tok = t * 8 + 2 * c + e;
            if (tok >= M) continue;
            if (out_mode == OUT_SILU_MUL) {
                // weight rows come in groups of 16: eight gate rows, then the eight up rows that belong to
                // them, so row ra is a gate and row rb its up: out[tok, r0 / 2 + g] = silu(gate) * up
                if (wb_ok) {
                    const float gt = acc[t][e], up = acc[t][2 + e];
                    reinterpret_cast<bf16*>(out)[(size_t)tok * out_stride + (r0 >> 1) + g] =
                        __float2bfloat16_rn(gt / (1.0f + expf(-gt)) * up);
                }
            } else if (out_mode == OUT_BF16) {
                bf16* o = reinterpret_cast<bf16*>(out) + (size_t)tok * out_stride;
                if (wa_ok) o[ra] = __float2bfloat16_rn(acc[t][e]);
                if (wb_ok) o[rb] = __float2bfloat16_rn(acc[t][2 + e]);
            } else {
                float* o = reinterpret_cast<float*>(out) +
                           (out_mode == OUT_PARTIAL ? ((size_t)blockIdx.y * M + tok) * out_stride : (size_t)tok * out_stride);
                if (wa_ok) o[ra] = acc[t][e];
                if (wb_ok) o[rb] = acc[t][2 + e];
            }
        }
    }
}

// Sum of the slices into a dense result (for consumers that cannot add slices themselves).
template <typename T>
__global__ void reduce_partial_kernel(T* __restrict__ out, const float* __restrict__ partial, int nsplit, long total) {
    TW_TIMELINE_SCOPE(TW_K_REDUCE_PARTIAL);
    tw_grid_wait();
    TW_TIMELINE_MARK();
    tw_grid_launch_dependents();
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    // the order every consumer of a split product uses: whole groups of four slices into four sums by slice mod 4,
    // the rest into the first, then (s0 + s1) + (s2 + s3)
    float s[4] = {0.f, 0.f, 0.f, 0.f};
    int i = 0;
    for (; i + 4 <= nsplit; i += 4) {
#pragma unroll
        for (int u = 0; u < 4; ++u) s[u] += partial[(size_t)(i + u) * total + idx];
    }
    for (; i < nsplit; ++i) s[0] += partial[(size_t)i * total + idx];
    out[idx] = tw_from_float<T>((s[0] + s[1]) + (s[2] + s[3]));
}

}  // namespace

// out_mode 0: bf16 [M, out_stride]; 1: fp32 [M, out_stride]; 2: fp32 partial sums [ksplit, M, out_stride]
// (then kper < K); 3: bf16 [M, out_stride] = silu(gate) * up for weights whose rows alternate between eight
// gate rows and their eight up rows (N a multiple of 16, no split).  K must be a multiple of 8; kper of 32.
TW_EXPORT int tw_gemm_smallm(const void* w, const void* x, int M, int N, int K, int kper, void* out, int out_mode,
                             int out_stride, const void* next_weights, long long next_bytes, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if ((uintptr_t)next_weights & 15) return (int)cudaErrorMisalignedAddress;
    if (!next_weights || next_bytes < 0) next_bytes = 0;
    if (M > 64 || K <= 0 || (K & 7) || kper <= 0 || (kper & 31) || (out_mode & ~OUT_EARLY_DEPENDENTS) < 0 || (out_mode & ~OUT_EARLY_DEPENDENTS) > 3 || ((out_mode & ~OUT_EARLY_DEPENDENTS) == OUT_SILU_MUL && (N & 15)))
        return (int)cudaErrorInvalidValue;
    const int ksplit = (K + kper - 1) / kper;
    if (ksplit > 1 && (out_mode & ~OUT_EARLY_DEPENDENTS) != OUT_PARTIAL) return (int)cudaErrorInvalidValue;
    dim3 grid((N + ROWS_PER_BLOCK - 1) / ROWS_PER_BLOCK, ksplit);
    const bf16* wp = (const bf16*)w;
    const bf16* xp = (const bf16*)x;
    static int sm_count = 0;
    if (!sm_count) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sm_count <= 0) sm_count = 148;
    }
    // few blocks for the GPU (under 3.2 per SM, five fit) and enough k for two warps: two warps per row tile
    const bool pair_warps = M <= 8 && (long)grid.x * grid.y * 10 <= (long)sm_count * 32 && kper >= 512;
    if (pair_warps) {
        grid.x = (N + (WARPS / 2) * 16 - 1) / ((WARPS / 2) * 16);
        tw_launch(gemm_smallm_kernel<1, 2>, dim3(grid), dim3(WARPS * 32), 0, stream, 1, wp, xp, M, N, K, kper, out, out_mode, out_stride,
                  next_weights, next_bytes);
    } else if (M <= 8)
        tw_launch(gemm_smallm_kernel<1, 1>, dim3(grid), dim3(WARPS * 32), 0, stream, 1, wp, xp, M, N, K, kper, out, out_mode, out_stride,
                  next_weights, next_bytes);
    else if (M <= 16)
        tw_launch(gemm_smallm_kernel<2, 1>, dim3(grid), dim3(WARPS * 32), 0, stream, 1, wp, xp, M, N, K, kper, out, out_mode, out_stride,
                  next_weights, next_bytes);
    else if (M <= 32)
        tw_launch(gemm_smallm_kernel<4, 1>, dim3(grid), dim3(WARPS * 32), 0, stream, 1, wp, xp, M, N, K, kper, out, out_mode, out_stride,
                  next_weights, next_bytes);
    else
        tw_launch(gemm_smallm_kernel<8, 1>, dim3(grid), dim3(WARPS * 32), 0, stream, 1, wp, xp, M, N, K, kper, out, out_mode, out_stride,
                  next_weights, next_bytes);
    return TW_LAUNCH_CHECK();
}

TW_EXPORT int tw_reduce_partial(void* out, const float* partial, int nsplit, long total, int dtype, cudaStream_t stream) {
    if (total <= 0) return 0;
    const int blocks = (int)((total + 255) / 256);
    if (dtype == TW_F32)
        tw_launch(reduce_partial_kernel<float>, dim3(blocks), dim3(256), 0, stream, 1, (float*)out, partial, nsplit, total);
    else
        tw_launch(reduce_partial_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, 1, (bf16*)out, partial, nsplit, total);
    return TW_LAUNCH_CHECK();
}
