// Paged causal attention for any mix of rows: one block per (token, query head).
//
// This is the exact-arithmetic kernel: fp32 scores, fp32 online softmax, fp32
// accumulation, any head size up to 256, any number of heads and groups, an
// optional window.  It serves the whole float32 path and any bfloat16 shape
// that the tensor-core kernels refuse.  Prompt portions and single decoded
// tokens are the same case here: each token row attends to the keys
// lo..position of its own request through that request's block table.
//
//   kv_head = head / (Hq / Hkv)
//   score_p = (q . k_p) * scale            p in [lo, position], lo = max(0, position - window + 1)
//   out     = softmax(score) @ v
// Reference: flow_engine/model.py:193-200 (mask p <= position), flow_engine/
// kernels/paged_decode.py:13-43 (online softmax in fp32, GQA head map).
//
// Key p is handled by warp p % 4, so the order of the sums at a position does
// not depend on how the request was cut into steps or on what else is in the
// batch.
#include "common.cuh"

#define TW_ATTN_WARPS 4
#define TW_ATTN_MAXR 8  // head_dim <= 32 * 8

template <typename T>
__global__ void attn_generic_kernel(T* __restrict__ out, int out_stride, const T* __restrict__ q, int q_stride,
                                    const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                                    const int* __restrict__ seq_slot, const int* __restrict__ block_table,
                                    int table_stride, const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                                    int Hq, int Hkv, int D, int page_size, int num_pages, int window, float scale,
                                    int* status) {
    extern __shared__ float smem[];  // TW_ATTN_WARPS * (D + 2)
    tw_grid_wait();
    tw_grid_launch_dependents();
    const int n = blockIdx.x, head = blockIdx.y;
    const int s = seq_of_token[n];
    if (s < 0) return;
    const int pos = positions[n];
    const int kvh = head / (Hq / Hkv);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int* table = block_table + (size_t)seq_slot[s] * table_stride;

    float qr[TW_ATTN_MAXR], acc[TW_ATTN_MAXR];
    const T* qrow = q + (size_t)n * q_stride + head * D;
#pragma unroll
    for (int j = 0; j < TW_ATTN_MAXR; ++j) {
        const int d = lane + 32 * j;
        qr[j] = d < D ? tw_to_float(qrow[d]) : 0.f;
        acc[j] = 0.f;
    }
    float m = -INFINITY, l = 0.f;
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    int p = lo + ((warp - lo) % TW_ATTN_WARPS + TW_ATTN_WARPS) % TW_ATTN_WARPS;
    for (; p <= pos; p += TW_ATTN_WARPS) {
        const int blk = p / page_size;
        const int page = blk < table_stride ? table[blk] : -1;
        if (page < 0 || page >= num_pages) {
            if (lane == 0) atomicOr(status, TW_ERR_PAGE);
            continue;
        }
        const size_t base = (((size_t)page * Hkv + kvh) * page_size + (p - blk * page_size)) * D;
        const T* kr = k_cache + base;
        const T* vr = v_cache + base;
        float dot = 0.f;
#pragma unroll
        for (int j = 0; j < TW_ATTN_MAXR; ++j) {
            const int d = lane + 32 * j;
            if (d < D) dot += qr[j] * tw_to_float(kr[d]);
        }
        dot = tw_warp_sum(dot) * scale;
        const float m_new = fmaxf(m, dot);
        const float alpha = expf(m - m_new);   // m == -inf gives 0
        const float w = expf(dot - m_new);
        l = l * alpha + w;
#pragma unroll
        for (int j = 0; j < TW_ATTN_MAXR; ++j) {
            const int d = lane + 32 * j;
            if (d < D) acc[j] = acc[j] * alpha + w * tw_to_float(vr[d]);
        }
        m = m_new;
    }
    // Merge the warps' partial softmaxes.
    float* my = smem + warp * (D + 2);
#pragma unroll
    for (int j = 0; j < TW_ATTN_MAXR; ++j) {
        const int d = lane + 32 * j;
        if (d < D) my[d] = acc[j];
    }
    if (lane == 0) { my[D] = m; my[D + 1] = l; }
    __syncthreads();
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < TW_ATTN_WARPS; ++w) M = fmaxf(M, smem[w * (D + 2) + D]);
    float f[TW_ATTN_WARPS], L = 0.f;
#pragma unroll
    for (int w = 0; w < TW_ATTN_WARPS; ++w) {
        const float mw = smem[w * (D + 2) + D];
        f[w] = (mw == -INFINITY) ? 0.f : expf(mw - M);
        L += smem[w * (D + 2) + D + 1] * f[w];
    }
    T* orow = out + (size_t)n * out_stride + head * D;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float o = 0.f;
#pragma unroll
        for (int w = 0; w < TW_ATTN_WARPS; ++w) o += smem[w * (D + 2) + d] * f[w];
        orow[d] = tw_from_float<T>(L > 0.f ? o / L : 0.f);
    }
}

TW_EXPORT int tw_attn_generic(void* out, int out_stride, const void* q, int q_stride, const int* positions,
                              const int* seq_of_token, const int* seq_slot, const int* block_table, int table_stride,
                              const void* k_cache, const void* v_cache, int n_tokens, int Hq, int Hkv, int D,
                              int page_size, int num_pages, int window, float scale, int dtype, int* status,
                              cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (D <= 0 || D > 32 * TW_ATTN_MAXR || Hkv <= 0 || Hq % Hkv) return (int)cudaErrorInvalidValue;
    dim3 grid(n_tokens, Hq);
    const size_t smem = (size_t)TW_ATTN_WARPS * (D + 2) * sizeof(float);
    if (dtype == TW_F32)
        tw_launch(attn_generic_kernel<float>, dim3(grid), dim3(32 * TW_ATTN_WARPS), smem, stream, 1, 
            (float*)out, out_stride, (const float*)q, q_stride, positions, seq_of_token, seq_slot, block_table,
            table_stride, (const float*)k_cache, (const float*)v_cache, Hq, Hkv, D, page_size, num_pages, window, scale,
            status);
    else
        tw_launch(attn_generic_kernel<__nv_bfloat16>, dim3(grid), dim3(32 * TW_ATTN_WARPS), smem, stream, 1, 
            (__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)q, q_stride, positions, seq_of_token, seq_slot,
            block_table, table_stride, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, Hq, Hkv, D,
            page_size, num_pages, window, scale, status);
    return TW_LAUNCH_CHECK();
}
