// Memory-bound kernels around the matrix products: embedding rows into the
// fp32 residual stream, residual add fused with RMSNorm, bias + rotary position
// encoding fused with the write of K and V into cache pages, SiLU(gate)*up.
//
// All statistics, angles and sums are fp32; `T` is the storage type of
// activations and cache (float or bf16).  Every kernel takes any row width.
#include "common.cuh"
#include <cooperative_groups.h>

namespace cg = cooperative_groups;

// ---------------------------------------------------------------------------
// Embedding: resid[n, :] = float(table[ids[n], :]).  No scaling
// (reference: flow_engine/model.py:176).  An id below zero names a token that is still on the
// device: -(i + 1) stands for device_tokens[i], the i-th token the previous step sampled, so a
// step can be launched before the host has seen its input tokens.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void embed_kernel(float* __restrict__ resid, const T* __restrict__ table,
                             const int* __restrict__ ids, const int* __restrict__ device_tokens, int n_device_tokens,
                             int hidden, int vocab, int* status) {
    TW_TIMELINE_SCOPE(TW_K_EMBED);
    tw_grid_wait();
    TW_TIMELINE_MARK();
    tw_grid_launch_dependents();
    const int n = blockIdx.x;
    int id = ids[n];
    if (id < 0 && device_tokens && -(id + 1) < n_device_tokens) id = device_tokens[-(id + 1)];
    if (id < 0 || id >= vocab) {
        if (threadIdx.x == 0) atomicOr(status, TW_ERR_TOKEN_ID);
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) resid[(size_t)n * hidden + i] = 0.f;
        return;
    }
    const T* row = table + (size_t)id * hidden;
    float* dst = resid + (size_t)n * hidden;
    if constexpr (sizeof(T) == 2) {
        // 16 bytes per load where the row allows: a decode step waits for this kernel's one round trip to memory
        if ((hidden & 7) == 0 && (reinterpret_cast<uintptr_t>(table) & 15) == 0 && (reinterpret_cast<uintptr_t>(resid) & 15) == 0) {
            for (int i = threadIdx.x; i < (hidden >> 3); i += blockDim.x) {
                const uint4 raw = reinterpret_cast<const uint4*>(row)[i];
                const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
                const float2 a = __bfloat1622float2(h2[0]), b = __bfloat1622float2(h2[1]);
                const float2 c = __bfloat1622float2(h2[2]), d = __bfloat1622float2(h2[3]);
                reinterpret_cast<float4*>(dst)[2 * i] = make_float4(a.x, a.y, b.x, b.y);
                reinterpret_cast<float4*>(dst)[2 * i + 1] = make_float4(c.x, c.y, d.x, d.y);
            }
            return;
        }
    }
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = tw_to_float(row[i]);
}

TW_EXPORT int tw_embed(void* resid, const void* table, const int* ids, const int* device_tokens, int n_device_tokens,
                       int n_tokens, int hidden, int vocab, int dtype, int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (dtype == TW_F32)
        tw_launch(embed_kernel<float>, dim3(n_tokens), dim3(256), 0, stream, 1, (float*)resid, (const float*)table, ids, device_tokens, n_device_tokens, hidden, vocab, status);
    else
        tw_launch(embed_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(256), 0, stream, 1, (float*)resid, (const __nv_bfloat16*)table, ids,
                                                                   device_tokens, n_device_tokens, hidden, vocab, status);
    return TW_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------
// Residual add + RMSNorm.
//   v = resid[src] + delta[src]            (delta may be null)
//   resid[src] = v                         (only when rows == null)
//   out[r] = T( (v * (1 / sqrt(mean(v^2) + eps))) * weight )
// rows != null selects source rows (the final norm runs on the wanted rows
// only); the residual stream is then left untouched.
// Reference: flow_engine/model.py:21-23 (fp32 statistics).  The reference casts
// the normalised value to the activation type before the multiply by the
// weight; here the product is formed in fp32 and rounded once.
// ---------------------------------------------------------------------------
// The delta is either a dense tensor of the activation type or `nsplit` fp32 slices of a
// split matrix product ([slice][row][hidden], slices `split_stride` floats apart), which
// are added here in slice order.
#define TW_NORM_THREADS 512
#define TW_NORM_MAXV 16          // values a thread keeps in registers: rows up to 512 * 16 wide take the one-pass path

template <typename T, bool ONE_PASS>
__global__ void __launch_bounds__(TW_NORM_THREADS)
add_rmsnorm_kernel(T* __restrict__ out, float* __restrict__ resid, const T* __restrict__ delta,
                   const float* __restrict__ partial, int nsplit, size_t split_stride,
                   const float* __restrict__ weight, float eps, int hidden, const int* __restrict__ rows) {
    __shared__ float scratch[33];
    const int r = blockIdx.x;
    TW_TIMELINE_SCOPE(TW_K_NORM);
    tw_grid_wait();
    TW_TIMELINE_MARK();
    tw_grid_launch_dependents();
    const int src = rows ? rows[r] : r;
    float* x = resid + (size_t)src * hidden;
    const T* d = delta ? delta + (size_t)src * hidden : nullptr;
    const float* ps = partial ? partial + (size_t)src * hidden : nullptr;
    const bool has_delta = d || ps;
    auto delta_at = [&](int i) -> float {
        if (d) return tw_to_float(d[i]);
        float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;      // fixed order: ((s0 + s1) + (s2 + s3)) over interleaved slices
        int k = 0;
        for (; k + 4 <= nsplit; k += 4) {
            s0 += ps[(size_t)k * split_stride + i];
            s1 += ps[(size_t)(k + 1) * split_stride + i];
            s2 += ps[(size_t)(k + 2) * split_stride + i];
            s3 += ps[(size_t)(k + 3) * split_stride + i];
        }
        for (; k < nsplit; ++k) s0 += ps[(size_t)k * split_stride + i];
        return (s0 + s1) + (s2 + s3);
    };
    T* o = out + (size_t)r * hidden;
    if (ONE_PASS) {
        float v[TW_NORM_MAXV];
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < TW_NORM_MAXV; ++j) {
            const int i = threadIdx.x + j * TW_NORM_THREADS;
            v[j] = 0.f;
            if (i < hidden) {
                v[j] = x[i];
                if (has_delta) v[j] += delta_at(i);
                if (!rows && has_delta) x[i] = v[j];
                ss += v[j] * v[j];
            }
        }
        ss = tw_block_sum(ss, scratch);
        const float inv = 1.0f / sqrtf(ss / (float)hidden + eps);
#pragma unroll
        for (int j = 0; j < TW_NORM_MAXV; ++j) {
            const int i = threadIdx.x + j * TW_NORM_THREADS;
            if (i < hidden) o[i] = tw_from_float<T>((v[j] * inv) * weight[i]);
        }
    } else {
        float ss = 0.f;
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
            float v = x[i];
            if (has_delta) v += delta_at(i);
            if (!rows && has_delta) x[i] = v;
            ss += v * v;
        }
        ss = tw_block_sum(ss, scratch);
        const float inv = 1.0f / sqrtf(ss / (float)hidden + eps);
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
            float v = x[i];
            if (rows && has_delta) v += delta_at(i);
            o[i] = tw_from_float<T>((v * inv) * weight[i]);
        }
    }
}

// The same for steps with few rows: a cluster of CTAs shares one row, each CTA owning a
// range of columns, and the partial sums of squares meet in distributed shared memory
// (added in rank order, so the result does not depend on timing).  With one CTA per row a
// decode step of 8 rows would keep only 8 SMs busy.
#define TW_NORM_CLUSTER 8
#define TW_NORM_CTHREADS 256
#define TW_NORM_CMAXV 4

template <typename T>
__global__ void __launch_bounds__(TW_NORM_CTHREADS)
add_rmsnorm_cluster_kernel(T* __restrict__ out, float* __restrict__ resid, const T* __restrict__ delta,
                           const float* __restrict__ partial, int nsplit, size_t split_stride,
                           const float* __restrict__ weight, float eps, int hidden, const int* __restrict__ rows) {
    __shared__ float scratch[33];
    __shared__ float all_ss[TW_NORM_CLUSTER];      // every block's sum of squares, written here by the blocks themselves
    TW_TIMELINE_SCOPE(TW_K_NORM_CLUSTER);
    // What no kernel of the step writes (the row indices, the norm's weights) is read before the wait for the
    // kernel before this one: this kernel is a chain of round trips, and these two need not be in it.
    cg::cluster_group cluster = cg::this_cluster();
    const int rank = (int)cluster.block_rank();
    const int r = blockIdx.x / TW_NORM_CLUSTER;
    const int src = rows ? rows[r] : r;
    const int chunk = (hidden + TW_NORM_CLUSTER - 1) / TW_NORM_CLUSTER;
    const int c0 = rank * chunk, c1 = min(hidden, c0 + chunk);
    float wv[TW_NORM_CMAXV];
#pragma unroll
    for (int j = 0; j < TW_NORM_CMAXV; ++j) {
        const int i = c0 + threadIdx.x + j * TW_NORM_CTHREADS;
        wv[j] = i < c1 ? weight[i] : 0.f;
    }
    tw_grid_wait();
    TW_TIMELINE_MARK();
    tw_launch_dependents_now();     // 64 small blocks: the product that follows may settle on the SMs meanwhile (1 % of a decode step)
    float* x = resid + (size_t)src * hidden;
    const T* d = delta ? delta + (size_t)src * hidden : nullptr;
    const float* ps = partial ? partial + (size_t)src * hidden : nullptr;
    const bool has_delta = d || ps;
    float v[TW_NORM_CMAXV];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < TW_NORM_CMAXV; ++j) {
        const int i = c0 + threadIdx.x + j * TW_NORM_CTHREADS;
        v[j] = 0.f;
        if (i < c1) {
            float dv = 0.f;
            if (d) {
                dv = tw_to_float(d[i]);
            } else if (ps) {
                // The slices are summed in the order every consumer of a split product uses: whole groups of
                // four into four sums by k mod 4, the rest into the first, then (s0 + s1) + (s2 + s3).  The
                // first sixteen are loaded before anything is added, so that they are one round trip to L2
                // and not one per group (this kernel is nothing but latency).
                float t[16];
#pragma unroll
                for (int u = 0; u < 16; ++u) t[u] = u < nsplit ? ps[(size_t)u * split_stride + i] : 0.f;
                const int full = nsplit & ~3;
                float sum[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int u = 0; u < 16; ++u) {
                    if (u < full) sum[u & 3] += t[u];
                }
                int k = 16;
                for (; k + 4 <= nsplit; k += 4) {
                    sum[0] += ps[(size_t)k * split_stride + i];
                    sum[1] += ps[(size_t)(k + 1) * split_stride + i];
                    sum[2] += ps[(size_t)(k + 2) * split_stride + i];
                    sum[3] += ps[(size_t)(k + 3) * split_stride + i];
                }
#pragma unroll
                for (int u = 0; u < 16; ++u) {
                    if (u >= full && u < nsplit) sum[0] += t[u];
                }
                for (k = max(k, full); k < nsplit; ++k) sum[0] += ps[(size_t)k * split_stride + i];
                dv = (sum[0] + sum[1]) + (sum[2] + sum[3]);
            }
            v[j] = x[i] + dv;
            if (!rows && has_delta) x[i] = v[j];
            ss += v[j] * v[j];
        }
    }
    ss = tw_block_sum(ss, scratch);
    // every block hands its sum to all blocks of the cluster (one remote store each), so that after one
    // cluster barrier each block finds the eight sums in its own shared memory and nobody reads a neighbour's
    if (threadIdx.x < TW_NORM_CLUSTER) *cluster.map_shared_rank(&all_ss[rank], threadIdx.x) = ss;
    cluster.sync();
    float total = 0.f;
#pragma unroll
    for (int k = 0; k < TW_NORM_CLUSTER; ++k) total += all_ss[k];       // in rank order
    const float inv = 1.0f / sqrtf(total / (float)hidden + eps);
    T* o = out + (size_t)r * hidden;
#pragma unroll
    for (int j = 0; j < TW_NORM_CMAXV; ++j) {
        const int i = c0 + threadIdx.x + j * TW_NORM_CTHREADS;
        if (i < c1) o[i] = tw_from_float<T>((v[j] * inv) * wv[j]);
    }
}

__device__ __forceinline__ float4 tw_load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 tw_load4(const __nv_bfloat16* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void tw_store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void tw_store4(__nv_bfloat16* p, float4 v) {
    uint2 raw;
    *reinterpret_cast<__nv_bfloat162*>(&raw.x) = __floats2bfloat162_rn(v.x, v.y);
    *reinterpret_cast<__nv_bfloat162*>(&raw.y) = __floats2bfloat162_rn(v.z, v.w);
    *reinterpret_cast<uint2*>(p) = raw;
}

// Many rows (prompt portions): four values per thread and access, one pass, values kept in registers.
// Dense delta only; hidden a multiple of 4 and at most 4 * 256 * V4 wide.  V4 = float4 per thread: 4 for rows up
// to 4,096 wide (half the registers, twice the blocks per SM), 8 up to 8,192.
#define TW_NORM_V4 8
template <typename T, int V4>
__global__ void __launch_bounds__(256)
add_rmsnorm_vec4_kernel(T* __restrict__ out, float* __restrict__ resid, const T* __restrict__ delta,
                        const float* __restrict__ weight, float eps, int hidden, const int* __restrict__ rows) {
    __shared__ float scratch[33];
    TW_TIMELINE_SCOPE(TW_K_NORM);
    tw_grid_wait();
    TW_TIMELINE_MARK();
    tw_grid_launch_dependents();
    const int r = blockIdx.x;
    const int src = rows ? rows[r] : r;
    float4* x4 = reinterpret_cast<float4*>(resid + (size_t)src * hidden);
    const int n4 = hidden >> 2;
    float4 v[V4];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < V4; ++j) {
        const int i = threadIdx.x + j * 256;
        v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i < n4) {
            v[j] = x4[i];
            if (delta) {
                const float4 d = tw_load4(delta + (size_t)src * hidden + 4 * i);
                v[j].x += d.x; v[j].y += d.y; v[j].z += d.z; v[j].w += d.w;
                if (!rows) x4[i] = v[j];
            }
            ss += v[j].x * v[j].x + v[j].y * v[j].y + v[j].z * v[j].z + v[j].w * v[j].w;
        }
    }
    ss = tw_block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)hidden + eps);
    const float4* w4 = reinterpret_cast<const float4*>(weight);
#pragma unroll
    for (int j = 0; j < V4; ++j) {
        const int i = threadIdx.x + j * 256;
        if (i < n4) {
            const float4 w = w4[i];
            tw_store4(out + (size_t)r * hidden + 4 * i,
                      make_float4((v[j].x * inv) * w.x, (v[j].y * inv) * w.y, (v[j].z * inv) * w.z, (v[j].w * inv) * w.w));
        }
    }
}

template <typename T>
static int launch_add_rmsnorm(T* out, float* resid, const T* delta, const float* partial, int nsplit,
                              size_t split_stride, const float* weight, float eps, int n_rows, int hidden,
                              const int* rows, cudaStream_t stream) {
    if (n_rows <= 64 && hidden >= 1024 && hidden <= TW_NORM_CLUSTER * TW_NORM_CTHREADS * TW_NORM_CMAXV) {
        return tw_launch(add_rmsnorm_cluster_kernel<T>, dim3(n_rows * TW_NORM_CLUSTER), dim3(TW_NORM_CTHREADS), 0, stream,
                         TW_NORM_CLUSTER, out, resid, delta, partial, nsplit, split_stride, weight, eps, hidden, rows);
    }
    if (!partial && (hidden & 3) == 0 && hidden <= 4 * 256 * TW_NORM_V4) {
        if (hidden <= 4 * 256 * 4)
            tw_launch(add_rmsnorm_vec4_kernel<T, 4>, dim3(n_rows), dim3(256), 0, stream, 1, out, resid, delta, weight, eps,
                      hidden, rows);
        else
            tw_launch(add_rmsnorm_vec4_kernel<T, TW_NORM_V4>, dim3(n_rows), dim3(256), 0, stream, 1, out, resid, delta, weight,
                      eps, hidden, rows);
        return TW_LAUNCH_CHECK();
    }
    if (hidden <= TW_NORM_THREADS * TW_NORM_MAXV)
        tw_launch(add_rmsnorm_kernel<T, true>, dim3(n_rows), dim3(TW_NORM_THREADS), 0, stream, 1, out, resid, delta, partial, nsplit,
                                                                            split_stride, weight, eps, hidden, rows);
    else
        tw_launch(add_rmsnorm_kernel<T, false>, dim3(n_rows), dim3(TW_NORM_THREADS), 0, stream, 1, out, resid, delta, partial, nsplit,
                                                                             split_stride, weight, eps, hidden, rows);
    return TW_LAUNCH_CHECK();
}

TW_EXPORT int tw_add_rmsnorm(void* out, float* resid, const void* delta, const float* partial, int nsplit,
                             long split_stride, const float* weight, float eps, int n_rows, int hidden,
                             const int* rows, int dtype, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (delta && partial) return (int)cudaErrorInvalidValue;
    if (dtype == TW_F32)
        return launch_add_rmsnorm<float>((float*)out, resid, (const float*)delta, partial, nsplit, (size_t)split_stride,
                                         weight, eps, n_rows, hidden, rows, stream);
    return launch_add_rmsnorm<__nv_bfloat16>((__nv_bfloat16*)out, resid, (const __nv_bfloat16*)delta, partial, nsplit,
                                             (size_t)split_stride, weight, eps, n_rows, hidden, rows, stream);
}

// ---------------------------------------------------------------------------
// Bias + rotary position encoding + cache write, one block per token.
//
// qkv row layout: [q heads | k heads | v heads], each head `D` wide.
//   x += bias                                       (bias may be null)
//   angle_i = float(position) * inv_freq[i]         (fp32; inv_freq may be null: no rotation)
//   y[i]        = x[i] * cos - x[i + D/2] * sin     (rotate-half pairing)
//   y[i + D/2]  = x[i + D/2] * cos + x[i] * sin
// q is rewritten in place; rotated k and v go to the page that the request's
// block table names for this position:
//   page = table[slot_row][pos / P];  element ((page * Hkv + h) * P + pos % P) * D + d
// Reference: flow_engine/model.py:26-33,184-187; flow_engine/cache.py:93-100.
// ---------------------------------------------------------------------------
// The source of a row is the qkv buffer itself or, when the projection was split over k,
// the sum of `nsplit` fp32 slices [slice][token][width]; q always lands in the qkv buffer.
#define TW_ROPE_THREADS 128

template <typename T>
__global__ void __launch_bounds__(TW_ROPE_THREADS)
rope_kv_write_kernel(T* __restrict__ qkv, int qkv_stride, const float* __restrict__ partial, int nsplit,
                     size_t split_stride, const float* __restrict__ bias, const int* __restrict__ positions,
                     const int* __restrict__ seq_of_token, const int* __restrict__ seq_slot,
                     const int* __restrict__ block_table, int table_stride, const float* __restrict__ inv_freq,
                     T* __restrict__ k_cache, T* __restrict__ v_cache, int Hq, int Hkv, int D, int page_size,
                     int num_pages, int write_cache, int* status) {
    TW_TIMELINE_SCOPE(TW_K_ROPE);
    tw_grid_wait();
    TW_TIMELINE_MARK();
    tw_grid_launch_dependents();
    const int n = blockIdx.x;
    const int s = seq_of_token[n];
    if (s < 0) return;  // padding row of a fixed-size batch
    const int pos = positions[n];
    const int half = D >> 1;
    T* row = qkv + (size_t)n * qkv_stride;
    const int width = (Hq + 2 * Hkv) * D;
    const float* prow = partial ? partial + (size_t)n * width : nullptr;
    auto src_at = [&](int col) -> float {
        if (!prow) return tw_to_float(row[col]);
        float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
        int k = 0;
        for (; k + 4 <= nsplit; k += 4) {
            s0 += prow[(size_t)k * split_stride + col];
            s1 += prow[(size_t)(k + 1) * split_stride + col];
            s2 += prow[(size_t)(k + 2) * split_stride + col];
            s3 += prow[(size_t)(k + 3) * split_stride + col];
        }
        for (; k < nsplit; ++k) s0 += prow[(size_t)k * split_stride + col];
        return (s0 + s1) + (s2 + s3);
    };

    int page = -1;
    if (write_cache) {
        const int blk = pos / page_size;
        page = blk < table_stride ? block_table[(size_t)seq_slot[s] * table_stride + blk] : -1;
        if (page < 0 || page >= num_pages) {
            if (threadIdx.x == 0 && blockIdx.y == 0) atomicOr(status, TW_ERR_PAGE);
            page = -1;
        }
    }
    const int in_page = pos % page_size;
    const int rot_pairs = (write_cache ? Hq + Hkv : Hq) * half;     // rotated (q, then k) pairs
    const int v_pairs = write_cache ? Hkv * half : 0;               // v is copied pair-wise, unrotated
    const int idx = blockIdx.y * TW_ROPE_THREADS + threadIdx.x;
    if (idx < rot_pairs) {
        const int head = idx / half, i = idx - head * half;
        const int col = head * D + i;
        float x1 = src_at(col), x2 = src_at(col + half);
        if (bias) { x1 += bias[col]; x2 += bias[col + half]; }
        float y1 = x1, y2 = x2;
        if (inv_freq) {
            const float ang = (float)pos * inv_freq[i];
            float sn, cs;
            sincosf(ang, &sn, &cs);
            y1 = x1 * cs - x2 * sn;
            y2 = x2 * cs + x1 * sn;
        }
        if (head < Hq) {
            row[col] = tw_from_float<T>(y1);
            row[col + half] = tw_from_float<T>(y2);
        } else if (page >= 0) {
            const int kvh = head - Hq;
            T* dst = k_cache + (((size_t)page * Hkv + kvh) * page_size + in_page) * D;
            dst[i] = tw_from_float<T>(y1);
            dst[i + half] = tw_from_float<T>(y2);
        }
    } else if (idx < rot_pairs + v_pairs && page >= 0) {
        const int j = idx - rot_pairs;
        const int kvh = j / half, i = j - kvh * half;
        const int col = (Hq + Hkv) * D + kvh * D + i;
        float v1 = src_at(col), v2 = src_at(col + half);
        if (bias) { v1 += bias[col]; v2 += bias[col + half]; }
        T* dst = v_cache + (((size_t)page * Hkv + kvh) * page_size + in_page) * D;
        dst[i] = tw_from_float<T>(v1);
        dst[i + half] = tw_from_float<T>(v2);
    }
}

// bf16, dense source, head size a multiple of 16: a thread rotates eight neighbouring pairs with 16-byte accesses
// (or copies sixteen values of v).  Same arithmetic as the kernel above.
__global__ void __launch_bounds__(TW_ROPE_THREADS)
rope_kv_write_bf16x8_kernel(__nv_bfloat16* __restrict__ qkv, int qkv_stride, const float* __restrict__ bias,
                            const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                            const int* __restrict__ seq_slot, const int* __restrict__ block_table, int table_stride,
                            const float* __restrict__ inv_freq, __nv_bfloat16* __restrict__ k_cache,
                            __nv_bfloat16* __restrict__ v_cache, int Hq, int Hkv, int D, int page_size, int num_pages,
                            int write_cache, int* status) {
    TW_TIMELINE_SCOPE(TW_K_ROPE);
    tw_grid_wait();
    TW_TIMELINE_MARK();
    tw_grid_launch_dependents();
    const int n = blockIdx.x;
    const int s = seq_of_token[n];
    if (s < 0) return;
    const int pos = positions[n];
    const int half = D >> 1, groups = half >> 3;           // groups of 8 pairs per head
    __nv_bfloat16* row = qkv + (size_t)n * qkv_stride;
    int page = -1;
    if (write_cache) {
        const int blk = pos / page_size;
        page = blk < table_stride ? block_table[(size_t)seq_slot[s] * table_stride + blk] : -1;
        if (page < 0 || page >= num_pages) {
            if (threadIdx.x == 0 && blockIdx.y == 0) atomicOr(status, TW_ERR_PAGE);
            page = -1;
        }
    }
    const int in_page = pos % page_size;
    // the angles depend on the position and the pair only: each is evaluated once per block, not once per head
    __shared__ float s_cos[128], s_sin[128];
    if (inv_freq) {
        for (int i = threadIdx.x; i < half; i += TW_ROPE_THREADS) sincosf((float)pos * inv_freq[i], &s_sin[i], &s_cos[i]);
    }
    __syncthreads();
    const int rot_items = (write_cache ? Hq + Hkv : Hq) * groups;
    const int v_items = write_cache ? Hkv * groups : 0;      // v: 8 values of each half per item
    const int idx = blockIdx.y * TW_ROPE_THREADS + threadIdx.x;
    if (idx >= rot_items + v_items) return;
    const bool is_v = idx >= rot_items;
    const int item = is_v ? idx - rot_items : idx;
    const int head = item / groups, i0 = (item - head * groups) * 8;
    const int col = (is_v ? (Hq + Hkv) * D : 0) + head * D + i0;
    uint4 lo = *reinterpret_cast<const uint4*>(row + col), hi = *reinterpret_cast<const uint4*>(row + col + half);
    __nv_bfloat162* lo2 = reinterpret_cast<__nv_bfloat162*>(&lo);
    __nv_bfloat162* hi2 = reinterpret_cast<__nv_bfloat162*>(&hi);
    float blo[8], bhi[8];                       // col and half are multiples of 8: 32-byte aligned reads of the bias
    if (bias) {
        *reinterpret_cast<float4*>(blo) = *reinterpret_cast<const float4*>(bias + col);
        *reinterpret_cast<float4*>(blo + 4) = *reinterpret_cast<const float4*>(bias + col + 4);
        *reinterpret_cast<float4*>(bhi) = *reinterpret_cast<const float4*>(bias + col + half);
        *reinterpret_cast<float4*>(bhi + 4) = *reinterpret_cast<const float4*>(bias + col + half + 4);
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        float2 x1 = __bfloat1622float2(lo2[e]), x2 = __bfloat1622float2(hi2[e]);
        if (bias) {
            x1.x += blo[2 * e]; x1.y += blo[2 * e + 1];
            x2.x += bhi[2 * e]; x2.y += bhi[2 * e + 1];
        }
        float2 y1 = x1, y2 = x2;
        if (inv_freq && !is_v) {
            float sn = s_sin[i0 + 2 * e], cs = s_cos[i0 + 2 * e];
            y1.x = x1.x * cs - x2.x * sn; y2.x = x2.x * cs + x1.x * sn;
            sn = s_sin[i0 + 2 * e + 1]; cs = s_cos[i0 + 2 * e + 1];
            y1.y = x1.y * cs - x2.y * sn; y2.y = x2.y * cs + x1.y * sn;
        }
        lo2[e] = __floats2bfloat162_rn(y1.x, y1.y);
        hi2[e] = __floats2bfloat162_rn(y2.x, y2.y);
    }
    __nv_bfloat16* dst;
    if (!is_v && head < Hq) {
        dst = row + col;
    } else {
        if (page < 0) return;
        const int kvh = is_v ? head : head - Hq;
        dst = (is_v ? v_cache : k_cache) + (((size_t)page * Hkv + kvh) * page_size + in_page) * D + i0;
    }
    *reinterpret_cast<uint4*>(dst) = lo;
    *reinterpret_cast<uint4*>(dst + half) = hi;
}

TW_EXPORT int tw_rope_kv_write(void* qkv, int qkv_stride, const float* partial, int nsplit, long split_stride,
                               const float* bias, const int* positions,
                               const int* seq_of_token, const int* seq_slot, const int* block_table, int table_stride,
                               const float* inv_freq, void* k_cache, void* v_cache, int n_tokens, int Hq, int Hkv,
                               int D, int page_size, int num_pages, int write_cache, int dtype, int* status,
                               cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (D <= 0 || (D & 1)) return (int)cudaErrorInvalidValue;
    if (dtype == TW_BF16 && !partial && (D & 15) == 0 && D <= 256 && (qkv_stride & 7) == 0 && (reinterpret_cast<uintptr_t>(bias) & 15) == 0 &&
        (reinterpret_cast<uintptr_t>(qkv) & 15) == 0) {
        const int items = (Hq + 2 * Hkv) * (D / 16);
        const dim3 vgrid(n_tokens, (items + TW_ROPE_THREADS - 1) / TW_ROPE_THREADS);
        return tw_launch(rope_kv_write_bf16x8_kernel, vgrid, dim3(TW_ROPE_THREADS), 0, stream, 1, (__nv_bfloat16*)qkv,
                         qkv_stride, bias, positions, seq_of_token, seq_slot, block_table, table_stride, inv_freq,
                         (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, Hq, Hkv, D, page_size, num_pages,
                         write_cache, status);
    }
    const int work = (Hq + 2 * Hkv) * (D / 2);
    const dim3 grid(n_tokens, (work + TW_ROPE_THREADS - 1) / TW_ROPE_THREADS);
    const int threads = TW_ROPE_THREADS;
    if (dtype == TW_F32)
        tw_launch(rope_kv_write_kernel<float>, dim3(grid), dim3(threads), 0, stream, 1, 
            (float*)qkv, qkv_stride, partial, nsplit, (size_t)split_stride, bias, positions, seq_of_token, seq_slot,
            block_table, table_stride, inv_freq,
            (float*)k_cache, (float*)v_cache, Hq, Hkv, D, page_size, num_pages, write_cache, status);
    else
        tw_launch(rope_kv_write_kernel<__nv_bfloat16>, dim3(grid), dim3(threads), 0, stream, 1, 
            (__nv_bfloat16*)qkv, qkv_stride, partial, nsplit, (size_t)split_stride, bias, positions, seq_of_token,
            seq_slot, block_table, table_stride, inv_freq, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, Hq, Hkv, D, page_size, num_pages, write_cache,
            status);
    return TW_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------
// SwiGLU activation: out[n, i] = silu(gate[n, i]) * up[n, i], silu(z) = z / (1 + exp(-z)),
// with gate = gate_up[n, i] and up = gate_up[n, I + i] (rows packed [gate; up]).
// Reference: flow_engine/model.py:76-80.
// ---------------------------------------------------------------------------
// With `interleaved` the columns come in groups of 16: eight gates, then their eight ups
// (the packing the fused small-batch kernel wants); otherwise all gates, then all ups.
template <typename T>
__global__ void silu_mul_kernel(T* __restrict__ out, const T* __restrict__ gate_up, int inter, long total,
                                int interleaved) {
    TW_TIMELINE_SCOPE(TW_K_SILU_MUL);
    tw_grid_wait();
    TW_TIMELINE_MARK();
    tw_grid_launch_dependents();
    long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    const long step = (long)gridDim.x * blockDim.x;
    for (; idx < total; idx += step) {
        const long n = idx / inter;
        const int i = (int)(idx - n * inter);
        const int gcol = interleaved ? ((i >> 3) << 4) + (i & 7) : i;
        const int ucol = interleaved ? gcol + 8 : inter + i;
        const float g = tw_to_float(gate_up[n * 2 * inter + gcol]);
        const float u = tw_to_float(gate_up[n * 2 * inter + ucol]);
        const float act = g / (1.0f + expf(-g));
        out[idx] = tw_from_float<T>(act * u);
    }
}

// bf16 with the intermediate size a multiple of 8: a thread handles 8 outputs with 16-byte accesses.
__global__ void silu_mul_bf16x8_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ gate_up,
                                       int inter, long total8, int interleaved) {
    TW_TIMELINE_SCOPE(TW_K_SILU_MUL);
    tw_grid_wait();
    TW_TIMELINE_MARK();
    tw_grid_launch_dependents();
    long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    const long step = (long)gridDim.x * blockDim.x;
    const int groups = inter >> 3;
    for (; idx < total8; idx += step) {
        const long n = idx / groups;
        const int j = (int)(idx - n * groups);
        const __nv_bfloat16* row = gate_up + n * 2 * (long)inter;
        const uint4 gv = *reinterpret_cast<const uint4*>(row + (interleaved ? j * 16 : j * 8));
        const uint4 uv = *reinterpret_cast<const uint4*>(row + (interleaved ? j * 16 + 8 : inter + j * 8));
        const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gv);
        const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&uv);
        uint4 ov;
        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 g = __bfloat1622float2(g2[e]), u = __bfloat1622float2(u2[e]);
            o2[e] = __floats2bfloat162_rn(g.x / (1.0f + expf(-g.x)) * u.x, g.y / (1.0f + expf(-g.y)) * u.y);
        }
        *reinterpret_cast<uint4*>(out + n * (long)inter + j * 8) = ov;
    }
}

// The same from the fp32 slices of a gate/up product split over k ([slice][row][2 * inter], `split_stride` floats
// apart): the slices are added in the order every consumer of a split product uses (whole groups of four into
// four sums by slice mod 4, the rest into the first, then (s0 + s1) + (s2 + s3)), then silu(gate) * up, bf16 out.
// Four outputs per thread; inter a multiple of 8 when interleaved, of 4 otherwise.
__device__ __forceinline__ float4 tw_sum_slices4(const float* p, int nsplit, size_t split_stride) {
    float4 s[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) s[u] = make_float4(0.f, 0.f, 0.f, 0.f);
    int k = 0;
    for (; k + 4 <= nsplit; k += 4) {
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const float4 v = *reinterpret_cast<const float4*>(p + (size_t)(k + u) * split_stride);
            s[u].x += v.x; s[u].y += v.y; s[u].z += v.z; s[u].w += v.w;
        }
    }
    for (; k < nsplit; ++k) {
        const float4 v = *reinterpret_cast<const float4*>(p + (size_t)k * split_stride);
        s[0].x += v.x; s[0].y += v.y; s[0].z += v.z; s[0].w += v.w;
    }
    return make_float4((s[0].x + s[1].x) + (s[2].x + s[3].x), (s[0].y + s[1].y) + (s[2].y + s[3].y),
                       (s[0].z + s[1].z) + (s[2].z + s[3].z), (s[0].w + s[1].w) + (s[2].w + s[3].w));
}

__global__ void silu_mul_slices_kernel(__nv_bfloat16* __restrict__ out, const float* __restrict__ partial, int nsplit,
                                       size_t split_stride, int inter, long total4, int interleaved) {
    TW_TIMELINE_SCOPE(TW_K_SILU_MUL);
    tw_grid_wait();
    TW_TIMELINE_MARK();
    tw_grid_launch_dependents();
    long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    const long step = (long)gridDim.x * blockDim.x;
    const int quads = inter >> 2;
    for (; idx < total4; idx += step) {
        const long n = idx / quads;
        const int i = (int)(idx - n * quads) * 4;                       // first of this thread's four outputs
        const int gcol = interleaved ? ((i >> 3) << 4) + (i & 7) : i;
        const int ucol = interleaved ? gcol + 8 : inter + i;
        const float* row = partial + (size_t)n * 2 * inter;
        const float4 g = tw_sum_slices4(row + gcol, nsplit, split_stride);
        const float4 u = tw_sum_slices4(row + ucol, nsplit, split_stride);
        uint2 packed;
        *reinterpret_cast<__nv_bfloat162*>(&packed.x) =
            __floats2bfloat162_rn(g.x / (1.0f + expf(-g.x)) * u.x, g.y / (1.0f + expf(-g.y)) * u.y);
        *reinterpret_cast<__nv_bfloat162*>(&packed.y) =
            __floats2bfloat162_rn(g.z / (1.0f + expf(-g.z)) * u.z, g.w / (1.0f + expf(-g.w)) * u.w);
        *reinterpret_cast<uint2*>(out + n * (long)inter + i) = packed;
    }
}

TW_EXPORT int tw_silu_mul_slices(void* out, const float* partial, int nsplit, long split_stride, int n_rows, int inter,
                                 int interleaved, cudaStream_t stream) {
    if (n_rows <= 0 || inter <= 0) return 0;
    if (nsplit < 1 || (inter & 3) || (interleaved && (inter & 7)) || (split_stride & 3) ||
        ((uintptr_t)partial & 15) || ((uintptr_t)out & 7))
        return (int)cudaErrorInvalidValue;
    const long total4 = (long)n_rows * (inter >> 2);
    const long blocks = (total4 + 255) / 256;
    tw_launch(silu_mul_slices_kernel, dim3((int)(blocks > 4096 ? 4096 : blocks)), dim3(256), 0, stream, 1, (__nv_bfloat16*)out,
              partial, nsplit, (size_t)split_stride, inter, total4, interleaved);
    return TW_LAUNCH_CHECK();
}

TW_EXPORT int tw_silu_mul(void* out, const void* gate_up, int n_rows, int inter, int interleaved, int dtype,
                          cudaStream_t stream) {
    const long total = (long)n_rows * inter;
    if (total <= 0) return 0;
    long blocks = (total + 255) / 256;
    if (blocks > 148L * 16) blocks = 148L * 16;
    if (dtype == TW_BF16 && (inter & 7) == 0) {
        const long total8 = total >> 3;
        long b8 = (total8 + 255) / 256;
        if (b8 > 148L * 16) b8 = 148L * 16;
        tw_launch(silu_mul_bf16x8_kernel, dim3((int)b8), dim3(256), 0, stream, 1, (__nv_bfloat16*)out, (const __nv_bfloat16*)gate_up, inter,
                                                            total8, interleaved);
        return TW_LAUNCH_CHECK();
    }
    if (dtype == TW_F32)
        tw_launch(silu_mul_kernel<float>, dim3((int)blocks), dim3(256), 0, stream, 1, (float*)out, (const float*)gate_up, inter, total,
                                                                interleaved);
    else
        tw_launch(silu_mul_kernel<__nv_bfloat16>, dim3((int)blocks), dim3(256), 0, stream, 1, (__nv_bfloat16*)out,
                                                                        (const __nv_bfloat16*)gate_up, inter, total,
                                                                        interleaved);
    return TW_LAUNCH_CHECK();
}
