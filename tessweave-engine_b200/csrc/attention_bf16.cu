// Paged grouped-query attention in bfloat16 on the tensor cores, for one head size
// (compile with -DTW_HEAD_DIM=<multiple of 16, 16..256>).
//
// Two kernels share the tile machinery:
//   * decode:  requests that bring ONE token.  A block serves one (request, key/value head,
//     slice of the keys); all query heads of the group are the rows of one MMA tile, so keys
//     and values are read once for the whole group.  The keys are split over blocks
//     ("split-KV"); partial results (fp32 accumulator, running maximum, sum) go to scratch
//     memory, and the block that finishes last merges them in slice order.
//   * prefill: requests that bring several tokens.  A block serves 64 rows, a row being a
//     (token, query head of the group) pair, and walks the keys up to the last visible one.
// Scores, softmax statistics and the accumulator are fp32; probabilities are rounded to
// bf16 only as the operand of the P.V product.  Keys beyond the visible range are never
// read: their shared-memory rows are zero-filled, so stale page contents cannot leak in.
//
//   score = (q . k) * scale,  visible iff  position - window < p <= position
// Reference: flow_engine/model.py:193-200 and flow_engine/kernels/paged_decode.py:13-43.
#include "common.cuh"

#ifndef TW_HEAD_DIM
#define TW_HEAD_DIM 128
#endif

namespace {

constexpr int D = TW_HEAD_DIM;
static_assert(D % 16 == 0 && D >= 16 && D <= 256, "head size must be a multiple of 16 in 16..256");
constexpr int DP = D + 8;        // padded row: consecutive rows fall into different 16-byte bank groups
constexpr int KSTEPS = D / 16;   // k-steps of Q.K^T
constexpr int NT_O = D / 8;      // n-tiles of P.V
constexpr int CHUNKS = D / 8;    // 16-byte chunks of a row
constexpr float NEG_INF = -INFINITY;

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}

// 16-byte asynchronous copy; src_bytes == 0 writes zeros and reads nothing.
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, int src_bytes) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(a), "l"(gmem), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Element offset of key p's row in the cache, or -1 if p is outside [0, limit) or has no page.
__device__ __forceinline__ long long key_offset(int p, int limit, const int* table, int table_stride, int page_size,
                                                int num_pages, int Hkv, int kvh, int* status) {
    if (p < 0 || p >= limit) return -1;
    const int blk = p / page_size;
    const int page = blk < table_stride ? table[blk] : -1;
    if (page < 0 || page >= num_pages) {
        atomicOr(status, TW_ERR_PAGE);
        return -1;
    }
    return (((long long)page * Hkv + kvh) * page_size + (p - blk * page_size)) * D;
}

// ---------------------------------------------------------------------------------------
// decode
// ---------------------------------------------------------------------------------------
constexpr int DEC_WARPS = 4;
constexpr int DEC_TILE = 64;                                  // keys per block and iteration (16 per warp)
constexpr int DEC_STAGES = 3;                                 // tiles of a warp in shared memory (2 in flight)
constexpr int DEC_STAGE = 2 * 16 * DP;                        // elements of one warp stage: K then V
constexpr int DEC_PAGE_CACHE = 1024;                          // block-table entries kept in shared memory
constexpr int DEC_SMEM_STAGES = DEC_WARPS * DEC_STAGES * DEC_STAGE * 2;
constexpr int DEC_SMEM_OFFS = DEC_WARPS * DEC_STAGES * 16 * 8;  // row offsets of the tiles in flight
constexpr int DEC_SMEM = DEC_SMEM_STAGES + DEC_SMEM_OFFS + DEC_PAGE_CACHE * 4;

__global__ void __launch_bounds__(DEC_WARPS * 32)
attn_decode_kernel(bf16* __restrict__ out, int out_stride, const bf16* __restrict__ q, int q_stride,
                   const int* __restrict__ seq_q_start, const int* __restrict__ seq_q_len,
                   const int* __restrict__ seq_kv_len, const int* __restrict__ seq_slot,
                   const int* __restrict__ block_table, int table_stride, const bf16* __restrict__ k_cache,
                   const bf16* __restrict__ v_cache, int Hq, int Hkv, int page_size, int num_pages, int window,
                   float scale_log2e, int nsplit, float* __restrict__ partial_o, float* __restrict__ partial_ml,
                   int* __restrict__ counters, int* status) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __shared__ int s_is_last;
    __shared__ float s_row_max[16];
    tw_grid_wait();
    const int s = blockIdx.z, kvh = blockIdx.y;
    const int split = blockIdx.x % nsplit, ht = blockIdx.x / nsplit;
    if (seq_q_len[s] != 1) return;
    const int G = Hq / Hkv, h0 = ht * 16;
    const int nheads = min(16, G - h0);
    const int n = seq_q_start[s];
    const int pos = seq_kv_len[s] - 1;
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int nkeys = pos + 1 - lo;
    const int per = ((nkeys + nsplit - 1) / nsplit + DEC_TILE - 1) / DEC_TILE * DEC_TILE;
    const int k_begin = lo + split * per;
    const int k_end = min(pos + 1, k_begin + per);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, c = lane & 3;
    const int* table = block_table + (size_t)seq_slot[s] * table_stride;

    bf16* stage_base = reinterpret_cast<bf16*>(smem_raw) + warp * DEC_STAGES * DEC_STAGE;
    long long* offs_base = reinterpret_cast<long long*>(smem_raw + DEC_SMEM_STAGES) + warp * DEC_STAGES * 16;
    int* page_cache = reinterpret_cast<int*>(smem_raw + DEC_SMEM_STAGES + DEC_SMEM_OFFS);

    // the block-table entries of this block's keys, read once
    const int first_blk = k_begin / page_size;
    if (k_begin < k_end) {
        const int last_blk = (k_end - 1) / page_size;
        const int nblk = min(DEC_PAGE_CACHE, last_blk - first_blk + 1);
        for (int i = threadIdx.x; i < nblk; i += DEC_WARPS * 32)
            page_cache[i] = first_blk + i < table_stride ? table[first_blk + i] : -1;
    }
    __syncthreads();

    // query fragments: rows g and g + 8 are heads h0 + g and h0 + g + 8 of this group
    uint32_t qf[KSTEPS][4];
    {
        const bf16* q0 = q + (size_t)n * q_stride + (size_t)(kvh * G + h0 + g) * D;
        const bf16* q1 = q0 + 8 * D;
        const bool v0 = g < nheads, v1 = g + 8 < nheads;
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) {
            const int d = ks * 16 + 2 * c;
            qf[ks][0] = v0 ? *reinterpret_cast<const uint32_t*>(q0 + d) : 0u;
            qf[ks][1] = v1 ? *reinterpret_cast<const uint32_t*>(q1 + d) : 0u;
            qf[ks][2] = v0 ? *reinterpret_cast<const uint32_t*>(q0 + d + 8) : 0u;
            qf[ks][3] = v1 ? *reinterpret_cast<const uint32_t*>(q1 + d + 8) : 0u;
        }
    }

    float oacc[NT_O][4];
#pragma unroll
    for (int i = 0; i < NT_O; ++i) { oacc[i][0] = oacc[i][1] = oacc[i][2] = oacc[i][3] = 0.f; }
    float m0 = NEG_INF, m1 = NEG_INF, l0 = 0.f, l1 = 0.f;

    const int ntiles = k_begin < k_end ? (k_end - k_begin + DEC_TILE - 1) / DEC_TILE : 0;

    // lanes 0..15 find the row offsets of the warp's 16 keys from the cached block-table entries
    auto load_tile = [&](int t, int st) {
        if (t < ntiles) {
            const int kb = k_begin + t * DEC_TILE + warp * 16;
            long long* offs = offs_base + st * 16;
            if (lane < 16) {
                const int p = kb + lane;
                long long off = -1;
                if (p < k_end) {
                    const int blk = p / page_size;
                    const int page = blk - first_blk < DEC_PAGE_CACHE ? page_cache[blk - first_blk]
                                                                      : (blk < table_stride ? table[blk] : -1);
                    if (page < 0 || page >= num_pages) atomicOr(status, TW_ERR_PAGE);
                    else off = (((long long)page * Hkv + kvh) * page_size + (p - blk * page_size)) * D;
                }
                offs[lane] = off;
            }
            __syncwarp();
            bf16* ks_ = stage_base + st * DEC_STAGE;
            bf16* vs_ = ks_ + 16 * DP;
#pragma unroll
            for (int i = lane; i < 16 * CHUNKS; i += 32) {
                const int row = i / CHUNKS, col = i - row * CHUNKS;
                const long long off = offs[row];
                const int bytes = off >= 0 ? 16 : 0;
                const long long src = off >= 0 ? off + col * 8 : 0;
                cp_async16(ks_ + row * DP + col * 8, k_cache + src, bytes);
                cp_async16(vs_ + row * DP + col * 8, v_cache + src, bytes);
            }
        }
        cp_async_commit();      // one group per tile slot, empty past the end, so the wait count is constant
    };

#pragma unroll
    for (int t = 0; t < DEC_STAGES - 1; ++t) load_tile(t, t);
    for (int t = 0; t < ntiles; ++t) {
        const int st = t % DEC_STAGES;
        load_tile(t + DEC_STAGES - 1, (t + DEC_STAGES - 1) % DEC_STAGES);
        cp_async_wait<DEC_STAGES - 1>();
        __syncwarp();
        const int kb = k_begin + t * DEC_TILE + warp * 16;
        if (kb < k_end) {
            const bf16* ks_ = stage_base + st * DEC_STAGE;
            const bf16* vs_ = ks_ + 16 * DP;
            float sacc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
            const int j = lane >> 3, r = lane & 7;
#pragma unroll
            for (int ks = 0; ks < KSTEPS; ++ks) {
                uint32_t b[4];
                ldmatrix_x4(b, ks_ + ((j >> 1) * 8 + r) * DP + ks * 16 + (j & 1) * 8);
                mma_bf16(sacc[0], qf[ks], b[0], b[1]);
                mma_bf16(sacc[1], qf[ks], b[2], b[3]);
            }
            // mask, scale, online softmax (rows g and g + 8)
            float rmax0 = NEG_INF, rmax1 = NEG_INF;
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const bool ok = kb + nt * 8 + 2 * c + e < k_end;
                    sacc[nt][e] = ok ? sacc[nt][e] * scale_log2e : NEG_INF;
                    sacc[nt][2 + e] = ok ? sacc[nt][2 + e] * scale_log2e : NEG_INF;
                    rmax0 = fmaxf(rmax0, sacc[nt][e]);
                    rmax1 = fmaxf(rmax1, sacc[nt][2 + e]);
                }
            }
            rmax0 = fmaxf(rmax0, __shfl_xor_sync(0xffffffffu, rmax0, 1));
            rmax0 = fmaxf(rmax0, __shfl_xor_sync(0xffffffffu, rmax0, 2));
            rmax1 = fmaxf(rmax1, __shfl_xor_sync(0xffffffffu, rmax1, 1));
            rmax1 = fmaxf(rmax1, __shfl_xor_sync(0xffffffffu, rmax1, 2));
            const float mn0 = fmaxf(m0, rmax0), mn1 = fmaxf(m1, rmax1);
            const float mu0 = mn0 == NEG_INF ? 0.f : mn0, mu1 = mn1 == NEG_INF ? 0.f : mn1;
            const float a0 = exp2f(m0 - mu0), a1 = exp2f(m1 - mu1);
            m0 = mn0; m1 = mn1;
            float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    sacc[nt][e] = exp2f(sacc[nt][e] - mu0);
                    sacc[nt][2 + e] = exp2f(sacc[nt][2 + e] - mu1);
                    ps0 += sacc[nt][e];
                    ps1 += sacc[nt][2 + e];
                }
            }
            l0 = l0 * a0 + ps0;
            l1 = l1 * a1 + ps1;
            uint32_t pa[4];
            pa[0] = pack_bf16(sacc[0][0], sacc[0][1]);
            pa[1] = pack_bf16(sacc[0][2], sacc[0][3]);
            pa[2] = pack_bf16(sacc[1][0], sacc[1][1]);
            pa[3] = pack_bf16(sacc[1][2], sacc[1][3]);
#pragma unroll
            for (int nt2 = 0; nt2 < NT_O / 2; ++nt2) {
                uint32_t b[4];
                ldmatrix_x4_trans(b, vs_ + ((j & 1) * 8 + r) * DP + nt2 * 16 + (j >> 1) * 8);
                float* o0 = oacc[2 * nt2];
                float* o1 = oacc[2 * nt2 + 1];
                o0[0] *= a0; o0[1] *= a0; o0[2] *= a1; o0[3] *= a1;
                o1[0] *= a0; o1[1] *= a0; o1[2] *= a1; o1[3] *= a1;
                mma_bf16(oacc[2 * nt2], pa, b[0], b[1]);
                mma_bf16(oacc[2 * nt2 + 1], pa, b[2], b[3]);
            }
        }
        __syncwarp();
    }
    cp_async_wait<0>();
    tw_grid_launch_dependents();     // all keys are read: the next kernel may be scheduled
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);

    // merge the warps through shared memory (the stage buffers are free now)
    __syncthreads();
    float* mo = reinterpret_cast<float*>(smem_raw);              // [warps][16][D]
    float* mml = mo + DEC_WARPS * 16 * D;                        // [warps][16][2]
#pragma unroll
    for (int nt = 0; nt < NT_O; ++nt) {
        const int d = nt * 8 + 2 * c;
        float* p0 = mo + ((warp * 16 + g) * D + d);
        float* p1 = mo + ((warp * 16 + g + 8) * D + d);
        p0[0] = oacc[nt][0]; p0[1] = oacc[nt][1];
        p1[0] = oacc[nt][2]; p1[1] = oacc[nt][3];
    }
    if (c == 0) {
        mml[(warp * 16 + g) * 2] = m0; mml[(warp * 16 + g) * 2 + 1] = l0;
        mml[(warp * 16 + g + 8) * 2] = m1; mml[(warp * 16 + g + 8) * 2 + 1] = l1;
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < nheads * D; idx += DEC_WARPS * 32) {
        const int row = idx / D, d = idx - row * D;
        float M = NEG_INF;
#pragma unroll
        for (int w = 0; w < DEC_WARPS; ++w) M = fmaxf(M, mml[(w * 16 + row) * 2]);
        float L = 0.f, o = 0.f;
        if (M != NEG_INF) {
#pragma unroll
            for (int w = 0; w < DEC_WARPS; ++w) {
                const float mw = mml[(w * 16 + row) * 2];
                const float f = mw == NEG_INF ? 0.f : exp2f(mw - M);
                L += mml[(w * 16 + row) * 2 + 1] * f;
                o += mo[(w * 16 + row) * D + d] * f;
            }
        }
        const int head = kvh * G + h0 + row;
        if (nsplit == 1) {
            out[(size_t)n * out_stride + (size_t)head * D + d] = __float2bfloat16_rn(L > 0.f ? o / L : 0.f);
        } else {
            const size_t base = ((size_t)s * Hq + head) * nsplit + split;
            partial_o[base * D + d] = o;
            if (d == 0) { partial_ml[base * 2] = M; partial_ml[base * 2 + 1] = L; }
        }
    }
    if (nsplit == 1) return;

    // The block that finishes last among the slices of this (request, head tile) merges them, in
    // slice order, so the result does not depend on which block that is:
    //   out = sum_i o_i 2^(m_i - M) / sum_i l_i 2^(m_i - M)
    __threadfence();
    __syncthreads();
    int* counter = counters + ((size_t)s * Hkv + kvh) * (gridDim.x / nsplit) + ht;
    if (threadIdx.x == 0) {
        const int done = atomicAdd(counter, 1);
        s_is_last = done == nsplit - 1;
        if (s_is_last) *counter = 0;         // ready for the next launch
    }
    __syncthreads();
    if (!s_is_last) return;
    __threadfence();
    // factors 2^(m_i - M) and weighted sums l_i 2^(m_i - M) of every (head, slice), loaded in parallel
    float* fac = reinterpret_cast<float*>(smem_raw);              // [nheads][nsplit]
    float* lsum = fac + 16 * nsplit;                              // [nheads][nsplit]
    const size_t group_base = ((size_t)s * Hq + kvh * G + h0) * nsplit;      // slices of head h0 start here
    for (int idx = threadIdx.x; idx < nheads * nsplit; idx += DEC_WARPS * 32) {
        fac[idx] = __ldcg(partial_ml + (group_base + idx) * 2);
        lsum[idx] = __ldcg(partial_ml + (group_base + idx) * 2 + 1);
    }
    __syncthreads();
    if (threadIdx.x < nheads) {
        float M = NEG_INF;
        for (int i = 0; i < nsplit; ++i) M = fmaxf(M, fac[threadIdx.x * nsplit + i]);
        s_row_max[threadIdx.x] = M;
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < nheads * nsplit; idx += DEC_WARPS * 32) {
        const float M = s_row_max[idx / nsplit];
        const float mi = fac[idx];
        const float f = (mi == NEG_INF || M == NEG_INF) ? 0.f : exp2f(mi - M);
        fac[idx] = f;
        lsum[idx] *= f;
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < nheads * D; idx += DEC_WARPS * 32) {
        const int row = idx / D, d = idx - row * D;
        const float* f = fac + row * nsplit;
        const float* po = partial_o + (group_base + (size_t)row * nsplit) * D + d;
        float L = 0.f, o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
        for (int i = 0; i < nsplit; ++i) L += lsum[row * nsplit + i];
        int i = 0;
        for (; i + 4 <= nsplit; i += 4) {          // four independent loads in flight; fixed order of the sums
            o0 += __ldcg(po + (size_t)i * D) * f[i];
            o1 += __ldcg(po + (size_t)(i + 1) * D) * f[i + 1];
            o2 += __ldcg(po + (size_t)(i + 2) * D) * f[i + 2];
            o3 += __ldcg(po + (size_t)(i + 3) * D) * f[i + 3];
        }
        for (; i < nsplit; ++i) o0 += __ldcg(po + (size_t)i * D) * f[i];
        const float o = (o0 + o1) + (o2 + o3);
        out[(size_t)n * out_stride + (size_t)(kvh * G + h0 + row) * D + d] = __float2bfloat16_rn(L > 0.f ? o / L : 0.f);
    }
}

// ---------------------------------------------------------------------------------------
// prefill
// ---------------------------------------------------------------------------------------
constexpr int PF_WARPS = 4;
constexpr int PF_BM = 16 * PF_WARPS;                          // rows (token, head) per block
constexpr int PF_BN = 64;                                     // keys per iteration
constexpr int PF_STAGE = 2 * PF_BN * DP;                      // K then V
constexpr int PF_SMEM = 2 * PF_STAGE * 2 + 2 * PF_BN * 8;

__global__ void __launch_bounds__(PF_WARPS * 32)
attn_prefill_kernel(bf16* __restrict__ out, int out_stride, const bf16* __restrict__ q, int q_stride,
                    const int* __restrict__ seq_q_start, const int* __restrict__ seq_q_len,
                    const int* __restrict__ seq_kv_len, const int* __restrict__ seq_slot,
                    const int* __restrict__ block_table, int table_stride, const bf16* __restrict__ k_cache,
                    const bf16* __restrict__ v_cache, int Hq, int Hkv, int page_size, int num_pages, int window,
                    float scale_log2e, int skip_single, int* status) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    tw_grid_wait();
    tw_grid_launch_dependents();
    const int s = blockIdx.z, kvh = blockIdx.y;
    const int q_len = seq_q_len[s];
    if (q_len <= 0 || (skip_single && q_len == 1)) return;
    const int G = Hq / Hkv;
    const int rows_total = q_len * G;
    const int row0 = blockIdx.x * PF_BM;
    if (row0 >= rows_total) return;
    const int kv_len = seq_kv_len[s];
    const int pos0 = kv_len - q_len;                             // position of the first token of this portion
    const int n0 = seq_q_start[s];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, c = lane & 3;
    const int* table = block_table + (size_t)seq_slot[s] * table_stride;

    bf16* stages = reinterpret_cast<bf16*>(smem_raw);
    long long* offs_all = reinterpret_cast<long long*>(smem_raw + 2 * PF_STAGE * 2);

    // rows of this thread
    const int ra = row0 + warp * 16 + g, rb = ra + 8;
    const bool va = ra < rows_total, vb = rb < rows_total;
    const int ta = ra / G, tb = rb / G;
    const int pa_ = pos0 + ta, pb_ = pos0 + tb;                  // positions of the two rows
    const int loa = (window > 0 && pa_ - window + 1 > 0) ? pa_ - window + 1 : 0;
    const int lob = (window > 0 && pb_ - window + 1 > 0) ? pb_ - window + 1 : 0;

    uint32_t qf[KSTEPS][4];
    {
        const bf16* q0 = q + (size_t)(n0 + (va ? ta : 0)) * q_stride + (size_t)(kvh * G + (va ? ra - ta * G : 0)) * D;
        const bf16* q1 = q + (size_t)(n0 + (vb ? tb : 0)) * q_stride + (size_t)(kvh * G + (vb ? rb - tb * G : 0)) * D;
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) {
            const int d = ks * 16 + 2 * c;
            qf[ks][0] = va ? *reinterpret_cast<const uint32_t*>(q0 + d) : 0u;
            qf[ks][1] = vb ? *reinterpret_cast<const uint32_t*>(q1 + d) : 0u;
            qf[ks][2] = va ? *reinterpret_cast<const uint32_t*>(q0 + d + 8) : 0u;
            qf[ks][3] = vb ? *reinterpret_cast<const uint32_t*>(q1 + d + 8) : 0u;
        }
    }
    float oacc[NT_O][4];
#pragma unroll
    for (int i = 0; i < NT_O; ++i) { oacc[i][0] = oacc[i][1] = oacc[i][2] = oacc[i][3] = 0.f; }
    float m0 = NEG_INF, m1 = NEG_INF, l0 = 0.f, l1 = 0.f;

    // keys this block has to look at: from the first row's window start to the last row's position
    const int t_last = min(q_len - 1, (row0 + PF_BM - 1) / G);
    const int key_end = pos0 + t_last + 1;
    const int t_first = row0 / G;
    const int lo_block = (window > 0 && pos0 + t_first - window + 1 > 0) ? pos0 + t_first - window + 1 : 0;
    const int key_begin = lo_block / PF_BN * PF_BN;
    const int ntiles = (key_end - key_begin + PF_BN - 1) / PF_BN;
    // warp-level bounds, to skip tiles no row of the warp can see
    const int wr0 = row0 + warp * 16, wr1 = min(rows_total - 1, wr0 + 15);
    const int warp_hi = pos0 + wr1 / G;
    const int warp_lo = (window > 0 && pos0 + wr0 / G - window + 1 > 0) ? pos0 + wr0 / G - window + 1 : 0;

    auto load_tile = [&](int t, int st) {
        const int kb = key_begin + t * PF_BN;
        long long* offs = offs_all + st * PF_BN;
        if (threadIdx.x < PF_BN)
            offs[threadIdx.x] = key_offset(kb + threadIdx.x, key_end, table, table_stride, page_size, num_pages, Hkv,
                                           kvh, status);
        __syncthreads();
        bf16* ks_ = stages + st * PF_STAGE;
        bf16* vs_ = ks_ + PF_BN * DP;
        for (int i = threadIdx.x; i < PF_BN * CHUNKS; i += PF_WARPS * 32) {
            const int row = i / CHUNKS, col = i - row * CHUNKS;
            const long long off = offs[row];
            const int bytes = off >= 0 ? 16 : 0;
            const long long src = off >= 0 ? off + col * 8 : 0;
            cp_async16(ks_ + row * DP + col * 8, k_cache + src, bytes);
            cp_async16(vs_ + row * DP + col * 8, v_cache + src, bytes);
        }
        cp_async_commit();
    };

    load_tile(0, 0);
    for (int t = 0; t < ntiles; ++t) {
        const int st = t & 1;
        if (t + 1 < ntiles) {
            load_tile(t + 1, st ^ 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const int kb = key_begin + t * PF_BN;
        if (wr0 < rows_total && kb <= warp_hi && kb + PF_BN > warp_lo) {
            const bf16* ks_ = stages + st * PF_STAGE;
            const bf16* vs_ = ks_ + PF_BN * DP;
            float sacc[PF_BN / 8][4];
#pragma unroll
            for (int i = 0; i < PF_BN / 8; ++i) { sacc[i][0] = sacc[i][1] = sacc[i][2] = sacc[i][3] = 0.f; }
            const int j = lane >> 3, r = lane & 7;
#pragma unroll
            for (int ks = 0; ks < KSTEPS; ++ks) {
#pragma unroll
                for (int np = 0; np < PF_BN / 16; ++np) {
                    uint32_t b[4];
                    ldmatrix_x4(b, ks_ + (np * 16 + (j >> 1) * 8 + r) * DP + ks * 16 + (j & 1) * 8);
                    mma_bf16(sacc[2 * np], qf[ks], b[0], b[1]);
                    mma_bf16(sacc[2 * np + 1], qf[ks], b[2], b[3]);
                }
            }
            float rmax0 = NEG_INF, rmax1 = NEG_INF;
#pragma unroll
            for (int nt = 0; nt < PF_BN / 8; ++nt) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int key = kb + nt * 8 + 2 * c + e;
                    const bool oka = va && key <= pa_ && key >= loa;
                    const bool okb = vb && key <= pb_ && key >= lob;
                    sacc[nt][e] = oka ? sacc[nt][e] * scale_log2e : NEG_INF;
                    sacc[nt][2 + e] = okb ? sacc[nt][2 + e] * scale_log2e : NEG_INF;
                    rmax0 = fmaxf(rmax0, sacc[nt][e]);
                    rmax1 = fmaxf(rmax1, sacc[nt][2 + e]);
                }
            }
            rmax0 = fmaxf(rmax0, __shfl_xor_sync(0xffffffffu, rmax0, 1));
            rmax0 = fmaxf(rmax0, __shfl_xor_sync(0xffffffffu, rmax0, 2));
            rmax1 = fmaxf(rmax1, __shfl_xor_sync(0xffffffffu, rmax1, 1));
            rmax1 = fmaxf(rmax1, __shfl_xor_sync(0xffffffffu, rmax1, 2));
            const float mn0 = fmaxf(m0, rmax0), mn1 = fmaxf(m1, rmax1);
            const float mu0 = mn0 == NEG_INF ? 0.f : mn0, mu1 = mn1 == NEG_INF ? 0.f : mn1;
            const float a0 = exp2f(m0 - mu0), a1 = exp2f(m1 - mu1);
            m0 = mn0; m1 = mn1;
            float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
            for (int nt = 0; nt < PF_BN / 8; ++nt) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    sacc[nt][e] = exp2f(sacc[nt][e] - mu0);
                    sacc[nt][2 + e] = exp2f(sacc[nt][2 + e] - mu1);
                    ps0 += sacc[nt][e];
                    ps1 += sacc[nt][2 + e];
                }
            }
            l0 = l0 * a0 + ps0;
            l1 = l1 * a1 + ps1;
#pragma unroll
            for (int nt = 0; nt < NT_O; ++nt) {
                oacc[nt][0] *= a0; oacc[nt][1] *= a0; oacc[nt][2] *= a1; oacc[nt][3] *= a1;
            }
#pragma unroll
            for (int kk = 0; kk < PF_BN / 16; ++kk) {
                uint32_t pa[4];
                pa[0] = pack_bf16(sacc[2 * kk][0], sacc[2 * kk][1]);
                pa[1] = pack_bf16(sacc[2 * kk][2], sacc[2 * kk][3]);
                pa[2] = pack_bf16(sacc[2 * kk + 1][0], sacc[2 * kk + 1][1]);
                pa[3] = pack_bf16(sacc[2 * kk + 1][2], sacc[2 * kk + 1][3]);
#pragma unroll
                for (int nt2 = 0; nt2 < NT_O / 2; ++nt2) {
                    uint32_t b[4];
                    ldmatrix_x4_trans(b, vs_ + (kk * 16 + (j & 1) * 8 + r) * DP + nt2 * 16 + (j >> 1) * 8);
                    mma_bf16(oacc[2 * nt2], pa, b[0], b[1]);
                    mma_bf16(oacc[2 * nt2 + 1], pa, b[2], b[3]);
                }
            }
        }
        __syncthreads();
    }
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const float i0 = l0 > 0.f ? 1.f / l0 : 0.f, i1 = l1 > 0.f ? 1.f / l1 : 0.f;
    bf16* oa = out + (size_t)(n0 + ta) * out_stride + (size_t)(kvh * G + ra - ta * G) * D;
    bf16* ob = out + (size_t)(n0 + tb) * out_stride + (size_t)(kvh * G + rb - tb * G) * D;
#pragma unroll
    for (int nt = 0; nt < NT_O; ++nt) {
        const int d = nt * 8 + 2 * c;
        if (va) *reinterpret_cast<uint32_t*>(oa + d) = pack_bf16(oacc[nt][0] * i0, oacc[nt][1] * i0);
        if (vb) *reinterpret_cast<uint32_t*>(ob + d) = pack_bf16(oacc[nt][2] * i1, oacc[nt][3] * i1);
    }
}

bool g_attrs_set = false;

int set_attrs() {
    if (g_attrs_set) return 0;
    cudaError_t e = cudaFuncSetAttribute(attn_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, DEC_SMEM);
    if (e != cudaSuccess) return (int)e;
    e = cudaFuncSetAttribute(attn_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PF_SMEM);
    if (e != cudaSuccess) return (int)e;
    g_attrs_set = true;
    return 0;
}

}  // namespace

TW_EXPORT int tw_attn_head_dim() { return D; }

// Scratch floats the decode kernel needs for `n_seqs` requests: partial accumulators, then (max, sum) pairs.
// Beside them it needs one int32 counter per (request, key/value head, tile of 16 heads), zero before the
// first launch; the kernel leaves them zero.
TW_EXPORT long long tw_attn_decode_scratch_floats(int n_seqs, int Hq, int nsplit) {
    return (long long)n_seqs * Hq * nsplit * (D + 2);
}

TW_EXPORT int tw_attn_decode(void* out, int out_stride, const void* q, int q_stride, const int* seq_q_start,
                             const int* seq_q_len, const int* seq_kv_len, const int* seq_slot, const int* block_table,
                             int table_stride, const void* k_cache, const void* v_cache, int n_seqs, int Hq, int Hkv,
                             int page_size, int num_pages, int window, float scale, int nsplit, float* scratch,
                             int* counters, int* status, cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (Hkv <= 0 || Hq % Hkv || nsplit < 1 || (nsplit > 1 && (!scratch || !counters))) return (int)cudaErrorInvalidValue;
    if (int e = set_attrs()) return e;
    const int G = Hq / Hkv, htiles = (G + 15) / 16;
    float* partial_o = scratch;
    float* partial_ml = scratch ? scratch + (size_t)n_seqs * Hq * nsplit * D : nullptr;
    dim3 grid(nsplit * htiles, Hkv, n_seqs);
    tw_launch(attn_decode_kernel, dim3(grid), dim3(DEC_WARPS * 32), DEC_SMEM, stream, 1, 
        (bf16*)out, out_stride, (const bf16*)q, q_stride, seq_q_start, seq_q_len, seq_kv_len, seq_slot, block_table,
        table_stride, (const bf16*)k_cache, (const bf16*)v_cache, Hq, Hkv, page_size, num_pages, window,
        scale * 1.4426950408889634f, nsplit, partial_o, partial_ml, counters, status);
    return TW_LAUNCH_CHECK();
}

TW_EXPORT int tw_attn_prefill(void* out, int out_stride, const void* q, int q_stride, const int* seq_q_start,
                              const int* seq_q_len, const int* seq_kv_len, const int* seq_slot, const int* block_table,
                              int table_stride, const void* k_cache, const void* v_cache, int n_seqs, int max_q_len,
                              int Hq, int Hkv, int page_size, int num_pages, int window, float scale, int skip_single,
                              int* status, cudaStream_t stream) {
    if (n_seqs <= 0 || max_q_len <= 0) return 0;
    if (Hkv <= 0 || Hq % Hkv) return (int)cudaErrorInvalidValue;
    if (int e = set_attrs()) return e;
    const int G = Hq / Hkv;
    dim3 grid((max_q_len * G + PF_BM - 1) / PF_BM, Hkv, n_seqs);
    tw_launch(attn_prefill_kernel, dim3(grid), dim3(PF_WARPS * 32), PF_SMEM, stream, 1, 
        (bf16*)out, out_stride, (const bf16*)q, q_stride, seq_q_start, seq_q_len, seq_kv_len, seq_slot, block_table,
        table_stride, (const bf16*)k_cache, (const bf16*)v_cache, Hq, Hkv, page_size, num_pages, window,
        scale * 1.4426950408889634f, skip_single, status);
    return TW_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------------------
// The same decode attention for callers that must not allocate: scratch in the device image.
// See attention_no_alloc.h for what a caller has to know.
// ---------------------------------------------------------------------------------------
#include "attention_no_alloc.h"
#include <stdio.h>

// Counters first (they must be zero when a launch starts), then the partial results.  In host
// code this name is only a handle for cudaGetSymbolAddress, never a device address.
static __device__ __align__(256) unsigned char tw_attn_static_scratch[TW_ATTN_STATIC_SCRATCH_BYTES];

namespace {
constexpr int kMaxDevices = 64;
unsigned char* g_static_scratch_ptr[kMaxDevices] = {};     // device address of the array, per GPU
thread_local char g_static_error[256] = "";
}  // namespace

TW_EXPORT const char* tw_attn_decode_static_last_error(void) { return g_static_error; }

TW_EXPORT int tw_attn_decode_static(void* out, int out_stride, const void* q, int q_stride, const int* seq_q_start,
                                    const int* seq_q_len, const int* seq_kv_len, const int* seq_slot,
                                    const int* block_table, int table_stride, const void* k_cache, const void* v_cache,
                                    int n_seqs, int Hq, int Hkv, int page_size, int num_pages, int window, float scale,
                                    int nsplit, int* status, cudaStream_t stream) {
    g_static_error[0] = 0;
    if (n_seqs <= 0) return 0;
    if (Hkv <= 0 || Hq % Hkv || nsplit < 1) return (int)cudaErrorInvalidValue;
    const int G = Hq / Hkv, htiles = (G + 15) / 16;
    const size_t partial_bytes = sizeof(float) * (size_t)n_seqs * Hq * nsplit * (D + 2);
    const size_t counter_bytes = sizeof(int) * (size_t)n_seqs * Hkv * htiles;
    if (counter_bytes > TW_ATTN_STATIC_COUNTER_BYTES ||
        partial_bytes > TW_ATTN_STATIC_SCRATCH_BYTES - TW_ATTN_STATIC_COUNTER_BYTES) {
        snprintf(g_static_error, sizeof(g_static_error),
                 "tw_attn_decode_static: %d requests x %d heads x %d slices need %zu bytes of partial results and "
                 "%zu bytes of counters; the static array holds %u and %u",
                 n_seqs, Hq, nsplit, partial_bytes, counter_bytes,
                 TW_ATTN_STATIC_SCRATCH_BYTES - TW_ATTN_STATIC_COUNTER_BYTES, TW_ATTN_STATIC_COUNTER_BYTES);
        return TW_ATTN_STATIC_TOO_LARGE;
    }
    // set-up, once per GPU, with that GPU current: the device address of the array
    int device = -1;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return (int)e;
    if (device < 0 || device >= kMaxDevices) return (int)cudaErrorInvalidDevice;
    if (!g_static_scratch_ptr[device]) {
        unsigned char* ptr = nullptr;
        e = cudaGetSymbolAddress((void**)&ptr, tw_attn_static_scratch);
        if (e != cudaSuccess || !ptr) {
            snprintf(g_static_error, sizeof(g_static_error),
                     "tw_attn_decode_static: cudaGetSymbolAddress failed on device %d: %s", device,
                     cudaGetErrorString(e));
            return TW_ATTN_STATIC_NO_SYMBOL;
        }
        g_static_scratch_ptr[device] = ptr;
    }
    unsigned char* base = g_static_scratch_ptr[device];
    int* counters = reinterpret_cast<int*>(base);
    float* partial_o = reinterpret_cast<float*>(base + TW_ATTN_STATIC_COUNTER_BYTES);
    float* partial_ml = partial_o + (size_t)n_seqs * Hq * nsplit * D;
    if (int a = set_attrs()) return a;
    // the array keeps what the last call left; only the counters need a defined start
    e = cudaMemsetAsync(counters, 0, counter_bytes, stream);
    if (e != cudaSuccess) return (int)e;
    dim3 grid(nsplit * htiles, Hkv, n_seqs);
    tw_launch(attn_decode_kernel, dim3(grid), dim3(DEC_WARPS * 32), DEC_SMEM, stream, 1, 
        (bf16*)out, out_stride, (const bf16*)q, q_stride, seq_q_start, seq_q_len, seq_kv_len, seq_slot, block_table,
        table_stride, (const bf16*)k_cache, (const bf16*)v_cache, Hq, Hkv, page_size, num_pages, window,
        scale * 1.4426950408889634f, nsplit, partial_o, partial_ml, counters, status);
    return TW_LAUNCH_CHECK();
}
