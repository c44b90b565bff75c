// Paged grouped-query attention in bfloat16 on the tensor cores, for one head size
// (compile with -DTW_HEAD_DIM=<multiple of 16, 16..256>).
//
// Two kernels share the tile machinery:
//   * decode:  requests that bring ONE token.  A block serves one (request, key/value head,
//     slice of the keys); the query heads of the group are the columns of one MMA tile, so keys
//     and values are read once for the whole group.  The keys are split over blocks
//     ("split-KV").  Up to 16 slices form one thread-block cluster: the partial results (fp32
//     accumulator, running maximum, sum) stay in shared memory and every block of the cluster
//     merges its share of the outputs by reading its neighbours' shared memory.  With more
//     slices the partial results go to scratch memory and the block that finishes last merges
//     them.  Both merge in slice order.
//   * prefill: requests that bring several tokens.  A block serves 128 rows (64 for head sizes
//     above 128), a row being a (token, query head of the group) pair, and walks the keys up
//     to the last visible one; a warp holds two 16-row tiles, so that every key and value
//     fragment it reads from shared memory feeds two MMAs.
// Scores, softmax statistics and the accumulator are fp32; probabilities are rounded to
// bf16 only as the operand of the P.V product.  Keys beyond the visible range are never
// read: their shared-memory rows are zero-filled, so stale page contents cannot leak in.
//
//   score = (q . k) * scale,  visible iff  position - window < p <= position
// Reference: flow_engine/model.py:193-200 and flow_engine/kernels/paged_decode.py:13-43.
#include "common.cuh"
#include "attention_common.cuh"
#include <cooperative_groups.h>

namespace cg = cooperative_groups;

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

using namespace tw_attn;

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
// A warp works on 16 keys at a time with the roles of the MMA operands swapped against the
// prefill kernel: S^T[key, head] = K[key, :] . Q^T, so the (at most 8) query heads of a tile are
// the 8 columns of mma.m16n8k16 and nothing is padded to 16 rows; O^T[d, head] += V^T P^T.
// K goes straight from global memory into A fragments, one tile ahead (the order of d inside a
// dot product does not matter, so a thread reads 16 contiguous bytes of its two key rows per 32
// values of d and q is read with the same permutation); V goes through shared memory, three
// tiles deep, because the product needs it transposed (ldmatrix.trans).  P^T is obtained from the
// S^T fragments with movmatrix.
constexpr int DEC_WARPS = 4;
constexpr int DEC_TILE = DEC_WARPS * 16;                      // keys per block and iteration
constexpr int DEC_HEADS = 8;                                  // query heads per block (columns of the MMA)
constexpr int DEC_STAGES = 3;                                 // V tiles of a warp in shared memory (2 in flight)
constexpr int DEC_STAGE = 16 * DP;                            // elements of one warp stage of V
constexpr int DEC_PAGE_CACHE = 256;                           // block-table entries kept in shared memory
constexpr int DEC_SMEM_STAGES = DEC_WARPS * DEC_STAGES * DEC_STAGE * 2;
constexpr int DEC_SMEM_OFFS = DEC_WARPS * DEC_STAGES * 16 * 8;  // row offsets of the tiles in flight
constexpr int DEC_SMEM = DEC_SMEM_STAGES + DEC_SMEM_OFFS + DEC_PAGE_CACHE * 4;
constexpr int DB32 = D / 32;                                  // whole 32-wide blocks of d
constexpr bool DTAIL16 = (D % 32) != 0;                       // plus one 16-wide block
constexpr int MT_O = D / 16;                                  // m-tiles of O^T
constexpr int DEC_MAX_CLUSTER = 16;                           // slices that can merge through distributed shared memory
// after the last tile the stage buffers hold the warps' partial results and this block's merged slice
static_assert((DEC_WARPS + 1) * DEC_HEADS * (D + 2) * 4 <= DEC_SMEM_STAGES, "merge area must fit the stage buffers");

struct KFrag {                    // the d values of one key row this thread feeds to the MMAs
    uint4 blk[DB32 > 0 ? DB32 : 1];
    uint2 tail;
};

// -DTW_TRACE: every block of the decode kernel records clock64() at its phase boundaries and the global
// timer (ns) at its start and end, for a timeline of one launch (tw_attn_decode_trace_ptr gives the
// buffer: [block][slot]).  Off in the product.
#ifdef TW_TRACE
constexpr int DTRACE_BLOCKS = 2048, DTRACE_SLOTS = 12;
__device__ long long g_dec_trace[DTRACE_BLOCKS * DTRACE_SLOTS];
__device__ __forceinline__ long long global_ns() {
    long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
#define TW_DTRACE(slot)                                                                                 \
    do {                                                                                                \
        const int b_ = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);                  \
        if (threadIdx.x == 0 && b_ < DTRACE_BLOCKS)                                                     \
            g_dec_trace[b_ * DTRACE_SLOTS + (slot)] = ((slot) >= 10) ? global_ns() : clock64();         \
    } while (0)
#else
#define TW_DTRACE(slot) do {} while (0)
#endif

template <bool CLUSTER, bool FUSED>
__global__ void __launch_bounds__(DEC_WARPS * 32, (D <= 128 ? 4 : 2))
attn_decode_kernel(bf16* __restrict__ out, int out_stride, const bf16* __restrict__ q, int q_stride,
                   const int* __restrict__ seq_q_start, const int* __restrict__ seq_q_len,
                   const int* __restrict__ seq_kv_len, const int* __restrict__ seq_slot,
                   const int* __restrict__ block_table, int table_stride, const bf16* k_cache,
                   const bf16* v_cache, int Hq, int Hkv, int page_size, int num_pages, int window,
                   float scale_log2e, int nsplit, float* __restrict__ partial_o, float* __restrict__ partial_ml,
                   int* __restrict__ counters, int* status, const FusedQkv fq) {
    // k_cache and v_cache carry no __restrict__: with FUSED the block that holds the newest position writes that
    // position's key and value through fq.k_cache / fq.v_cache, which are the same memory, and reads them back
    // below: that one key row with ld.global.cg (L2, coherent) and the values with cp.async.cg, never through
    // the non-coherent path, which may hold a line from before the write.
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __shared__ int s_is_last;
    __shared__ float s_row_max[DEC_HEADS];
    __shared__ __align__(16) bf16 s_q[FUSED ? DEC_HEADS * D : 8];      // the rotated query heads, when the kernel makes them
    // The request arrays and the block table are written before the step's first kernel starts, not by the
    // kernel before this one: they are read before the wait for that kernel, while it is still finishing.
    const int s = blockIdx.z, kvh = blockIdx.y;
    const int split = blockIdx.x % nsplit, ht = blockIdx.x / nsplit;
    TW_TIMELINE_SCOPE(TW_K_ATTN_DECODE);
    TW_DTRACE(10);
    TW_DTRACE(0);
    if (seq_q_len[s] != 1) {
        tw_grid_wait();             // a block never finishes before the kernel before this one has
        return;
    }
    const int G = Hq / Hkv, h0 = ht * DEC_HEADS;
    const int nheads = min(DEC_HEADS, G - h0);
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
    TW_DTRACE(1);
    tw_grid_wait();
    TW_TIMELINE_MARK();
    TW_DTRACE(2);

    // ---- with FUSED: bias, rotation by position and the cache write of the step's new token, done here instead
    // of in a kernel of their own (same arithmetic and the same order of the slice sums as that kernel).
    constexpr int half = D / 2;
    const int width = (Hq + 2 * Hkv) * D;
    if constexpr (FUSED) {
        // The block whose slice holds the newest position writes that position's key and value before any of its
        // copies starts (its slice is the last one with keys, and as a rule the shortest).
        if (fq.k_cache && pos >= k_begin && pos < k_end) {
            const int blk = pos / page_size;
            const int page = blk < table_stride ? table[blk] : -1;
            if (page < 0 || page >= num_pages) {
                if (threadIdx.x == 0) atomicOr(status, TW_ERR_PAGE);
            } else {
                const size_t off = (((size_t)page * Hkv + kvh) * page_size + (pos - blk * page_size)) * D;
                for (int i = threadIdx.x; i < D; i += DEC_WARPS * 32) {
                    // thread i: pair i of the key if i < D / 2, and element i of the value
                    const int ik = i < half ? i : 0;
                    const int cols[3] = {(Hq + kvh) * D + ik, (Hq + kvh) * D + ik + half, (Hq + Hkv + kvh) * D + i};
                    float x[3];
                    product_cols<3>(fq, (size_t)n, width, cols, x);
                    if (i < half) {
                        float sn = 0.f, cs = 1.f;
                        if (fq.inv_freq) sincosf((float)pos * fq.inv_freq[i], &sn, &cs);
                        fq.k_cache[off + i] = __float2bfloat16_rn(x[0] * cs - x[1] * sn);
                        fq.k_cache[off + i + half] = __float2bfloat16_rn(x[1] * cs + x[0] * sn);
                    }
                    fq.v_cache[off + i] = __float2bfloat16_rn(x[2]);
                }
            }
            __threadfence();
            __syncthreads();
        }
    }

    // q as the B operand: head h0 + g, with the same order of d as the key fragments
    KFrag qf;
    if constexpr (!FUSED) {
        const bool valid = g < nheads;
        const bf16* qrow = q + (size_t)n * q_stride + (size_t)(kvh * G + h0 + (valid ? g : 0)) * D;
#pragma unroll
        for (int jb = 0; jb < DB32; ++jb)
            qf.blk[jb] = valid ? *reinterpret_cast<const uint4*>(qrow + 32 * jb + 8 * c) : make_uint4(0u, 0u, 0u, 0u);
        qf.tail = (DTAIL16 && valid) ? *reinterpret_cast<const uint2*>(qrow + 32 * DB32 + 4 * c) : make_uint2(0u, 0u);
    }

    float oacc[MT_O][4];
#pragma unroll
    for (int i = 0; i < MT_O; ++i) { oacc[i][0] = oacc[i][1] = oacc[i][2] = oacc[i][3] = 0.f; }
    float m0 = NEG_INF, m1 = NEG_INF, l0 = 0.f, l1 = 0.f;      // heads 2c and 2c + 1 of the tile

    const int ntiles = k_begin < k_end ? (k_end - k_begin + DEC_TILE - 1) / DEC_TILE : 0;

    // lanes 0..15 find the row offsets of the warp's 16 keys of tile t; V of the tile is copied to stage st
    auto stage_tile = [&](int t, int st) {
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
            bf16* vs_ = stage_base + st * DEC_STAGE;
#pragma unroll
            for (int i = lane; i < 16 * CHUNKS; i += 32) {
                const int row = i / CHUNKS, col = i - row * CHUNKS;
                const long long off = offs[row];
                cp_async16(vs_ + row * DP + col * 8, v_cache + (off >= 0 ? off + col * 8 : 0), off >= 0 ? 16 : 0);
            }
        }
        cp_async_commit();      // one group per tile slot, empty past the end, so the wait count is constant
    };
    // K of tile t (rows g and g + 8 of the warp's 16 keys), straight into registers; zero where there is no key.
    // Keys that earlier steps wrote come through the read-only path (ld.global.nc).  With FUSED the row of the
    // newest position was written by this very block a moment ago: it alone is read with ld.global.cg, because
    // the read-only path may still hold its line from before the write.
    auto load_row = [&](long long off, bool fresh, KFrag& k) {
#pragma unroll
        for (int jb = 0; jb < DB32; ++jb) {
            const uint4* p = reinterpret_cast<const uint4*>(k_cache + off + 32 * jb + 8 * c);
            k.blk[jb] = off < 0 ? make_uint4(0u, 0u, 0u, 0u) : (fresh ? __ldcg(p) : __ldg(p));
        }
        const uint2* pt = reinterpret_cast<const uint2*>(k_cache + off + 32 * DB32 + 4 * c);
        k.tail = (!DTAIL16 || off < 0) ? make_uint2(0u, 0u) : (fresh ? __ldcg(pt) : __ldg(pt));
    };
    auto load_k = [&](int t, int st, KFrag& ka, KFrag& kb_) {
        const long long* offs = offs_base + st * 16;
        const long long oa = t < ntiles ? offs[g] : -1, ob = t < ntiles ? offs[g + 8] : -1;
        const int pa = k_begin + t * DEC_TILE + warp * 16 + g;
        load_row(oa, FUSED && pa == pos, ka);
        load_row(ob, FUSED && pa + 8 == pos, kb_);
    };

    KFrag ka_next, kb_next;
    TW_DTRACE(3);
    // With FUSED: this block's query heads (computed once per block, rotated, into shared memory, from where every
    // warp takes its fragments).  Their loads go out first: they come from L2, and issued behind the first keys
    // and values they would stand in the same queue as those.  Up to four slices are kept apart in registers
    // while the keys' copies are issued; more are added afterwards, with the keys on their way.
    constexpr int PQ = (DEC_HEADS * half + DEC_WARPS * 32 - 1) / (DEC_WARPS * 32);     // pairs per thread
    int cols[FUSED ? 2 * PQ : 1];
    float x[FUSED ? 2 * PQ : 1];
    float raw[FUSED ? 2 * PQ : 1][4];
    float freq[FUSED ? PQ : 1];
    const bool early_q = FUSED && fq.partial && fq.nslices <= 4;
    if constexpr (FUSED) {
#pragma unroll
        for (int j = 0; j < PQ; ++j) {
            const int p = threadIdx.x + j * DEC_WARPS * 32;
            const int head = p / half, i = p - head * half;
            const bool live = p < DEC_HEADS * half && head < nheads;
            cols[2 * j] = live ? (kvh * G + h0 + head) * D + i : 0;
            cols[2 * j + 1] = cols[2 * j] + half;
            freq[j] = (fq.inv_freq && live) ? fq.inv_freq[i] : 0.f;
        }
        if (early_q) {
            const float* prow = fq.partial + (size_t)n * width;
#pragma unroll
            for (int j = 0; j < 2 * PQ; ++j) {
#pragma unroll
                for (int u = 0; u < 4; ++u) raw[j][u] = u < fq.nslices ? prow[(size_t)u * fq.slice_stride + cols[j]] : 0.f;
                x[j] = fq.bias ? fq.bias[cols[j]] : 0.f;
            }
        }
    }
    stage_tile(0, 0);
    load_k(0, 0, ka_next, kb_next);
    stage_tile(1, 1);
    TW_DTRACE(4);
    if constexpr (FUSED) {
        if (early_q) {
            // the sums product_cols makes: four slices pairwise, fewer one after the other
#pragma unroll
            for (int j = 0; j < 2 * PQ; ++j) {
                const float sum = fq.nslices == 4 ? (raw[j][0] + raw[j][1]) + (raw[j][2] + raw[j][3])
                                                  : ((raw[j][0] + raw[j][1]) + raw[j][2]);
                x[j] = fq.bias ? sum + x[j] : sum;
            }
        } else {
            product_cols<2 * PQ>(fq, (size_t)n, width, cols, x);
        }
        TW_DTRACE(5);
#pragma unroll
        for (int j = 0; j < PQ; ++j) {
            const int p = threadIdx.x + j * DEC_WARPS * 32;
            if (p < DEC_HEADS * half) {
                const int head = p / half, i = p - head * half;
                float y1 = 0.f, y2 = 0.f;
                if (head < nheads) {
                    float sn = 0.f, cs = 1.f;
                    if (fq.inv_freq) sincosf((float)pos * freq[j], &sn, &cs);
                    y1 = x[2 * j] * cs - x[2 * j + 1] * sn;
                    y2 = x[2 * j + 1] * cs + x[2 * j] * sn;
                }
                s_q[head * D + i] = __float2bfloat16_rn(y1);
                s_q[head * D + i + half] = __float2bfloat16_rn(y2);
            }
        }
        __syncthreads();
        const bf16* qrow = s_q + g * D;                     // zero beyond nheads
#pragma unroll
        for (int jb = 0; jb < DB32; ++jb) qf.blk[jb] = *reinterpret_cast<const uint4*>(qrow + 32 * jb + 8 * c);
        qf.tail = DTAIL16 ? *reinterpret_cast<const uint2*>(qrow + 32 * DB32 + 4 * c) : make_uint2(0u, 0u);
    }
    TW_DTRACE(6);
    for (int t = 0; t < ntiles; ++t) {
        const int st = t % DEC_STAGES;
        const KFrag ka = ka_next, kb_ = kb_next;
        stage_tile(t + 2, (t + 2) % DEC_STAGES);
        load_k(t + 1, (t + 1) % DEC_STAGES, ka_next, kb_next);      // in flight while this tile is worked on
        const int key0 = k_begin + t * DEC_TILE + warp * 16;
        if (key0 < k_end) {
            // S^T = K Q^T: rows = keys g, g + 8; columns = heads 2c, 2c + 1
            float sacc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int jb = 0; jb < DB32; ++jb) {
                mma_bf16_regs(sacc, ka.blk[jb].x, kb_.blk[jb].x, ka.blk[jb].y, kb_.blk[jb].y, qf.blk[jb].x, qf.blk[jb].y);
                mma_bf16_regs(sacc, ka.blk[jb].z, kb_.blk[jb].z, ka.blk[jb].w, kb_.blk[jb].w, qf.blk[jb].z, qf.blk[jb].w);
            }
            if (DTAIL16) mma_bf16_regs(sacc, ka.tail.x, kb_.tail.x, ka.tail.y, kb_.tail.y, qf.tail.x, qf.tail.y);
            const bool oka = key0 + g < k_end, okb = key0 + g + 8 < k_end;
            sacc[0] = oka ? sacc[0] * scale_log2e : NEG_INF;
            sacc[1] = oka ? sacc[1] * scale_log2e : NEG_INF;
            sacc[2] = okb ? sacc[2] * scale_log2e : NEG_INF;
            sacc[3] = okb ? sacc[3] * scale_log2e : NEG_INF;
            // maxima over the 16 keys: over the lanes that share c
            float r0 = fmaxf(sacc[0], sacc[2]), r1 = fmaxf(sacc[1], sacc[3]);
#pragma unroll
            for (int o = 4; o < 32; o <<= 1) {
                r0 = fmaxf(r0, __shfl_xor_sync(0xffffffffu, r0, o));
                r1 = fmaxf(r1, __shfl_xor_sync(0xffffffffu, r1, o));
            }
            const float mn0 = fmaxf(m0, r0), mn1 = fmaxf(m1, r1);
            const float mu0 = mn0 == NEG_INF ? 0.f : mn0, mu1 = mn1 == NEG_INF ? 0.f : mn1;
            const float a0 = exp2f(m0 - mu0), a1 = exp2f(m1 - mu1);
            const bool rescale = (mn0 != m0) || (mn1 != m1);
            m0 = mn0; m1 = mn1;
            sacc[0] = exp2f(sacc[0] - mu0); sacc[1] = exp2f(sacc[1] - mu1);
            sacc[2] = exp2f(sacc[2] - mu0); sacc[3] = exp2f(sacc[3] - mu1);
            l0 = l0 * a0 + sacc[0] + sacc[2];          // this thread's keys only; summed over g at the end
            l1 = l1 * a1 + sacc[1] + sacc[3];
            // P^T as the B operand: keys 2c, 2c + 1 (and + 8) of head g
            const uint32_t pb0 = movmatrix_trans(pack_bf16(sacc[0], sacc[1]));
            const uint32_t pb1 = movmatrix_trans(pack_bf16(sacc[2], sacc[3]));
            if (__any_sync(0xffffffffu, rescale)) {
#pragma unroll
                for (int mt = 0; mt < MT_O; ++mt) {
                    oacc[mt][0] *= a0; oacc[mt][1] *= a1; oacc[mt][2] *= a0; oacc[mt][3] *= a1;
                }
            }
            cp_async_wait<DEC_STAGES - 1>();            // V of this tile has landed
            __syncwarp();
            const bf16* vs_ = stage_base + st * DEC_STAGE;
            const int j = lane >> 3, r = lane & 7;
#pragma unroll
            for (int mt = 0; mt < MT_O; ++mt) {
                uint32_t a[4];
                ldmatrix_x4_trans(a, vs_ + ((j >> 1) * 8 + r) * DP + mt * 16 + (j & 1) * 8);
                mma_bf16_regs(oacc[mt], a[0], a[1], a[2], a[3], pb0, pb1);
            }
        }
        __syncwarp();
    }
    cp_async_wait<0>();
    // the keys and values are in: while the slices merge, the memory system may fetch the next kernel's weights
    if constexpr (FUSED) {
        if (threadIdx.x == 0) tw_prefetch_l2_share(fq.next_weights, fq.next_bytes);
    }
    TW_DTRACE(7);
    // sums over the keys of the other threads with the same heads
#pragma unroll
    for (int o = 4; o < 32; o <<= 1) {
        l0 += __shfl_xor_sync(0xffffffffu, l0, o);
        l1 += __shfl_xor_sync(0xffffffffu, l1, o);
    }

    // merge the warps through shared memory (the stage buffers are free now)
    __syncthreads();
    float* mo = reinterpret_cast<float*>(smem_raw);              // [warps][heads][D]
    float* mml = mo + DEC_WARPS * DEC_HEADS * D;                 // [warps][heads][2]
#pragma unroll
    for (int mt = 0; mt < MT_O; ++mt) {
        const int d = mt * 16 + g;
        float* p0 = mo + (warp * DEC_HEADS + 2 * c) * D;
        float* p1 = p0 + D;
        p0[d] = oacc[mt][0]; p1[d] = oacc[mt][1];
        p0[d + 8] = oacc[mt][2]; p1[d + 8] = oacc[mt][3];
    }
    if (g == 0) {
        mml[(warp * DEC_HEADS + 2 * c) * 2] = m0; mml[(warp * DEC_HEADS + 2 * c) * 2 + 1] = l0;
        mml[(warp * DEC_HEADS + 2 * c + 1) * 2] = m1; mml[(warp * DEC_HEADS + 2 * c + 1) * 2 + 1] = l1;
    }
    float* part_o = mml + DEC_WARPS * DEC_HEADS * 2;             // [heads][D]: this block's slice, for the cluster
    float* part_ml = part_o + DEC_HEADS * D;                     // [heads][2]
    __syncthreads();
    for (int idx = threadIdx.x; idx < nheads * D; idx += DEC_WARPS * 32) {
        const int row = idx / D, d = idx - row * D;
        float M = NEG_INF;
#pragma unroll
        for (int w = 0; w < DEC_WARPS; ++w) M = fmaxf(M, mml[(w * DEC_HEADS + row) * 2]);
        float L = 0.f, o = 0.f;
        if (M != NEG_INF) {
#pragma unroll
            for (int w = 0; w < DEC_WARPS; ++w) {
                const float mw = mml[(w * DEC_HEADS + row) * 2];
                const float f = mw == NEG_INF ? 0.f : exp2f(mw - M);
                L += mml[(w * DEC_HEADS + row) * 2 + 1] * f;
                o += mo[(w * DEC_HEADS + row) * D + d] * f;
            }
        }
        const int head = kvh * G + h0 + row;
        if (nsplit == 1) {
            out[(size_t)n * out_stride + (size_t)head * D + d] = __float2bfloat16_rn(L > 0.f ? o / L : 0.f);
        } else if (CLUSTER) {
            part_o[row * D + d] = o;
            if (d == 0) { part_ml[row * 2] = M; part_ml[row * 2 + 1] = L; }
        } else {
            const size_t base = ((size_t)s * Hq + head) * nsplit + split;
            partial_o[base * D + d] = o;
            if (d == 0) { partial_ml[base * 2] = M; partial_ml[base * 2 + 1] = L; }
        }
    }
    tw_grid_launch_dependents_late();
    if (nsplit == 1) return;

    if constexpr (CLUSTER) {
        // The slices of this (request, head tile) are the blocks of one cluster, slice i being block
        // i.  Every block merges its share of the outputs, reading all slices in slice order:
        //   out = sum_i o_i 2^(m_i - M) / sum_i l_i 2^(m_i - M)
        cg::cluster_group cluster = cg::this_cluster();
        TW_DTRACE(8);
        cluster.sync();
        for (int idx = split * (DEC_WARPS * 32) + threadIdx.x; idx < nheads * D; idx += nsplit * (DEC_WARPS * 32)) {
            const int row = idx / D, d = idx - row * D;
            float M = NEG_INF;
            for (int i = 0; i < nsplit; ++i) M = fmaxf(M, *cluster.map_shared_rank(part_ml + row * 2, i));
            float L = 0.f, o = 0.f;
            for (int i = 0; i < nsplit; ++i) {
                const float* ml = cluster.map_shared_rank(part_ml + row * 2, i);
                const float mi = ml[0];
                const float f = (mi == NEG_INF || M == NEG_INF) ? 0.f : exp2f(mi - M);
                L += ml[1] * f;
                o += *cluster.map_shared_rank(part_o + row * D + d, i) * f;
            }
            out[(size_t)n * out_stride + (size_t)(kvh * G + h0 + row) * D + d] = __float2bfloat16_rn(L > 0.f ? o / L : 0.f);
        }
        cluster.sync();          // nobody leaves while a neighbour may still read its shared memory
        TW_DTRACE(9);
        TW_DTRACE(11);
        return;
    }

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
    float* lsum = fac + DEC_HEADS * nsplit;                       // [nheads][nsplit]
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
    // four values of d per thread and eight slices in flight at once: the merge is a chain of
    // L2 round trips on one block while the rest of the GPU waits, so it is kept short
    constexpr int D4 = D / 4;
    for (int idx = threadIdx.x; idx < nheads * D4; idx += DEC_WARPS * 32) {
        const int row = idx / D4, d4 = idx - row * D4;
        const float* f = fac + row * nsplit;
        const float4* po = reinterpret_cast<const float4*>(partial_o + (group_base + (size_t)row * nsplit) * D) + d4;
        float L = 0.f;
        for (int i = 0; i < nsplit; ++i) L += lsum[row * nsplit + i];
        float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
        int i = 0;
        for (; i + 8 <= nsplit; i += 8) {          // fixed order of the sums: slice 0, 1, 2, ...
            float4 v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = __ldcg(po + (size_t)(i + j) * D4);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float fj = f[i + j];
                o.x += v[j].x * fj; o.y += v[j].y * fj; o.z += v[j].z * fj; o.w += v[j].w * fj;
            }
        }
        for (; i < nsplit; ++i) {
            const float4 v = __ldcg(po + (size_t)i * D4);
            const float fj = f[i];
            o.x += v.x * fj; o.y += v.y * fj; o.z += v.z * fj; o.w += v.w * fj;
        }
        const float inv = L > 0.f ? 1.f / L : 0.f;
        uint2 packed;
        packed.x = pack_bf16(o.x * inv, o.y * inv);
        packed.y = pack_bf16(o.z * inv, o.w * inv);
        *reinterpret_cast<uint2*>(out + (size_t)n * out_stride + (size_t)(kvh * G + h0 + row) * D + 4 * d4) = packed;
    }
}

// ---------------------------------------------------------------------------------------
// prefill
// ---------------------------------------------------------------------------------------
constexpr int PF_WARPS = 4;
constexpr int PF_MT = D <= 128 ? 2 : 1;                       // 16-row tiles per warp (the accumulators must fit the registers)
constexpr int PF_BM = 16 * PF_MT * PF_WARPS;                  // rows (token, head) per block
constexpr int PF_BN = 64;                                     // keys per iteration
constexpr int PF_STAGE = 2 * PF_BN * DP;                      // K then V
constexpr int PF_Q_ELEMS = PF_BM * DP;
constexpr int PF_SMEM = PF_Q_ELEMS * 2 + 2 * PF_STAGE * 2 + 2 * PF_BN * 8;

__global__ void __launch_bounds__(PF_WARPS * 32, (D <= 128 ? 2 : 1))
attn_prefill_kernel(bf16* __restrict__ out, int out_stride, const bf16* __restrict__ q, int q_stride,
                    const int* __restrict__ seq_q_start, const int* __restrict__ seq_q_len,
                    const int* __restrict__ seq_kv_len, const int* __restrict__ seq_slot,
                    const int* __restrict__ block_table, int table_stride, const bf16* __restrict__ k_cache,
                    const bf16* __restrict__ v_cache, int Hq, int Hkv, int page_size, int num_pages, int window,
                    float scale_log2e, int skip_single, int* status) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    TW_TIMELINE_SCOPE(TW_K_ATTN_PREFILL);
    tw_grid_wait();
    TW_TIMELINE_MARK();
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

    bf16* q_tile = reinterpret_cast<bf16*>(smem_raw);
    bf16* stages = q_tile + PF_Q_ELEMS;
    long long* offs_all = reinterpret_cast<long long*>(smem_raw + PF_Q_ELEMS * 2 + 2 * PF_STAGE * 2);

    // the block's query rows into shared memory (rows beyond the portion are zero)
    for (int i = threadIdx.x; i < PF_BM * CHUNKS; i += PF_WARPS * 32) {
        const int rr = i / CHUNKS, col = i - rr * CHUNKS;
        const int r = row0 + rr;
        const bool v = r < rows_total;
        const int t = v ? r / G : 0;
        const bf16* src = q + (size_t)(n0 + t) * q_stride + (size_t)(kvh * G + (v ? r - t * G : 0)) * D + col * 8;
        cp_async16(q_tile + rr * DP + col * 8, src, v ? 16 : 0);
    }
    cp_async_commit();

    // rows of this thread: m-tile mt holds rows wbase + 16 mt + g and + 8
    const int wbase = row0 + warp * 16 * PF_MT;
    int rpos[PF_MT][2], rlo[PF_MT][2];
    bool rvalid[PF_MT][2];
#pragma unroll
    for (int mt = 0; mt < PF_MT; ++mt) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int r = wbase + 16 * mt + g + 8 * h;
            rvalid[mt][h] = r < rows_total;
            rpos[mt][h] = pos0 + r / G;
            rlo[mt][h] = (window > 0 && rpos[mt][h] - window + 1 > 0) ? rpos[mt][h] - window + 1 : 0;
        }
    }
    float oacc[PF_MT][NT_O][4];
    float mrow[PF_MT][2], lrow[PF_MT][2];
#pragma unroll
    for (int mt = 0; mt < PF_MT; ++mt) {
        mrow[mt][0] = mrow[mt][1] = NEG_INF;
        lrow[mt][0] = lrow[mt][1] = 0.f;
#pragma unroll
        for (int i = 0; i < NT_O; ++i) { oacc[mt][i][0] = oacc[mt][i][1] = oacc[mt][i][2] = oacc[mt][i][3] = 0.f; }
    }

    // keys this block has to look at: from the first row's window start to the last row's position
    const int t_last = min(q_len - 1, (row0 + PF_BM - 1) / G);
    const int key_end = pos0 + t_last + 1;
    const int t_first = row0 / G;
    const int lo_block = (window > 0 && pos0 + t_first - window + 1 > 0) ? pos0 + t_first - window + 1 : 0;
    const int key_begin = lo_block / PF_BN * PF_BN;
    const int ntiles = (key_end - key_begin + PF_BN - 1) / PF_BN;
    // warp-level bounds, to skip tiles no row of the warp can see
    const int wr1 = min(rows_total - 1, wbase + 16 * PF_MT - 1);
    const int warp_hi = pos0 + wr1 / G;
    const int warp_lo = (window > 0 && pos0 + wbase / G - window + 1 > 0) ? pos0 + wbase / G - window + 1 : 0;

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

    const int j = lane >> 3, r8 = lane & 7;
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
        if (wbase < rows_total && kb <= warp_hi && kb + PF_BN > warp_lo) {
            const bf16* ks_ = stages + st * PF_STAGE;
            const bf16* vs_ = ks_ + PF_BN * DP;
            float sacc[PF_MT][PF_BN / 8][4];
#pragma unroll
            for (int mt = 0; mt < PF_MT; ++mt)
#pragma unroll
                for (int i = 0; i < PF_BN / 8; ++i) { sacc[mt][i][0] = sacc[mt][i][1] = sacc[mt][i][2] = sacc[mt][i][3] = 0.f; }
#pragma unroll
            for (int ks = 0; ks < KSTEPS; ++ks) {
                uint32_t qa[PF_MT][4];
#pragma unroll
                for (int mt = 0; mt < PF_MT; ++mt)
                    ldmatrix_x4(qa[mt], q_tile + ((warp * PF_MT + mt) * 16 + (j & 1) * 8 + r8) * DP + ks * 16 + (j >> 1) * 8);
#pragma unroll
                for (int np = 0; np < PF_BN / 16; ++np) {
                    uint32_t b[4];
                    ldmatrix_x4(b, ks_ + (np * 16 + (j >> 1) * 8 + r8) * DP + ks * 16 + (j & 1) * 8);
#pragma unroll
                    for (int mt = 0; mt < PF_MT; ++mt) {
                        mma_bf16(sacc[mt][2 * np], qa[mt], b[0], b[1]);
                        mma_bf16(sacc[mt][2 * np + 1], qa[mt], b[2], b[3]);
                    }
                }
            }
            uint32_t pfrag[PF_MT][PF_BN / 16][4];
#pragma unroll
            for (int mt = 0; mt < PF_MT; ++mt) {
                float rmax0 = NEG_INF, rmax1 = NEG_INF;
#pragma unroll
                for (int nt = 0; nt < PF_BN / 8; ++nt) {
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int key = kb + nt * 8 + 2 * c + e;
                        const bool oka = rvalid[mt][0] && key <= rpos[mt][0] && key >= rlo[mt][0];
                        const bool okb = rvalid[mt][1] && key <= rpos[mt][1] && key >= rlo[mt][1];
                        sacc[mt][nt][e] = oka ? sacc[mt][nt][e] * scale_log2e : NEG_INF;
                        sacc[mt][nt][2 + e] = okb ? sacc[mt][nt][2 + e] * scale_log2e : NEG_INF;
                        rmax0 = fmaxf(rmax0, sacc[mt][nt][e]);
                        rmax1 = fmaxf(rmax1, sacc[mt][nt][2 + e]);
                    }
                }
                rmax0 = fmaxf(rmax0, __shfl_xor_sync(0xffffffffu, rmax0, 1));
                rmax0 = fmaxf(rmax0, __shfl_xor_sync(0xffffffffu, rmax0, 2));
                rmax1 = fmaxf(rmax1, __shfl_xor_sync(0xffffffffu, rmax1, 1));
                rmax1 = fmaxf(rmax1, __shfl_xor_sync(0xffffffffu, rmax1, 2));
                const float mn0 = fmaxf(mrow[mt][0], rmax0), mn1 = fmaxf(mrow[mt][1], rmax1);
                const float mu0 = mn0 == NEG_INF ? 0.f : mn0, mu1 = mn1 == NEG_INF ? 0.f : mn1;
                const float a0 = exp2f(mrow[mt][0] - mu0), a1 = exp2f(mrow[mt][1] - mu1);
                mrow[mt][0] = mn0; mrow[mt][1] = mn1;
                float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
                for (int nt = 0; nt < PF_BN / 8; ++nt) {
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        sacc[mt][nt][e] = exp2f(sacc[mt][nt][e] - mu0);
                        sacc[mt][nt][2 + e] = exp2f(sacc[mt][nt][2 + e] - mu1);
                        ps0 += sacc[mt][nt][e];
                        ps1 += sacc[mt][nt][2 + e];
                    }
                }
                lrow[mt][0] = lrow[mt][0] * a0 + ps0;
                lrow[mt][1] = lrow[mt][1] * a1 + ps1;
#pragma unroll
                for (int nt = 0; nt < NT_O; ++nt) {
                    oacc[mt][nt][0] *= a0; oacc[mt][nt][1] *= a0; oacc[mt][nt][2] *= a1; oacc[mt][nt][3] *= a1;
                }
#pragma unroll
                for (int kk = 0; kk < PF_BN / 16; ++kk) {
                    pfrag[mt][kk][0] = pack_bf16(sacc[mt][2 * kk][0], sacc[mt][2 * kk][1]);
                    pfrag[mt][kk][1] = pack_bf16(sacc[mt][2 * kk][2], sacc[mt][2 * kk][3]);
                    pfrag[mt][kk][2] = pack_bf16(sacc[mt][2 * kk + 1][0], sacc[mt][2 * kk + 1][1]);
                    pfrag[mt][kk][3] = pack_bf16(sacc[mt][2 * kk + 1][2], sacc[mt][2 * kk + 1][3]);
                }
            }
#pragma unroll
            for (int kk = 0; kk < PF_BN / 16; ++kk) {
#pragma unroll
                for (int nt2 = 0; nt2 < NT_O / 2; ++nt2) {
                    uint32_t b[4];
                    ldmatrix_x4_trans(b, vs_ + (kk * 16 + (j & 1) * 8 + r8) * DP + nt2 * 16 + (j >> 1) * 8);
#pragma unroll
                    for (int mt = 0; mt < PF_MT; ++mt) {
                        mma_bf16(oacc[mt][2 * nt2], pfrag[mt][kk], b[0], b[1]);
                        mma_bf16(oacc[mt][2 * nt2 + 1], pfrag[mt][kk], b[2], b[3]);
                    }
                }
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int mt = 0; mt < PF_MT; ++mt) {
        float l0 = lrow[mt][0], l1 = lrow[mt][1];
        l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
        l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
        l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
        l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
        const float i0 = l0 > 0.f ? 1.f / l0 : 0.f, i1 = l1 > 0.f ? 1.f / l1 : 0.f;
        const int ra = wbase + 16 * mt + g, rb = ra + 8;
        const int ta = ra / G, tb = rb / G;
        bf16* oa = out + (size_t)(n0 + ta) * out_stride + (size_t)(kvh * G + ra - ta * G) * D;
        bf16* ob = out + (size_t)(n0 + tb) * out_stride + (size_t)(kvh * G + rb - tb * G) * D;
#pragma unroll
        for (int nt = 0; nt < NT_O; ++nt) {
            const int d = nt * 8 + 2 * c;
            if (rvalid[mt][0]) *reinterpret_cast<uint32_t*>(oa + d) = pack_bf16(oacc[mt][nt][0] * i0, oacc[mt][nt][1] * i0);
            if (rvalid[mt][1]) *reinterpret_cast<uint32_t*>(ob + d) = pack_bf16(oacc[mt][nt][2] * i1, oacc[mt][nt][3] * i1);
        }
    }
}

bool g_attrs_set = false;

int set_attrs() {
    if (g_attrs_set) return 0;
    cudaError_t e = cudaFuncSetAttribute(attn_decode_kernel<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, DEC_SMEM);
    if (e != cudaSuccess) return (int)e;
    e = cudaFuncSetAttribute(attn_decode_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, DEC_SMEM);
    if (e != cudaSuccess) return (int)e;
    e = cudaFuncSetAttribute(attn_decode_kernel<true, false>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
    if (e != cudaSuccess) return (int)e;
    e = cudaFuncSetAttribute(attn_decode_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, DEC_SMEM);
    if (e != cudaSuccess) return (int)e;
    e = cudaFuncSetAttribute(attn_decode_kernel<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, DEC_SMEM);
    if (e != cudaSuccess) return (int)e;
    e = cudaFuncSetAttribute(attn_decode_kernel<true, true>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
    if (e != cudaSuccess) return (int)e;
    e = cudaFuncSetAttribute(attn_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PF_SMEM);
    if (e != cudaSuccess) return (int)e;
    g_attrs_set = true;
    return 0;
}

// Whether clusters of `size` decode blocks can be resident on this GPU (asked once per size).
int g_cluster_ok[DEC_MAX_CLUSTER + 1];          // 0 = not asked yet, 1 = yes, -1 = no

bool decode_cluster_ok(int size) {
    if (size < 2 || size > DEC_MAX_CLUSTER) return false;
    if (g_cluster_ok[size] == 0) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(size);
        cfg.blockDim = dim3(DEC_WARPS * 32);
        cfg.dynamicSmemBytes = DEC_SMEM;
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = size;
        attr.val.clusterDim.y = 1;
        attr.val.clusterDim.z = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        int clusters = 0;
        const cudaError_t e = cudaOccupancyMaxActiveClusters(&clusters, attn_decode_kernel<true, false>, &cfg);
        if (e != cudaSuccess) (void)cudaGetLastError();
        g_cluster_ok[size] = (e == cudaSuccess && clusters >= 1) ? 1 : -1;
    }
    return g_cluster_ok[size] > 0;
}

}  // namespace

TW_EXPORT int tw_attn_head_dim() { return D; }

#ifdef TW_TRACE
TW_EXPORT int tw_attn_decode_trace_ptr(void** ptr, int* blocks, int* slots) {
    *blocks = DTRACE_BLOCKS; *slots = DTRACE_SLOTS;
    return (int)cudaGetSymbolAddress(ptr, g_dec_trace);
}
#endif

// Most slices that merge through a cluster; more go through scratch memory.
TW_EXPORT int tw_attn_decode_cluster_slices() { return DEC_MAX_CLUSTER; }

// Scratch floats the decode kernel needs for `n_seqs` requests: partial accumulators, then (max, sum) pairs.
// Beside them it needs one int32 counter per (request, key/value head, tile of 8 heads), zero before the
// first launch; the kernel leaves them zero.
TW_EXPORT long long tw_attn_decode_scratch_floats(int n_seqs, int Hq, int nsplit) {
    return (long long)n_seqs * Hq * nsplit * (D + 2);
}

// Most slices a request's keys may be cut into.  The merge through scratch memory keeps two floats per
// (head, slice) in the block's dynamic shared memory; beyond this limit they would not fit at every head size.
constexpr int DEC_MAX_SPLITS = 128;
static_assert(2 * DEC_HEADS * DEC_MAX_SPLITS * 4 <= DEC_SMEM, "the merge factors of the most slices must fit the block's shared memory");

TW_EXPORT int tw_attn_decode_max_splits() { return DEC_MAX_SPLITS; }

// What every decode entry point refuses before it launches: more slices than the merge has room for, and a
// query that the kernel's 16-byte loads cannot read.
static int decode_refuses(int nsplit, const void* q, int q_stride) {
    if (nsplit < 1 || nsplit > DEC_MAX_SPLITS) return (int)cudaErrorInvalidValue;
    if (q && (((uintptr_t)q & 15) || (q_stride & 7))) return (int)cudaErrorMisalignedAddress;
    return 0;
}

TW_EXPORT int tw_attn_decode(void* out, int out_stride, const void* q, int q_stride, const int* seq_q_start,
                             const int* seq_q_len, const int* seq_kv_len, const int* seq_slot, const int* block_table,
                             int table_stride, const void* k_cache, const void* v_cache, int n_seqs, int Hq, int Hkv,
                             int page_size, int num_pages, int window, float scale, int nsplit, int flags,
                             float* scratch, int* counters, int* status, cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (Hkv <= 0 || Hq % Hkv || nsplit < 1 || (nsplit > 1 && (!scratch || !counters))) return (int)cudaErrorInvalidValue;
    if (int r = decode_refuses(nsplit, q, q_stride)) return r;
    // the merge reads the partial results 16 bytes at a time and writes 8 bytes of the result at a time
    if (((uintptr_t)out & 7) || (out_stride & 3) || ((uintptr_t)scratch & 15)) return (int)cudaErrorMisalignedAddress;
    if (int e = set_attrs()) return e;
    const int G = Hq / Hkv, htiles = (G + DEC_HEADS - 1) / DEC_HEADS;
    float* partial_o = scratch;
    float* partial_ml = scratch ? scratch + (size_t)n_seqs * Hq * nsplit * D : nullptr;
    dim3 grid(nsplit * htiles, Hkv, n_seqs);
    if (nsplit > 1 && !(flags & 1) && decode_cluster_ok(nsplit))
        return tw_launch(attn_decode_kernel<true, false>, dim3(grid), dim3(DEC_WARPS * 32), DEC_SMEM, stream, nsplit,
            (bf16*)out, out_stride, (const bf16*)q, q_stride, seq_q_start, seq_q_len, seq_kv_len, seq_slot, block_table,
            table_stride, (const bf16*)k_cache, (const bf16*)v_cache, Hq, Hkv, page_size, num_pages, window,
            scale * 1.4426950408889634f, nsplit, partial_o, partial_ml, counters, status, FusedQkv{});
    tw_launch(attn_decode_kernel<false, false>, dim3(grid), dim3(DEC_WARPS * 32), DEC_SMEM, stream, 1, 
        (bf16*)out, out_stride, (const bf16*)q, q_stride, seq_q_start, seq_q_len, seq_kv_len, seq_slot, block_table,
        table_stride, (const bf16*)k_cache, (const bf16*)v_cache, Hq, Hkv, page_size, num_pages, window,
        scale * 1.4426950408889634f, nsplit, partial_o, partial_ml, counters, status, FusedQkv{});
    return TW_LAUNCH_CHECK();
}

// The same for a decode-only step whose q/k/v product has not been touched yet: the kernel adds the bias,
// rotates q and k by position, writes the new key and value to their cache pages and attends, so the step
// needs no kernel between the product and the attention.  The product is given as fp32 slices
// [nslices][rows][(Hq + 2 Hkv) D] (`partial`) or as bf16 rows (`dense`); `bias` and `inv_freq` may be null;
// with write_cache 0 the cache is read only (the new position must then be in it already).
TW_EXPORT int tw_attn_decode_fused(void* out, int out_stride, const float* partial, int nslices, long long slice_stride,
                                   const void* dense, int dense_stride, const float* bias, const float* inv_freq,
                                   int write_cache, const int* seq_q_start, const int* seq_q_len, const int* seq_kv_len,
                                   const int* seq_slot, const int* block_table, int table_stride, void* k_cache,
                                   void* v_cache, int n_seqs, int Hq, int Hkv, int page_size, int num_pages, int window,
                                   float scale, int nsplit, int flags, float* scratch, int* counters, int* status,
                                   const void* next_weights, long long next_bytes, cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if ((uintptr_t)next_weights & 15) return (int)cudaErrorMisalignedAddress;
    if (Hkv <= 0 || Hq % Hkv || nsplit < 1 || (nsplit > 1 && (!scratch || !counters)) || (!partial && !dense) ||
        (partial && nslices < 1))
        return (int)cudaErrorInvalidValue;
    if (int r = decode_refuses(nsplit, nullptr, 0)) return r;
    if (((uintptr_t)out & 7) || (out_stride & 3) || ((uintptr_t)scratch & 15)) return (int)cudaErrorMisalignedAddress;
    if (int e = set_attrs()) return e;
    const int G = Hq / Hkv, htiles = (G + DEC_HEADS - 1) / DEC_HEADS;
    float* partial_o = scratch;
    float* partial_ml = scratch ? scratch + (size_t)n_seqs * Hq * nsplit * D : nullptr;
    FusedQkv fq;
    fq.partial = partial; fq.nslices = nslices; fq.slice_stride = slice_stride;
    fq.dense = (const bf16*)dense; fq.dense_stride = dense_stride; fq.bias = bias; fq.inv_freq = inv_freq;
    fq.k_cache = write_cache ? (bf16*)k_cache : nullptr;
    fq.v_cache = write_cache ? (bf16*)v_cache : nullptr;
    fq.next_weights = next_weights; fq.next_bytes = next_weights ? next_bytes : 0;
    dim3 grid(nsplit * htiles, Hkv, n_seqs);
    if (nsplit > 1 && !(flags & 1) && decode_cluster_ok(nsplit))
        return tw_launch(attn_decode_kernel<true, true>, dim3(grid), dim3(DEC_WARPS * 32), DEC_SMEM, stream, nsplit,
            (bf16*)out, out_stride, (const bf16*)nullptr, 0, seq_q_start, seq_q_len, seq_kv_len, seq_slot, block_table,
            table_stride, (const bf16*)k_cache, (const bf16*)v_cache, Hq, Hkv, page_size, num_pages, window,
            scale * 1.4426950408889634f, nsplit, partial_o, partial_ml, counters, status, fq);
    tw_launch(attn_decode_kernel<false, true>, dim3(grid), dim3(DEC_WARPS * 32), DEC_SMEM, stream, 1,
        (bf16*)out, out_stride, (const bf16*)nullptr, 0, seq_q_start, seq_q_len, seq_kv_len, seq_slot, block_table,
        table_stride, (const bf16*)k_cache, (const bf16*)v_cache, Hq, Hkv, page_size, num_pages, window,
        scale * 1.4426950408889634f, nsplit, partial_o, partial_ml, counters, status, fq);
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
    if (((uintptr_t)out & 7) || (out_stride & 3)) return (int)cudaErrorMisalignedAddress;
    if (int r = decode_refuses(nsplit, q, q_stride)) {
        snprintf(g_static_error, sizeof(g_static_error),
                 "tw_attn_decode_static: at most %d slices; q must be 16-byte aligned with a row stride that is a multiple of 8",
                 DEC_MAX_SPLITS);
        return r;
    }
    const int G = Hq / Hkv, htiles = (G + DEC_HEADS - 1) / DEC_HEADS;
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
    tw_launch(attn_decode_kernel<false, false>, dim3(grid), dim3(DEC_WARPS * 32), DEC_SMEM, stream, 1, 
        (bf16*)out, out_stride, (const bf16*)q, q_stride, seq_q_start, seq_q_len, seq_kv_len, seq_slot, block_table,
        table_stride, (const bf16*)k_cache, (const bf16*)v_cache, Hq, Hkv, page_size, num_pages, window,
        scale * 1.4426950408889634f, nsplit, partial_o, partial_ml, counters, status, FusedQkv{});
    return TW_LAUNCH_CHECK();
}
