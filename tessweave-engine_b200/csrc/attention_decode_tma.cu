// Paged split-KV decode attention in bfloat16 with keys and values brought in by TMA, for head sizes
// that are multiples of 64 (compile with -DTW_HEAD_DIM=64, 128, 192 or 256).
//
// A block serves one (request, key/value head, slice of the request's keys) for requests that bring ONE
// token; the up to 8 query heads of the group are the columns of one MMA tile, so keys and values are read
// once for the whole group.  One warp is the producer: for every tile of 64 keys it issues one
// cp.async.bulk.tensor.2d per cache page and 64 columns of d (no multicast) into a ring of stages in shared
// memory, in the 128-byte swizzle, and never touches the data.  Four consumer warps each own 16 keys of a
// tile: S^T = K Q^T and O^T += V^T P^T on mma.sync with fragments read by ldmatrix (conflict-free under the
// swizzle), online softmax in fp32.  How many bytes a block keeps in flight is the depth of the ring (up to
// 200 KB per SM), not a matter of registers, and the producer starts before the kernel ahead of this one has
// finished wherever the cache it reads was written by earlier steps.  When its last copy has landed the
// producer asks for weights of a later kernel to be brought into L2 (`fq.next_weights`) and leaves; the merges
// below are the consumer warps' alone.
//
// With `fq` (a decode-only step whose q/k/v product has not been touched yet) the block adds the bias,
// rotates q and k by position, and writes the new key and value to their cache page itself; the block whose
// slice holds that newest position takes the row from its own registers (through shared memory), not from
// the copy, which may have read the page before the write.
//
// Slices of a request merge, in slice order, inside a thread-block cluster (every block sends its slice to
// the shared memory of the block that merges those values), or -- when there are more slices than a cluster
// can hold -- through scratch memory in the block that finishes last.
//
//   score = (q . k) * scale,  visible iff  position - window < p <= position
// Reference: flow_engine/model.py:193-200 and flow_engine/kernels/paged_decode.py:13-43.
//
// Every wait on an mbarrier is bounded; a wait that runs out sets TW_ERR_WAIT in the status word, every role
// stops, the producer waits (bounded) for its copies in flight, and the block writes zeros and returns.
#include "tcgen05.cuh"
#include "attention_common.cuh"
#include <cooperative_groups.h>

namespace cg = cooperative_groups;

#ifndef TW_HEAD_DIM
#define TW_HEAD_DIM 128
#endif

namespace {

typedef __nv_bfloat16 bf16;
using tc5::mbar_arrive;
using tc5::mbar_expect_tx;
using tc5::mbar_fence_init;
using tc5::mbar_init;
using tc5::mbar_wait;
using tc5::tma_load_2d;
using tw_attn::FusedQkv;
using tw_attn::ldmatrix_x4;
using tw_attn::ldmatrix_x4_trans;
using tw_attn::mma_bf16_regs;
using tw_attn::movmatrix_trans;
using tw_attn::pack_bf16;
using tw_attn::product_cols;

constexpr int D = TW_HEAD_DIM;
static_assert(D % 64 == 0 && D >= 64 && D <= 256, "the TMA decode attention takes head sizes 64, 128, 192 and 256");
constexpr int KB = D / 64;                         // 64-column blocks of a row of k or v
constexpr int TILE = 64;                           // keys per stage
constexpr int CWARPS = 4;                          // consumer warps: warp w owns keys 16 w .. 16 w + 15 of a tile
constexpr int CTHREADS = CWARPS * 32;
constexpr int THREADS = CTHREADS + 32;             // plus the producer warp
constexpr int HEADS = 8;                           // query heads per block (columns of the MMA)
constexpr int BLKB = TILE * 128;                   // bytes of a [64 keys][64 values of d] swizzled block
constexpr int STAGE_BYTES = 2 * KB * BLKB;         // K, then V
constexpr int MAX_STAGES = 8;
constexpr int STATIC_SMEM_ROOM = 9 * 1024 + HEADS * D * 4;   // barriers, block-table entries, query heads, the cluster's merge, alignment slack
constexpr int DEEPEST = (227 * 1024 - STATIC_SMEM_ROOM) / STAGE_BYTES < MAX_STAGES ? (227 * 1024 - STATIC_SMEM_ROOM) / STAGE_BYTES : MAX_STAGES;
constexpr int PAGE_CACHE = 512;                    // block-table entries kept in shared memory
constexpr int KSTEPS = D / 16;
constexpr int MT_O = D / 16;                       // m-tiles of O^T
constexpr int MAX_CLUSTER = 16;

// -DTW_TRACE: the first consumer thread and the producer of every block record the global timer (ns) at
// their phase boundaries, for a timeline of one launch (tw_attn_decode_tma_trace_ptr gives the buffer:
// [block][slot]).  Off in the product.
#ifdef TW_TRACE
constexpr int TRACE_BLOCKS = 2048, TRACE_SLOTS = 12;
__device__ long long g_trace[TRACE_BLOCKS * TRACE_SLOTS];
#define TW_TTRACE(slot)                                                                                      \
    do {                                                                                                     \
        const int b_ = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);                       \
        if ((threadIdx.x & 31) == 0 && b_ < TRACE_BLOCKS) {                                                  \
            long long t_;                                                                                    \
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));                                           \
            g_trace[b_ * TRACE_SLOTS + (slot)] = t_;                                                         \
        }                                                                                                    \
    } while (0)
#else
#define TW_TTRACE(slot) do {} while (0)
#endif
constexpr float NEG_INF = -INFINITY;
// after the last tile the ring holds the warps' partial results
constexpr int MERGE_BYTES = CWARPS * HEADS * (D + 2) * 4;
constexpr int MIN_STAGES = (MERGE_BYTES + STAGE_BYTES - 1) / STAGE_BYTES < 2 ? 2 : (MERGE_BYTES + STAGE_BYTES - 1) / STAGE_BYTES;

// byte offset of (key row, 16-byte chunk of d) inside a K or V tile of a stage
__device__ __forceinline__ int tile_offset(int row, int chunk) {
    return (chunk >> 3) * BLKB + row * 128 + (((chunk & 7) ^ (row & 7)) << 4);
}

__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(CTHREADS) : "memory"); }

template <bool CLUSTER, bool FUSED>
__global__ void __launch_bounds__(THREADS, 2)
attn_decode_tma_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                       bf16* __restrict__ out, int out_stride, const bf16* __restrict__ q, int q_stride,
                       const int* __restrict__ seq_q_start, const int* __restrict__ seq_q_len,
                       const int* __restrict__ seq_kv_len, const int* __restrict__ seq_slot,
                       const int* __restrict__ block_table, int table_stride, int Hq, int Hkv, int page_size,
                       int num_pages, int window, float scale_log2e, int nsplit, int nstages,
                       float* __restrict__ partial_o, float* __restrict__ partial_ml, int* __restrict__ counters,
                       int* status, const FusedQkv fq) {
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t full[MAX_STAGES];
    __shared__ __align__(8) uint64_t empty[MAX_STAGES];
    __shared__ int page_cache[PAGE_CACHE];
    __shared__ __align__(16) bf16 s_q[HEADS * D];                 // the block's query heads (zero beyond the group)
    __shared__ __align__(16) bf16 s_fresh[2 * D];                 // the newest position's key and value, when this block made them
    __shared__ int s_is_last, s_aborted;
    __shared__ float s_row_max[HEADS];
    __shared__ float2 s_row_ml[HEADS];                            // this block's (maximum, sum) per head, warps merged
    // what the other blocks of the cluster send this one to merge: their slices of the groups of four values it
    // owns, and their maxima and sums.  Of its own, not in the ring: a neighbour may be done before this block is.
    __shared__ __align__(16) float4 s_recv_o[HEADS * D / 4 + MAX_CLUSTER];
    __shared__ float2 s_recv_ml[MAX_CLUSTER][HEADS];

    const int s = blockIdx.z, kvh = blockIdx.y;
    const int split = blockIdx.x % nsplit, ht = blockIdx.x / nsplit;
    TW_TIMELINE_SCOPE(TW_K_ATTN_DECODE);
    // The request arrays and the block table are written before the step's first kernel starts, not by the
    // kernel before this one: they are read before the wait for that kernel.
    if (seq_q_len[s] != 1) {
        tw_grid_wait();             // a block never finishes before the kernel before this one has
        return;
    }
    const int G = Hq / Hkv, h0 = ht * HEADS;
    const int nheads = min(HEADS, G - h0);
    const int n = seq_q_start[s];
    const int pos = seq_kv_len[s] - 1;
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    // tiles start at multiples of 64 keys, so that a tile is a whole number of pages (or a part of one)
    const int base = (lo / TILE) * TILE;
    const int per = (((pos + 1 - base) + nsplit - 1) / nsplit + TILE - 1) / TILE * TILE;
    const int k_begin = base + split * per;
    const int k_end = min(pos + 1, k_begin + per);
    const int first_key = max(lo, k_begin);                          // visible keys of this block: first_key .. k_end - 1
    const int ntiles = k_begin < k_end ? (k_end - k_begin + TILE - 1) / TILE : 0;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int* table = block_table + (size_t)seq_slot[s] * table_stride;
    unsigned char* ring = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

    const int first_blk = k_begin / page_size;
    if (threadIdx.x == 0) {
        for (int i = 0; i < nstages; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], CWARPS); }
        s_aborted = 0;
        mbar_fence_init();
    }
    if (ntiles > 0) {
        const int nblk = min(PAGE_CACHE, (k_end - 1) / page_size - first_blk + 1);
        for (int i = threadIdx.x; i < nblk; i += THREADS)
            page_cache[i] = first_blk + i < table_stride ? table[first_blk + i] : -1;
    }
    __syncthreads();
    volatile int* aborted = &s_aborted;
    const bool makes_newest = FUSED && fq.k_cache && pos >= k_begin && pos < k_end;   // this block writes the new key and value

    float oacc[MT_O][4];
#pragma unroll
    for (int i = 0; i < MT_O; ++i) { oacc[i][0] = oacc[i][1] = oacc[i][2] = oacc[i][3] = 0.f; }
    float m0 = NEG_INF, m1 = NEG_INF, l0 = 0.f, l1 = 0.f;           // heads 2c and 2c + 1 of the tile
    const int g = lane >> 2, c = lane & 3;

    if (warp == CWARPS) {
        // ---- producer.  Where this kernel itself writes the step's new key and value, everything else in the
        // cache is from earlier steps and may be fetched at once; otherwise the kernel before this one (or
        // one before that) wrote the newest position, and the copies wait for it.
        if (!(FUSED && fq.k_cache)) tw_grid_wait();
        TW_TTRACE(9);
        const int box_rows = min(page_size, TILE);
        const int boxes = TILE / box_rows;
        int issued = 0;
        for (int i = 0; i < ntiles; ++i) {
            const int st = i % nstages;
            const uint32_t parity = (i / nstages) & 1;
            int row_coord = -1;
            if (lane < boxes) {
                const int key0 = k_begin + i * TILE + lane * box_rows;
                if (key0 < k_end && key0 + box_rows > first_key) {
                    const int blk = key0 / page_size;
                    const int page = blk - first_blk < PAGE_CACHE ? page_cache[blk - first_blk]
                                                                  : (blk < table_stride ? table[blk] : -1);
                    if (page < 0 || page >= num_pages) atomicOr(status, TW_ERR_PAGE);
                    else row_coord = (page * Hkv + kvh) * page_size + (key0 - blk * page_size);
                }
            }
            const uint32_t bytes = (uint32_t)__popc(__ballot_sync(0xffffffffu, row_coord >= 0)) * (2 * KB * box_rows * 128);
            int ok = 1;
            if (lane == 0) {
                ok = (!*aborted && mbar_wait(&empty[st], parity ^ 1, status)) ? 1 : 0;
                if (ok) mbar_expect_tx(&full[st], bytes); else *aborted = 1;
            }
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) break;
            if (row_coord >= 0) {
                unsigned char* dst = ring + st * STAGE_BYTES + lane * box_rows * 128;
#pragma unroll
                for (int kb = 0; kb < KB; ++kb) {
                    tma_load_2d(dst + kb * BLKB, &map_k, &full[st], kb * 64, row_coord);
                    tma_load_2d(dst + (KB + kb) * BLKB, &map_v, &full[st], kb * 64, row_coord);
                }
            }
            issued = i + 1;
        }
        TW_TTRACE(10);
        // The producer takes no part in the merges.  It arrives at the cluster's one barrier now (it has nothing to
        // publish) and leaves when its own work is done; the barrier counts the threads that have not exited.
        if (CLUSTER && nsplit > 1) cg::this_cluster().barrier_arrive();
        if (lane == 0) {
            if (*aborted) {
                // wait (bounded) for the copies already in flight, so that none lands after the block has gone
                for (int i = max(0, issued - nstages); i < issued; ++i) mbar_wait(&full[i % nstages], (i / nstages) & 1, status);
            } else if (FUSED && fq.next_weights) {
                // The last keys and values are on their way.  Once they are in, the memory system has little to do
                // while the slices merge: it may fetch weights of the kernels that follow.  Asked for from here,
                // not by a consumer: the requests take a thread one or two microseconds to issue.
                if (issued > 0) mbar_wait(&full[(issued - 1) % nstages], ((issued - 1) / nstages) & 1, status);
                tw_prefetch_l2_share(fq.next_weights, fq.next_bytes);
            }
        }
        if (FUSED && fq.k_cache) tw_grid_wait();
        return;
    } else {
        // ---- consumers
        if (warp == 0) TW_TTRACE(0);
        tw_grid_wait();
        if (warp == 0) TW_TTRACE(1);
        TW_TIMELINE_MARK();
        constexpr int half = D / 2;
        const int width = (Hq + 2 * Hkv) * D;
        if constexpr (FUSED) {
            // The block whose slice holds the newest position makes that position's key and value (bias, rotation):
            // into the cache for later steps, and into shared memory for this one.
            if (makes_newest) {
                const int blk = pos / page_size;
                const int page = blk < table_stride ? table[blk] : -1;
                const bool page_ok = page >= 0 && page < num_pages;
                if (!page_ok && threadIdx.x == 0) atomicOr(status, TW_ERR_PAGE);
                const size_t off = page_ok ? (((size_t)page * Hkv + kvh) * page_size + (pos - blk * page_size)) * D : 0;
                for (int i = threadIdx.x; i < D; i += CTHREADS) {
                    // thread i: pair i of the key if i < D / 2, and element i of the value
                    const int ik = i < half ? i : 0;
                    const int cols[3] = {(Hq + kvh) * D + ik, (Hq + kvh) * D + ik + half, (Hq + Hkv + kvh) * D + i};
                    float x[3];
                    product_cols<3>(fq, (size_t)n, width, cols, x);
                    if (i < half) {
                        float sn = 0.f, cs = 1.f;
                        if (fq.inv_freq) sincosf((float)pos * fq.inv_freq[i], &sn, &cs);
                        const bf16 k1 = __float2bfloat16_rn(x[0] * cs - x[1] * sn), k2 = __float2bfloat16_rn(x[1] * cs + x[0] * sn);
                        s_fresh[i] = k1; s_fresh[i + half] = k2;
                        if (page_ok) { fq.k_cache[off + i] = k1; fq.k_cache[off + i + half] = k2; }
                    }
                    const bf16 v = __float2bfloat16_rn(x[2]);
                    s_fresh[D + i] = v;
                    if (page_ok) fq.v_cache[off + i] = v;
                }
            }
            // this block's query heads, rotated, into shared memory.  All of a thread's columns are loaded before
            // anything is added: one round trip to L2, not one per pair.
            constexpr int PQ = (HEADS * half + CTHREADS - 1) / CTHREADS;     // pairs per thread
            int cols[2 * PQ];
            float x[2 * PQ];
#pragma unroll
            for (int j = 0; j < PQ; ++j) {
                const int p = threadIdx.x + j * CTHREADS;
                const int head = p / half, i = p - head * half;
                const bool live = p < HEADS * half && head < nheads;
                cols[2 * j] = live ? (kvh * G + h0 + head) * D + i : 0;
                cols[2 * j + 1] = cols[2 * j] + half;
            }
            product_cols<2 * PQ>(fq, (size_t)n, width, cols, x);
#pragma unroll
            for (int j = 0; j < PQ; ++j) {
                const int p = threadIdx.x + j * CTHREADS;
                if (p < HEADS * half) {
                    const int head = p / half, i = p - head * half;
                    float y1 = 0.f, y2 = 0.f;
                    if (head < nheads) {
                        float sn = 0.f, cs = 1.f;
                        if (fq.inv_freq) sincosf((float)pos * fq.inv_freq[i], &sn, &cs);
                        y1 = x[2 * j] * cs - x[2 * j + 1] * sn;
                        y2 = x[2 * j + 1] * cs + x[2 * j] * sn;
                    }
                    s_q[head * D + i] = __float2bfloat16_rn(y1);
                    s_q[head * D + i + half] = __float2bfloat16_rn(y2);
                }
            }
        } else {
            for (int idx = threadIdx.x; idx < HEADS * (D / 8); idx += CTHREADS) {
                const int head = idx / (D / 8), ch = idx - head * (D / 8);
                uint4 v = make_uint4(0u, 0u, 0u, 0u);
                if (head < nheads) v = *reinterpret_cast<const uint4*>(q + (size_t)n * q_stride + (size_t)(kvh * G + h0 + head) * D + ch * 8);
                *reinterpret_cast<uint4*>(s_q + head * D + ch * 8) = v;
            }
        }
        consumer_sync();
        if (warp == 0) TW_TTRACE(2);
        // q as the B operand: head g, values of d 16 ks + 2c, + 1 and + 8, + 9
        uint32_t qb[KSTEPS][2];
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) {
            qb[ks][0] = *reinterpret_cast<const uint32_t*>(s_q + g * D + 16 * ks + 2 * c);
            qb[ks][1] = *reinterpret_cast<const uint32_t*>(s_q + g * D + 16 * ks + 2 * c + 8);
        }
        bool ok = true;
        for (int i = 0; i < ntiles && ok; ++i) {
            const int st = i % nstages;
            ok = !*aborted && mbar_wait(&full[st], (i / nstages) & 1, status);
            if (!ok) { *aborted = 1; break; }
            if (warp == 0 && i == 0) TW_TTRACE(3);
            const int key0 = k_begin + i * TILE + warp * 16;
            if (key0 < k_end && key0 + 16 > first_key) {
                unsigned char* ks_ = ring + st * STAGE_BYTES;
                unsigned char* vs_ = ks_ + KB * BLKB;
                // Value rows of keys this block must not see -- beyond the request's last key, before the window,
                // or of a page that was never copied -- hold whatever was there: zero them (0 x NaN is NaN).
                if (key0 < first_key || key0 + 16 > k_end) {
                    for (int idx = lane; idx < 16 * (D / 8); idx += 32) {
                        const int r = idx / (D / 8), ch = idx - r * (D / 8);
                        if (key0 + r < first_key || key0 + r >= k_end)
                            *reinterpret_cast<uint4*>(vs_ + tile_offset(warp * 16 + r, ch)) = make_uint4(0u, 0u, 0u, 0u);
                    }
                    tc5::fence_proxy_async();      // these stores stay ahead of the copy that fills the stage next
                }
                if constexpr (FUSED) {
                    // the newest position's row comes from this block's own arithmetic, not from the copy
                    if (makes_newest && pos >= key0 && pos < key0 + 16) {
                        const int r = warp * 16 + (pos - key0);
                        for (int idx = lane; idx < 2 * (D / 8); idx += 32) {
                            const int which = idx / (D / 8), ch = idx - which * (D / 8);
                            *reinterpret_cast<uint4*>((which ? vs_ : ks_) + tile_offset(r, ch)) =
                                *reinterpret_cast<const uint4*>(s_fresh + which * D + ch * 8);
                        }
                        tc5::fence_proxy_async();
                    }
                }
                __syncwarp();
                // S^T = K Q^T: rows = keys g, g + 8; columns = heads 2c, 2c + 1
                float sacc[4] = {0.f, 0.f, 0.f, 0.f};
                const int krow = warp * 16 + (lane & 15);
#pragma unroll
                for (int ks = 0; ks < KSTEPS; ++ks) {
                    uint32_t a[4];
                    ldmatrix_x4(a, ks_ + tile_offset(krow, 2 * ks + (lane >> 4)));
                    mma_bf16_regs(sacc, a[0], a[1], a[2], a[3], qb[ks][0], qb[ks][1]);
                }
                const bool oka = key0 + g >= first_key && key0 + g < k_end;
                const bool okb = key0 + g + 8 >= first_key && key0 + g + 8 < k_end;
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
                // O^T += V^T P^T: V read transposed, 8 keys x 8 values of d per matrix
                const int j = lane >> 3, r = lane & 7;
                const int vrow = warp * 16 + (j >> 1) * 8 + r;
#pragma unroll
                for (int mt = 0; mt < MT_O; ++mt) {
                    uint32_t a[4];
                    ldmatrix_x4_trans(a, vs_ + tile_offset(vrow, 2 * mt + (j & 1)));
                    mma_bf16_regs(oacc[mt], a[0], a[1], a[2], a[3], pb0, pb1);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[st]);
        }
        if (warp == 0) TW_TTRACE(4);
        // sums over the keys of the other threads with the same heads
#pragma unroll
        for (int o = 4; o < 32; o <<= 1) {
            l0 += __shfl_xor_sync(0xffffffffu, l0, o);
            l1 += __shfl_xor_sync(0xffffffffu, l1, o);
        }
    }

    // ---- merge the warps (the ring is free: every copy that was issued has been waited for).  The warps exchange
    // their maxima, each scales its sums to the block's maximum in registers, and the four are added in warp order.
    // Only the consumer warps are here: the producer has left (see above), so every barrier below is theirs.
    consumer_sync();
    const bool failed = *aborted != 0;
    float* mo = reinterpret_cast<float*>(ring);                  // [warps][heads][D]
    float* wml = mo + CWARPS * HEADS * D;                        // [warps][heads][2]
    if (g == 0) {
        wml[(warp * HEADS + 2 * c) * 2] = m0; wml[(warp * HEADS + 2 * c) * 2 + 1] = l0;
        wml[(warp * HEADS + 2 * c + 1) * 2] = m1; wml[(warp * HEADS + 2 * c + 1) * 2 + 1] = l1;
    }
    consumer_sync();
    {
        float M0 = NEG_INF, M1 = NEG_INF;
#pragma unroll
        for (int w = 0; w < CWARPS; ++w) {
            M0 = fmaxf(M0, wml[(w * HEADS + 2 * c) * 2]);
            M1 = fmaxf(M1, wml[(w * HEADS + 2 * c + 1) * 2]);
        }
        if (failed) M0 = M1 = NEG_INF;
        const float f0 = (m0 == NEG_INF || M0 == NEG_INF) ? 0.f : exp2f(m0 - M0);
        const float f1 = (m1 == NEG_INF || M1 == NEG_INF) ? 0.f : exp2f(m1 - M1);
        float* p0 = mo + (warp * HEADS + 2 * c) * D;
        float* p1 = p0 + D;
#pragma unroll
        for (int mt = 0; mt < MT_O; ++mt) {
            const int d = mt * 16 + g;
            p0[d] = oacc[mt][0] * f0; p1[d] = oacc[mt][1] * f1;
            p0[d + 8] = oacc[mt][2] * f0; p1[d + 8] = oacc[mt][3] * f1;
        }
        if (warp == 0 && g == 0) {
            float L0 = 0.f, L1 = 0.f;
#pragma unroll
            for (int w = 0; w < CWARPS; ++w) {
                const float w0 = wml[(w * HEADS + 2 * c) * 2], w1 = wml[(w * HEADS + 2 * c + 1) * 2];
                L0 += wml[(w * HEADS + 2 * c) * 2 + 1] * ((w0 == NEG_INF || M0 == NEG_INF) ? 0.f : exp2f(w0 - M0));
                L1 += wml[(w * HEADS + 2 * c + 1) * 2 + 1] * ((w1 == NEG_INF || M1 == NEG_INF) ? 0.f : exp2f(w1 - M1));
            }
            s_row_ml[2 * c] = make_float2(M0, L0);
            s_row_ml[2 * c + 1] = make_float2(M1, L1);
        }
    }
    consumer_sync();
    // Four values of d at a time: the block's slice of (head, d .. d + 3).  It goes to the output (one slice), to
    // the block of the cluster that merges these four values (see below), or to scratch memory.
    constexpr int D4 = D / 4;
    const int n4 = nheads * D4;
    const int own4 = (n4 + nsplit - 1) / nsplit;                 // groups of four a block of the cluster merges
    const float4* mo4 = reinterpret_cast<const float4*>(mo);
    for (int j = threadIdx.x; j < n4; j += CTHREADS) {
        const int row = j / D4, d4 = j - row * D4;
        float4 o = mo4[j];
#pragma unroll
        for (int w = 1; w < CWARPS; ++w) {
            const float4 v = mo4[w * HEADS * D4 + j];
            o.x += v.x; o.y += v.y; o.z += v.z; o.w += v.w;
        }
        const int head = kvh * G + h0 + row;
        if (nsplit == 1) {
            const float L = s_row_ml[row].y;
            const float inv = L > 0.f ? 1.f / L : 0.f;
            uint2 packed;
            packed.x = pack_bf16(o.x * inv, o.y * inv);
            packed.y = pack_bf16(o.z * inv, o.w * inv);
            *reinterpret_cast<uint2*>(out + (size_t)n * out_stride + (size_t)head * D + 4 * d4) = packed;
        } else if (CLUSTER) {
            cg::cluster_group cluster = cg::this_cluster();
            *cluster.map_shared_rank(s_recv_o + split * own4 + j / nsplit, j % nsplit) = o;
        } else {
            const size_t at = ((size_t)s * Hq + head) * nsplit + split;
            *reinterpret_cast<float4*>(partial_o + at * D + 4 * d4) = o;
            if (d4 == 0) { partial_ml[at * 2] = s_row_ml[row].x; partial_ml[at * 2 + 1] = s_row_ml[row].y; }
        }
    }
    if (nsplit == 1) return;
    if (warp == 0) TW_TTRACE(5);

    if constexpr (CLUSTER) {
        // The slices of this (request, head tile) are the blocks of one cluster, slice i being block i.  Block r
        // merges the groups of four values j with j mod nsplit = r: every block has written its slice of them, and
        // its maxima and sums, into r's shared memory; after the cluster's barrier r reads its own memory only, so
        // nobody waits for a neighbour before it leaves.
        //   out = sum_i o_i 2^(m_i - M) / sum_i l_i 2^(m_i - M),   slices added in slice order
        cg::cluster_group cluster = cg::this_cluster();
        for (int t = threadIdx.x; t < nsplit * nheads; t += CTHREADS) {
            const int r = t / nheads, row = t - r * nheads;
            *cluster.map_shared_rank(&s_recv_ml[split][row], r) = s_row_ml[row];
        }
        cluster.barrier_arrive();
        cluster.barrier_wait();
        if (warp == 0) TW_TTRACE(6);
        for (int e = threadIdx.x; e < own4 * 4; e += CTHREADS) {
            const int jj = e >> 2, comp = e & 3;
            const int j = jj * nsplit + split;
            if (j >= n4) continue;
            const int row = j / D4, d = (j - row * D4) * 4 + comp;
            float M = NEG_INF;
            for (int i = 0; i < nsplit; ++i) M = fmaxf(M, s_recv_ml[i][row].x);
            float L = 0.f, o = 0.f;
            const float* mine = reinterpret_cast<const float*>(s_recv_o) + comp;
            for (int i = 0; i < nsplit; ++i) {
                const float2 ml = s_recv_ml[i][row];
                const float f = (ml.x == NEG_INF || M == NEG_INF) ? 0.f : exp2f(ml.x - M);
                L += ml.y * f;
                o += mine[(i * own4 + jj) * 4] * f;
            }
            out[(size_t)n * out_stride + (size_t)(kvh * G + h0 + row) * D + d] = __float2bfloat16_rn(L > 0.f ? o / L : 0.f);
        }
        if (warp == 0) TW_TTRACE(7);
        return;
    }

    // The block that finishes last among the slices of this (request, head tile) merges them, in slice order,
    // so the result does not depend on which block that is.
    __threadfence();
    consumer_sync();
    int* counter = counters + ((size_t)s * Hkv + kvh) * (gridDim.x / nsplit) + ht;
    if (threadIdx.x == 0) {
        const int done = atomicAdd(counter, 1);
        s_is_last = done == nsplit - 1;
        if (s_is_last) *counter = 0;         // ready for the next launch
    }
    consumer_sync();
    if (!s_is_last) return;
    __threadfence();
    float* fac = reinterpret_cast<float*>(ring);                  // [nheads][nsplit]
    float* lsum = fac + HEADS * nsplit;                           // [nheads][nsplit]
    const size_t group_base = ((size_t)s * Hq + kvh * G + h0) * nsplit;      // slices of head h0 start here
    for (int idx = threadIdx.x; idx < nheads * nsplit; idx += CTHREADS) {
        fac[idx] = __ldcg(partial_ml + (group_base + idx) * 2);
        lsum[idx] = __ldcg(partial_ml + (group_base + idx) * 2 + 1);
    }
    consumer_sync();
    if (threadIdx.x < nheads) {
        float M = NEG_INF;
        for (int i = 0; i < nsplit; ++i) M = fmaxf(M, fac[threadIdx.x * nsplit + i]);
        s_row_max[threadIdx.x] = M;
    }
    consumer_sync();
    for (int idx = threadIdx.x; idx < nheads * nsplit; idx += CTHREADS) {
        const float M = s_row_max[idx / nsplit];
        const float mi = fac[idx];
        const float f = (mi == NEG_INF || M == NEG_INF) ? 0.f : exp2f(mi - M);
        fac[idx] = f;
        lsum[idx] *= f;
    }
    consumer_sync();
    for (int idx = threadIdx.x; idx < nheads * D4; idx += CTHREADS) {
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

constexpr int DEC_MAX_SPLITS = 128;
static_assert(2 * HEADS * DEC_MAX_SPLITS * 4 <= MIN_STAGES * STAGE_BYTES, "the merge factors of the most slices must fit the ring");

size_t smem_bytes(int nstages);

template <bool CLUSTER, bool FUSED>
int prepare() {
    static bool done = false;
    if (done) return 0;
    cudaError_t e = cudaFuncSetAttribute(attn_decode_tma_kernel<CLUSTER, FUSED>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem_bytes(DEEPEST));
    if (e != cudaSuccess) return (int)e;
    if (CLUSTER) {
        e = cudaFuncSetAttribute(attn_decode_tma_kernel<CLUSTER, FUSED>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
        if (e != cudaSuccess) return (int)e;
    }
    done = true;
    return 0;
}

int g_cluster_ok[MAX_CLUSTER + 1][MAX_STAGES + 1] = {};      // 0 unknown, 1 fits, -1 does not

bool cluster_fits(int size, int nstages) {
    if (size < 2 || size > MAX_CLUSTER) return false;
    int& known = g_cluster_ok[size][nstages];
    if (known == 0) {
        if (prepare<true, false>() != 0) return false;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(size);
        cfg.blockDim = dim3(THREADS);
        cfg.dynamicSmemBytes = smem_bytes(nstages);
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = size;
        attr.val.clusterDim.y = 1;
        attr.val.clusterDim.z = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        int clusters = 0;
        const cudaError_t e = cudaOccupancyMaxActiveClusters(&clusters, attn_decode_tma_kernel<true, false>, &cfg);
        if (e != cudaSuccess) (void)cudaGetLastError();
        known = (e == cudaSuccess && clusters >= 1) ? 1 : -1;
    }
    return known > 0;
}

size_t smem_bytes(int nstages) { return (size_t)nstages * STAGE_BYTES + 1024; }

int g_sm_count = 0;

}  // namespace

#ifdef TW_TRACE
TW_EXPORT int tw_attn_decode_tma_trace_ptr(void** ptr, int* blocks, int* slots) {
    *blocks = TRACE_BLOCKS; *slots = TRACE_SLOTS;
    return (int)cudaGetSymbolAddress(ptr, g_trace);
}
#endif

TW_EXPORT int tw_attn_decode_tma_head_dim() { return D; }
TW_EXPORT int tw_attn_decode_tma_max_splits() { return DEC_MAX_SPLITS; }
TW_EXPORT int tw_attn_decode_tma_max_stages() { return DEEPEST; }
// Pages must be a whole fraction of a tile of 64 keys (at least 4 keys, so that a box is 512 bytes or more) or a
// whole number of tiles.
TW_EXPORT int tw_attn_decode_tma_supported(int page_size) {
    if (page_size < 4) return 0;
    return (TILE % page_size == 0 || page_size % TILE == 0) ? 1 : 0;
}

// Split-KV decode attention for the requests of the batch that bring one token.  Either `q` (bf16 rows
// [tokens, Hq * D], 16-byte aligned) is given, or the step's untouched q/k/v product (`partial`: fp32 slices
// [nslices][rows][(Hq + 2 Hkv) D], or `dense`: bf16 rows) with `bias`, `inv_freq` and, with write_cache, the
// duty to store the new key and value.  `nstages` is the depth of the ring (0: as deep as one block per SM
// allows while the launch has no more blocks than SMs, else half of that so that two blocks share an SM).
// `scratch` and `counters` as for tw_attn_decode; they are used when the slices do not fit a cluster.
TW_EXPORT int tw_attn_decode_tma(void* out, int out_stride, const void* q, int q_stride, const float* partial, int nslices,
                                 long long slice_stride, const void* dense, int dense_stride, const float* bias,
                                 const float* inv_freq, int write_cache, const int* seq_q_start, const int* seq_q_len,
                                 const int* seq_kv_len, const int* seq_slot, const int* block_table, int table_stride,
                                 void* k_cache, void* v_cache, int n_seqs, int Hq, int Hkv, int page_size, int num_pages,
                                 int window, float scale, int nsplit, int nstages, int flags, float* scratch, int* counters,
                                 int* status, const void* next_weights, long long next_bytes, cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    const bool fused = partial || dense;
    if (Hkv <= 0 || Hq % Hkv || nsplit < 1 || nsplit > DEC_MAX_SPLITS || !tw_attn_decode_tma_supported(page_size) ||
        (!fused && !q) || (partial && nslices < 1) || (nsplit > 1 && (!scratch || !counters)))
        return (int)cudaErrorInvalidValue;
    if (((uintptr_t)out & 7) || (out_stride & 3) || ((uintptr_t)scratch & 15) || ((uintptr_t)k_cache & 15) ||
        ((uintptr_t)v_cache & 15) || ((uintptr_t)next_weights & 15) || (!fused && (((uintptr_t)q & 15) || (q_stride & 7))))
        return (int)cudaErrorMisalignedAddress;
    if (!g_sm_count) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
            g_sm_count = 148;
    }
    const int G = Hq / Hkv, htiles = (G + HEADS - 1) / HEADS;
    const long long blocks = (long long)nsplit * htiles * Hkv * n_seqs;
    const int deepest = tw_attn_decode_tma_max_stages();
    if (nstages <= 0) nstages = blocks <= g_sm_count ? deepest : (113 * 1024 - STATIC_SMEM_ROOM) / STAGE_BYTES;
    if (nstages > deepest) nstages = deepest;
    if (nstages < MIN_STAGES) nstages = MIN_STAGES;
    const long long rows = (long long)num_pages * Hkv * page_size;
    if (rows >= (1ll << 31)) return (int)cudaErrorInvalidValue;
    const int box_rows = page_size < TILE ? page_size : TILE;
    CUtensorMap mk, mv;
    if (int e = tc5::get_map(k_cache, rows, D, box_rows, &mk)) return e;
    if (int e = tc5::get_map(v_cache, rows, D, box_rows, &mv)) return e;
    float* partial_o = scratch;
    float* partial_ml = scratch ? scratch + (size_t)n_seqs * Hq * nsplit * D : nullptr;
    FusedQkv fq = {};
    if (fused) {
        fq.partial = partial; fq.nslices = nslices; fq.slice_stride = slice_stride;
        fq.dense = (const bf16*)dense; fq.dense_stride = dense_stride; fq.bias = bias; fq.inv_freq = inv_freq;
        fq.k_cache = write_cache ? (bf16*)k_cache : nullptr;
        fq.v_cache = write_cache ? (bf16*)v_cache : nullptr;
        fq.next_weights = next_weights; fq.next_bytes = next_weights ? next_bytes : 0;
    }
    const dim3 grid(nsplit * htiles, Hkv, n_seqs);
    const size_t smem = smem_bytes(nstages);
    const float scale_log2e = scale * 1.4426950408889634f;
    const bool cluster = nsplit > 1 && !(flags & 1) && cluster_fits(nsplit, nstages);
#define TW_DECODE_TMA_LAUNCH(CL, FU)                                                                                   \
    do {                                                                                                               \
        if (int e = prepare<CL, FU>()) return e;                                                                       \
        return tw_launch(attn_decode_tma_kernel<CL, FU>, grid, dim3(THREADS), smem, stream, CL ? nsplit : 1, mk, mv,    \
                         (bf16*)out, out_stride, (const bf16*)q, q_stride, seq_q_start, seq_q_len, seq_kv_len, seq_slot, \
                         block_table, table_stride, Hq, Hkv, page_size, num_pages, window, scale_log2e, nsplit, nstages, \
                         partial_o, partial_ml, counters, status, fq);                                                 \
    } while (0)
    if (cluster && fused) TW_DECODE_TMA_LAUNCH(true, true);
    if (cluster) TW_DECODE_TMA_LAUNCH(true, false);
    if (fused) TW_DECODE_TMA_LAUNCH(false, true);
    TW_DECODE_TMA_LAUNCH(false, false);
#undef TW_DECODE_TMA_LAUNCH
}
