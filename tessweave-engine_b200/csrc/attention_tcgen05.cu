// Paged causal attention for prompt portions on the 5th-generation tensor cores, for one head
// size (compile with -DTW_HEAD_DIM=64 or 128).
//
// A block serves up to 256 rows of one (request, key/value head), a row being a (token, query
// head of the group) pair, as two tiles of 128 rows, and walks the request's keys in tiles of
// 128.  Per key tile and row tile:
//     S = Q K^T        tcgen05.mma, both operands K-major in shared memory, S (fp32) in tensor memory
//     P = 2^(S c - m)  four warps, one row (one TMEM lane) per thread: tcgen05.ld, fp32 maximum
//                      and sum, P rounded to bf16 and stored over S in tensor memory (tcgen05.st)
//     O += P V         tcgen05.mma with P as the operand in tensor memory and V read "MN-major"
//                      straight from the page layout [key][d]; O (fp32) stays in tensor memory
//                      for the whole walk
// The two row tiles alternate, so the tensor cores work on one while the softmax warps work on
// the other.  Keys and values travel by TMA (cp.async.bulk.tensor.2d, no multicast), one box
// per page and 64 columns of d, into the swizzled layout the MMAs read; a warp of its own
// issues them.  Another warp issues every MMA.
//
// O is only rescaled when a row's maximum grows by more than 2^8 (the sums carry the same
// stale maximum, so the quotient is exact); rows of values beyond the request's last key are
// zeroed in shared memory, so stale page contents cannot reach a product.
//
//   score = (q . k) * scale,  visible iff  position - window < p <= position
// Reference: flow_engine/model.py:193-200 (the reference calls a library's attention here).
//
// Every wait on an mbarrier is bounded; a wait that runs out sets TW_ERR_WAIT in the status
// word, every role stops, the block waits (bounded) for its copies in flight, frees its tensor
// memory and returns.
#include "tcgen05.cuh"

#ifndef TW_HEAD_DIM
#define TW_HEAD_DIM 128
#endif

namespace {

using namespace tc5;

constexpr int D = TW_HEAD_DIM;
static_assert(D == 64 || D == 128, "the tcgen05 attention is built for head sizes 64 and 128");

constexpr int BM = 128;                       // rows of a query tile = TMEM lanes
constexpr int NQ = 2;                         // query tiles per block
constexpr int BN = 128;                       // keys per tile
constexpr int KB = D / 64;                    // 64-column blocks of a row of q, k or v
constexpr int BLK = 128 * 128;                // bytes of a [128 rows][64 columns] swizzled block
constexpr int KV_STAGES = D == 128 ? 2 : 4;   // K and V have rings of their own
constexpr int Q_BYTES = NQ * KB * BLK;
constexpr int KV_STAGE_BYTES = KB * BLK;
constexpr int SMEM_TILES = Q_BYTES + 2 * KV_STAGES * KV_STAGE_BYTES;
constexpr int SMEM = SMEM_TILES + 1024 /* alignment slack */ + 256 /* barriers */;
constexpr int THREADS = 320;                  // warp 0: TMA, warp 1: MMA, warps 2-5 / 6-9: softmax of tile 0 / 1
constexpr int TMEM_COLS = 512;                // S of both tiles (2 x 128 columns; P over its first 64), O of both tiles (2 x D)
constexpr int O_COL = 256;
constexpr float RESCALE_THRESHOLD = 8.f;      // log2 units
#define NEG_INF (-INFINITY)

// -DTW_TRACE: block (0, 0, 0) records clock64() at the hand-over points of its roles, for a
// timeline of one block (tw_attn_tc5_trace_ptr gives the buffer).  Off in the product.
#ifdef TW_TRACE
constexpr int TRACE_SLOTS = 12, TRACE_TILES = 80, TRACE_ROLES = 10;     // a role = a warp
__device__ long long g_trace[TRACE_ROLES * TRACE_TILES * TRACE_SLOTS];
#define TW_TRACE_AT(role, tile, slot)                                                              \
    do {                                                                                           \
        if (blockIdx.x == 0 && blockIdx.y == 0 && (tile) < TRACE_TILES)         \
            g_trace[((role) * TRACE_TILES + (tile)) * TRACE_SLOTS + (slot)] = clock64();           \
    } while (0)
#else
#define TW_TRACE_AT(role, tile, slot) do {} while (0)
#endif

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
// (a0, a1) * b + c and (a0, a1) + (b0, b1) as one packed instruction each
__device__ __forceinline__ float2 fma2(float a0, float a1, float b, float c) {
    float2 d;
    asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\t"
        "mov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %4};\n\tmov.b64 rc, {%5, %5};\n\t"
        "fma.rn.f32x2 rd, ra, rb, rc;\n\t"
        "mov.b64 {%0, %1}, rd;\n\t}"
        : "=f"(d.x), "=f"(d.y) : "f"(a0), "f"(a1), "f"(b), "f"(c));
    return d;
}
__device__ __forceinline__ float2 add2(float2 a, float2 b) {
    float2 d;
    asm("{\n\t.reg .b64 ra, rb, rd;\n\t"
        "mov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
        "add.rn.f32x2 rd, ra, rb;\n\t"
        "mov.b64 {%0, %1}, rd;\n\t}"
        : "=f"(d.x), "=f"(d.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
    return d;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

__global__ void __launch_bounds__(THREADS, 1)
attn_prefill_tc5_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                        bf16* __restrict__ out, int out_stride, const bf16* __restrict__ q, int q_stride,
                        const int* __restrict__ seq_q_start, const int* __restrict__ seq_q_len,
                        const int* __restrict__ seq_kv_len, const int* __restrict__ seq_slot,
                        const int* __restrict__ block_table, int table_stride, int Hq, int Hkv, int page_size,
                        int num_pages, int window, float scale_log2e, int skip_single, int* status) {
    extern __shared__ unsigned char smem_raw[];
    TW_TIMELINE_SCOPE(TW_K_ATTN_PREFILL);
    if (threadIdx.x == 0) TW_TRACE_AT(0, 0, 5);
    tw_grid_wait();
    TW_TIMELINE_MARK();
    // Blocks start in the order of blockIdx.x, and a block's work grows with the position of its rows: x counts
    // (row tile, key/value head) with the head fastest and the last row tile first, so that the longest blocks of
    // all heads start first and the short ones fill the gaps (with the head as blockIdx.y, the long blocks of
    // the last heads started late: 78 us against 58 us for 2,048 tokens).
    const int s = blockIdx.y, kvh = (int)blockIdx.x % Hkv, xt = (int)blockIdx.x / Hkv;
    const int q_len = seq_q_len[s];
    if (q_len <= 0 || (skip_single && q_len == 1)) return;
    const int G = Hq / Hkv;
    const int rows_total = q_len * G;
    const int mtiles = (rows_total + NQ * BM - 1) / (NQ * BM);
    if (xt >= mtiles) return;
    const int row0 = (mtiles - 1 - xt) * (NQ * BM);                  // the rows with the most keys first
    const int kv_len = seq_kv_len[s];
    const int pos0 = kv_len - q_len;                                 // position of the first token of this portion
    const int n0 = seq_q_start[s];
    const int* table = block_table + (size_t)seq_slot[s] * table_stride;
    const int row_end = min(rows_total, row0 + NQ * BM);
    const int nq = row_end - row0 > BM ? 2 : 1;
    const int pos_first = pos0 + row0 / G, pos_last = pos0 + (row_end - 1) / G;
    const int j_begin = (window > 0 && pos_first - window + 1 > 0) ? (pos_first - window + 1) / BN : 0;
    const int ntiles = pos_last / BN + 1 - j_begin;
    const int tail_rows = max(0, (j_begin + ntiles) * BN - kv_len);  // rows of the last tile that hold no key

    unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* q_s = tiles;                                      // [NQ][KB][128 rows][128 B]
    unsigned char* k_s = q_s + Q_BYTES;                              // [KV_STAGES][KB][128 keys][128 B]
    unsigned char* v_s = k_s + KV_STAGES * KV_STAGE_BYTES;           // [KV_STAGES][KB][128 keys][128 B]
    uint64_t* k_full = reinterpret_cast<uint64_t*>(tiles + SMEM_TILES);
    uint64_t* k_empty = k_full + KV_STAGES;
    uint64_t* v_full = k_empty + KV_STAGES;
    uint64_t* v_empty = v_full + KV_STAGES;
    uint64_t* s_full = v_empty + KV_STAGES;                          // S of tile X is complete
    uint64_t* p_full = s_full + NQ;                                  // P of tile X is written, S read, O rescaled
    uint64_t* o_done = p_full + NQ;                                  // the P V products of tile X so far have retired
    uint64_t* v_fixed = o_done + NQ;                                 // value rows past the last key are zeroed
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(v_fixed + 1);
    volatile int* aborted = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int i = 0; i < KV_STAGES; ++i) {
            mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1);
            mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1);
        }
        for (int x = 0; x < NQ; ++x) { mbar_init(&s_full[x], 1); mbar_init(&p_full[x], BM / 32); mbar_init(&o_done[x], 1); }
        mbar_init(v_fixed, 1);
        *aborted = 0;
        mbar_fence_init();
    }
    // The producer's work for key tile i: one TMA box per page (and 64 columns of d) for the keys, then for the
    // values; lane b owns box b of a tile.  False if a wait ran out.
    const int box_rows = min(page_size, BN);
    const int boxes = BN / box_rows;
    auto issue_tile = [&](int i) -> bool {
        const int st = i % KV_STAGES;
        const uint32_t parity = (i / KV_STAGES) & 1;
        int row_coord = -1;
        if (lane < boxes) {
            const int key0 = (j_begin + i) * BN + lane * box_rows;
            if (key0 < kv_len) {
                const int blk = key0 / page_size;
                const int page = blk < table_stride ? table[blk] : -1;
                if (page < 0 || page >= num_pages) atomicOr(status, TW_ERR_PAGE);
                else row_coord = (page * Hkv + kvh) * page_size + (key0 - blk * page_size);
            }
        }
        const uint32_t bytes = (uint32_t)__popc(__ballot_sync(0xffffffffu, row_coord >= 0)) * KB * box_rows * 128;
        int ok = 1;
        if (lane == 0) {
            ok = (!*aborted && mbar_wait(&k_empty[st], parity ^ 1, status)) ? 1 : 0;
            if (ok) mbar_expect_tx(&k_full[st], bytes); else *aborted = 1;
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) return false;
        if (lane == 0) TW_TRACE_AT(0, i, 0);
        if (row_coord >= 0) {
#pragma unroll
            for (int kb = 0; kb < KB; ++kb)
                tma_load_2d(k_s + st * KV_STAGE_BYTES + kb * BLK + lane * box_rows * 128, &map_k, &k_full[st], kb * 64, row_coord);
        }
        if (lane == 0) {
            ok = (!*aborted && mbar_wait(&v_empty[st], parity ^ 1, status)) ? 1 : 0;
            if (ok) mbar_expect_tx(&v_full[st], bytes); else *aborted = 1;
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) {                                   // K of this tile is in flight: let it land
            if (lane == 0) mbar_wait(&k_full[st], parity, status);
            return false;
        }
        if (lane == 0) TW_TRACE_AT(1, i, 2);
        if (row_coord >= 0) {
#pragma unroll
            for (int kb = 0; kb < KB; ++kb)
                tma_load_2d(v_s + st * KV_STAGE_BYTES + kb * BLK + lane * box_rows * 128, &map_v, &v_full[st], kb * 64, row_coord);
        }
        return true;
    };
    if (warp == 1) tmem_alloc(tmem_slot, TMEM_COLS);
    // The first key and value tiles need nothing of what follows: the producer warp (whose first thread has just
    // set up the barriers) asks for them now, and the other warps bring the query rows in meanwhile.
    int issued = 0;
    if (warp == 0) {
        __syncwarp();
        while (issued < ntiles && issued < KV_STAGES && issue_tile(issued)) ++issued;
    }

    // the block's query rows into shared memory, in the swizzled K-major layout (rows beyond the portion are zero).
    // All of a thread's loads are issued before the first store: one round trip to L2, not thirteen in a row
    // (which was 9 of the 13 us a block spent outside its key tiles).
    {
        constexpr int Q_ITEMS = NQ * BM * (D / 8);
        constexpr int Q_THREADS = THREADS - 32;                          // every warp but the producer
        constexpr int Q_PER_THREAD = (Q_ITEMS + Q_THREADS - 1) / Q_THREADS;
        uint4 vals[Q_PER_THREAD];
#pragma unroll
        for (int j = 0; j < Q_PER_THREAD; ++j) {
            const int i = (int)threadIdx.x - 32 + j * Q_THREADS;
            const int rr = i / (D / 8), c = i - rr * (D / 8);
            const int r = row0 + rr;
            vals[j] = make_uint4(0u, 0u, 0u, 0u);
            if (warp != 0 && i < Q_ITEMS && r < rows_total) {
                const int t = r / G;
                vals[j] = *reinterpret_cast<const uint4*>(q + (size_t)(n0 + t) * q_stride + (size_t)(kvh * G + (r - t * G)) * D + c * 8);
            }
        }
#pragma unroll
        for (int j = 0; j < Q_PER_THREAD; ++j) {
            const int i = (int)threadIdx.x - 32 + j * Q_THREADS;
            if (warp != 0 && i < Q_ITEMS) {
                const int rr = i / (D / 8), c = i - rr * (D / 8);
                const int x = rr / BM, rt = rr - x * BM;
                *reinterpret_cast<uint4*>(q_s + (x * KB + (c >> 3)) * BLK + rt * 128 + (((c & 7) ^ (rt & 7)) << 4)) = vals[j];
            }
        }
    }
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    if (threadIdx.x == 0) TW_TRACE_AT(0, 0, 6);

    if (warp == 0) {
        // ---- producer: the remaining tiles, each as soon as its stage is free
        while (issued < ntiles && !*aborted && issue_tile(issued)) ++issued;
        if (tail_rows && issued == ntiles) {
            // The last tile reaches past the request's last key.  What its value rows hold there (the rest
            // of a page, or whatever the stage held before) must not reach a product, since 0 x NaN is NaN:
            // zero them once the copies have landed, then tell the MMA thread.
            const int last = ntiles - 1;
            if (mbar_wait(&v_full[last % KV_STAGES], (last / KV_STAGES) & 1, status)) {
                unsigned char* vt = v_s + (last % KV_STAGES) * KV_STAGE_BYTES;
                for (int idx = lane; idx < tail_rows * KB * 8; idx += 32) {
                    const int r = BN - tail_rows + idx / (KB * 8), rest = idx % (KB * 8);
                    *reinterpret_cast<uint4*>(vt + (rest >> 3) * BLK + r * 128 + ((rest & 7) << 4)) = make_uint4(0u, 0u, 0u, 0u);
                }
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) mbar_arrive(v_fixed);
            } else {
                *aborted = 1;
            }
        }
        if (*aborted && lane == 0) {
            // wait (bounded) for the copies already in flight, so that none lands after the block has gone
            for (int i = max(0, issued - KV_STAGES); i < issued; ++i) {
                mbar_wait(&k_full[i % KV_STAGES], (i / KV_STAGES) & 1, status);
                mbar_wait(&v_full[i % KV_STAGES], (i / KV_STAGES) & 1, status);
            }
        }
    } else if (warp == 1) {
        // ---- tensor cores: lane 0 issues every MMA of the block.  The tensor pipe runs dry as soon as
        // this thread does anything else, so whatever a group of MMAs needs beside P (V of the tile, K of
        // the next one) is waited for before P, and the groups follow one another without a break.
        if (lane == 0 && ntiles > 0) {
            const uint32_t idesc_s = instr_desc(BN), idesc_o = instr_desc(D, true);
            // Descriptors are built once; per MMA only a constant is added to the address field (a thread
            // that computes a descriptor from scratch before each MMA issues them slower than they execute).
            const uint64_t q_desc = smem_desc(q_s, 0), k_desc = smem_desc(k_s, 0), v_desc = smem_desc_mn_major(v_s, BLK);
            auto issue_s = [&](int x, int i) {
                const uint64_t kd = k_desc + (uint64_t)((i % KV_STAGES) * (KV_STAGE_BYTES >> 4));
                const uint64_t qd = q_desc + (uint64_t)(x * KB * (BLK >> 4));
#pragma unroll
                for (int kb = 0; kb < KB; ++kb)
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        umma_bf16(tmem_base + x * BN, qd + (uint64_t)(kb * (BLK >> 4) + k * 2), kd + (uint64_t)(kb * (BLK >> 4) + k * 2),
                                  idesc_s, (kb > 0 || k > 0) ? 1u : 0u);
                umma_commit(&s_full[x]);
            };
            auto issue_o = [&](int x, int i) {
                const uint64_t vd = v_desc + (uint64_t)((i % KV_STAGES) * (KV_STAGE_BYTES >> 4));
#pragma unroll
                for (int k = 0; k < BN / 16; ++k)
                    umma_bf16_ts(tmem_base + O_COL + x * D, tmem_base + x * BN + k * 8, vd + (uint64_t)(k * (2048 >> 4)),
                                 idesc_o, (i > 0 || k > 0) ? 1u : 0u);
                umma_commit(&o_done[x]);
            };
            bool ok = mbar_wait(&k_full[0], 0, status);
            if (ok) {
                tc_fence_after();
                for (int x = 0; x < nq; ++x) issue_s(x, 0);
                umma_commit(&k_empty[0]);
            }
            for (int i = 0; ok && i < ntiles; ++i) {
                const int st = i % KV_STAGES;
                TW_TRACE_AT(1, i, 10);
                ok = mbar_wait(&v_full[st], (i / KV_STAGES) & 1, status);
                TW_TRACE_AT(1, i, 2);
                if (ok && i == ntiles - 1 && tail_rows) ok = mbar_wait(v_fixed, 0, status);
                if (ok && i + 1 < ntiles) ok = mbar_wait(&k_full[(i + 1) % KV_STAGES], ((i + 1) / KV_STAGES) & 1, status);
                TW_TRACE_AT(1, i, 4);
                for (int x = 0; ok && x < nq; ++x) {
                    TW_TRACE_AT(1, i, x * 6 + 0);
                    ok = mbar_wait(&p_full[x], i & 1, status);
                    if (!ok) break;
                    TW_TRACE_AT(1, i, x * 6 + 1);
                    tc_fence_after();
                    issue_o(x, i);
                    TW_TRACE_AT(1, i, x * 6 + 3);
                    if (i + 1 < ntiles) issue_s(x, i + 1);
                    TW_TRACE_AT(1, i, x * 6 + 5);
                }
                if (ok) {
                    umma_commit(&v_empty[st]);
                    if (i + 1 < ntiles) umma_commit(&k_empty[(i + 1) % KV_STAGES]);
                }
                TW_TRACE_AT(1, i, 8);
            }
            if (!ok) *aborted = 1;
        }
        __syncwarp();
    } else if ((warp - 2) / 4 < nq) {
        // ---- softmax: thread = row rt of tile x = TMEM lane rt
        const int x = (warp - 2) / 4;
        const int quarter = warp & 3;                        // the TMEM lanes this warp may touch
        const int rt = quarter * 32 + lane;
        const int r = row0 + x * BM + rt;
        const bool valid = r < rows_total;
        const int t = valid ? r / G : (rows_total - 1) / G;
        const int pos = pos0 + t;
        const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
        const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
        const uint32_t s_addr = lane_addr + x * BN, o_addr = lane_addr + O_COL + x * D;
        float m_used = NEG_INF, l = 0.f;
        bool ok = true;
        for (int i = 0; i < ntiles; ++i) {
            const int kbase = (j_begin + i) * BN;
            if (lane == 0) TW_TRACE_AT(warp, i, 0);
            ok = !*aborted && mbar_wait(&s_full[x], i & 1, status);
            if (!ok) break;
            if (lane == 0) TW_TRACE_AT(warp, i, 1);
            tc_fence_after();
            uint32_t v[BN];
#pragma unroll
            for (int c = 0; c < BN; c += 32) tmem_ld32_nowait(s_addr + c, v + c);
            tmem_wait_ld();
            if (lane == 0) TW_TRACE_AT(warp, i, 2);
            const bool all_visible = kbase + BN - 1 <= pos && kbase >= lo;
            if (!__all_sync(0xffffffffu, all_visible)) {
#pragma unroll
                for (int c = 0; c < BN; ++c) {
                    const int key = kbase + c;
                    if (key > pos || key < lo) v[c] = __float_as_uint(NEG_INF);
                }
            }
            // four independent chains of three-input maxima
            float mx[4] = {NEG_INF, NEG_INF, NEG_INF, NEG_INF};
#pragma unroll
            for (int c = 0; c < BN; c += 8) {
#pragma unroll
                for (int k = 0; k < 4; ++k) mx[k] = max3(mx[k], __uint_as_float(v[c + 2 * k]), __uint_as_float(v[c + 2 * k + 1]));
            }
            const float mt = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * scale_log2e;   // scale > 0: the maximum commutes with it
            const bool rescale = mt > m_used + RESCALE_THRESHOLD;     // also the first finite maximum (m_used = -inf)
            float factor = 1.f;
            if (rescale) {
                factor = m_used == NEG_INF ? 0.f : ex2(m_used - mt);
                m_used = mt;
            }
            const float neg_mu = m_used == NEG_INF ? 0.f : -m_used;
            // p = 2^(s c - m) two at a time (packed fp32 multiply-add and add), four independent sums of pairs
            float2 acc[4] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll
            for (int c = 0; c < BN; c += 8) {
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    float2 e = fma2(__uint_as_float(v[c + 2 * k]), __uint_as_float(v[c + 2 * k + 1]), scale_log2e, neg_mu);
                    e.x = ex2(e.x);
                    e.y = ex2(e.y);
                    acc[k] = add2(acc[k], e);
                    v[(c >> 1) + k] = pack_bf16(e.x, e.y);
                }
            }
            const float sum = ((acc[0].x + acc[0].y) + (acc[1].x + acc[1].y)) + ((acc[2].x + acc[2].y) + (acc[3].x + acc[3].y));
            l = l * factor + sum;
            if (i > 0 && __any_sync(0xffffffffu, rescale)) {
                // P V of the tile before has retired (it was issued before the S just read): O is complete up to it
                ok = mbar_wait(&o_done[x], (i - 1) & 1, status);
                if (!ok) break;
                tc_fence_after();
                {
#pragma unroll
                    for (int c = 0; c < D; c += 32) {
                        uint32_t o[32];
                        tmem_ld32_nowait(o_addr + c, o);
                        tmem_wait_ld();
#pragma unroll
                        for (int k = 0; k < 32; ++k) o[k] = __float_as_uint(__uint_as_float(o[k]) * factor);
                        tmem_st32_nowait(o_addr + c, o);
                    }
                    tmem_wait_st();
                }
            }
            if (lane == 0) TW_TRACE_AT(warp, i, 3);
            // P over the first 64 columns of S: the whole row of S is in registers by now
            tmem_st32_nowait(s_addr, v);
            tmem_st32_nowait(s_addr + 32, v + 32);
            tmem_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_full[x]);      // one arrival per warp: 128 arrivals on one barrier take 450 cycles
            if (lane == 0) TW_TRACE_AT(warp, i, 4);
        }
        if (ok && ntiles > 0) ok = mbar_wait(&o_done[x], (ntiles - 1) & 1, status);
        if (lane == 0) TW_TRACE_AT(warp, TRACE_TILES - 1, 0);
        if (!ok) {
            *aborted = 1;
        } else if (ntiles > 0) {
            tc_fence_after();
            const float inv = l > 0.f ? 1.f / l : 0.f;
            bf16* orow = out + (size_t)(n0 + t) * out_stride + (size_t)(kvh * G + (r - t * G)) * D;
#pragma unroll
            for (int c = 0; c < D; c += 32) {
                uint32_t o[32];
                tmem_ld32_nowait(o_addr + c, o);
                tmem_wait_ld();
                if (valid) {
#pragma unroll
                    for (int k = 0; k < 32; k += 8) {
                        uint4 w;
                        w.x = pack_bf16(__uint_as_float(o[k]) * inv, __uint_as_float(o[k + 1]) * inv);
                        w.y = pack_bf16(__uint_as_float(o[k + 2]) * inv, __uint_as_float(o[k + 3]) * inv);
                        w.z = pack_bf16(__uint_as_float(o[k + 4]) * inv, __uint_as_float(o[k + 5]) * inv);
                        w.w = pack_bf16(__uint_as_float(o[k + 6]) * inv, __uint_as_float(o[k + 7]) * inv);
                        *reinterpret_cast<uint4*>(orow + c + k) = w;
                    }
                }
            }
        }
    }
    if (lane == 0) TW_TRACE_AT(warp, TRACE_TILES - 1, 1);
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
    if (threadIdx.x == 32) TW_TRACE_AT(0, 0, 7);
}

}  // namespace

TW_EXPORT int tw_attn_tc5_head_dim() { return D; }

#ifdef TW_TRACE
TW_EXPORT int tw_attn_tc5_trace_ptr(long long** ptr, int* roles, int* tiles, int* slots) {
    *roles = TRACE_ROLES; *tiles = TRACE_TILES; *slots = TRACE_SLOTS;
    return (int)cudaGetSymbolAddress((void**)ptr, g_trace);
}
#endif

// Whether the kernel takes this page size: a key tile is a whole number of pages, or a page a
// whole number of key tiles, and a tile has at most 32 boxes.
TW_EXPORT int tw_attn_prefill_tc5_supported(int page_size) {
    if (page_size < 4) return 0;
    return (BN % page_size == 0 || page_size % BN == 0) ? 1 : 0;
}

// Attention for the requests of the batch that bring several tokens (with skip_single, requests
// with one token are left to the decode kernel).  q [tokens, Hq * D] and out [tokens, Hq * D] are
// bf16 with 16-byte aligned rows; the cache is [pages, Hkv, page_size, D] bf16.
TW_EXPORT int tw_attn_prefill_tc5(void* out, int out_stride, const void* q, int q_stride, const int* seq_q_start,
                                  const int* seq_q_len, const int* seq_kv_len, const int* seq_slot,
                                  const int* block_table, int table_stride, const void* k_cache, const void* v_cache,
                                  int n_seqs, int max_q_len, int Hq, int Hkv, int page_size, int num_pages, int window,
                                  float scale, int skip_single, int* status, cudaStream_t stream) {
    if (n_seqs <= 0 || max_q_len <= 0) return 0;
    if (Hkv <= 0 || Hq % Hkv || !tw_attn_prefill_tc5_supported(page_size) || scale <= 0.f) return (int)cudaErrorInvalidValue;
    if ((reinterpret_cast<uintptr_t>(out) & 15) || (reinterpret_cast<uintptr_t>(q) & 15) || (out_stride & 7) || (q_stride & 7) ||
        (reinterpret_cast<uintptr_t>(k_cache) & 15) || (reinterpret_cast<uintptr_t>(v_cache) & 15))
        return (int)cudaErrorMisalignedAddress;
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc5_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e != cudaSuccess) return (int)e;
        attr_set = true;
    }
    const int box_rows = page_size < BN ? page_size : BN;
    const long long rows = (long long)num_pages * Hkv * page_size;
    if (rows >= (1ll << 31)) return (int)cudaErrorInvalidValue;
    CUtensorMap mk, mv;
    if (int e = get_map(k_cache, rows, D, box_rows, &mk)) return e;
    if (int e = get_map(v_cache, rows, D, box_rows, &mv)) return e;
    const int G = Hq / Hkv;
    dim3 grid(((max_q_len * G + NQ * BM - 1) / (NQ * BM)) * Hkv, n_seqs);
    return tw_launch(attn_prefill_tc5_kernel, grid, dim3(THREADS), (size_t)SMEM, stream, 1, mk, mv, (bf16*)out, out_stride,
                     (const bf16*)q, q_stride, seq_q_start, seq_q_len, seq_kv_len, seq_slot, block_table, table_stride,
                     Hq, Hkv, page_size, num_pages, window, scale * 1.4426950408889634f, skip_single, status);
}
