// bf16 matrix products for many rows (prompt steps) on CTA pairs: out = x @ w.T, fp32 accumulation.
//
// Two thread blocks on neighbouring SMs (a cluster of two) compute one 256 x 256 tile with
// tcgen05.mma.cta_group::2: block r of the pair holds rows 128 r .. 128 r + 127 of the token
// operand and of the accumulator, and half of the 256 weight rows of the tile; the tensor cores
// of both SMs read the weight rows from both blocks' shared memory.  Per k-block a block
// therefore loads 16 KB of tokens and 16 KB of weights instead of 16 + 32 KB for a 128 x 256
// tile of its own, and it is the traffic from L2 to the SMs that bounds these products.
//
//   * every block loads its own tiles by TMA (no multicast); the copies of both blocks complete
//     on the mbarrier of the pair's first block, whose one thread issues every MMA;
//   * tcgen05.commit with a multicast mask hands a stage back to the producers of both blocks and
//     tells both blocks' epilogue warps when the accumulator is complete;
//   * the kernel is persistent: a pair walks its tiles with the shared-memory ring kept full across
//     tiles, and two accumulators in tensor memory let four epilogue warps per block read one tile
//     (tcgen05.ld, one TMEM lane per thread) while the tensor cores work on the next; they write bf16,
//     fp32, or silu(gate) * up for weights whose rows come in groups of eight gates and eight ups.
//
// Measured on B200 (2,048 x 37,888 x 3,584): 391 us, 0.88 of the library's product; with the
// SiLU.mul epilogue it equals the library's product plus the separate SiLU.mul kernel.  Per k-block
// the copies alone take 560 cycles, the MMAs alone 660 (512 of them in the tensor pipe), both
// together 830.  Tried and measured no better: tiles of 256 x 512 (the accumulator then fills the
// tensor memory and the epilogue no longer overlaps), L2 prefetch of the weight tiles ahead of
// the copies, the next k-block's wait between the MMAs of the current one, spinning waits.
//
// Every wait on an mbarrier is bounded; a wait that runs out sets TW_ERR_WAIT in the status word,
// the role stops, and the block goes on to the common end (cluster barrier, tensor memory freed).
//
// The reference runs these products through a library (nn.Linear: flow_engine/model.py:54,
// 76-80,201,204).
#include "tcgen05.cuh"

namespace {

using namespace tc5;

constexpr int BM = 128;            // rows per block (256 per pair)
constexpr int BN = 256;            // weight rows per pair tile
constexpr int BNH = BN / 2;        // weight rows a block loads
constexpr int BK = 64;            // four MMAs of 16 values of k per k-block (the issue loop is written out for four)
constexpr int EPI_WARPS = 4;
constexpr int THREADS = 64 + EPI_WARPS * 32;   // warp 0: TMA, warp 1: MMA, warps 2-5: epilogue
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BNH * BK * 2;
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int STAGES = 7;
constexpr int TMEM_COLS = 512;         // two accumulators of 256 columns: the epilogue of a tile overlaps the next tile's MMAs
constexpr int SMEM = STAGES * STAGE_BYTES + 1024 /* alignment slack */ + 256 /* barriers */;

enum : int { OUT_BF16 = 0, OUT_F32 = 1, OUT_SILU_MUL = 3 };

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t map_to_rank(const void* smem, uint32_t rank) {
    uint32_t out;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(smem_u32(smem)), "r"(rank));
    return out;
}
__device__ __forceinline__ void tma_load_2d_pair(void* smem, const CUtensorMap* map, uint32_t bar_cluster_addr, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(smem)), "l"(map), "r"(bar_cluster_addr), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(ncols));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::);
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols));
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// arrive on the barrier at this offset in both blocks of the pair once the MMAs issued so far have retired
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smem_u32(bar)), "h"((uint16_t)3) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Instruction descriptor of the pair: D fp32, A and B bf16 K-major, M = 256 over the two blocks, N = 256.
__device__ __forceinline__ uint32_t instr_desc_pair() {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
}

// One accumulator row of 16 columns, written the way `out_mode` says.
__device__ __forceinline__ void store_chunk(const uint32_t (&v)[16], void* out, int out_mode, int out_stride, int row, int col,
                                            int rows_b) {
    if (out_mode == OUT_SILU_MUL) {
        // columns col .. col + 7 are gates, col + 8 .. col + 15 their ups (rows_b is a multiple of 16)
        uint4 p;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&p);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float g0 = __uint_as_float(v[2 * j]), g1 = __uint_as_float(v[2 * j + 1]);
            const float u0 = __uint_as_float(v[8 + 2 * j]), u1 = __uint_as_float(v[8 + 2 * j + 1]);
            h[j] = __floats2bfloat162_rn(g0 / (1.f + __expf(-g0)) * u0, g1 / (1.f + __expf(-g1)) * u1);
        }
        *reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(out) + (size_t)row * out_stride + (col >> 1)) = p;
        return;
    }
    const int n = min(16, rows_b - col);
    if (out_mode == OUT_BF16) {
        bf16* o = reinterpret_cast<bf16*>(out) + (size_t)row * out_stride + col;
        if (n == 16 && ((reinterpret_cast<uintptr_t>(o) & 15) == 0)) {
            uint4 p0, p1;
            __nv_bfloat162* h0 = reinterpret_cast<__nv_bfloat162*>(&p0);
            __nv_bfloat162* h1 = reinterpret_cast<__nv_bfloat162*>(&p1);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                h0[j] = __floats2bfloat162_rn(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1]));
                h1[j] = __floats2bfloat162_rn(__uint_as_float(v[8 + 2 * j]), __uint_as_float(v[8 + 2 * j + 1]));
            }
            reinterpret_cast<uint4*>(o)[0] = p0;
            reinterpret_cast<uint4*>(o)[1] = p1;
        } else {
            for (int j = 0; j < n; ++j) o[j] = __float2bfloat16_rn(__uint_as_float(v[j]));
        }
    } else {
        float* o = reinterpret_cast<float*>(out) + (size_t)row * out_stride + col;
        for (int j = 0; j < n; ++j) o[j] = __uint_as_float(v[j]);
    }
}

// Persistent: a pair walks the tiles pair, pair + pairs, ...; tile t covers token rows 256 (t % tiles_m) ..
// and weight rows 256 (t / tiles_m) .., so that the pairs at work at one time share weight tiles.
__global__ void __launch_bounds__(THREADS)
gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, int rows_a,
                 int rows_b, int K, void* __restrict__ out, int out_mode, int out_stride, int* status) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full = reinterpret_cast<uint64_t*>(tiles + STAGES * STAGE_BYTES);     // used in the pair's first block
    uint64_t* empty = full + STAGES;
    uint64_t* acc_full = empty + STAGES;            // [2]: accumulator b is complete (both blocks)
    uint64_t* acc_empty = acc_full + 2;             // [2]: accumulator b has been read by every epilogue warp of the pair (first block)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);

    tw_grid_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();
    const int pair = (int)(blockIdx.x >> 1), pairs = (int)(gridDim.x >> 1);
    const int tiles_m = (rows_a + 2 * BM - 1) / (2 * BM), tiles_n = (rows_b + BN - 1) / BN;
    const int n_tiles = tiles_m * tiles_n;
    const int num_kb = (K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 2 * EPI_WARPS); }
        mbar_fence_init();
    }
    if (warp == 1) tmem_alloc_pair(tmem_slot, TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                 // both blocks' barriers exist before either block signals the other's
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            // ---- producer of this block: its 128 token rows and its 128 weight rows of every k-block of every tile
            int it = 0;
            bool ok = true;
            for (int t = pair; ok && t < n_tiles; t += pairs) {
                const int a_row0 = (t % tiles_m) * 2 * BM + (int)rank * BM;
                const int b_row0 = (t / tiles_m) * BN + (int)rank * BNH;
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    ok = mbar_wait(&empty[s], ((it / STAGES) & 1) ^ 1, status);
                    if (!ok) break;
                    const uint32_t full_addr = map_to_rank(&full[s], 0);
                    // The first block announces the bytes of both blocks.  The other block's copies may land
                    // before that: the phase cannot complete while the first block's arrival is outstanding.
                    if (rank == 0) mbar_expect_tx(&full[s], 2 * STAGE_BYTES);
                    unsigned char* a_tile = tiles + s * STAGE_BYTES;
                    tma_load_2d_pair(a_tile, &map_a, full_addr, kb * BK, a_row0);
                    tma_load_2d_pair(a_tile + A_BYTES, &map_b, full_addr, kb * BK, b_row0);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            // ---- tensor cores of both SMs: one thread of the pair's first block issues every MMA
            const uint32_t idesc = instr_desc_pair();
            const uint64_t a_desc = smem_desc(tiles, 0), b_desc = smem_desc(tiles + A_BYTES, 0);
            // An MMA is not accepted before the one before it has retired, so whatever this thread does
            // between the last MMA of a k-block and the first of the next leaves the tensor pipe idle.  The
            // test of the next k-block's barrier is therefore made before the last MMA is issued, while the
            // third one runs; only if the copies have not landed by then does the thread wait for them later.
            int s = 0, lt = 0;
            uint32_t phase = 0;
            bool ok = true, ready = false;
            for (int t = pair; ok && t < n_tiles; t += pairs, ++lt) {
                const int b = lt & 1;
                ok = mbar_wait(&acc_empty[b], ((lt >> 1) & 1) ^ 1, status);       // the epilogues have read what was there
                if (!ok) break;
                tc_fence_after();
                const uint32_t acc = tmem_base + b * BN;
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!ready) ok = mbar_wait(&full[s], phase, status);
                    if (!ok) break;
                    const uint64_t ad = a_desc + (uint64_t)(s * (STAGE_BYTES >> 4)), bd = b_desc + (uint64_t)(s * (STAGE_BYTES >> 4));
                    const int s_next = s + 1 == STAGES ? 0 : s + 1;
                    const uint32_t phase_next = s + 1 == STAGES ? phase ^ 1u : phase;
                    umma_bf16_pair(acc, ad, bd, idesc, kb > 0 ? 1u : 0u);
                    umma_bf16_pair(acc, ad + 2, bd + 2, idesc, 1u);
                    umma_bf16_pair(acc, ad + 4, bd + 4, idesc, 1u);
                    ready = mbar_test_wait(&full[s_next], phase_next);     // usually true: the copies run stages ahead
                    umma_bf16_pair(acc, ad + 6, bd + 6, idesc, 1u);
                    umma_commit_pair(&empty[s]);
                    s = s_next;
                    phase = phase_next;
                }
                if (ok) umma_commit_pair(&acc_full[b]);
            }
        }
    } else {
        // ---- epilogue warps of both blocks; warp w may touch TMEM lanes 32 (w % 4) .. + 31 = 32 rows of this block
        const int quarter = warp & 3;
        const uint32_t empty_addr = map_to_rank(&acc_empty[0], 0);
        int lt = 0;
        bool ok = num_kb > 0;
        for (int t = pair; ok && t < n_tiles; t += pairs, ++lt) {
            const int b = lt & 1;
            ok = mbar_wait(&acc_full[b], (lt >> 1) & 1, status);
            if (!ok) break;
            tc_fence_after();
            const int row = (t % tiles_m) * 2 * BM + (int)rank * BM + quarter * 32 + lane;
            const int col0 = (t / tiles_m) * BN;
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 16) {
                uint32_t v[16];
                tmem_ld16(tmem_base + ((uint32_t)(quarter * 32) << 16) + b * BN + c0, v);
                if (row < rows_a && col0 + c0 < rows_b) store_chunk(v, out, out_mode, out_stride, row, col0 + c0, rows_b);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0)          // the MMA thread of the first block may write this accumulator again
                asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(empty_addr + 8u * b) : "memory");
        }
    }
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                 // neither block leaves (or frees tensor memory) while the other may still use its shared memory
    if (warp == 1) tmem_dealloc_pair(tmem_base, TMEM_COLS);
}

}  // namespace

// out[m, n] = x[m, k] @ w[n, k].T, bf16 operands (k a multiple of 8, both 16-byte aligned), for m of
// a few hundred rows and more.  out_mode 0: bf16 [m, out_stride]; 1: fp32 [m, out_stride]; 3: bf16
// [m, out_stride] = silu(gate) * up with n / 2 columns, for w whose rows come in groups of eight
// gates followed by their eight ups (n a multiple of 16).
TW_EXPORT int tw_gemm_tcgen05_pair(const void* x, const void* w, int m, int n, int k, void* out, int out_mode,
                                   int out_stride, int* status, cudaStream_t stream) {
    if (m <= 0 || n <= 0) return 0;
    if (k <= 0 || (k & 7) || (out_mode != OUT_BF16 && out_mode != OUT_F32 && out_mode != OUT_SILU_MUL) ||
        (out_mode == OUT_SILU_MUL && ((n & 15) || (out_stride & 7) || (reinterpret_cast<uintptr_t>(out) & 15))) ||
        (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w) & 15))
        return (int)cudaErrorInvalidValue;
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(gemm_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e != cudaSuccess) return (int)e;
        attr_set = true;
    }
    CUtensorMap ma, mb;
    if (int e = get_map(x, m, k, BM, &ma)) return e;
    if (int e = get_map(w, n, k, BNH, &mb)) return e;
    static int sm_count = 0;
    if (!sm_count) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
        if (sm_count < 2) sm_count = 2;
    }
    const int n_tiles = ((m + 2 * BM - 1) / (2 * BM)) * ((n + BN - 1) / BN);
    const int pairs = n_tiles < sm_count / 2 ? n_tiles : sm_count / 2;
    dim3 grid(2 * pairs);
    return tw_launch(gemm_pair_kernel, grid, dim3(THREADS), (size_t)SMEM, stream, 2, ma, mb, m, n, k, out, out_mode,
                     out_stride, status);
}
