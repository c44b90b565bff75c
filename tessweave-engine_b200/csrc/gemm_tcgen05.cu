// bf16 matrix products on the 5th-generation tensor cores: out = x @ w.T with fp32 accumulation.
//
//   * operands travel global -> shared memory by TMA (cp.async.bulk.tensor.2d, 128-byte swizzle),
//     one elected thread issuing, completion counted on mbarriers, STAGES tiles in flight;
//   * one elected thread issues tcgen05.mma (cta_group::1, kind::f16, M = 128, N = BN, K = 16 per
//     instruction) straight from shared-memory descriptors; the accumulator lives in tensor
//     memory (TMEM), not in registers;
//   * tcgen05.commit hands shared-memory stages back to the producer and, after the last k-block,
//     tells the four epilogue warps that the accumulator is complete; they read it with
//     tcgen05.ld (one TMEM lane per thread) and write the result.
//
// The 128-row operand ("A") and the BN-row operand ("B") are both [rows, K] with K contiguous.
// Two uses:
//   swap-AB  (few tokens: decode):  A = w [n, k], B = x [m <= 64, k]; D[w row, token]; the weights
//            stream through a deep pipeline once, which is what bounds a decode step;
//   normal   (many tokens: prefill): A = x [m, k] in tiles of 128 tokens, B = w [n, k] in tiles of
//            BN rows; D[token, feature].
// k may be split over blockIdx.z; each slice then writes fp32 partial sums [slice][token][n].
// No load is multicast; every block fetches its own tiles.
//
// Every wait on an mbarrier is bounded (about a second of clock cycles).  A wait that runs out
// sets TW_ERR_WAIT in the status word, the block stops issuing work, waits (bounded) for the
// copies it has in flight, frees its tensor memory and returns.
//
// The reference runs these products through a library (nn.Linear: flow_engine/model.py:54,
// 76-80,201,204).
#include "tcgen05.cuh"

namespace {

using namespace tc5;

constexpr int BM = 128;            // rows of the A tile = TMEM lanes
constexpr int BK = 64;             // k per stage: 64 bf16 = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int THREADS = 128;

enum : int { OUT_BF16 = 0, OUT_F32 = 1, OUT_PARTIAL = 2 };

template <int BN> struct Config {
    static constexpr int A_BYTES = BM * BK * 2;
    static constexpr int B_BYTES = BN * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + (B_BYTES < 1024 ? 1024 : B_BYTES);
    static constexpr int STAGES = (200 * 1024) / STAGE_BYTES > 10 ? 10 : (200 * 1024) / STAGE_BYTES;
    static constexpr int TMEM_COLS = BN < 32 ? 32 : BN;
    static constexpr int SMEM = STAGES * STAGE_BYTES + 1024 /* alignment slack */ + 256 /* barriers */;
};

// out_mode / layout of the result:
//   swap == 1: D[w row, token]: out[token * out_stride + row]   (rows of A are output features)
//   swap == 0: D[token, feature]: out[token * out_stride + feature]
template <int BN>
__global__ void __launch_bounds__(THREADS)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    int rows_a, int rows_b, int K, int kper, void* __restrict__ out, int out_mode, int out_stride,
                    int swap, int* status) {
    using C = Config<BN>;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full = reinterpret_cast<uint64_t*>(tiles + C::STAGES * C::STAGE_BYTES);
    uint64_t* empty = full + C::STAGES;
    uint64_t* acc_full = empty + C::STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
    volatile int* aborted = reinterpret_cast<volatile int*>(tmem_slot + 1);

    tw_grid_wait();
    tw_grid_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int a_row0 = blockIdx.x * BM, b_row0 = blockIdx.y * BN;
    const int kbeg = blockIdx.z * kper, kend = min(K, kbeg + kper);
    const int num_kb = (kend - kbeg + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        mbar_init(acc_full, 1);
        *aborted = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(tmem_slot, C::TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0 && lane == 0) {
        // ---- producer: TMA loads, STAGES tiles ahead of the tensor cores
        int issued = 0;
        for (int kb = 0; kb < num_kb; ++kb) {
            const int s = kb % C::STAGES;
            const uint32_t parity = ((kb / C::STAGES) & 1) ^ 1;
            if (*aborted || !mbar_wait(&empty[s], parity, status)) { *aborted = 1; break; }
            unsigned char* a_tile = tiles + s * C::STAGE_BYTES;
            unsigned char* b_tile = a_tile + C::A_BYTES;
            mbar_expect_tx(&full[s], C::A_BYTES + C::B_BYTES);
            tma_load_2d(a_tile, &map_a, &full[s], kbeg + kb * BK, a_row0);
            tma_load_2d(b_tile, &map_b, &full[s], kbeg + kb * BK, b_row0);
            issued = kb + 1;
        }
        if (*aborted) {
            // wait (bounded) for the copies already in flight, so that none lands after the block has gone
            for (int kb = max(0, issued - C::STAGES); kb < issued; ++kb)
                mbar_wait(&full[kb % C::STAGES], (kb / C::STAGES) & 1, status);
        }
    } else if (warp == 1 && lane == 0) {
        // ---- tensor cores: one thread issues every MMA of the block
        const uint32_t idesc = instr_desc(BN);
        for (int kb = 0; kb < num_kb; ++kb) {
            const int s = kb % C::STAGES;
            if (*aborted || !mbar_wait(&full[s], (kb / C::STAGES) & 1, status)) { *aborted = 1; break; }
            tc_fence_after();
            const unsigned char* a_tile = tiles + s * C::STAGE_BYTES;
            const unsigned char* b_tile = a_tile + C::A_BYTES;
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k)
                umma_bf16(tmem_base, smem_desc(a_tile, k * UMMA_K * 2), smem_desc(b_tile, k * UMMA_K * 2), idesc,
                          (kb > 0 || k > 0) ? 1u : 0u);
            umma_commit(&empty[s]);           // the stage is free once these MMAs have read it
        }
        umma_commit(acc_full);                // the accumulator is complete once every MMA has retired
    }
    __syncwarp();

    // ---- epilogue: all four warps; warp w owns TMEM lanes 32 w .. 32 w + 31
    bool ok = num_kb > 0 ? mbar_wait(acc_full, 0, status) : true;
    if (*aborted) ok = false;
    tc_fence_after();
    if (ok) {
        const int row = a_row0 + warp * 32 + lane;          // row of A this thread holds
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 16) {
            uint32_t v[16];
            if (num_kb > 0) {
                tmem_ld16(tmem_base + ((uint32_t)(warp * 32) << 16) + c0, v);
            } else {
#pragma unroll
                for (int j = 0; j < 16; ++j) v[j] = 0u;
            }
            if (row >= rows_a) continue;
            if (swap) {
                // row = output feature, columns = tokens
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const int tok = b_row0 + c0 + j;
                    if (tok >= rows_b) break;
                    const float f = __uint_as_float(v[j]);
                    if (out_mode == OUT_BF16)
                        reinterpret_cast<bf16*>(out)[(size_t)tok * out_stride + row] = __float2bfloat16_rn(f);
                    else if (out_mode == OUT_F32)
                        reinterpret_cast<float*>(out)[(size_t)tok * out_stride + row] = f;
                    else
                        reinterpret_cast<float*>(out)[((size_t)blockIdx.z * rows_b + tok) * out_stride + row] = f;
                }
            } else {
                // row = token, columns = output features (16 contiguous values per step)
                const int col = b_row0 + c0;
                if (col >= rows_b) continue;
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
                    float* o = reinterpret_cast<float*>(out) +
                               (out_mode == OUT_PARTIAL ? ((size_t)blockIdx.z * rows_a + row) * out_stride
                                                        : (size_t)row * out_stride) + col;
                    for (int j = 0; j < n; ++j) o[j] = __uint_as_float(v[j]);
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, C::TMEM_COLS);
}

template <int BN>
int launch(const void* a, int rows_a, const void* b, int rows_b, int K, int kper, void* out, int out_mode,
           int out_stride, int swap, int* status, cudaStream_t stream) {
    using C = Config<BN>;
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM);
        if (e != cudaSuccess) return (int)e;
        attr_set = true;
    }
    CUtensorMap ma, mb;
    if (int e = get_map(a, rows_a, K, BM, &ma)) return e;
    if (int e = get_map(b, rows_b, K, BN, &mb)) return e;
    const int ksplit = (K + kper - 1) / kper;
    dim3 grid((rows_a + BM - 1) / BM, (rows_b + BN - 1) / BN, ksplit);
    return tw_launch(gemm_tcgen05_kernel<BN>, grid, dim3(THREADS), (size_t)C::SMEM, stream, 1, ma, mb, rows_a, rows_b, K,
                     kper, out, out_mode, out_stride, swap, status);
}

}  // namespace

// out[m, n] = x[m, k] @ w[n, k].T, bf16 operands (k a multiple of 8, both 16-byte aligned).
//   swap = 1 (m <= 64): the weights are the 128-row operand; kper < k splits k into slices and
//                       out is then fp32 [slices, m, n] (out_mode 2).
//   swap = 0: tokens are the 128-row operand, the weights come in tiles of 256 (or 128) rows.
// out_mode 0: bf16 [m, out_stride]; 1: fp32 [m, out_stride]; 2: fp32 slices.  kper a multiple of 64.
TW_EXPORT int tw_gemm_tcgen05(const void* x, const void* w, int m, int n, int k, int kper, void* out, int out_mode,
                              int out_stride, int swap, int* status, cudaStream_t stream) {
    if (m <= 0 || n <= 0) return 0;
    if (k <= 0 || (k & 7) || kper <= 0 || (kper & 63) || out_mode < 0 || out_mode > 2 ||
        (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w) & 15))
        return (int)cudaErrorInvalidValue;
    const int ksplit = (k + kper - 1) / kper;
    if (ksplit > 1 && out_mode != OUT_PARTIAL) return (int)cudaErrorInvalidValue;
    if (swap) {
        if (m > 64) return (int)cudaErrorInvalidValue;
        if (m <= 16) return launch<16>(w, n, x, m, k, kper, out, out_mode, out_stride, 1, status, stream);
        if (m <= 32) return launch<32>(w, n, x, m, k, kper, out, out_mode, out_stride, 1, status, stream);
        return launch<64>(w, n, x, m, k, kper, out, out_mode, out_stride, 1, status, stream);
    }
    if (n >= 256) return launch<256>(x, m, w, n, k, kper, out, out_mode, out_stride, 0, status, stream);
    return launch<128>(x, m, w, n, k, kper, out, out_mode, out_stride, 0, status, stream);
}
