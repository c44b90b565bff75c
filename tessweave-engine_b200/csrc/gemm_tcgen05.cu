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
#include "common.cuh"

#include <cuda.h>
#include <mutex>
#include <unordered_map>

namespace {

typedef __nv_bfloat16 bf16;

constexpr int BM = 128;            // rows of the A tile = TMEM lanes
constexpr int BK = 64;             // k per stage: 64 bf16 = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int THREADS = 128;
constexpr long long WAIT_CYCLES = 2000000000ll;      // bound of every mbarrier wait

enum : int { OUT_BF16 = 0, OUT_F32 = 1, OUT_PARTIAL = 2 };

// ---- PTX wrappers ------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait: false (and the error bit set) if the phase did not complete in time.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* status) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long start = clock64();
    while (!mbar_try_wait(bar, parity)) {
        if (clock64() - start > WAIT_CYCLES) {
            atomicOr(status, TW_ERR_WAIT);
            return false;
        }
    }
    return true;
}
__device__ __forceinline__ void tma_load_2d(void* smem, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(smem)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(ncols));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols));
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor of a [rows][64] bf16 tile written by TMA with the 128-byte
// swizzle: K-major, rows 128 bytes apart, groups of 8 rows 1024 bytes apart (stride byte offset),
// leading byte offset 1 (unused for swizzled K-major), descriptor version 1, layout SWIZZLE_128B.
__device__ __forceinline__ uint64_t smem_desc(const void* tile, int k_byte_offset) {
    const uint32_t addr = smem_u32(tile) + k_byte_offset;
    return (uint64_t)((addr & 0x3FFFF) >> 4) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor: D fp32, A and B bf16, both K-major, N = bn, M = 128, dense, no negate.
__device__ __forceinline__ uint32_t instr_desc(int bn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}

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

// ---- host side: tensor maps -----------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

struct MapKey {
    const void* ptr; int rows, k, box_rows;
    bool operator==(const MapKey& o) const { return ptr == o.ptr && rows == o.rows && k == o.k && box_rows == o.box_rows; }
};
struct MapKeyHash {
    size_t operator()(const MapKey& m) const {
        return std::hash<const void*>()(m.ptr) ^ (size_t)m.rows * 1000003u ^ (size_t)m.k * 7919u ^ (size_t)m.box_rows * 31u;
    }
};
std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_maps;
std::mutex g_maps_mutex;

// A [rows, k] bf16 matrix with k contiguous, read in boxes of [box_rows, 64] with the 128-byte swizzle;
// what lies outside the matrix reads as zero.
int get_map(const void* ptr, int rows, int k, int box_rows, CUtensorMap* out) {
    std::lock_guard<std::mutex> lock(g_maps_mutex);
    const MapKey key{ptr, rows, k, box_rows};
    auto it = g_maps.find(key);
    if (it != g_maps.end()) { *out = it->second; return 0; }
    EncodeTiledFn fn = encode_fn();
    if (!fn) return (int)cudaErrorNotSupported;
    const cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)k * 2};
    const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    CUtensorMap m;
    const CUresult r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return 1000 + (int)r;
    if (g_maps.size() > 4096) g_maps.clear();
    g_maps[key] = m;
    *out = m;
    return 0;
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
