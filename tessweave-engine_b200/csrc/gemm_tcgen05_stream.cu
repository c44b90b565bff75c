// bf16 matrix products for a few dozen rows (decode steps of 9 to 128 requests) on the 5th-generation
// tensor cores: out = x @ w.T with fp32 accumulation, bound by reading w once.
//
// The weights are the 128-row operand of tcgen05.mma (M = 128 weight rows, N = the tokens, padded to
// 16, 32, 64 or 128), so a k-block of a weight tile is one 16 KB TMA copy whatever the number of tokens.
// The kernel is persistent, one block per SM: a block walks its work items (a 128-row tile of w and a
// slice of k each) with the ring of shared-memory stages kept full across items, so the weights stream
// without a gap from the kernel's first copy to its last; two accumulators in tensor memory let the four
// epilogue warps write one item's result while the tensor cores work on the next.
//
//   warp 0: one thread issues the TMA copies (weights 128 x 64, tokens N x 64, 128-byte swizzle, no multicast);
//   warp 1: one thread issues the MMAs (descriptors built once, a constant added per MMA) and hands stages
//           back with tcgen05.commit;
//   warps 2-5: epilogue, one TMEM lane (= weight row) per thread: fp32 or bf16 rows, fp32 slices of a
//           product split over k, or silu(gate) * up for weights whose rows come in groups of eight gates and
//           their eight ups (the up of a gate sits eight lanes further: one shuffle).
//
// Every wait on an mbarrier is bounded; a wait that runs out sets TW_ERR_WAIT in the status word, the role
// stops, the producer waits (bounded) for the copies it has in flight, and the block goes on to the common
// end, where it frees its tensor memory.
//
// The reference runs these products through a library (nn.Linear: flow_engine/model.py:54,76-80,201,204).
#include "tcgen05.cuh"

namespace {

using namespace tc5;

constexpr int BM = 128;            // weight rows per item = TMEM lanes
constexpr int BK = 64;             // values of k per stage: one 128-byte swizzle row, four MMAs
constexpr int EPI_WARPS = 4;
constexpr int THREADS = 64 + EPI_WARPS * 32;
constexpr int A_BYTES = BM * BK * 2;

enum : int { OUT_BF16 = 0, OUT_F32 = 1, OUT_PARTIAL = 2, OUT_SILU_MUL = 3, OUT_EARLY_DEPENDENTS = 16 /* flag, or-ed in */ };

template <int BN> struct Config {
    static constexpr int B_BYTES = BN * BK * 2 < 1024 ? 1024 : BN * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int STAGES = (208 * 1024) / STAGE_BYTES > 12 ? 12 : (208 * 1024) / STAGE_BYTES;
    static constexpr int ACC_COLS = BN < 32 ? 32 : BN;             // columns between the two accumulators
    static constexpr int TMEM_COLS = 2 * ACC_COLS;
    static constexpr int SMEM = STAGES * STAGE_BYTES + 1024 /* alignment slack */ + 512 /* barriers */;
};

// Item i of the kernel: weight rows 128 (i / ksplit) .., k from (i % ksplit) * kper.
template <int BN>
__global__ void __launch_bounds__(THREADS)
gemm_stream_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, int n_rows,
                   int m_tokens, int K, int kper, int ksplit, void* __restrict__ out, int out_mode, int out_stride,
                   int* status, const void* next_weights, long long next_bytes) {
    using C = Config<BN>;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full = reinterpret_cast<uint64_t*>(tiles + C::STAGES * C::STAGE_BYTES);
    uint64_t* empty = full + C::STAGES;
    uint64_t* acc_full = empty + C::STAGES;         // [2]: accumulator b is complete
    uint64_t* acc_empty = acc_full + 2;             // [2]: accumulator b has been read by every epilogue warp
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);

    TW_TIMELINE_SCOPE(TW_K_OTHER);
    tw_grid_wait();
    TW_TIMELINE_MARK();
    // a small kernel after this one (a norm) may become resident at once; it waits for the result itself
    if (out_mode & OUT_EARLY_DEPENDENTS) tw_launch_dependents_now();
    out_mode &= ~OUT_EARLY_DEPENDENTS;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_items = ((n_rows + BM - 1) / BM) * ksplit;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], EPI_WARPS); }
        mbar_fence_init();
    }
    if (warp == 1) tmem_alloc(tmem_slot, C::TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            // ---- producer: the copies of every k-block of every item of this block, STAGES ahead of the tensor cores
            int it = 0;
            bool ok = true;
            for (int item = blockIdx.x; ok && item < n_items; item += gridDim.x) {
                const int row0 = (item / ksplit) * BM;
                const int kbeg = (item % ksplit) * kper, kend = min(K, kbeg + kper);
                for (int k0 = kbeg; k0 < kend; k0 += BK, ++it) {
                    const int s = it % C::STAGES;
                    ok = mbar_wait(&empty[s], ((it / C::STAGES) & 1) ^ 1, status);
                    if (!ok) break;
                    unsigned char* a_tile = tiles + s * C::STAGE_BYTES;
                    mbar_expect_tx(&full[s], A_BYTES + BN * BK * 2);
                    tma_load_2d(a_tile, &map_w, &full[s], k0, row0);
                    tma_load_2d(a_tile + A_BYTES, &map_x, &full[s], k0, 0);
                }
            }
            // this block's last copy is on its way: its share of what the kernel after this one streams may follow
            if (ok) tw_prefetch_l2_share(next_weights, next_bytes);
            if (!ok) {
                // wait (bounded) for the copies already in flight, so that none lands after the block has gone
                for (int j = max(0, it - C::STAGES); j < it; ++j) mbar_wait(&full[j % C::STAGES], (j / C::STAGES) & 1, status);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ---- tensor cores.  An MMA is not accepted before the one before it has retired, so the look at the
            // next stage's barrier is taken while the third MMA of a k-block runs, and the thread only waits for
            // the copies if they have not landed by then.
            const uint32_t idesc = instr_desc(BN);
            const uint64_t a_desc = smem_desc(tiles, 0), b_desc = smem_desc(tiles + A_BYTES, 0);
            int s = 0, li = 0;
            uint32_t phase = 0;
            bool ok = true, ready = false;
            for (int item = blockIdx.x; ok && item < n_items; item += gridDim.x, ++li) {
                const int b = li & 1;
                const int kbeg = (item % ksplit) * kper, kend = min(K, kbeg + kper);
                const int num_kb = (kend - kbeg + BK - 1) / BK;
                ok = mbar_wait(&acc_empty[b], ((li >> 1) & 1) ^ 1, status);      // the epilogue has read what was there
                if (!ok) break;
                tc_fence_after();
                const uint32_t acc = tmem_base + b * C::ACC_COLS;
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!ready) ok = mbar_wait(&full[s], phase, status);
                    if (!ok) break;
                    tc_fence_after();
                    const uint64_t ad = a_desc + (uint64_t)(s * (C::STAGE_BYTES >> 4)), bd = b_desc + (uint64_t)(s * (C::STAGE_BYTES >> 4));
                    const int s_next = s + 1 == C::STAGES ? 0 : s + 1;
                    const uint32_t phase_next = s + 1 == C::STAGES ? phase ^ 1u : phase;
                    umma_bf16(acc, ad, bd, idesc, kb > 0 ? 1u : 0u);
                    umma_bf16(acc, ad + 2, bd + 2, idesc, 1u);
                    umma_bf16(acc, ad + 4, bd + 4, idesc, 1u);
                    ready = mbar_test_wait(&full[s_next], phase_next);
                    umma_bf16(acc, ad + 6, bd + 6, idesc, 1u);
                    umma_commit(&empty[s]);
                    s = s_next;
                    phase = phase_next;
                }
                if (ok) umma_commit(&acc_full[b]);
            }
        }
    } else {
        // ---- epilogue; warp w may touch TMEM lanes 32 (w % 4) .. + 31 = 32 weight rows of the item
        const int quarter = warp & 3;
        int li = 0;
        bool ok = true;
        for (int item = blockIdx.x; ok && item < n_items; item += gridDim.x, ++li) {
            const int b = li & 1;
            const int slice = item % ksplit;                  // every slice has values of k: ksplit = ceil(K / kper)
            ok = mbar_wait(&acc_full[b], (li >> 1) & 1, status);
            if (!ok) break;
            tc_fence_after();
            const int row = (item / ksplit) * BM + quarter * 32 + lane;          // weight row = output feature
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 16) {
                if (c0 >= m_tokens) break;
                uint32_t v[16];
                tmem_ld16(tmem_base + ((uint32_t)(quarter * 32) << 16) + b * C::ACC_COLS + c0, v);
                if (out_mode == OUT_SILU_MUL) {
                    // rows 16 g .. 16 g + 7 are gates, the eight after them their ups: lane l < 8 (mod 16) takes the up from lane l + 8
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const float up = __shfl_down_sync(0xffffffffu, __uint_as_float(v[j]), 8);
                        const float gt = __uint_as_float(v[j]);
                        const int tok = c0 + j;
                        if ((lane & 8) == 0 && row < n_rows && tok < m_tokens)
                            reinterpret_cast<bf16*>(out)[(size_t)tok * out_stride + (row >> 4) * 8 + (lane & 7)] =
                                __float2bfloat16_rn(gt / (1.0f + expf(-gt)) * up);
                    }
                    continue;
                }
                if (row >= n_rows) continue;
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const int tok = c0 + j;
                    if (tok >= m_tokens) break;
                    const float f = __uint_as_float(v[j]);
                    if (out_mode == OUT_BF16)
                        reinterpret_cast<bf16*>(out)[(size_t)tok * out_stride + row] = __float2bfloat16_rn(f);
                    else if (out_mode == OUT_F32)
                        reinterpret_cast<float*>(out)[(size_t)tok * out_stride + row] = f;
                    else
                        reinterpret_cast<float*>(out)[((size_t)slice * m_tokens + tok) * out_stride + row] = f;
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[b]);      // the MMA thread may write this accumulator again
        }
    }
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, C::TMEM_COLS);
}

template <int BN>
int launch(const void* w, int n, const void* x, int m, int K, int kper, int ksplit, void* out, int out_mode, int out_stride,
           int* status, int blocks, const void* next_weights, long long next_bytes, cudaStream_t stream) {
    using C = Config<BN>;
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(gemm_stream_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM);
        if (e != cudaSuccess) return (int)e;
        attr_set = true;
    }
    CUtensorMap mw, mx;
    if (int e = get_map(w, n, K, BM, &mw)) return e;
    if (int e = get_map(x, m, K, BN, &mx)) return e;
    return tw_launch(gemm_stream_kernel<BN>, dim3(blocks), dim3(THREADS), (size_t)C::SMEM, stream, 1, mw, mx, n, m, K, kper, ksplit,
                     out, out_mode, out_stride, status, next_weights, next_bytes);
}

}  // namespace

// out[m, n] = x[m, k] @ w[n, k].T for m <= 128 rows, bf16 operands (k a multiple of 8, both 16-byte aligned).
// kper (a multiple of 64) < k splits k into slices; out is then fp32 [slices, m, n] (out_mode 2).
// out_mode 0: bf16 [m, out_stride]; 1: fp32 [m, out_stride]; 3: bf16 [m, out_stride] = silu(gate) * up with n / 2
// columns, for w whose rows come in groups of eight gates followed by their eight ups (n a multiple of 16, no slices).
TW_EXPORT int tw_gemm_tcgen05_stream(const void* x, const void* w, int m, int n, int k, int kper, void* out, int out_mode,
                                     int out_stride, int* status, const void* next_weights, long long next_bytes,
                                     cudaStream_t stream) {
    if (m <= 0 || n <= 0) return 0;
    if ((uintptr_t)next_weights & 15) return (int)cudaErrorMisalignedAddress;
    if (!next_weights || next_bytes < 0) next_bytes = 0;
    const int mode = out_mode & ~OUT_EARLY_DEPENDENTS;
    if (m > 128 || k <= 0 || (k & 7) || kper <= 0 || (kper & 63) || mode < 0 || mode > 3 ||
        (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w) & 15))
        return (int)cudaErrorInvalidValue;
    const int ksplit = (k + kper - 1) / kper;
    if (ksplit > 1 && mode != OUT_PARTIAL) return (int)cudaErrorInvalidValue;
    if (mode == OUT_SILU_MUL && (n & 15)) return (int)cudaErrorInvalidValue;
    static int sm_count = 0;
    if (!sm_count) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sm_count <= 0) sm_count = 148;
    }
    const long long items = (long long)((n + BM - 1) / BM) * ksplit;
    const int blocks = (int)(items < sm_count ? items : sm_count);
    if (m <= 16) return launch<16>(w, n, x, m, k, kper, ksplit, out, out_mode, out_stride, status, blocks, next_weights, next_bytes, stream);
    if (m <= 32) return launch<32>(w, n, x, m, k, kper, ksplit, out, out_mode, out_stride, status, blocks, next_weights, next_bytes, stream);
    if (m <= 64) return launch<64>(w, n, x, m, k, kper, ksplit, out, out_mode, out_stride, status, blocks, next_weights, next_bytes, stream);
    return launch<128>(w, n, x, m, k, kper, ksplit, out, out_mode, out_stride, status, blocks, next_weights, next_bytes, stream);
}

TW_EXPORT int tw_gemm_tcgen05_stream_sm_count() {
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
    return sms;
}
