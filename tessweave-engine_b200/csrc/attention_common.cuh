// What the bfloat16 attention kernels share: tensor-core and shared-memory instruction wrappers, and the
// description of a decode step's q/k/v product for the kernels that turn it into query, key and value
// themselves.
#pragma once

#include "common.cuh"

namespace tw_attn {

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

__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t v) {
    uint32_t r;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(r) : "r"(v));
    return r;
}
__device__ __forceinline__ void mma_bf16_regs(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                              uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Where a decode step's query, key and value come from when the kernel makes them itself: the rows of the
// q/k/v product (fp32 slices of a product split over k, or one bf16 row), its bias, the rotation table.
struct FusedQkv {
    const float* partial;        // [slices][rows][width] fp32, or null
    int nslices;
    long long slice_stride;      // elements between slices
    const bf16* dense;           // [rows][dense_stride] bf16, used when partial is null
    int dense_stride;
    const float* bias;           // [width] or null
    const float* inv_freq;       // [D / 2]; null: no rotation
    bf16* k_cache;               // where the new key and value go; null: the cache is not written
    bf16* v_cache;
    const void* next_weights;    // what the kernel after this one streams (or null): prefetched into L2 after the keys
    long long next_bytes;
};

// fp32 values of NC columns of one row of the q/k/v product, bias included.  The slices of a split product are
// summed (0 + 4 + 8 ..), (1 + 5 + ..), .. first and then ((.) + (.)) + ((.) + (.)), as the kernel that otherwise
// does this work sums them; the loads of all columns and of four slices are independent of one another.
template <int NC>
__device__ __forceinline__ void product_cols(const FusedQkv& fq, size_t row, int width, const int (&cols)[NC], float (&out)[NC]) {
    if (fq.partial) {
        const float* prow = fq.partial + row * width;
        float acc[NC][4];
#pragma unroll
        for (int j = 0; j < NC; ++j) { acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f; }
        int k = 0;
        for (; k + 4 <= fq.nslices; k += 4) {
#pragma unroll
            for (int j = 0; j < NC; ++j) {
#pragma unroll
                for (int u = 0; u < 4; ++u) acc[j][u] += prow[(size_t)(k + u) * fq.slice_stride + cols[j]];
            }
        }
        for (; k < fq.nslices; ++k) {
#pragma unroll
            for (int j = 0; j < NC; ++j) acc[j][0] += prow[(size_t)k * fq.slice_stride + cols[j]];
        }
#pragma unroll
        for (int j = 0; j < NC; ++j) out[j] = (acc[j][0] + acc[j][1]) + (acc[j][2] + acc[j][3]);
    } else {
#pragma unroll
        for (int j = 0; j < NC; ++j) out[j] = __bfloat162float(fq.dense[row * fq.dense_stride + cols[j]]);
    }
    if (fq.bias) {
#pragma unroll
        for (int j = 0; j < NC; ++j) out[j] += fq.bias[cols[j]];
    }
}

}  // namespace tw_attn
