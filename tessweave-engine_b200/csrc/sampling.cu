// Token selection on fp32 logits: a cluster of eight blocks per greedy row, one block per row with a temperature.
//
//   temperature == 0:  the largest logit; the lowest index wins a tie
//                      (reference: flow_engine/engine.py:155-156, argmax).
//   temperature  > 0:  e_v = exp((x_v - max) / temperature);  u = uniform(seed, counter);
//                      the first index whose running sum of e exceeds u * sum(e)
//                      (reference: flow_engine/engine.py:157-158 samples from
//                      softmax(logits / T) with a per-request seeded generator; its CPU
//                      stream cannot be reproduced on the device, so the engine defines
//                      its own counter-based uniform, below).
//
// uniform(seed, counter): splitmix64 of seed + (counter + 1) * 0x9E3779B97F4A7C15,
// top 24 bits, times 2^-24.  A request's draws depend on its own seed and on how
// many tokens it has drawn, never on its neighbours in the batch.
#include "common.cuh"
#include <cooperative_groups.h>

namespace cg = cooperative_groups;

__host__ __device__ inline float tw_uniform(unsigned long long seed, unsigned long long counter) {
    unsigned long long z = seed + (counter + 1ull) * 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z = z ^ (z >> 31);
    return (float)(z >> 40) * (1.0f / 16777216.0f);
}

#define TW_SAMPLE_THREADS 1024
#define TW_SAMPLE_CLUSTER 8          // blocks that share a greedy row

// One block chooses the token of row r: the whole procedure of the file's head.
__device__ void sample_whole_row(int* __restrict__ out, const float* __restrict__ logits, int vocab,
                                 const float* __restrict__ temperature, const long long* __restrict__ seed,
                                 const long long* __restrict__ counter, int r) {
    __shared__ float sval[32];
    __shared__ int sidx[32];
    __shared__ float swarp[32];
    __shared__ float sbcast[2];
    __shared__ int sbest;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* x = logits + (size_t)r * vocab;
    const int chunk = (vocab + TW_SAMPLE_THREADS - 1) / TW_SAMPLE_THREADS;
    const int begin = tid * chunk, end = min(vocab, begin + chunk);

    // -- maximum and its lowest index: the threads stride over the row together (16 bytes each where the
    //    row allows), indices rise within a thread, and ties between threads go to the lower index
    float best = -INFINITY;
    int besti = 0x7fffffff;
    if ((vocab & 3) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
        const float4* x4 = reinterpret_cast<const float4*>(x);
        for (int v4 = tid; v4 < (vocab >> 2); v4 += TW_SAMPLE_THREADS) {
            const float4 f = x4[v4];
            if (f.x > best) { best = f.x; besti = 4 * v4; }
            if (f.y > best) { best = f.y; besti = 4 * v4 + 1; }
            if (f.z > best) { best = f.z; besti = 4 * v4 + 2; }
            if (f.w > best) { best = f.w; besti = 4 * v4 + 3; }
        }
    } else {
        for (int v = tid; v < vocab; v += TW_SAMPLE_THREADS) {
            const float f = x[v];
            if (f > best) { best = f; besti = v; }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, besti, o);
        if (ob > best || (ob == best && oi < besti)) { best = ob; besti = oi; }
    }
    if (lane == 0) { sval[warp] = best; sidx[warp] = besti; }
    __syncthreads();
    if (warp == 0) {
        best = sval[lane]; besti = sidx[lane];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, besti, o);
            if (ob > best || (ob == best && oi < besti)) { best = ob; besti = oi; }
        }
        if (lane == 0) { sbcast[0] = best; sbest = besti; }
    }
    __syncthreads();
    const float mx = sbcast[0];
    const float temp = temperature ? temperature[r] : 0.f;
    if (!(temp > 0.f)) {
        if (tid == 0) out[r] = sbest < vocab ? sbest : 0;
        return;
    }

    // -- running sums of e in index order: per-thread chunk sums, then a block scan
    float local = 0.f;
    for (int v = begin; v < end; ++v) local += expf((x[v] - mx) / temp);
    float incl = local;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float t = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += t;
    }
    if (lane == 31) swarp[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        float w = swarp[lane];
        float wi = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float t = __shfl_up_sync(0xffffffffu, wi, o);
            if (lane >= o) wi += t;
        }
        swarp[lane] = wi - w;  // exclusive prefix of the warp totals
        if (lane == 31) sbcast[1] = wi;
    }
    if (tid == 0) sbest = 0x7fffffff;
    __syncthreads();
    const float total = sbcast[1];
    const float u = tw_uniform((unsigned long long)seed[r], (unsigned long long)counter[r]);
    const float target = u * total;
    // Every thread walks its own chunk from its exclusive prefix; the lowest index at
    // which a running sum passes the target wins.
    float c = swarp[warp] + (incl - local);
    int cand = 0x7fffffff;
    for (int v = begin; v < end; ++v) {
        c += expf((x[v] - mx) / temp);
        if (c > target) { cand = v; break; }
    }
    if (cand != 0x7fffffff) atomicMin(&sbest, cand);
    __syncthreads();
    if (tid == 0) out[r] = sbest < vocab ? sbest : vocab - 1;
}

// Greedy rows are shared by a cluster of eight blocks: each finds the largest logit (lowest index at a tie) of its
// eighth of the row, sends it to the first block's shared memory, and that block takes the best of the eight
// (8 rows of 152,064 logits: 8.3 -> 3 us).  A row with a temperature is the first block's alone.
__global__ void __launch_bounds__(TW_SAMPLE_THREADS)
sample_kernel(int* __restrict__ out, const float* __restrict__ logits, int vocab,
              const float* __restrict__ temperature, const long long* __restrict__ seed,
              const long long* __restrict__ counter) {
    __shared__ float pval[32];
    __shared__ int pidx[32];
    __shared__ float cval[TW_SAMPLE_CLUSTER];
    __shared__ int cidx[TW_SAMPLE_CLUSTER];
    TW_TIMELINE_SCOPE(TW_K_SAMPLE);
    tw_grid_wait();
    TW_TIMELINE_MARK();
    tw_grid_launch_dependents();
    cg::cluster_group cluster = cg::this_cluster();
    const int rank = (int)cluster.block_rank();
    const int r = blockIdx.x / TW_SAMPLE_CLUSTER;
    const float temp = temperature ? temperature[r] : 0.f;
    if (temp > 0.f) {                      // the same for all blocks of the cluster: nobody waits at a barrier below
        if (rank == 0) sample_whole_row(out, logits, vocab, temperature, seed, counter, r);
        return;
    }
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* x = logits + (size_t)r * vocab;
    float best = -INFINITY;
    int besti = 0x7fffffff;
    if ((vocab & 3) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
        const float4* x4 = reinterpret_cast<const float4*>(x);
        const int n4 = vocab >> 2, per = (n4 + TW_SAMPLE_CLUSTER - 1) / TW_SAMPLE_CLUSTER;
        const int lo = rank * per, hi = min(n4, lo + per);
        for (int v4 = lo + tid; v4 < hi; v4 += TW_SAMPLE_THREADS) {
            const float4 f = x4[v4];
            if (f.x > best) { best = f.x; besti = 4 * v4; }
            if (f.y > best) { best = f.y; besti = 4 * v4 + 1; }
            if (f.z > best) { best = f.z; besti = 4 * v4 + 2; }
            if (f.w > best) { best = f.w; besti = 4 * v4 + 3; }
        }
    } else {
        const int per = (vocab + TW_SAMPLE_CLUSTER - 1) / TW_SAMPLE_CLUSTER;
        const int lo = rank * per, hi = min(vocab, lo + per);
        for (int v = lo + tid; v < hi; v += TW_SAMPLE_THREADS) {
            const float f = x[v];
            if (f > best) { best = f; besti = v; }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, besti, o);
        if (ob > best || (ob == best && oi < besti)) { best = ob; besti = oi; }
    }
    if (lane == 0) { pval[warp] = best; pidx[warp] = besti; }
    __syncthreads();
    if (warp == 0) {
        best = pval[lane]; besti = pidx[lane];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, besti, o);
            if (ob > best || (ob == best && oi < besti)) { best = ob; besti = oi; }
        }
        if (lane == 0) {
            *cluster.map_shared_rank(&cval[rank], 0) = best;
            *cluster.map_shared_rank(&cidx[rank], 0) = besti;
        }
    }
    cluster.sync();
    if (rank == 0 && tid == 0) {
        best = cval[0]; besti = cidx[0];
#pragma unroll
        for (int k = 1; k < TW_SAMPLE_CLUSTER; ++k)
            if (cval[k] > best || (cval[k] == best && cidx[k] < besti)) { best = cval[k]; besti = cidx[k]; }
        out[r] = besti < vocab ? besti : 0;
    }
}

// temperature, seed and counter may be null: every row is then greedy.
TW_EXPORT int tw_sample(int* out, const float* logits, int n_rows, int vocab, const float* temperature,
                        const long long* seed, const long long* counter, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (vocab <= 0) return (int)cudaErrorInvalidValue;
    tw_launch(sample_kernel, dim3(n_rows * TW_SAMPLE_CLUSTER), dim3(TW_SAMPLE_THREADS), 0, stream, TW_SAMPLE_CLUSTER, out, logits,
              vocab, temperature, seed, counter);
    return TW_LAUNCH_CHECK();
}

// Host-side copy of the uniform, for tools that want to predict a draw.
TW_EXPORT float tw_uniform_host(unsigned long long seed, unsigned long long counter) {
    return tw_uniform(seed, counter);
}
