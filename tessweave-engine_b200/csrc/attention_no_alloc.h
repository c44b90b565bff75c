// Split-KV decode attention for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference project; it exists for users of this
// library only.  Some callers cannot call cudaMalloc at the moment they need attention: a
// serving loop with a latency bound, because cudaMalloc and cudaFree synchronise the whole
// device and stall every stream; an application that hands each component a fixed memory budget
// at start-up and forbids allocation afterwards; a plug-in inside a host program that owns all
// device memory and gives none away at run time.  The ordinary entry point (tw_attn_decode)
// asks its caller for a scratch buffer and a counter array, which such a caller would have to
// allocate.  tw_attn_decode_static keeps both in one
// array that is part of the library's device image instead, so calling it allocates nothing,
// neither directly nor through any library.
//
// What to know before using it:
//   * The array is TW_ATTN_STATIC_SCRATCH_BYTES (8 MiB) per loaded library and GPU, held from
//     the moment the library is loaded on that GPU until the process exits.
//   * A call needs 4 * n_seqs * n_q_heads * nsplit * (head_dim + 2) bytes of it for partial
//     results plus 64 KiB for counters.  A call that needs more is refused with
//     TW_ATTN_STATIC_TOO_LARGE before anything is launched; tw_attn_decode_static_last_error()
//     then says how many bytes were asked for and how many there are.  Lower nsplit, or use
//     tw_attn_decode with a buffer of your own.
//   * The first call on each GPU looks up the array's device address (cudaGetSymbolAddress,
//     with that GPU current).  Make that first call outside of any stream capture.
//   * Every call uses the same array and finds in it what the previous call left.  The
//     counters, which must start at zero, are cleared on the stream at the start of every
//     call; nothing else needs a defined start.  Two calls that run on the GPU at the same
//     time (different streams, or different threads without ordering) race on the array and
//     give wrong results: order them on one stream or with events.
//   * nsplit is at most 128 (tw_attn_decode_max_splits()), q must be 16-byte aligned and q_stride a
//     multiple of 8 elements: the kernel reads the query 16 bytes at a time.  Other values are refused
//     with cudaErrorInvalidValue / cudaErrorMisalignedAddress before anything is launched.
//   * Inputs and outputs are passed exactly as to tw_attn_decode (see attention_bf16.cu);
//     only `scratch` and `counters` are gone.  The head size is the one the library was
//     compiled for (tw_attn_head_dim()).
#pragma once

#include <cuda_runtime.h>

#define TW_ATTN_STATIC_SCRATCH_BYTES (8u << 20)
#define TW_ATTN_STATIC_COUNTER_BYTES (64u << 10)
#define TW_ATTN_STATIC_TOO_LARGE (-2)     // the call needs more scratch than the static array holds
#define TW_ATTN_STATIC_NO_SYMBOL (-3)     // the array's device address could not be looked up

#ifdef __cplusplus
extern "C" {
#endif

// Returns 0, a CUDA error code (> 0), or one of the negative codes above.
int tw_attn_decode_static(void* out, int out_stride, const void* q, int q_stride, const int* seq_q_start,
                          const int* seq_q_len, const int* seq_kv_len, const int* seq_slot, const int* block_table,
                          int table_stride, const void* k_cache, const void* v_cache, int n_seqs, int Hq, int Hkv,
                          int page_size, int num_pages, int window, float scale, int nsplit, int* status,
                          cudaStream_t stream);

// Text of the last refusal of tw_attn_decode_static in this thread ("" if there was none).
const char* tw_attn_decode_static_last_error(void);

#ifdef __cplusplus
}
#endif
