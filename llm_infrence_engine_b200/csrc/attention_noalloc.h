/* Paged attention for callers that must not allocate device memory.
 *
 * This entry point has no counterpart in the reference project (which has no kernels of its own
 * at all); it exists for users of this library.
 *
 * Some callers cannot call cudaMalloc, directly or through a framework's allocator: code that runs
 * inside a host whose memory budget is fixed at start-up and fully handed out, plugin or callback
 * contexts in which allocation calls are forbidden or may deadlock against the host's own allocator
 * lock, and processes that have already given every free byte of the device to a cache pool. The
 * ordinary entry points llmie_paged_attention_f32 / _bf16 need scratch memory from the caller when
 * the keys are cut into several slices (num_splits > 1). This variant brings its own: a fixed array
 * that is part of the library's image on the device.
 *
 * What that costs and how it behaves:
 *  - The array holds LLMIE_NOALLOC_SCRATCH_FLOATS floats (8 MiB). Every GPU on which the library is
 *    loaded holds these bytes from load until the process exits, whether or not this function is
 *    ever called.
 *  - A call needs tokens * num_heads * num_splits * (head_dim + 2) floats. A call that needs more
 *    is refused with LLMIE_ERR_SCRATCH_TOO_SMALL and launches nothing; use fewer splits or fewer
 *    tokens per call. llmie_noalloc_error_string() turns the code into a sentence.
 *  - The first call on each device looks up the array's device address (cudaGetSymbolAddress, with
 *    that device current) and remembers it. Make that first call before any stream capture begins.
 *  - All calls share the one array, and it keeps what the last call left there. Nothing in it has to
 *    start at zero: every (token, head, slice) cell that the merge step reads is written by the
 *    slice's own block first, empty slices included. Two calls that overlap in time on the same
 *    GPU (different streams, or different host threads) race on the array and give wrong results;
 *    order them on one stream or with events.
 *  - Inputs and outputs are the caller's, exactly as for the ordinary entry points. The function
 *    calls no cudaMalloc, cudaFree or other allocating routine.
 *
 * dtype: 0 = float32, 1 = bfloat16 (q, pools and out share it). All other arguments as
 * llmie_paged_attention_f32 / _bf16. Returns 0, a CUDA error code, or one of the codes below.
 */
#pragma once
#include <cuda_runtime.h>

#define LLMIE_NOALLOC_SCRATCH_FLOATS (2u * 1024u * 1024u)
#define LLMIE_ERR_SCRATCH_TOO_SMALL 100002
#define LLMIE_ERR_SCRATCH_SETUP 100003

#ifdef __cplusplus
extern "C" {
#endif

int llmie_paged_attention_noalloc(const void* q, int q_stride, const void* k_pool, const void* v_pool, const int* block_table,
                                  int max_blocks, const int* token_seq, const int* positions, void* out, int num_tokens,
                                  int num_heads, int num_kv_heads, int head_dim, int page_size, float scale, int window,
                                  int num_splits, int dtype, cudaStream_t stream);

/* A sentence for a code returned by llmie_paged_attention_noalloc (static storage, never NULL). */
const char* llmie_noalloc_error_string(int code);

#ifdef __cplusplus
}
#endif
