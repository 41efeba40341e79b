// bfloat16 instantiation of the generic paged attention (any head size and group; 32-bit arithmetic).
#include "attention_generic.cuh"

LLMIE_API int llmie_paged_attention_bf16(const bf16* q, int q_stride, const bf16* k_pool, const bf16* v_pool,
                                         const int* block_table, int max_blocks, const int* token_seq, const int* positions,
                                         bf16* out, float* scratch, int N, int nq, int nkv, int d, int page_size, float scale,
                                         int window, int num_splits, int slice_keys, cudaStream_t s) {
    return attn_generic::paged_attention<bf16>(q, q_stride, k_pool, v_pool, block_table, max_blocks, token_seq, positions, out,
                                               scratch, N, nq, nkv, d, page_size, scale, window, num_splits, slice_keys, s);
}
