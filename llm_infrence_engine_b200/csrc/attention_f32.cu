// float32 instantiation of the generic paged attention (the true 32-bit path).
#include "attention_generic.cuh"

LLMIE_API int llmie_paged_attention_f32(const float* q, int q_stride, const float* k_pool, const float* v_pool,
                                        const int* block_table, int max_blocks, const int* token_seq, const int* positions,
                                        float* out, float* scratch, int N, int nq, int nkv, int d, int page_size, float scale,
                                        int window, int num_splits, int slice_keys, cudaStream_t s) {
    return attn_generic::paged_attention<float>(q, q_stride, k_pool, v_pool, block_table, max_blocks, token_seq, positions, out,
                                                scratch, N, nq, nkv, d, page_size, scale, window, num_splits, slice_keys, s);
}
