// The allocation-free variant of paged attention: same kernels, scratch in a fixed device array.
// See attention_noalloc.h for who needs this and what the limits are.
#include <mutex>

#include "attention_generic.cuh"
#include "attention_noalloc.h"

namespace {

// Part of the library's device image: present on every GPU that loads the library, until exit.
static __device__ __align__(256) float g_noalloc_scratch[LLMIE_NOALLOC_SCRATCH_FLOATS];

constexpr int MAX_DEVICES = 64;
std::mutex g_setup_lock;
float* g_scratch_address[MAX_DEVICES] = {};  // device address of the array, per device, looked up once

// In host code `g_noalloc_scratch` is only a handle for the runtime, not an address a kernel could
// use; the address on the current device comes from cudaGetSymbolAddress.
int scratch_for_current_device(float** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= MAX_DEVICES) return LLMIE_ERR_SCRATCH_SETUP;
    std::lock_guard<std::mutex> hold(g_setup_lock);
    if (!g_scratch_address[dev]) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess) return (int)e;
        if (!p) return LLMIE_ERR_SCRATCH_SETUP;
        g_scratch_address[dev] = static_cast<float*>(p);
    }
    *out = g_scratch_address[dev];
    return 0;
}

}  // namespace

LLMIE_API int llmie_paged_attention_noalloc(const void* q, int q_stride, const void* k_pool, const void* v_pool,
                                            const int* block_table, int max_blocks, const int* token_seq, const int* positions,
                                            void* out, int num_tokens, int num_heads, int num_kv_heads, int head_dim, int page_size,
                                            float scale, int window, int num_splits, int dtype, cudaStream_t stream) {
    if (num_tokens <= 0) return 0;
    if (num_heads <= 0 || head_dim <= 0 || num_splits < 1 || (dtype != DT_F32 && dtype != DT_BF16)) return LLMIE_ERR_BAD_ARGUMENT;
    const size_t need = attn_generic::scratch_floats(num_tokens, num_heads, head_dim, num_splits);
    if (num_splits > 1 && need > (size_t)LLMIE_NOALLOC_SCRATCH_FLOATS) return LLMIE_ERR_SCRATCH_TOO_SMALL;
    float* scratch = nullptr;
    const int rc = scratch_for_current_device(&scratch);
    if (rc) return rc;
    if (dtype == DT_F32)
        return attn_generic::paged_attention<float>((const float*)q, q_stride, (const float*)k_pool, (const float*)v_pool, block_table,
                                                    max_blocks, token_seq, positions, (float*)out, scratch, num_tokens, num_heads,
                                                    num_kv_heads, head_dim, page_size, scale, window, num_splits, 0, stream);
    return attn_generic::paged_attention<bf16>((const bf16*)q, q_stride, (const bf16*)k_pool, (const bf16*)v_pool, block_table,
                                               max_blocks, token_seq, positions, (bf16*)out, scratch, num_tokens, num_heads,
                                               num_kv_heads, head_dim, page_size, scale, window, num_splits, 0, stream);
}

LLMIE_API const char* llmie_noalloc_error_string(int code) {
    switch (code) {
        case 0: return "no error";
        case LLMIE_ERR_BAD_ARGUMENT: return "an argument is outside what the attention kernel accepts (head sizes, head counts, splits or dtype)";
        case LLMIE_ERR_SCRATCH_TOO_SMALL:
            return "tokens * num_heads * num_splits * (head_dim + 2) exceeds the fixed scratch array of 2,097,152 floats; "
                   "use fewer splits or fewer tokens per call";
        case LLMIE_ERR_SCRATCH_SETUP: return "the device address of the fixed scratch array could not be looked up on the current device";
        default: return cudaGetErrorString((cudaError_t)code);
    }
}
