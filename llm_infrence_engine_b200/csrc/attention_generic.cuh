// Grouped-query attention of single tokens over a paged cache, for any mix of prompt portions and
// decoded tokens, in float32 or bfloat16 storage with all arithmetic in 32-bit.
//
// One block serves one token, one key/value head and up to GC of the query heads that share it,
// over one slice of the token's keys (split-KV): grid = (tokens, kv heads * head chunks, splits).
// A token at position p of request r reads keys max(0, p - window + 1) .. p through r's row of the
// block table; its own key is already in the cache (the rotation kernel wrote it), so prompt
// portions, decoded tokens and any way of cutting take the same path. Each of the four warps
// walks 32 keys at a time: lane j scores key j against the GC queries (the key row is read once for
// all of them), the warp does one online-softmax update, then every lane accumulates its own
// dimensions of the value rows. The warps are merged in shared memory; with one split the block
// writes the output row, otherwise its partial (max, sum, accumulator) goes to scratch memory and
// `attn_combine_kernel` merges the splits.
#pragma once
#include <math.h>

#include "common.cuh"

namespace attn_generic {

constexpr int WARPS = 4;

template <typename T, int DPL, int GC>
__global__ void __launch_bounds__(WARPS * 32) paged_attn_kernel(
    const T* __restrict__ q, int q_stride, const T* __restrict__ k_pool, const T* __restrict__ v_pool,
    const int* __restrict__ block_table, int max_blocks, const int* __restrict__ token_seq, const int* __restrict__ positions,
    T* __restrict__ out, float* __restrict__ part_acc, float* __restrict__ part_ml, int nq, int nkv, int d, int page_size,
    float scale, int window, int num_splits, int slice_keys) {
    constexpr int DMAX = DPL * 32;
    __shared__ float qs[GC][DMAX];
    __shared__ float ps[WARPS][GC][32];
    __shared__ float acc_s[WARPS][GC][DMAX];
    __shared__ float m_s[WARPS][GC], l_s[WARPS][GC];

    const int n = blockIdx.x;
    const int G = nq / nkv;
    const int chunks = (G + GC - 1) / GC;
    const int kvh = blockIdx.y / chunks;
    const int g0 = (blockIdx.y % chunks) * GC;
    const int ng = min(GC, G - g0);
    const int split = blockIdx.z;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

    const int p = positions[n];
    const int lo = window > 0 ? max(0, p - window + 1) : 0;
    const int hi = p + 1;
    // Two ways of cutting the keys into slices. `slice_keys` > 0: slice s holds the keys [s * slice_keys, (s + 1) * slice_keys)
    // of the request, whatever else is in the batch and however many slices are launched (slices beyond the token's
    // position are empty), so a token's arithmetic, and with it every bit of its result, depends on its own position
    // alone. Otherwise the token's visible keys are cut into `num_splits` equal runs.
    int start, end;
    if (slice_keys > 0) {
        start = split * slice_keys;
        end = min(hi, start + slice_keys);
    } else {
        int per = (hi - lo + num_splits - 1) / num_splits;
        per = (per + 31) & ~31;
        start = lo + split * per;
        end = min(hi, start + per);
    }
    const int* table = block_table + (size_t)token_seq[n] * max_blocks;

    for (int i = threadIdx.x; i < GC * DMAX; i += blockDim.x) {
        const int g = i / DMAX, c = i % DMAX;
        float v = 0.f;
        if (g < ng && c < d) v = to_f32(q[(size_t)n * q_stride + (size_t)(kvh * G + g0 + g) * d + c]) * scale;
        qs[g][c] = v;
    }
    __syncthreads();

    float m[GC], l[GC], acc[GC][DPL];
#pragma unroll
    for (int g = 0; g < GC; ++g) {
        m[g] = -INFINITY;
        l[g] = 0.f;
#pragma unroll
        for (int i = 0; i < DPL; ++i) acc[g][i] = 0.f;
    }

    constexpr int VN = Vec16<T>::N;
    for (int base = start + warp * 32; base < end; base += WARPS * 32) {
        if (base + 32 <= lo) continue;  // (absolute slices only) every key of the chunk lies before the window
        const int key = base + lane;
        const bool valid = key < end && key >= lo;
        int row = 0;
        float s[GC];
#pragma unroll
        for (int g = 0; g < GC; ++g) s[g] = 0.f;
        if (valid) {
            const int blk = table[key / page_size];
            row = (blk * nkv + kvh) * page_size + key % page_size;
            const T* kr = k_pool + (size_t)row * d;
            for (int c = 0; c < d; c += VN) {
                float kf[VN];
                Vec16<T>::load(kr + c, kf);
#pragma unroll
                for (int g = 0; g < GC; ++g)
#pragma unroll
                    for (int i = 0; i < VN; ++i) s[g] = fmaf(qs[g][c + i], kf[i], s[g]);
            }
        }
        float corr[GC];
#pragma unroll
        for (int g = 0; g < GC; ++g) {
            const float sv = valid ? s[g] : -INFINITY;
            const float m_new = fmaxf(m[g], warp_max(sv));
            const float pv = valid ? expf(sv - m_new) : 0.f;
            corr[g] = expf(m[g] - m_new);
            l[g] = l[g] * corr[g] + warp_sum(pv);
            m[g] = m_new;
            ps[warp][g][lane] = pv;
        }
        __syncwarp();
#pragma unroll
        for (int g = 0; g < GC; ++g)
#pragma unroll
            for (int i = 0; i < DPL; ++i) acc[g][i] *= corr[g];
        const int count = min(32, end - base);
        for (int j = max(0, lo - base); j < count; ++j) {
            const int rj = __shfl_sync(0xffffffffu, row, j);
            const T* vr = v_pool + (size_t)rj * d;
            float vv[DPL];
#pragma unroll
            for (int i = 0; i < DPL; ++i) {
                const int dim = lane + 32 * i;
                vv[i] = dim < d ? to_f32(vr[dim]) : 0.f;
            }
#pragma unroll
            for (int g = 0; g < GC; ++g) {
                const float pj = ps[warp][g][j];
#pragma unroll
                for (int i = 0; i < DPL; ++i) acc[g][i] = fmaf(pj, vv[i], acc[g][i]);
            }
        }
        __syncwarp();
    }

#pragma unroll
    for (int g = 0; g < GC; ++g) {
        if (lane == 0) { m_s[warp][g] = m[g]; l_s[warp][g] = l[g]; }
#pragma unroll
        for (int i = 0; i < DPL; ++i) acc_s[warp][g][lane + 32 * i] = acc[g][i];
    }
    __syncthreads();

    for (int i = threadIdx.x; i < ng * d; i += blockDim.x) {
        const int g = i / d, dim = i % d;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) M = fmaxf(M, m_s[w][g]);
        float L = 0.f, A = 0.f;
        if (M > -INFINITY) {
#pragma unroll
            for (int w = 0; w < WARPS; ++w) {
                const float f = expf(m_s[w][g] - M);
                L = fmaf(l_s[w][g], f, L);
                A = fmaf(acc_s[w][g][dim], f, A);
            }
        }
        const int head = kvh * G + g0 + g;
        if (num_splits == 1) {
            out[(size_t)n * nq * d + (size_t)head * d + dim] = from_f32<T>(A / L);
        } else {
            const size_t slot = ((size_t)n * nq + head) * num_splits + split;
            part_acc[slot * d + dim] = A;
            if (dim == 0) { part_ml[slot * 2] = M; part_ml[slot * 2 + 1] = L; }
        }
    }
}

// out[n, head, :] = sum_s acc_s e^(m_s - M) / sum_s l_s e^(m_s - M) over the splits of one (token, head).
template <typename T>
__global__ void attn_combine_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml, T* __restrict__ out,
                                    int d, int num_splits) {
    const size_t th = blockIdx.x;  // token * nq + head
    const float* ml = part_ml + th * num_splits * 2;
    float M = -INFINITY;
    for (int s = 0; s < num_splits; ++s) M = fmaxf(M, ml[2 * s]);
    float L = 0.f;
    for (int s = 0; s < num_splits; ++s) L = fmaf(ml[2 * s + 1], expf(ml[2 * s] - M), L);
    for (int dim = threadIdx.x; dim < d; dim += blockDim.x) {
        float A = 0.f;
        for (int s = 0; s < num_splits; ++s) A = fmaf(part_acc[(th * num_splits + s) * d + dim], expf(ml[2 * s] - M), A);
        out[th * d + dim] = from_f32<T>(A / L);
    }
}

template <typename T, int DPL>
int launch_gc(int GC, dim3 grid, cudaStream_t s, const T* q, int q_stride, const T* k_pool, const T* v_pool,
              const int* block_table, int max_blocks, const int* token_seq, const int* positions, T* out, float* part_acc,
              float* part_ml, int nq, int nkv, int d, int page_size, float scale, int window, int num_splits, int slice_keys) {
#define LLMIE_ATTN_LAUNCH(GCV)                                                                                              \
    paged_attn_kernel<T, DPL, GCV><<<grid, WARPS * 32, 0, s>>>(q, q_stride, k_pool, v_pool, block_table, max_blocks,          \
                                                               token_seq, positions, out, part_acc, part_ml, nq, nkv, d,     \
                                                               page_size, scale, window, num_splits, slice_keys)
    switch (GC) {
        case 1: LLMIE_ATTN_LAUNCH(1); break;
        case 2: LLMIE_ATTN_LAUNCH(2); break;
        case 4: LLMIE_ATTN_LAUNCH(4); break;
        default: LLMIE_ATTN_LAUNCH(8); break;
    }
#undef LLMIE_ATTN_LAUNCH
    return launch_status();
}

// Scratch needed for `num_splits` > 1, in floats: accumulators, then (max, sum) pairs.
inline size_t scratch_floats(int N, int nq, int d, int num_splits) {
    return (size_t)N * nq * num_splits * (d + 2);
}

template <typename T>
int paged_attention(const T* q, int q_stride, const T* k_pool, const T* v_pool, const int* block_table, int max_blocks,
                    const int* token_seq, const int* positions, T* out, float* scratch, int N, int nq, int nkv, int d,
                    int page_size, float scale, int window, int num_splits, int slice_keys, cudaStream_t s) {
    if (N <= 0) return 0;
    if (nkv <= 0 || nq % nkv || d <= 0 || d > 256 || d % Vec16<T>::N || page_size <= 0 || num_splits < 1 || slice_keys < 0 || slice_keys % 32 ||
        (num_splits > 1 && !scratch) || q_stride % Vec16<T>::N)
        return LLMIE_ERR_BAD_ARGUMENT;
    const int G = nq / nkv;
    const int GC = G >= 5 ? 8 : (G >= 3 ? 4 : G);
    const int chunks = (G + GC - 1) / GC;
    if ((long long)nkv * chunks > 65535 || num_splits > 65535) return LLMIE_ERR_BAD_ARGUMENT;
    const dim3 grid(N, nkv * chunks, num_splits);
    float* part_acc = scratch;
    float* part_ml = scratch ? scratch + (size_t)N * nq * num_splits * d : nullptr;
    int rc;
    if (d <= 32) rc = launch_gc<T, 1>(GC, grid, s, q, q_stride, k_pool, v_pool, block_table, max_blocks, token_seq, positions, out, part_acc, part_ml, nq, nkv, d, page_size, scale, window, num_splits, slice_keys);
    else if (d <= 64) rc = launch_gc<T, 2>(GC, grid, s, q, q_stride, k_pool, v_pool, block_table, max_blocks, token_seq, positions, out, part_acc, part_ml, nq, nkv, d, page_size, scale, window, num_splits, slice_keys);
    else if (d <= 128) rc = launch_gc<T, 4>(GC, grid, s, q, q_stride, k_pool, v_pool, block_table, max_blocks, token_seq, positions, out, part_acc, part_ml, nq, nkv, d, page_size, scale, window, num_splits, slice_keys);
    else rc = launch_gc<T, 8>(GC, grid, s, q, q_stride, k_pool, v_pool, block_table, max_blocks, token_seq, positions, out, part_acc, part_ml, nq, nkv, d, page_size, scale, window, num_splits, slice_keys);
    if (rc) return rc;
    if (num_splits > 1) {
        attn_combine_kernel<T><<<N * nq, 64, 0, s>>>(part_acc, part_ml, out, d, num_splits);
        rc = launch_status();
    }
    return rc;
}

}  // namespace attn_generic
