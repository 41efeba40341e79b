// Choosing the next token on the device: argmax, and temperature / top-k / top-p sampling.
//
// One block per row of float32 logits. The sampled distribution is: x = logit / temperature; keep
// x >= the k-th largest x (ties kept); in descending order drop a token once the mass before it
// reaches top_p; softmax over what is left. The token drawn for the uniform number u is the first
// one, in index order, whose running mass exceeds u * total mass.
//
// No sort is needed for either threshold. Logits map to 32-bit keys that order like the floats;
// the k-th largest key is found by a 4-pass radix select, and the top-p threshold is the smallest
// key t with mass(keys > t) < top_p * total, found bit by bit (32 passes, each a masked sum over the
// row, which sits in L2 by then).
#include <math.h>

#include "common.cuh"

namespace {

constexpr int THREADS = 1024;

__device__ __forceinline__ uint32_t order_key(float x) {
    const uint32_t b = __float_as_uint(x);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__device__ __forceinline__ double block_sum_f64(double v, double* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        double t = lane < (THREADS >> 5) ? scratch[lane] : 0.0;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

// Lowest index among the largest values. Stage 1: grid (parts, rows), each block scans one slice of a row and
// writes its best (value, index) to `part`; stage 2: one block per row picks among the parts.
constexpr int ARG_THREADS = 256;

__device__ __forceinline__ void arg_better(float& best, int& idx, float ov, int oi) {
    if (oi >= 0 && (idx < 0 || ov > best || (ov == best && oi < idx))) { best = ov; idx = oi; }
}

__device__ __forceinline__ void arg_block_reduce(float& best, int& idx) {
    __shared__ float bv[ARG_THREADS / 32];
    __shared__ int bi[ARG_THREADS / 32];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) arg_better(best, idx, __shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, idx, o));
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { bv[warp] = best; bi[warp] = idx; }
    __syncthreads();
    if (warp == 0) {
        best = lane < ARG_THREADS / 32 ? bv[lane] : 0.f;
        idx = lane < ARG_THREADS / 32 ? bi[lane] : -1;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) arg_better(best, idx, __shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, idx, o));
    }
}

__global__ void __launch_bounds__(ARG_THREADS) argmax_part_kernel(const float* __restrict__ logits, float* __restrict__ part_v,
                                                                 int* __restrict__ part_i, int V, int per) {
    pdl_trigger();
    pdl_wait();
    const float* x = logits + (size_t)blockIdx.y * V;
    const int lo = blockIdx.x * per, hi = min(V, lo + per);
    float best = 0.f;
    int idx = -1;
    for (int i = lo + threadIdx.x; i < hi; i += ARG_THREADS) arg_better(best, idx, x[i], i);
    arg_block_reduce(best, idx);
    if (threadIdx.x == 0) { part_v[blockIdx.y * gridDim.x + blockIdx.x] = best; part_i[blockIdx.y * gridDim.x + blockIdx.x] = idx; }
}

__global__ void __launch_bounds__(ARG_THREADS) argmax_final_kernel(const float* __restrict__ part_v, const int* __restrict__ part_i,
                                                                  int* __restrict__ out, int parts) {
    pdl_trigger();
    pdl_wait();
    float best = 0.f;
    int idx = -1;
    for (int i = threadIdx.x; i < parts; i += ARG_THREADS) arg_better(best, idx, part_v[blockIdx.x * parts + i], part_i[blockIdx.x * parts + i]);
    arg_block_reduce(best, idx);
    if (threadIdx.x == 0) out[blockIdx.x] = idx < 0 ? 0 : idx;
}

__global__ void __launch_bounds__(THREADS) sample_kernel(const float* __restrict__ logits, const float* __restrict__ temperature,
                                                        const int* __restrict__ top_k, const float* __restrict__ top_p,
                                                        const float* __restrict__ uniform, int* __restrict__ out, int V) {
    __shared__ double red[33];
    __shared__ float redf[33];
    __shared__ unsigned int hist[256];
    __shared__ unsigned int sel_prefix, sel_remaining;
    __shared__ double chunk_sum[THREADS];
    __shared__ int winner;

    const int row = blockIdx.x;
    const float* x = logits + (size_t)row * V;
    const float temp = temperature[row];
    const int tid = threadIdx.x;

    if (!(temp > 0.f)) {  // greedy row inside a sampled batch: lowest index among the largest
        float best = -INFINITY;
        int idx = V;
        for (int i = tid; i < V; i += THREADS) {
            const float v = x[i];
            if (v > best || (v == best && i < idx) || idx == V) { best = v; idx = i; }
        }
        // reduce through shared memory, simplest form
        __shared__ float sv[THREADS];
        __shared__ int si[THREADS];
        sv[tid] = best; si[tid] = idx;
        __syncthreads();
        for (int o = THREADS / 2; o > 0; o >>= 1) {
            if (tid < o) {
                const float ov = sv[tid + o]; const int oi = si[tid + o];
                if (oi < V && (si[tid] >= V || ov > sv[tid] || (ov == sv[tid] && oi < si[tid]))) { sv[tid] = ov; si[tid] = oi; }
            }
            __syncthreads();
        }
        if (tid == 0) out[row] = si[0] < V ? si[0] : 0;
        return;
    }

    // ---- top-k: the key of the k-th largest scaled logit (0 keeps everything)
    uint32_t min_key = 0;
    const int k = top_k[row];
    if (k > 0 && k < V) {
        if (tid == 0) { sel_prefix = 0; sel_remaining = (unsigned)k; }
        __syncthreads();
        for (int shift = 24; shift >= 0; shift -= 8) {
            for (int i = tid; i < 256; i += THREADS) hist[i] = 0;
            __syncthreads();
            const uint32_t prefix = sel_prefix;
            const uint32_t mask = shift == 24 ? 0u : (0xffffffffu << (shift + 8));
            for (int i = tid; i < V; i += THREADS) {
                const uint32_t key = order_key(x[i] / temp);
                if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1u);
            }
            __syncthreads();
            if (tid == 0) {
                unsigned rem = sel_remaining;
                int b = 255;
                for (; b > 0; --b) {
                    if (hist[b] >= rem) break;
                    rem -= hist[b];
                }
                sel_prefix = prefix | ((uint32_t)b << shift);
                sel_remaining = rem;
            }
            __syncthreads();
        }
        min_key = sel_prefix;
    }

    // ---- maximum and total mass of the kept set
    float mx = -INFINITY;
    for (int i = tid; i < V; i += THREADS) {
        const float v = x[i] / temp;
        if (order_key(v) >= min_key) mx = fmaxf(mx, v);
    }
    mx = warp_max(mx);
    __syncthreads();
    if ((tid & 31) == 0) redf[tid >> 5] = mx;
    __syncthreads();
    if (tid < 32) {
        float t = redf[tid];
        t = warp_max(t);
        if (tid == 0) redf[32] = t;
    }
    __syncthreads();
    mx = redf[32];

    double part = 0.0;
    for (int i = tid; i < V; i += THREADS) {
        const float v = x[i] / temp;
        if (order_key(v) >= min_key) part += (double)expf(v - mx);
    }
    double total = block_sum_f64(part, red);

    // ---- top-p: smallest key t with mass(keys > t) < top_p * total; tokens with key >= t stay
    const float tp = top_p[row];
    if (tp < 1.0f) {
        const double limit = (double)tp * total;
        uint32_t t = 0;
        for (int bit = 31; bit >= 0; --bit) {
            const uint32_t cand = t | ((1u << bit) - 1u);  // this bit 0, everything below 1
            double above = 0.0;
            for (int i = tid; i < V; i += THREADS) {
                const float v = x[i] / temp;
                const uint32_t key = order_key(v);
                if (key >= min_key && key > cand) above += (double)expf(v - mx);
            }
            above = block_sum_f64(above, red);
            if (!(above < limit)) t |= (1u << bit);
        }
        if (t > min_key) min_key = t;
        part = 0.0;
        for (int i = tid; i < V; i += THREADS) {
            const float v = x[i] / temp;
            if (order_key(v) >= min_key) part += (double)expf(v - mx);
        }
        total = block_sum_f64(part, red);
    }

    // ---- the draw: each thread owns a run of consecutive tokens
    const int per = (V + THREADS - 1) / THREADS;
    const int lo = min(V, tid * per), hi = min(V, lo + per);
    double mine = 0.0;
    for (int i = lo; i < hi; ++i) {
        const float v = x[i] / temp;
        if (order_key(v) >= min_key) mine += (double)expf(v - mx);
    }
    chunk_sum[tid] = mine;
    if (tid == 0) winner = -1;
    __syncthreads();
    if (tid == 0) {
        const double target = (double)uniform[row] * total;
        double run = 0.0;
        int w = -1, last = -1;
        for (int c = 0; c < THREADS; ++c) {
            if (chunk_sum[c] > 0.0) last = c;
            if (run + chunk_sum[c] > target) { w = c; break; }
            run += chunk_sum[c];
        }
        if (w < 0) { w = last; run = -1.0; }  // rounding left u * total at or past the end: the last kept token
        winner = w;
        red[0] = run;
        red[1] = target;
    }
    __syncthreads();
    if (tid == winner) {
        double run = red[0];
        const double target = red[1];
        int pick = -1, last_kept = -1;
        for (int i = lo; i < hi; ++i) {
            const float v = x[i] / temp;
            if (order_key(v) < min_key) continue;
            last_kept = i;
            if (run >= 0.0) {
                run += (double)expf(v - mx);
                if (run > target) { pick = i; break; }
            }
        }
        out[row] = pick >= 0 ? pick : (last_kept >= 0 ? last_kept : 0);
    }
}

}  // namespace

// `part_v` / `part_i`: scratch of M * ARGMAX_PARTS floats / ints.
LLMIE_API int llmie_argmax(const float* logits, int* out, float* part_v, int* part_i, int M, int V, cudaStream_t s) {
    if (M <= 0) return 0;
    if (V <= 0 || M > 65535) return LLMIE_ERR_BAD_ARGUMENT;
    const int parts = 64;
    const int per = (V + parts - 1) / parts;
    int rc = launch_kernel(argmax_part_kernel, dim3(parts, M), dim3(ARG_THREADS), 0, s, logits, part_v, part_i, V, per);
    if (rc) return rc;
    return launch_kernel(argmax_final_kernel, dim3(M), dim3(ARG_THREADS), 0, s, (const float*)part_v, (const int*)part_i, out, parts);
}

LLMIE_API int llmie_sample(const float* logits, const float* temperature, const int* top_k, const float* top_p,
                           const float* uniform, int* out, int M, int V, cudaStream_t s) {
    if (M <= 0) return 0;
    if (V <= 0) return LLMIE_ERR_BAD_ARGUMENT;
    sample_kernel<<<M, THREADS, 0, s>>>(logits, temperature, top_k, top_p, uniform, out, V);
    return launch_status();
}
