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

// ------------------------------------------------------------------------------------------------
// The same distribution and the same draw as sample_kernel, for a thread-block CLUSTER per row. Each block of the cluster
// keeps its slice of the row (already divided by the temperature) in shared memory, so every pass after the first reads
// shared memory, and what the blocks must tell each other (histograms, maxima, masses) crosses through the cluster's
// distributed shared memory at a cluster barrier. Both thresholds come from a radix descent over the 32-bit keys, one byte
// per pass: the k-th largest key from histograms of counts, the top-p threshold from histograms of MASS (the smallest key t
// with mass(keys > t) < top_p * total has, byte by byte from the top, the smallest byte for which the mass above still stays
// below the limit). Four passes each where the single-block kernel needs 4 and 32 passes over global memory.
//
// Masses in the histograms are fixed-point integers (e^(x - max) * 2^40): sums of integers do not depend on the order of the
// additions, so every block of the cluster and every run arrive at the same threshold. A token below 2^-41 of the largest
// probability counts as nothing there (all of them together: below 1e-7 of the total); the draw itself adds up doubles.
constexpr int CL_THREADS = 512, CL_MAX = 8, CL_MAX_SLICE = 24576;  // floats of a slice: 96 KB of shared memory, two blocks per SM
constexpr double MASS_ONE = 1099511627776.0;                      // 2^40
static_assert(CL_THREADS == 512, "a histogram's 512 words are cleared by one thread each");

__device__ __forceinline__ uint32_t cluster_rank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r)); return r; }
__device__ __forceinline__ void cluster_barrier() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
__device__ __forceinline__ uint32_t peer_address(const void* own, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(r) : "r"((uint32_t)__cvta_generic_to_shared(own)), "r"(rank));
    return r;
}
__device__ __forceinline__ uint32_t peer_u32(const void* own, uint32_t rank) {
    uint32_t v; asm volatile("ld.shared::cluster.u32 %0, [%1];\n" : "=r"(v) : "r"(peer_address(own, rank)) : "memory"); return v;
}
__device__ __forceinline__ float peer_f32(const void* own, uint32_t rank) {
    float v; asm volatile("ld.shared::cluster.f32 %0, [%1];\n" : "=f"(v) : "r"(peer_address(own, rank)) : "memory"); return v;
}
__device__ __forceinline__ double peer_f64(const void* own, uint32_t rank) {
    double v; asm volatile("ld.shared::cluster.f64 %0, [%1];\n" : "=d"(v) : "r"(peer_address(own, rank)) : "memory"); return v;
}
__device__ __forceinline__ unsigned long long shfl_u64(unsigned long long v, int src) {
    return ((unsigned long long)__shfl_sync(0xffffffffu, (unsigned)(v >> 32), src) << 32) | __shfl_sync(0xffffffffu, (unsigned)v, src);
}
__device__ __forceinline__ unsigned long long mass_units(float v, float mx) { return (unsigned long long)((double)expf(v - mx) * MASS_ONE); }

// One warp: in a histogram g[256], going down from bucket 255, the first bucket at which the sum of the buckets so far (this
// one included) reaches `threshold`, or bucket 0; and the sum of the buckets above it. Lane i owns buckets 255 - 8 i .. 248 - 8 i.
__device__ __forceinline__ void first_bucket_reaching(const unsigned long long* g, unsigned long long threshold, int lane, int& bucket,
                                                      unsigned long long& above) {
    unsigned long long mine = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) mine += g[255 - 8 * lane - i];
    unsigned long long incl = mine;   // the sum over lanes 0 .. lane
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const unsigned long long up = shfl_u64(incl, max(lane - o, 0));
        if (lane >= o) incl += up;
    }
    const unsigned int reached = __ballot_sync(0xffffffffu, incl >= threshold);
    const int at = reached ? __ffs(reached) - 1 : 31;
    unsigned long long run = shfl_u64(incl - mine, at);   // the sum above the lane's first bucket
    int b = 255 - 8 * at;
    if (lane == at) {
        const int lowest = reached ? b - 7 : 0;
        while (b > lowest && run + g[b] < threshold) { run += g[b]; --b; }
    }
    bucket = __shfl_sync(0xffffffffu, b, at);
    above = shfl_u64(run, at);
}

__global__ void __launch_bounds__(CL_THREADS, 2) sample_cluster_kernel(const float* __restrict__ logits, const float* __restrict__ temperature,
                                                                      const int* __restrict__ top_k, const float* __restrict__ top_p,
                                                                      const float* __restrict__ uniform, int* __restrict__ out, int V, int C, int slice) {
    extern __shared__ float xs[];                 // [slice] this block's part of the row, divided by the temperature
    __shared__ unsigned int hist[2][512];         // a histogram of counts or of masses (256 low words, 256 high words): two sets,
                                                  //   taken in turn, so that a block that is a pass ahead does not clear what a
                                                  //   slower block still reads
    __shared__ unsigned long long gsum[256];      // a histogram added up over the cluster
    __shared__ double red[CL_THREADS / 32];
    __shared__ double slot_d;                     // what this block tells the others: a mass ...
    __shared__ unsigned int slot_m[2];            // ... a mass in fixed-point units (low word, high word) ...
    __shared__ float slot_f;                      // ... a maximum ...
    __shared__ int slot_i;                        // ... an index
    __shared__ unsigned int sel_prefix;
    __shared__ unsigned long long sel_remaining;  // top-k: how many of the bucket are still wanted; top-p: the mass above the prefix
    __shared__ int first_over, last_with_any;
    __shared__ float wv[CL_THREADS / 32];
    __shared__ int wi[CL_THREADS / 32];
    pdl_trigger();
    pdl_wait();

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t rank = cluster_rank();
    const int row = blockIdx.x / C;
    const float* x = logits + (size_t)row * V;
    const int lo = min(V, (int)rank * slice), n = min(V, lo + slice) - lo;   // this block's tokens: [lo, lo + n)
    const float temp = temperature[row];
    const bool greedy = !(temp > 0.f);

    // the slice into shared memory, and on the way its largest value with the lowest index that has it (the maximum of the
    // kept set whatever top-k and top-p keep: both keep the largest)
    float best = -INFINITY;
    int idx = -1;
    for (int j = tid; j < n; j += CL_THREADS) {
        const float v = greedy ? x[lo + j] : x[lo + j] / temp;
        xs[j] = v;
        if (idx < 0 || v > best) { best = v; idx = lo + j; }   // (a thread meets its indices in rising order)
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (oi >= 0 && (idx < 0 || ov > best || (ov == best && oi < idx))) { best = ov; idx = oi; }
    }
    if (lane == 0) { wv[warp] = best; wi[warp] = idx; }
    if (tid == 0) { first_over = CL_THREADS; last_with_any = -1; }
    __syncthreads();
    if (tid == 0) {
        for (int w = 1; w < CL_THREADS / 32; ++w)
            if (wi[w] >= 0 && (idx < 0 || wv[w] > best || (wv[w] == best && wi[w] < idx))) { best = wv[w]; idx = wi[w]; }
        slot_f = best; slot_i = idx;
    }
    cluster_barrier();
    if (greedy) {  // a greedy row inside a sampled batch: lowest index among the largest
        if (rank == 0 && tid == 0) {
            for (int r = 1; r < C; ++r) {
                const float ov = peer_f32(&slot_f, r);
                const int oi = (int)peer_u32(&slot_i, r);
                if (oi >= 0 && (idx < 0 || ov > best || (ov == best && oi < idx))) { best = ov; idx = oi; }
            }
            out[row] = idx >= 0 ? idx : 0;
        }
        cluster_barrier();  // nobody leaves while the first block may still read its slots
        return;
    }
    float mx = -INFINITY;
    for (int r = 0; r < C; ++r) mx = fmaxf(mx, peer_f32(&slot_f, r));

    // What a warp adds to a histogram. Amounts are 64-bit; shared memory adds 32 bits at a time natively, so a bucket is two
    // words and the adder that sees the low word wrap carries one into the high word (whoever comes first or last, the sum is
    // the same). A bucket that many lanes of the warp share (the top bytes of the keys hardly differ) gets the lanes' sum in
    // one addition; lanes in sparsely hit buckets add for themselves.
    auto add64 = [&](unsigned int* h, uint32_t bucket, unsigned long long v) {
        const unsigned int low = (unsigned int)v, high = (unsigned int)(v >> 32);
        const unsigned int old = atomicAdd(&h[bucket], low);
        const unsigned int carry = (old + low < old) ? 1u : 0u;
        if (high + carry) atomicAdd(&h[256 + bucket], high + carry);
    };
    auto add_into = [&](unsigned int* h, bool valid, uint32_t bucket, unsigned long long amount) {
        // two rounds: the lanes that share the bucket of the first lane still waiting add up among themselves and add once
        // (a vote, a shuffle, a vote: no search for all groups of equal buckets, which costs as many steps as there are groups)
        unsigned int waiting = __ballot_sync(0xffffffffu, valid);
#pragma unroll
        for (int round = 0; round < 2; ++round) {
            if (!waiting) return;
            const int leader = __ffs(waiting) - 1;
            const uint32_t lb = __shfl_sync(0xffffffffu, bucket, leader);
            const bool in = valid && bucket == lb && ((waiting >> lane) & 1u);
            const unsigned int group = __ballot_sync(0xffffffffu, in);
            if (__popc(group) >= 4) {
                unsigned long long v = in ? amount : 0ull;
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) v += shfl_u64(v, lane ^ o);
                if (lane == leader) add64(h, lb, v);
                waiting &= ~group;
            } else {
                break;   // sparse: everyone for themselves
            }
        }
        if ((waiting >> lane) & 1u) add64(h, bucket, amount);
    };
    // One pass of a descent: the histogram, over the whole row, of the byte at `shift` of the kept keys that agree with
    // `prefix` above it (counts, or masses); the same in every block afterwards, in gsum.
    int pass = 0;
    auto histogram = [&](uint32_t min_key, uint32_t prefix, int shift, bool masses) {
        unsigned int* h = hist[pass++ & 1];
        h[tid] = 0;   // 512 words: low halves, high halves
        __syncthreads();
        const uint32_t mask = shift == 24 ? 0u : (0xffffffffu << (shift + 8));
        for (int j0 = 0; j0 < n; j0 += CL_THREADS) {   // whole warps: the lanes of a warp vote together
            const int j = j0 + tid;
            const float v = j < n ? xs[j] : 0.f;
            const uint32_t key = j < n ? order_key(v) : 0u;
            const bool valid = j < n && key >= min_key && (key & mask) == prefix;
            add_into(h, valid, (key >> shift) & 255u, !valid ? 0ull : masses ? mass_units(v, mx) : 1ull);
        }
        cluster_barrier();
        if (tid < 256) {
            unsigned long long g = 0;
            for (int r = 0; r < C; ++r) g += ((unsigned long long)peer_u32(&h[256 + tid], r) << 32) + peer_u32(&h[tid], r);
            gsum[tid] = g;
        }
        __syncthreads();
    };

    // ---- top-k: the key of the k-th largest scaled logit (0 keeps everything)
    uint32_t min_key = 0;
    const int k = top_k[row];
    if (k > 0 && k < V) {
        if (tid == 0) { sel_prefix = 0; sel_remaining = (unsigned long long)k; }
        __syncthreads();
        for (int shift = 24; shift >= 0; shift -= 8) {
            const uint32_t prefix = sel_prefix;
            histogram(0u, prefix, shift, false);
            if (warp == 0) {
                int b;
                unsigned long long above;
                first_bucket_reaching(gsum, sel_remaining, lane, b, above);
                if (lane == 0) { sel_prefix = prefix | ((uint32_t)b << shift); sel_remaining -= above; }
            }
            __syncthreads();
        }
        min_key = sel_prefix;
    }

    // ---- top-p: the smallest key t with mass(keys > t) < top_p * total; tokens with key >= t stay
    const float tp = top_p[row];
    if (tp < 1.0f) {
        // the total mass of the kept set, in the units of the histograms
        unsigned long long part = 0;
        for (int j = tid; j < n; j += CL_THREADS)
            if (order_key(xs[j]) >= min_key) part += mass_units(xs[j], mx);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) part += shfl_u64(part, lane ^ o);
        if (tid == 0) { slot_m[0] = 0; slot_m[1] = 0; }
        __syncthreads();
        if (lane == 0) {
            const unsigned int low = (unsigned int)part, old = atomicAdd(&slot_m[0], low);
            atomicAdd(&slot_m[1], (unsigned int)(part >> 32) + ((old + low < old) ? 1u : 0u));
        }
        cluster_barrier();
        unsigned long long total = 0;
        for (int r = 0; r < C; ++r) total += ((unsigned long long)peer_u32(&slot_m[1], r) << 32) + peer_u32(&slot_m[0], r);
        // masses are whole numbers: mass < limit  <=>  mass < ceil(limit)
        const double limit = (double)tp * (double)total;
        unsigned long long limit_units = (unsigned long long)limit;
        if ((double)limit_units < limit) limit_units += 1;
        if (tid == 0) { sel_prefix = 0; sel_remaining = 0; }
        __syncthreads();
        for (int shift = 24; shift >= 0; shift -= 8) {
            const uint32_t prefix = sel_prefix;
            const unsigned long long above_prefix = sel_remaining;
            histogram(min_key, prefix, shift, true);
            if (warp == 0) {
                // going down from bucket 255: the mass above candidate (prefix | b | ones below) is above_prefix + the buckets
                // above b; the smallest b that keeps it below the limit is where adding bucket b itself would reach the limit
                int b;
                unsigned long long above;
                first_bucket_reaching(gsum, limit_units > above_prefix ? limit_units - above_prefix : 0ull, lane, b, above);
                if (lane == 0) { sel_prefix = prefix | ((uint32_t)b << shift); sel_remaining = above_prefix + above; }
            }
            __syncthreads();
        }
        if (sel_prefix > min_key) min_key = sel_prefix;
    }

    // ---- the draw: each thread owns a run of consecutive tokens of the block's slice, the blocks follow each other by rank;
    // the token is the first, in this order, at which the running mass exceeds u * total
    const int per = (n + CL_THREADS - 1) / CL_THREADS;
    const int jlo = min(n, tid * per), jhi = min(n, jlo + per);
    double mine = 0.0;
    for (int j = jlo; j < jhi; ++j)
        if (order_key(xs[j]) >= min_key) mine += (double)expf(xs[j] - mx);
    double upto = mine;   // the warp's threads up to this one
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const double up = __shfl_up_sync(0xffffffffu, upto, o);
        if (lane >= o) upto += up;
    }
    if (lane == 31) red[warp] = upto;
    __syncthreads();
    if (tid == 0) {
        double t = 0.0;
        for (int w = 0; w < CL_THREADS / 32; ++w) t += red[w];
        slot_d = t;
    }
    cluster_barrier();
    double before = 0.0, all = 0.0;   // the blocks before this one; everything
    for (int r = 0; r < C; ++r) {
        const double m = peer_f64(&slot_d, r);
        if (r < (int)rank) before += m;
        all += m;
    }
    const double target = (double)uniform[row] * all;
    for (int w = 0; w < warp; ++w) before += red[w];
    const double start = before + (upto - mine);
    if (mine > 0.0) {
        if (start + mine > target) atomicMin(&first_over, tid);
        atomicMax(&last_with_any, tid);
    }
    if (tid == 0) { slot_i = -1; slot_f = 0.f; }   // (everyone read the maxima long ago: a cluster barrier lies between)
    __syncthreads();
    // this block's candidate: where its first thread over the target finds the token, or, should no block find one (rounding
    // left the target at or past the end), its last kept token
    if (tid == first_over) {
        double run = start;
        int pick = -1, last_kept = -1;
        for (int j = jlo; j < jhi; ++j) {
            if (order_key(xs[j]) < min_key) continue;
            last_kept = lo + j;
            run += (double)expf(xs[j] - mx);
            if (run > target) { pick = lo + j; break; }
        }
        slot_i = pick >= 0 ? pick : last_kept;
        slot_f = 1.f;   // found by running mass
    } else if (first_over == CL_THREADS && tid == last_with_any) {
        int last_kept = -1;
        for (int j = jlo; j < jhi; ++j)
            if (order_key(xs[j]) >= min_key) last_kept = lo + j;
        slot_i = last_kept;
    }
    cluster_barrier();
    if (rank == 0 && tid == 0) {
        int pick = -1, last = -1;
        for (int r = 0; r < C; ++r) {
            const int cand = (int)peer_u32(&slot_i, r);
            if (cand < 0) continue;
            if (pick < 0 && peer_f32(&slot_f, r) > 0.f) pick = cand;   // the first block, by rank, that ran over the target
            last = cand;
        }
        out[row] = pick >= 0 ? pick : (last >= 0 ? last : 0);
    }
    cluster_barrier();  // nobody leaves while another block may still read its slots or histograms
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
                           const float* uniform, int* out, int M, int V, int single_block, cudaStream_t s) {
    if (M <= 0) return 0;
    if (V <= 0) return LLMIE_ERR_BAD_ARGUMENT;
    // a cluster per row: as few blocks as hold the row in their shared memory, but enough of them to spread a small batch
    // over the device (slices of at most 16 K tokens); rows too long for 8 blocks take the single-block kernel
    int C = 1;
    while (C < CL_MAX && ((V + C - 1) / C > 16384)) C *= 2;
    const int slice = (((V + C - 1) / C) + 3) & ~3;
    if (single_block || slice > CL_MAX_SLICE || (long long)M * C > 0x7fffffffLL) {
        sample_kernel<<<M, THREADS, 0, s>>>(logits, temperature, top_k, top_p, uniform, out, V);
        return launch_status();
    }
    static bool set = false;
    if (!set) {
        cudaError_t e = cudaFuncSetAttribute(sample_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(CL_MAX_SLICE * sizeof(float)));
        if (e != cudaSuccess) return (int)e;
        set = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(M * C));
    cfg.blockDim = dim3(CL_THREADS);
    cfg.dynamicSmemBytes = (size_t)slice * sizeof(float);
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)C;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = llmie_pdl_flag ? 2 : 1;
    return (int)cudaLaunchKernelEx(&cfg, sample_cluster_kernel, logits, temperature, top_k, top_p, uniform, out, V, C, slice);
}
