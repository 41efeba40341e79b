// The end of an attention tile, shared by the kernels that cut a tile's keys into slices.
#pragma once

#include "common.cuh"

namespace {

// `Params` has: out [tokens][nq * D] bfloat16, part_o [partials][ROWS][D] and part_ml [partials][ROWS][2] float32 scratch,
// counters (zero between launches), nq.
// The block's finished rows are in shared memory as (max, sum, output); write them out, or, with several key slices
// (`num_splits` of them for this tile and key/value head, this block's being number `split`), store the partial and let
// the last block merge all slices. Slice s keeps its partial at index part_base + s * part_stride; `counter` is the
// counter of this tile and key/value head; `sums` is shared memory for num_splits * nrows floats that nothing else uses
// (row_o must hold as many).
template <int D, int ROWS, int THREADS, typename Params>
__device__ __forceinline__ void finish_tile(const Params& p, const float* row_m, const float* row_l, const float* row_o, int num_splits,
                                            size_t part_base, size_t part_stride, int counter, int kvh, int split, int n0, int nrows,
                                            int G, int* flag_smem, float* sums) {
    const int tid = threadIdx.x;
    if (num_splits == 1) {
        for (int i = tid; i < nrows * D; i += THREADS) {
            const int r = i / D, dim = i % D;
            const float L = row_l[r];
            const float val = L > 0.f ? row_o[r * D + dim] / L : 0.f;
            p.out[(size_t)(n0 + r / G) * p.nq * D + (size_t)(kvh * G + r % G) * D + dim] = __float2bfloat16_rn(val);
        }
        return;
    }
    float* po = p.part_o + (part_base + split * part_stride) * ROWS * D;
    float* pml = p.part_ml + (part_base + split * part_stride) * ROWS * 2;
    for (int i = tid * 4; i < nrows * D; i += THREADS * 4) *reinterpret_cast<float4*>(po + i) = *reinterpret_cast<const float4*>(row_o + i);
    for (int r = tid; r < nrows; r += THREADS) { pml[2 * r] = row_m[r]; pml[2 * r + 1] = row_l[r]; }
    // The block's partial is complete once every thread has passed the barrier; thread 0 then counts the block in with an
    // atomic that RELEASES (what the block wrote is visible to whoever sees the count) and ACQUIRES (the last block sees what
    // the others wrote): one trip to memory instead of a fence followed by an atomic.
    __syncthreads();
    if (tid == 0) {
        int prev;
        asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;\n" : "=r"(prev) : "l"(p.counters + counter) : "memory");
        *flag_smem = prev == num_splits - 1;
    }
    __syncthreads();
    if (!*flag_smem) return;
    if constexpr (ROWS * D / 4 > THREADS) {
        // A tile of prompt rows, cut into a few slices: many steps per thread and few threads, so what a step costs in
        // instructions counts as much as the trips to memory. The block's own slice is still in shared memory; the first
        // steps' loads of the other slices leave at once, and while they travel one thread per row makes the slices' weights
        // e^(m_s - M) / L from the rows' (max, sum) pairs. A step is then four loads' worth of multiply-adds and a store.
        constexpr int STEPS = 4, OTHERS = 3;
        if (num_splits <= OTHERS + 1) {
            const int n = nrows * D;
            float4 a[STEPS][OTHERS];
            auto fetch = [&](int i0) {
#pragma unroll
                for (int u = 0; u < STEPS; ++u) {
                    const int i = i0 + u * THREADS * 4;
#pragma unroll
                    for (int k = 0; k < OTHERS; ++k) {
                        const int s = k < split ? k : k + 1;  // the slices that are not this block's
                        if (i < n && s < num_splits)
                            a[u][k] = __ldcg(reinterpret_cast<const float4*>(p.part_o + (part_base + s * part_stride) * ROWS * D + i));
                    }
                }
            };
            auto combine = [&](int i0) {
#pragma unroll
                for (int u = 0; u < STEPS; ++u) {
                    const int i = i0 + u * THREADS * 4;
                    if (i >= n) continue;
                    const int r = i / D, dim = i % D;
                    const float w_own = sums[r];
                    const float4 own = *reinterpret_cast<const float4*>(row_o + i);
                    float4 O = make_float4(own.x * w_own, own.y * w_own, own.z * w_own, own.w * w_own);
#pragma unroll
                    for (int k = 0; k < OTHERS; ++k) {
                        if (k + 1 < num_splits) {
                            const float w = sums[(k + 1) * nrows + r];
                            O.x = fmaf(a[u][k].x, w, O.x); O.y = fmaf(a[u][k].y, w, O.y); O.z = fmaf(a[u][k].z, w, O.z); O.w = fmaf(a[u][k].w, w, O.w);
                        }
                    }
                    const __nv_bfloat162 lo = __floats2bfloat162_rn(O.x, O.y), hi = __floats2bfloat162_rn(O.z, O.w);
                    uint2 packed;
                    packed.x = *reinterpret_cast<const uint32_t*>(&lo);
                    packed.y = *reinterpret_cast<const uint32_t*>(&hi);
                    *reinterpret_cast<uint2*>(p.out + (size_t)(n0 + r / G) * p.nq * D + (size_t)(kvh * G + r % G) * D + dim) = packed;
                }
            };
            fetch(tid * 4);
            for (int r = tid; r < nrows; r += THREADS) {
                float2 ml[OTHERS];
                float M = row_m[r];
#pragma unroll
                for (int k = 0; k < OTHERS; ++k) {
                    const int s = k < split ? k : k + 1;
                    ml[k] = make_float2(-INFINITY, 0.f);
                    if (s < num_splits) ml[k] = __ldcg(reinterpret_cast<const float2*>(p.part_ml + (part_base + s * part_stride) * ROWS * 2 + 2 * r));
                    M = fmaxf(M, ml[k].x);
                }
                float w[OTHERS + 1];
                w[0] = M > -INFINITY ? exp2f(row_m[r] - M) : 0.f;
                float L = row_l[r] * w[0];
#pragma unroll
                for (int k = 0; k < OTHERS; ++k) {
                    w[k + 1] = M > -INFINITY ? exp2f(ml[k].x - M) : 0.f;
                    L = fmaf(ml[k].y, w[k + 1], L);
                }
                const float inv = L > 0.f ? 1.f / L : 0.f;
#pragma unroll
                for (int k = 0; k <= OTHERS; ++k)
                    if (k < num_splits) sums[k * nrows + r] = w[k] * inv;  // [0] the block's own slice, [k + 1] the k-th other one
            }
            __syncthreads();
            combine(tid * 4);
            for (int i0 = tid * 4 + THREADS * 4 * STEPS; i0 < n; i0 += THREADS * 4 * STEPS) {
                fetch(i0);
                combine(i0);
            }
            if (tid == 0) p.counters[counter] = 0;  // ready for the next launch
            return;
        }
    }
    // Last block of the tile. One trip to memory brings every slice's (max, sum) pair into shared memory (the block's own
    // row_m / row_l / row_o are not needed any more); from these each row's thread makes the slices' weights
    // e^(m_s - M) and 1 / L; then every output element is one weighted sum whose loads do not depend on each other.
    float* wgt = const_cast<float*>(row_o);                 // [num_splits][nrows] maxima, then weights
    for (int i = tid; i < nrows * num_splits; i += THREADS) {
        const int s = i / nrows, r = i % nrows;
        const float2 ml = __ldcg(reinterpret_cast<const float2*>(p.part_ml + (part_base + s * part_stride) * ROWS * 2 + 2 * r));
        wgt[i] = ml.x;
        sums[i] = ml.y;
    }
    __syncthreads();
    for (int r = tid; r < nrows; r += THREADS) {
        float M = -INFINITY;
        for (int s = 0; s < num_splits; ++s) M = fmaxf(M, wgt[s * nrows + r]);
        float L = 0.f;
        for (int s = 0; s < num_splits; ++s) {
            const float w = M > -INFINITY ? exp2f(wgt[s * nrows + r] - M) : 0.f;
            wgt[s * nrows + r] = w;
            L = fmaf(sums[s * nrows + r], w, L);
        }
        const_cast<float*>(row_l)[r] = L > 0.f ? 1.f / L : 0.f;
    }
    __syncthreads();
    // four neighbouring outputs of a row per thread and step (16-byte loads that do not depend on each other)
    auto store4 = [&](int i, const float4& O) {
        const int r = i / D, dim = i % D;
        const float inv = row_l[r];
        const __nv_bfloat162 lo = __floats2bfloat162_rn(O.x * inv, O.y * inv), hi = __floats2bfloat162_rn(O.z * inv, O.w * inv);
        uint2 packed;
        packed.x = *reinterpret_cast<const uint32_t*>(&lo);
        packed.y = *reinterpret_cast<const uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(p.out + (size_t)(n0 + r / G) * p.nq * D + (size_t)(kvh * G + r % G) * D + dim) = packed;
    };
    if constexpr (ROWS * D / 4 <= THREADS) {
        // at most one step per thread (a decode tile): the slices in groups of GROUP whose loads all leave before the first of
        // them is used, one trip to memory per group
        for (int i = tid * 4; i < nrows * D; i += THREADS * 4) {
            const int r = i / D;
            float4 O = make_float4(0.f, 0.f, 0.f, 0.f);
            constexpr int GROUP = 12;
            for (int s0 = 0; s0 < num_splits; s0 += GROUP) {
                float4 a[GROUP];
#pragma unroll
                for (int k = 0; k < GROUP; ++k)
                    if (s0 + k < num_splits) a[k] = __ldcg(reinterpret_cast<const float4*>(p.part_o + (part_base + (s0 + k) * part_stride) * ROWS * D + i));
#pragma unroll
                for (int k = 0; k < GROUP; ++k) {
                    if (s0 + k < num_splits) {
                        const float w = wgt[(s0 + k) * nrows + r];
                        O.x = fmaf(a[k].x, w, O.x); O.y = fmaf(a[k].y, w, O.y); O.z = fmaf(a[k].z, w, O.z); O.w = fmaf(a[k].w, w, O.w);
                    }
                }
            }
            store4(i, O);
        }
    } else {
        // many steps per thread (a tile of prompt rows, few slices): four steps at a time, each with up to four slices, so that
        // sixteen loads are on their way together instead of one step's after the other's (a trip to memory per step was most
        // of what a slice cost)
        constexpr int STEPS = 4, GROUP = 4;
        for (int i0 = tid * 4; i0 < nrows * D; i0 += THREADS * 4 * STEPS) {
            float4 O[STEPS];
#pragma unroll
            for (int u = 0; u < STEPS; ++u) O[u] = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int s0 = 0; s0 < num_splits; s0 += GROUP) {
                float4 a[STEPS][GROUP];
#pragma unroll
                for (int u = 0; u < STEPS; ++u) {
                    const int i = i0 + u * THREADS * 4;
#pragma unroll
                    for (int k = 0; k < GROUP; ++k)
                        if (i < nrows * D && s0 + k < num_splits)
                            a[u][k] = __ldcg(reinterpret_cast<const float4*>(p.part_o + (part_base + (s0 + k) * part_stride) * ROWS * D + i));
                }
#pragma unroll
                for (int u = 0; u < STEPS; ++u) {
                    const int i = i0 + u * THREADS * 4;
                    if (i >= nrows * D) continue;
                    const int r = i / D;
#pragma unroll
                    for (int k = 0; k < GROUP; ++k) {
                        if (s0 + k < num_splits) {
                            const float w = wgt[(s0 + k) * nrows + r];
                            O[u].x = fmaf(a[u][k].x, w, O[u].x); O[u].y = fmaf(a[u][k].y, w, O[u].y);
                            O[u].z = fmaf(a[u][k].z, w, O[u].z); O[u].w = fmaf(a[u][k].w, w, O[u].w);
                        }
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < STEPS; ++u) {
                const int i = i0 + u * THREADS * 4;
                if (i < nrows * D) store4(i, O[u]);
            }
        }
    }
    if (tid == 0) p.counters[counter] = 0;  // ready for the next launch
}

}  // namespace
