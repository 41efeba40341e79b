// out[m, n] (+)= sum_k x[m, k] * w[n, k] for FEW rows m (a decode batch): the weights stream through the
// 5th-generation tensor cores of sm_100a at memory speed.
//
// The product is computed transposed ("swap A/B"): a tile of 128 weight rows is the M side of
// tcgen05.mma (cta_group::1, kind::f16, bfloat16 in, 32-bit accumulate), the TN <= 64 token rows are its
// N side, so no tensor-core work is wasted on padding tokens up to 128. Operands reach shared memory by
// TMA (cp.async.bulk.tensor, 128-byte swizzle, no multicast) through a ring of STAGES buffers guarded by
// mbarriers; the accumulator D[128 x TN] lives in tensor memory and is read back with tcgen05.ld.
//
//   warp 0, one lane   producer: waits for a free stage, arms its barrier with the byte count, issues the
//                      two TMA loads (weight tile 128 x 64, token tile TN x 64; rows or columns outside the
//                      matrices arrive as zeros)
//   warp 1, one lane   issues 4 MMAs (K = 16 each) per stage, commits the stage back to the producer,
//                      and after the last stage commits the accumulator barrier
//   all 4 warps        epilogue: each thread owns one weight row n (TMEM lane) and TN token columns;
//                      it stores, or adds with red.global.add.f32 when the K range is split over blocks
//
// grid = (ceil(N / 128), ceil(M / TN), k_splits). Splitting K gives small matrices enough blocks to pull
// the whole memory system; the partial sums meet in the float32 output by atomic addition, which is
// also how a projection adds itself into the residual stream without a separate kernel.
//
// Every wait on an mbarrier is bounded: after SPIN_LIMIT polls the block records an error in
// `error_flag`, stops issuing work, lets the copies it started land (again bounded), frees its tensor
// memory and returns. The host reads the flag and raises.
#include "common.cuh"
#include "tcgen05.cuh"

namespace {

constexpr int BM = 128, BK = 64, STAGES = 4, UMMA_K = 16;

template <int TN>
__global__ void __launch_bounds__(128) gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                                                      float* __restrict__ out, int ldo, int M, int N, int K, int kb_per_split,
                                                      int accumulate, int* error_flag) {
    constexpr int W_BYTES = BM * BK * 2, X_BYTES = TN * BK * 2, STAGE_BYTES = W_BYTES + X_BYTES;
    constexpr int COLS = TN < 32 ? 32 : TN;  // tensor-memory columns: a power of two, at least 32
    extern __shared__ unsigned char raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* full = reinterpret_cast<uint64_t*>(tiles + STAGES * STAGE_BYTES);
    uint64_t* empty = full + STAGES;
    uint64_t* accum = empty + STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile int* issued = abort_flag + 1;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n0 = blockIdx.x * BM, m0 = blockIdx.y * TN;
    const int nkb = (K + BK - 1) / BK;
    const int kb0 = blockIdx.z * kb_per_split, kb1 = min(nkb, kb0 + kb_per_split);
    const int iters = kb1 - kb0;

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full + s, 1); mbar_init(empty + s, 1); }
        mbar_init(accum, 1);
        *abort_flag = 0;
        *issued = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 0) {
        __syncwarp();  // lane 0 comes back from the initialisation above: the allocation is a warp-wide instruction
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(tmem_slot)), "n"(COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem = *tmem_slot;

    pdl_trigger();
    if (warp == 0 && lane == 0) {
        asm volatile("prefetch.tensormap [%0];\n" ::"l"(&tmap_w) : "memory");
        asm volatile("prefetch.tensormap [%0];\n" ::"l"(&tmap_x) : "memory");
        // The weights do not depend on the kernel before this one: the first stages' weight tiles are on their way
        // before the wait; the token tiles, which that kernel wrote, follow after it.
        const int early = min(iters, STAGES);
        constexpr uint32_t tx = STAGE_BYTES;
        for (int it = 0; it < early; ++it) {
            mbar_expect_tx(full + it, tx);
            tma_load_2d(tiles + it * STAGE_BYTES, &tmap_w, (kb0 + it) * BK, n0, full + it);
            *issued = it + 1;
        }
        pdl_wait();
        for (int it = 0; it < early; ++it) tma_load_2d(tiles + it * STAGE_BYTES + W_BYTES, &tmap_x, (kb0 + it) * BK, m0, full + it);
        for (int it = early; it < iters; ++it) {
            const int s = it % STAGES;
            if (!mbar_wait(empty + s, ((it / STAGES) & 1) ^ 1, abort_flag, error_flag, 1)) break;
            unsigned char* st = tiles + s * STAGE_BYTES;
            mbar_expect_tx(full + s, tx);
            tma_load_2d(st, &tmap_w, (kb0 + it) * BK, n0, full + s);
            tma_load_2d(st + W_BYTES, &tmap_x, (kb0 + it) * BK, m0, full + s);
            *issued = it + 1;
        }
    } else if (warp == 1 && lane == 0) {
        // instruction descriptor: D float32, A and B bfloat16, both K-major, N = TN, M = 128
        constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
        bool ok = true;
        for (int it = 0; it < iters && ok; ++it) {
            const int s = it % STAGES;
            ok = mbar_wait(full + s, (it / STAGES) & 1, abort_flag, error_flag, 2);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const uint32_t a_addr = smem_u32(tiles + s * STAGE_BYTES);
            const uint64_t a_desc = umma_desc(a_addr), b_desc = umma_desc(a_addr + W_BYTES);
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k)
                umma_bf16(tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, (it > 0 || k > 0) ? 1u : 0u);  // +32 bytes per K step
            umma_commit(empty + s);
        }
        if (ok) umma_commit(accum);
    }
    __syncwarp();
    pdl_wait();  // every thread: the epilogue writes where the kernel before may still read or write
    const bool done = __all_sync(0xffffffffu, mbar_wait(accum, 0, abort_flag, error_flag, 3));  // uniform per warp: tcgen05.ld is warp-wide
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    if (done) {
        const int n = n0 + warp * 32 + lane;
        const int rows = min(TN, M - m0);
#pragma unroll
        for (int c = 0; c < TN; c += 16) {
            uint32_t v[16];
            tmem_ld16(tmem + ((uint32_t)(warp * 32) << 16) + c, v);
            asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
            if (n < N) {
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const int m = c + j;
                    if (m < rows) {
                        float* dst = out + (size_t)(m0 + m) * ldo + n;
                        if (accumulate) atomicAdd(dst, __uint_as_float(v[j]));
                        else *dst = __uint_as_float(v[j]);
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (!done && tid == 0) {
        // gave up somewhere: let the copies that were started land before the block's shared memory goes away
        const int n_issued = *issued;
        for (int it = max(0, n_issued - STAGES); it < n_issued; ++it) {
            for (uint32_t i = 0; i < SPIN_LIMIT; ++i) {
                if (mbar_try_wait(full + it % STAGES, (it / STAGES) & 1)) break;
                __nanosleep(40);
            }
        }
    }
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "n"(COLS) : "memory");
}

// ------------------------------------------------------------------------------------------------ host side
template <int TN>
int launch(const CUtensorMap& mw, const CUtensorMap& mx, float* out, int ldo, int M, int N, int K, int k_splits, int accumulate,
           int* error_flag, cudaStream_t s) {
    constexpr size_t smem = (size_t)STAGES * (BM * BK * 2 + TN * BK * 2) + 1024 + 256;
    static bool set = false;
    if (!set) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<TN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        set = true;
    }
    const int nkb = (K + BK - 1) / BK;
    const int per = (nkb + k_splits - 1) / k_splits;
    const int splits = (nkb + per - 1) / per;  // no empty split
    const dim3 grid((N + BM - 1) / BM, (M + TN - 1) / TN, splits);
    return launch_kernel(gemm_tc_kernel<TN>, grid, dim3(128), smem, s, mw, mx, out, ldo, M, N, K, per, accumulate, error_flag);
}

static int run(const bf16* x, const bf16* w, float* out, int ldo, int M, int N, int K, int k_splits, int accumulate, int* error_flag,
               cudaStream_t s) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || K % 8 || ((uintptr_t)w & 15) || ((uintptr_t)x & 15) || k_splits < 1 || (!accumulate && k_splits != 1) || !error_flag ||
        ldo < N)
        return LLMIE_ERR_BAD_ARGUMENT;
    const int TN = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
    CUtensorMap mw, mx;
    int rc = tensor_map(w, N, K, BM, &mw);
    if (rc) return rc;
    rc = tensor_map(x, M, K, TN, &mx);
    if (rc) return rc;
    if (TN == 16) return launch<16>(mw, mx, out, ldo, M, N, K, k_splits, accumulate, error_flag, s);
    if (TN == 32) return launch<32>(mw, mx, out, ldo, M, N, K, k_splits, accumulate, error_flag, s);
    return launch<64>(mw, mx, out, ldo, M, N, K, k_splits, accumulate, error_flag, s);
}

}  // namespace

// x [M, K] and w [N, K] bfloat16 row-major (K a multiple of 8, bases 16-byte aligned), out float32 with row stride ldo.
// accumulate = 0 needs k_splits = 1 and stores; accumulate = 1 adds atomically into what `out` holds.
LLMIE_API int llmie_gemm_tc(const bf16* x, const bf16* w, float* out, int ldo, int M, int N, int K, int k_splits, int accumulate,
                            int* error_flag, cudaStream_t s) {
    return run(x, w, out, ldo, M, N, K, k_splits, accumulate, error_flag, s);
}
