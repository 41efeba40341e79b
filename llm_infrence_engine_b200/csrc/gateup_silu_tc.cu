// out[m, i] = silu(x W_gate^T)[m, i] * (x W_up^T)[m, i] for MANY rows m (prompt portions): the gate/up product of a gated
// feed-forward with the activation as its epilogue, on the tcgen05 tensor cores of sm_100a. The float32 gate and up sums
// never leave the chip: no [rows, 2 I] intermediate is written and read again, and no activation kernel runs.
//
// W is the fused matrix [2 I, K] (gate rows first, then up rows), x is [M, K], both bfloat16 row-major; out is bfloat16 [M, I].
//
// A tile of the output is 128 rows x 128 columns. Its accumulator is 128 lanes x 256 columns of tensor memory: columns 0-127
// the gate sums of the tile's output columns, 128-255 the up sums of the same columns. The B operand of a K step is therefore
// two boxes of weight rows, [n0, n0 + 128) of the gate half and [I + n0, I + n0 + 128) of the up half, side by side in shared
// memory: one MMA of N = 256 covers both. Tensor memory holds two such accumulators, so the epilogue of a tile runs while the
// MMAs of the next tile are issued.
//
// The kernel is persistent: one block per multiprocessor walks tiles blockIdx.x, + gridDim.x, ... (tiles that are neighbours
// in this order share their weight boxes, which therefore come from L2).
//
//   warp 0, one lane    producer: per K step of 64 one TMA box of x rows and two of weight rows (128-byte swizzle, no
//                       multicast) into a ring of 4 stages (mbarriers full / empty)
//   warp 1, one lane    issues 4 MMAs (128 x 256 x 16) per stage, frees the stage by tcgen05.commit, and after a tile's last
//                       stage commits the accumulator's barrier
//   warps 2-5           epilogue: thread = row; reads gate and up sums with tcgen05.ld, 16 columns at a time, computes
//                       silu(g) * u in 32-bit (fast exponential and division: the result is rounded to bfloat16) and stores
//                       16-byte pieces of the output row; then hands the accumulator back
//
// Every wait is bounded (tcgen05.cuh): a block that gives up sets the error flag, stops issuing, lets its copies land, frees
// its tensor memory and returns.
#include "common.cuh"
#include "tcgen05.cuh"

namespace {

constexpr int BM = 128, BK = 64, STAGES = 4, UMMA_K = 16;
constexpr int A_BYTES = BM * BK * 2;
constexpr int EPI_THREADS = 128, THREADS = 64 + EPI_THREADS;

template <int BN>
__global__ void __launch_bounds__(THREADS) gateup_silu_tc_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
                                                                  bf16* __restrict__ out, int M, int I, int K, int* error_flag) {
    constexpr int B_BYTES = 2 * BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;   // BN gate rows and BN up rows per K step
    extern __shared__ unsigned char raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* full = reinterpret_cast<uint64_t*>(tiles + STAGES * STAGE_BYTES);
    uint64_t* empty = full + STAGES;
    uint64_t* acc_full = empty + STAGES;   // [2] the MMAs of a tile have finished
    uint64_t* acc_free = acc_full + 2;     // [2] the epilogue has read the accumulator
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_free + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile int* issued = abort_flag + 1;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int m_tiles = (M + BM - 1) / BM, n_tiles = (I + BN - 1) / BN, num_tiles = m_tiles * n_tiles;
    const int nkb = (K + BK - 1) / BK;

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full + s, 1); mbar_init(empty + s, 1); }
        for (int s = 0; s < 2; ++s) { mbar_init(acc_full + s, 1); mbar_init(acc_free + s, EPI_THREADS / 32); }
        *abort_flag = 0;
        *issued = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(tmem_slot)), "n"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem = *tmem_slot;
    pdl_trigger();

    if (warp == 0) {
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];\n" ::"l"(&tmap_x) : "memory");
            asm volatile("prefetch.tensormap [%0];\n" ::"l"(&tmap_w) : "memory");
            pdl_wait();  // the rows are what the kernel before this one wrote
            int g = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
                const int m0 = (t % m_tiles) * BM, n0 = (t / m_tiles) * BN;
                for (int kb = 0; kb < nkb; ++kb, ++g) {
                    const int s = g % STAGES;
                    if (g >= STAGES && !mbar_wait(empty + s, ((g / STAGES) & 1) ^ 1, abort_flag, error_flag, 31)) { ok = false; break; }
                    unsigned char* st = tiles + s * STAGE_BYTES;
                    mbar_expect_tx(full + s, STAGE_BYTES);
                    tma_load_2d(st, &tmap_x, kb * BK, m0, full + s);
                    tma_load_2d(st + A_BYTES, &tmap_w, kb * BK, n0, full + s);                      // gate rows
                    tma_load_2d(st + A_BYTES + B_BYTES / 2, &tmap_w, kb * BK, I + n0, full + s);    // up rows of the same columns
                    *issued = g + 1;
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // instruction descriptor: D float32, A and B bfloat16, both K-major, N = 256, M = 128
            constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)((2 * BN) >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
            int g = 0, i = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++i) {
                const int buf = i & 1;
                if (i >= 2) ok = mbar_wait(acc_free + buf, ((i >> 1) & 1) ^ 1, abort_flag, error_flag, 32);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const uint32_t d = tmem + (uint32_t)(buf * 2 * BN);
                for (int kb = 0; kb < nkb; ++kb, ++g) {
                    const int s = g % STAGES;
                    ok = mbar_wait(full + s, (g / STAGES) & 1, abort_flag, error_flag, 33);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                    const uint32_t a_addr = smem_u32(tiles + s * STAGE_BYTES);
                    const uint64_t a_desc = umma_desc(a_addr), b_desc = umma_desc(a_addr + A_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) umma_bf16(d, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    umma_commit(empty + s);
                }
                if (ok) umma_commit(acc_full + buf);
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue
        const int quarter = warp & 3;               // the 32 lanes of tensor memory this warp may read
        const int row = quarter * 32 + lane;
        int i = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++i) {
            const int buf = i & 1;
            const int m = (t % m_tiles) * BM + row, n0 = (t / m_tiles) * BN;
            ok = __all_sync(0xffffffffu, mbar_wait(acc_full + buf, (i >> 1) & 1, abort_flag, error_flag, 34));
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const uint32_t base = tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * 2 * BN);
            bf16* dst = out + (size_t)m * I + n0;
#pragma unroll 2
            for (int c = 0; c < BN; c += 16) {
                uint32_t gv[16], uv[16];
                tmem_ld16(base + c, gv);
                tmem_ld16(base + BN + c, uv);
                asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
                uint32_t packed[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const float g0 = __uint_as_float(gv[2 * j]), g1 = __uint_as_float(gv[2 * j + 1]);
                    const float a = __fdividef(g0, 1.0f + __expf(-g0)) * __uint_as_float(uv[2 * j]);
                    const float b = __fdividef(g1, 1.0f + __expf(-g1)) * __uint_as_float(uv[2 * j + 1]);
                    const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
                    packed[j] = *reinterpret_cast<const uint32_t*>(&v);
                }
                if (m < M) {
                    if (n0 + c + 8 <= I) *reinterpret_cast<uint4*>(dst + c) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                    if (n0 + c + 16 <= I) *reinterpret_cast<uint4*>(dst + c + 8) = make_uint4(packed[4], packed[5], packed[6], packed[7]);
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(acc_free + buf)) : "memory");
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (*abort_flag && tid == 0) {
        // gave up somewhere: let the copies that were started land before the block's shared memory goes away
        const int n_issued = *issued;
        for (int g = max(0, n_issued - STAGES); g < n_issued; ++g) {
            for (uint32_t i = 0; i < SPIN_LIMIT; ++i) {
                if (mbar_try_wait(full + g % STAGES, (g / STAGES) & 1)) break;
                __nanosleep(40);
            }
        }
    }
    __syncthreads();
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "n"(512) : "memory");
}

// The tile's width in output columns: the one of 128, 112, 96, 80, 64 whose tiles fill the persistent grid's rounds best
// (608 tiles of 128 columns on 148 blocks are 4.1 rounds, so five; 704 tiles of 112 columns are 4.8 rounds, also five, of
// seven eighths the length).
inline int best_tile_width(long long m_tiles, int I, int blocks) {
    int best = 128;
    long long best_cost = -1;
    for (int bn = 128; bn >= 64; bn -= 16) {
        const long long tiles = m_tiles * ((I + bn - 1) / bn);
        const long long cost = ((tiles + blocks - 1) / blocks) * (bn + 8);   // + 8: what a tile costs whatever its width
        if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = bn; }
    }
    return best;
}

template <int BN>
int launch_gateup(const bf16* x, const bf16* w, bf16* out, int M, int I, int K, int num_blocks, int* error_flag, cudaStream_t s) {
    CUtensorMap mx, mw;
    int rc = tensor_map(x, M, K, BM, &mx);
    if (rc) return rc;
    rc = tensor_map(w, 2 * I, K, BN, &mw);
    if (rc) return rc;
    constexpr size_t smem = (size_t)STAGES * (A_BYTES + 2 * BN * BK * 2) + 1024 + 256;
    static bool set = false;
    if (!set) {
        cudaError_t e = cudaFuncSetAttribute(gateup_silu_tc_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        set = true;
    }
    const long long tiles = (long long)((M + BM - 1) / BM) * ((I + BN - 1) / BN);
    const int grid = (int)(tiles < num_blocks ? tiles : num_blocks);
    return launch_kernel(gateup_silu_tc_kernel<BN>, dim3(grid), dim3(THREADS), smem, s, mx, mw, out, M, I, K, error_flag);
}

}  // namespace

// x [M, K] and w [2 I, K] bfloat16 row-major (K and I multiples of 8, bases 16-byte aligned), out bfloat16 [M, I].
// num_blocks: the persistent grid (the number of multiprocessors; fewer if there are fewer tiles).
LLMIE_API int llmie_gateup_silu_tc(const bf16* x, const bf16* w, bf16* out, int M, int I, int K, int num_blocks, int* error_flag,
                                   cudaStream_t s) {
    if (M <= 0 || I <= 0) return 0;
    if (K <= 0 || K % 8 || I % 8 || ((uintptr_t)x & 15) || ((uintptr_t)w & 15) || ((uintptr_t)out & 15) || !error_flag || num_blocks < 1)
        return LLMIE_ERR_BAD_ARGUMENT;
    switch (best_tile_width((M + BM - 1) / BM, I, num_blocks)) {
        case 112: return launch_gateup<112>(x, w, out, M, I, K, num_blocks, error_flag, s);
        case 96: return launch_gateup<96>(x, w, out, M, I, K, num_blocks, error_flag, s);
        case 80: return launch_gateup<80>(x, w, out, M, I, K, num_blocks, error_flag, s);
        case 64: return launch_gateup<64>(x, w, out, M, I, K, num_blocks, error_flag, s);
        default: return launch_gateup<128>(x, w, out, M, I, K, num_blocks, error_flag, s);
    }
}
