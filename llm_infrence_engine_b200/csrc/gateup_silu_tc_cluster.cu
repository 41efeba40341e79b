// The gate/up product of prompt portions with silu(gate) * up as its epilogue (see gateup_silu_tc.cu, whose tiles, roles and
// epilogue this kernel shares), for PAIRS of blocks: the two blocks of a thread-block cluster work on two tiles of 128 rows
// that lie below each other, so they need the same 256 weight rows (128 gate rows, 128 up rows) in every K step. Each block
// fetches one half (block 0 the gate rows, block 1 the up rows) and the TMA copy delivers it to BOTH blocks' shared memory
// (cluster multicast); each block fetches its own 128 token rows. A K step therefore costs a block 32 KB from L2 instead of
// 48 KB. That matters because this product is bound by the path from L2 to the multiprocessors, not by the tensor cores:
// without sharing, 608 tiles x 687 KB = 418 MB cross it for 21 MB of distinct data.
//
// What the sharing adds to the protocol: a stage of the ring is written by both blocks, so a block may refill it only when
// the MMAs of BOTH blocks have read it: the stage's "empty" barrier counts two arrivals, and each block's MMA thread commits
// to the barrier of both blocks (tcgen05.commit with a cluster mask). Barriers are initialised before a cluster-wide barrier,
// and the blocks leave through another one, so nobody writes into a block that has gone.
//
// This file is the only one of the package that uses a TMA load with cluster multicast (of this GPU's own memory). It is
// optional: the library builds and runs without it (gateup_silu_tc.cu alone).
#include "common.cuh"
#include "tcgen05.cuh"

namespace {

constexpr int BM = 128, BK = 64, STAGES = 4, UMMA_K = 16;
constexpr int A_BYTES = BM * BK * 2;
constexpr int EPI_THREADS = 128, THREADS = 64 + EPI_THREADS;

__device__ __forceinline__ void tma_load_2d_multicast(void* dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar, uint16_t mask) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.multicast::cluster [%0], [%1, {%2, %3}], [%4], %5;\n" ::"r"(
            smem_u32(dst)), "l"(map), "r"(c0), "r"(c1), "r"(smem_u32(bar)), "h"(mask) : "memory");
}
__device__ __forceinline__ void umma_commit_multicast(uint64_t* bar, uint16_t mask) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n" ::"r"(smem_u32(bar)),
                 "h"(mask) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}

template <int BN>
__global__ void __launch_bounds__(THREADS) gateup_silu_tc_cluster_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
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
    // pairs of tiles: (m tile 2 j + rank, n tile) for the two blocks of a cluster
    const int rank = blockIdx.x & 1, pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
    const int m_pairs = ((M + BM - 1) / BM + 1) / 2, n_tiles = (I + BN - 1) / BN, num_tiles = m_pairs * n_tiles;
    const int nkb = (K + BK - 1) / BK;

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full + s, 1); mbar_init(empty + s, 2); }  // a stage is free when both blocks' MMAs have read it
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
    cluster_sync_all();  // the other block's barriers are initialised before anything of this block can reach them
    pdl_trigger();

    if (warp == 0) {
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];\n" ::"l"(&tmap_x) : "memory");
            asm volatile("prefetch.tensormap [%0];\n" ::"l"(&tmap_w) : "memory");
            pdl_wait();  // the rows are what the kernel before this one wrote
            int g = 0;
            bool ok = true;
            for (int t = pair; t < num_tiles && ok; t += num_pairs) {
                const int m0 = (2 * (t % m_pairs) + rank) * BM, n0 = (t / m_pairs) * BN;
                for (int kb = 0; kb < nkb; ++kb, ++g) {
                    const int s = g % STAGES;
                    if (g >= STAGES && !mbar_wait(empty + s, ((g / STAGES) & 1) ^ 1, abort_flag, error_flag, 31)) { ok = false; break; }
                    unsigned char* st = tiles + s * STAGE_BYTES;
                    mbar_expect_tx(full + s, STAGE_BYTES);   // own token rows + both halves of the weights, whoever fetches them
                    tma_load_2d(st, &tmap_x, kb * BK, m0, full + s);
                    // this block's half of the weight rows, delivered to both blocks: gate rows from block 0, up rows from block 1
                    tma_load_2d_multicast(st + A_BYTES + rank * (B_BYTES / 2), &tmap_w, kb * BK, (rank ? I : 0) + n0, full + s, (uint16_t)3);
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
            for (int t = pair; t < num_tiles && ok; t += num_pairs, ++i) {
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
                    umma_commit_multicast(empty + s, (uint16_t)3);   // both blocks learn that this block has read the stage
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
        for (int t = pair; t < num_tiles && ok; t += num_pairs, ++i) {
            const int buf = i & 1;
            const int m = (2 * (t % m_pairs) + rank) * BM + row, n0 = (t / m_pairs) * BN;
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
    cluster_sync_all();  // the other block may still send copies and arrivals here until it has come this far too
}

inline int best_tile_width(long long m_pairs, int I, int pairs_at_once) {
    int best = 128;
    long long best_cost = -1;
    for (int bn = 128; bn >= 64; bn -= 16) {
        const long long tiles = m_pairs * ((I + bn - 1) / bn);
        const long long cost = ((tiles + pairs_at_once - 1) / pairs_at_once) * (bn + 8);
        if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = bn; }
    }
    return best;
}

template <int BN>
int launch_gateup_cluster(const bf16* x, const bf16* w, bf16* out, int M, int I, int K, int num_blocks, int* error_flag, cudaStream_t s) {
    CUtensorMap mx, mw;
    int rc = tensor_map(x, M, K, BM, &mx);
    if (rc) return rc;
    rc = tensor_map(w, 2 * I, K, BN, &mw);
    if (rc) return rc;
    constexpr size_t smem = (size_t)STAGES * (A_BYTES + 2 * BN * BK * 2) + 1024 + 256;
    static bool set = false;
    if (!set) {
        cudaError_t e = cudaFuncSetAttribute(gateup_silu_tc_cluster_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        set = true;
    }
    const long long pairs = (long long)(((M + BM - 1) / BM + 1) / 2) * ((I + BN - 1) / BN);
    const long long want = pairs < num_blocks / 2 ? pairs : num_blocks / 2;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(2 * want));
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = llmie_pdl_flag ? 2 : 1;
    return (int)cudaLaunchKernelEx(&cfg, gateup_silu_tc_cluster_kernel<BN>, mx, mw, out, M, I, K, error_flag);
}

}  // namespace

// As llmie_gateup_silu_tc; num_blocks is rounded down to an even number (clusters of two blocks).
LLMIE_API int llmie_gateup_silu_tc_cluster(const bf16* x, const bf16* w, bf16* out, int M, int I, int K, int num_blocks, int* error_flag,
                                           cudaStream_t s) {
    if (M <= 0 || I <= 0) return 0;
    if (K <= 0 || K % 8 || I % 8 || ((uintptr_t)x & 15) || ((uintptr_t)w & 15) || ((uintptr_t)out & 15) || !error_flag || num_blocks < 2)
        return LLMIE_ERR_BAD_ARGUMENT;
    switch (best_tile_width(((M + BM - 1) / BM + 1) / 2, I, num_blocks / 2)) {
        case 112: return launch_gateup_cluster<112>(x, w, out, M, I, K, num_blocks, error_flag, s);
        case 96: return launch_gateup_cluster<96>(x, w, out, M, I, K, num_blocks, error_flag, s);
        case 80: return launch_gateup_cluster<80>(x, w, out, M, I, K, num_blocks, error_flag, s);
        case 64: return launch_gateup_cluster<64>(x, w, out, M, I, K, num_blocks, error_flag, s);
        default: return launch_gateup_cluster<128>(x, w, out, M, I, K, num_blocks, error_flag, s);
    }
}
