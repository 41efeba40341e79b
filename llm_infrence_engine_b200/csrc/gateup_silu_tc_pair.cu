// The gate/up product of prompt portions with silu(gate) * up as its epilogue (see gateup_silu_tc.cu, whose tiles, roles and
// epilogue this kernel shares), for PAIRS of multiprocessors working on one tile of 256 rows: tcgen05.mma with cta_group::2.
//
// The two blocks of a thread-block cluster own 128 rows each of a 256-row tile. One MMA instruction, issued by one thread of
// the first block (the leader), multiplies both blocks' token rows with ONE set of weight rows of which each block holds
// half in its shared memory: the leader the tile's gate rows, its peer the up rows. A K step therefore brings a block 16 KB
// of token rows and BN x 128 bytes of weights (32 KB at BN = 128) where the single-block kernel needs 48 KB for the same
// arithmetic per multiprocessor, and no copy is delivered twice (no multicast: every TMA copy goes to the shared memory of
// the block that issued it). That is what this product lacked: with 48 KB per 524 cycles of MMAs a multiprocessor must take
// in 92 bytes a cycle, more than it can; 61 bytes a cycle it can.
//
// What the pairing changes in the protocol:
//   * tensor memory is allocated, given up and freed with cta_group::2 by the same warp of both blocks;
//   * both blocks' TMA copies of a stage complete on the LEADER's "full" barrier (the copy is given the leader's barrier by
//     its address in the cluster; the leader's producer arms it with the bytes of both blocks);
//   * the leader's MMA thread frees a stage, and hands over an accumulator, in BOTH blocks by tcgen05.commit with a cluster
//     mask; the epilogue warps of both blocks give an accumulator back on the leader's barrier (a remote arrival);
//   * barriers are initialised before a cluster-wide barrier, and the blocks leave through another one.
// Each block's epilogue reads its own 128 rows of the accumulator from its own tensor memory, as before.
//
// Every wait on an mbarrier is bounded (tcgen05.cuh): a block that gives up sets the error flag, stops issuing, lets its
// copies land, and both blocks still meet at the final cluster barrier, free tensor memory and return.
#include "common.cuh"
#include "tcgen05.cuh"

namespace {

constexpr int BM = 128, BK = 64, UMMA_K = 16;
constexpr int A_BYTES = BM * BK * 2;
constexpr int EPI_THREADS = 128, THREADS = 64 + EPI_THREADS;

__device__ __forceinline__ uint32_t cluster_address_of(const void* own_smem, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(r) : "r"(smem_u32(own_smem)), "r"(rank));
    return r;
}
// A TMA copy into this block's shared memory whose bytes are counted on a barrier given by its cluster address (the leader's).
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, int c0, int c1, uint32_t bar_cluster_addr) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n" ::"r"(
                     smem_u32(dst)), "l"(map), "r"(c0), "r"(c1), "r"(bar_cluster_addr) : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(d_tmem),
                 "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// Arrives, once everything this thread has issued so far is complete, at the barrier of this offset in the blocks of `mask`.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar, uint16_t mask) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n" ::"r"(smem_u32(bar)),
                 "h"(mask) : "memory");
}
__device__ __forceinline__ void mbar_arrive_remote(uint32_t bar_cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];\n" ::"r"(bar_cluster_addr) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}

template <int BN, int STAGES>
__global__ void __launch_bounds__(THREADS) gateup_silu_tc_pair_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
                                                                       bf16* __restrict__ out, int M, int I, int K, int* error_flag) {
    constexpr int B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;   // this block's half of the weight rows of a K step
    extern __shared__ unsigned char raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* full = reinterpret_cast<uint64_t*>(tiles + STAGES * STAGE_BYTES);  // used in the leader only
    uint64_t* empty = full + STAGES;       // in both blocks: the MMAs that read the stage have finished
    uint64_t* acc_full = empty + STAGES;   // [2] in both blocks: the MMAs of a tile have finished
    uint64_t* acc_free = acc_full + 2;     // [2] used in the leader only: both blocks' epilogues have read the accumulator
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_free + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile int* issued = abort_flag + 1;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t rank = blockIdx.x & 1;   // clusters of two along x: block 2 j is the leader of pair j
    const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
    const int m_pairs = ((M + BM - 1) / BM + 1) / 2, n_tiles = (I + BN - 1) / BN, num_tiles = m_pairs * n_tiles;
    const int nkb = (K + BK - 1) / BK;

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full + s, 1); mbar_init(empty + s, 1); }
        for (int s = 0; s < 2; ++s) { mbar_init(acc_full + s, 1); mbar_init(acc_free + s, 2 * (EPI_THREADS / 32)); }
        *abort_flag = 0;
        *issued = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {  // the same warp of both blocks: the columns are the same in both
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(tmem_slot)), "n"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;\n" ::: "memory");
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
                const int m0 = (2 * (t % m_pairs) + (int)rank) * BM, n0 = (t / m_pairs) * BN;
                for (int kb = 0; kb < nkb; ++kb, ++g) {
                    const int s = g % STAGES;
                    if (g >= STAGES && !mbar_wait(empty + s, ((g / STAGES) & 1) ^ 1, abort_flag, error_flag, 41)) { ok = false; break; }
                    unsigned char* st = tiles + s * STAGE_BYTES;
                    const uint32_t leaders_full = cluster_address_of(full + s, 0);
                    if (rank == 0) mbar_expect_tx(full + s, 2 * STAGE_BYTES);   // what both blocks fetch for this stage
                    tma_load_2d_pair(st, &tmap_x, kb * BK, m0, leaders_full);
                    // the leader holds the gate rows of the tile's columns, its peer the up rows
                    tma_load_2d_pair(st + A_BYTES, &tmap_w, kb * BK, (rank ? I : 0) + n0, leaders_full);
                    *issued = g + 1;
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            // instruction descriptor: D float32, A and B bfloat16, both K-major, N = 2 BN (half of it from each block), M = 256
            constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)((2 * BN) >> 3) << 17) | ((uint32_t)((2 * BM) >> 4) << 24);
            int g = 0, i = 0;
            bool ok = true;
            for (int t = pair; t < num_tiles && ok; t += num_pairs, ++i) {
                const int buf = i & 1;
                if (i >= 2) ok = mbar_wait(acc_free + buf, ((i >> 1) & 1) ^ 1, abort_flag, error_flag, 42);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const uint32_t d = tmem + (uint32_t)(buf * 2 * BN);
                for (int kb = 0; kb < nkb; ++kb, ++g) {
                    const int s = g % STAGES;
                    ok = mbar_wait(full + s, (g / STAGES) & 1, abort_flag, error_flag, 43);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                    const uint32_t a_addr = smem_u32(tiles + s * STAGE_BYTES);
                    const uint64_t a_desc = umma_desc(a_addr), b_desc = umma_desc(a_addr + A_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) umma_bf16_pair(d, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    umma_commit_pair(empty + s, (uint16_t)3);   // the stage is free in both blocks
                }
                if (ok) umma_commit_pair(acc_full + buf, (uint16_t)3);
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue (both blocks, each its own 128 rows)
        const int quarter = warp & 3;               // the 32 lanes of tensor memory this warp may read
        const int row = quarter * 32 + lane;
        int i = 0;
        bool ok = true;
        for (int t = pair; t < num_tiles && ok; t += num_pairs, ++i) {
            const int buf = i & 1;
            const int m = (2 * (t % m_pairs) + (int)rank) * BM + row, n0 = (t / m_pairs) * BN;
            ok = __all_sync(0xffffffffu, mbar_wait(acc_full + buf, (i >> 1) & 1, abort_flag, error_flag, 44));
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
            if (lane == 0) mbar_arrive_remote(cluster_address_of(acc_free + buf, 0));
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (*abort_flag && tid == 0 && rank == 0) {
        // gave up somewhere: let the copies that were started land before the blocks' shared memory goes away (both blocks'
        // copies of a stage count on the leader's barrier, and the peer waits for the leader at the cluster barrier below)
        const int n_issued = *issued;
        for (int g = max(0, n_issued - STAGES); g < n_issued; ++g) {
            for (uint32_t i = 0; i < SPIN_LIMIT; ++i) {
                if (mbar_try_wait(full + g % STAGES, (g / STAGES) & 1)) break;
                __nanosleep(40);
            }
        }
    }
    cluster_sync_all();  // nobody frees tensor memory, or leaves, while the other block may still compute, copy or arrive here
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "n"(512) : "memory");
}

// The tile width with the fullest last round (see gateup_silu_tc.cu).
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
int launch_gateup_pair(const bf16* x, const bf16* w, bf16* out, int M, int I, int K, int num_blocks, int* error_flag, cudaStream_t s) {
    constexpr int STAGES = BN > 96 ? 6 : 7;   // 32 KB (BN = 128) to 24 KB (BN = 64) per stage
    CUtensorMap mx, mw;
    int rc = tensor_map(x, M, K, BM, &mx);
    if (rc) return rc;
    rc = tensor_map(w, 2 * I, K, BN, &mw);
    if (rc) return rc;
    constexpr size_t smem = (size_t)STAGES * (A_BYTES + BN * BK * 2) + 1024 + 256;
    static bool set = false;
    if (!set) {
        cudaError_t e = cudaFuncSetAttribute(gateup_silu_tc_pair_kernel<BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
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
    return (int)cudaLaunchKernelEx(&cfg, gateup_silu_tc_pair_kernel<BN, STAGES>, mx, mw, out, M, I, K, error_flag);
}

}  // namespace

// As llmie_gateup_silu_tc, by pairs of blocks on tiles of 256 rows; num_blocks is rounded down to an even number.
LLMIE_API int llmie_gateup_silu_tc_pair(const bf16* x, const bf16* w, bf16* out, int M, int I, int K, int num_blocks, int* error_flag,
                                        cudaStream_t s) {
    if (M <= 0 || I <= 0) return 0;
    if (K <= 0 || K % 8 || I % 8 || ((uintptr_t)x & 15) || ((uintptr_t)w & 15) || ((uintptr_t)out & 15) || !error_flag || num_blocks < 2)
        return LLMIE_ERR_BAD_ARGUMENT;
    switch (best_tile_width(((M + BM - 1) / BM + 1) / 2, I, num_blocks / 2)) {
        case 112: return launch_gateup_pair<112>(x, w, out, M, I, K, num_blocks, error_flag, s);
        case 96: return launch_gateup_pair<96>(x, w, out, M, I, K, num_blocks, error_flag, s);
        case 80: return launch_gateup_pair<80>(x, w, out, M, I, K, num_blocks, error_flag, s);
        case 64: return launch_gateup_pair<64>(x, w, out, M, I, K, num_blocks, error_flag, s);
        default: return launch_gateup_pair<128>(x, w, out, M, I, K, num_blocks, error_flag, s);
    }
}
