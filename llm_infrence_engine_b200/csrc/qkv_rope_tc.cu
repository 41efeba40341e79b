// The q/k/v projection of prompt portions with bias, rotation and cache write in its epilogue, on the 5th-generation
// tensor cores of sm_100a (bfloat16, head size 64).
//
//   D [128 tokens x 128 outputs] = X [128 x K] W^T [K x 128]     tcgen05.mma, D in tensor memory (float32), X and W tiles of
//                                                                64 columns by TMA (128-byte swizzle) into a ring of STAGES
//
// 128 outputs are two heads. Row i of the tile is lane i of tensor memory and thread i of the block: a thread reads its
// token's two heads from tensor memory and has both partners (j, j + 32) of every rotation pair in its own registers. It adds
// the bias, rotates query and key heads by the token's angle, rounds to bfloat16 and writes the head's 128 bytes to the
// token's row of `out`; key and value heads go into the token's cache slot as well. The product is not rounded before bias
// and rotation (the library product followed by the rotation kernel rounds it to bfloat16 in between).
//
//   warps 0-3  the 128 row threads (epilogue)
//   warp 4     fetches the tiles, up to four boxes at a time from four lanes
//   warp 5     one lane issues the MMAs
//
// Every wait on an mbarrier is bounded: after SPIN_LIMIT polls the block records an error, the roles leave their loops,
// copies in flight are given (bounded) time to land, tensor memory is freed and the block returns.
#include "common.cuh"
#include "tcgen05.cuh"

namespace {

constexpr int D = 64, BM = 128, BN = 128, BK = 64, STAGES = 4, THREADS = 192;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, TMEM_COLS = 128;

struct QkvParams {
    const float* bias;      // [heads * D] or nullptr
    const float* cos_t;     // [tokens][D / 2]
    const float* sin_t;
    const int* slots;       // [tokens] page * page_size + offset, or negative: no cache write for this token
    bf16* out;              // [tokens][heads * D]
    bf16* k_pool;           // [pages][nkv][page_size][D]
    bf16* v_pool;
    int* error_flag;
    int M, K, nq, nkv, page_size, write_kv;
};

__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

__global__ void __launch_bounds__(THREADS, 1) qkv_rope_tc_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
                                                                 const QkvParams p) {
    extern __shared__ unsigned char raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~(uintptr_t)1023);
    unsigned char* a_s = base;                      // [STAGES] token tiles
    unsigned char* b_s = base + STAGES * A_BYTES;   // [STAGES] weight tiles
    uint64_t* full = reinterpret_cast<uint64_t*>(b_s + STAGES * B_BYTES);
    uint64_t* empty = full + STAGES;
    uint64_t* done = empty + STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(done + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile int* issued = abort_flag + 1;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n0 = blockIdx.x * BN, m0 = blockIdx.y * BM;
    const int nkb = (p.K + BK - 1) / BK;

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full + s, 1); mbar_init(empty + s, 1); }
        mbar_init(done, 1);
        *abort_flag = 0;
        *issued = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(tmem_slot)), "n"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    if (warp == 4 && lane == 0) {
        asm volatile("prefetch.tensormap [%0];\n" ::"l"(&tmap_x) : "memory");
        asm volatile("prefetch.tensormap [%0];\n" ::"l"(&tmap_w) : "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem = *tmem_slot;

    pdl_trigger();
    if (warp == 4) {
        // Issuing a TMA copy occupies its thread for hundreds of cycles whatever the box's size, so the boxes of a step are
        // issued by different lanes side by side. The weights do not depend on the kernel before: the first STAGES tiles
        // of them are on their way before the dependency wait, the tokens' tiles follow after it.
        const int early = nkb < STAGES ? nkb : STAGES;
        if (lane == 0)
            for (int kb = 0; kb < early; ++kb) mbar_expect_tx(full + kb, A_BYTES + B_BYTES);
        __syncwarp();
        if (lane < early) tma_load_2d(b_s + lane * B_BYTES, &tmap_w, lane * BK, n0, full + lane);
        pdl_wait();
        if (lane < early) tma_load_2d(a_s + lane * A_BYTES, &tmap_x, lane * BK, m0, full + lane);
        __syncwarp();
        if (lane == 0) *issued = early;
        // from then on two steps of the ring at a time: lane 0 waits for both stages and announces the bytes, lanes 0 .. 3
        // issue the two token tiles and the two weight tiles
        bool ok = true;
        for (int kb0 = STAGES; kb0 < nkb; kb0 += 2) {
            const int n = nkb - kb0 < 2 ? nkb - kb0 : 2;
            if (lane == 0) {
                for (int i = 0; i < n && ok; ++i) {
                    const int st = (kb0 + i) % STAGES;
                    ok = mbar_wait(empty + st, (((kb0 + i) / STAGES) & 1) ^ 1, abort_flag, p.error_flag, 21);
                    if (ok) mbar_expect_tx(full + st, A_BYTES + B_BYTES);
                }
            }
            ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
            if (!ok) break;
            if (lane < 2 * n) {
                const int kb = kb0 + (lane >> 1), st = kb % STAGES;
                if (lane & 1) tma_load_2d(b_s + st * B_BYTES, &tmap_w, kb * BK, n0, full + st);
                else tma_load_2d(a_s + st * A_BYTES, &tmap_x, kb * BK, m0, full + st);
            }
            __syncwarp();
            if (lane == 0) *issued = kb0 + n;
        }
    } else if (warp == 5) {
        pdl_wait();
        if (lane == 0) {
            constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
            bool ok = true;
            for (int kb = 0; kb < nkb && ok; ++kb) {
                const int st = kb % STAGES;
                ok = mbar_wait(full + st, (kb / STAGES) & 1, abort_flag, p.error_flag, 22);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const uint64_t a_desc = umma_desc(smem_u32(a_s + st * A_BYTES)), b_desc = umma_desc(smem_u32(b_s + st * B_BYTES));
#pragma unroll
                for (int k = 0; k < BK / 16; ++k) umma_bf16(tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                umma_commit(empty + st);
            }
            if (ok) umma_commit(done);
        }
    } else {
        // ---------------------------------------------------------------- the 128 row threads
        pdl_wait();  // the tables of angles and the cache slots come from kernels before this one
        const int t = m0 + tid;
        const bool row_ok = t < p.M;
        const int heads = p.nq + 2 * p.nkv;
        const uint32_t lane_base = tmem + ((uint32_t)(warp * 32) << 16);
        float cs[D / 2], sn[D / 2];
        if (row_ok) {
#pragma unroll
            for (int j = 0; j < D / 2; j += 4) {
                const float4 a = *reinterpret_cast<const float4*>(p.cos_t + (size_t)t * (D / 2) + j);
                const float4 b = *reinterpret_cast<const float4*>(p.sin_t + (size_t)t * (D / 2) + j);
                cs[j] = a.x; cs[j + 1] = a.y; cs[j + 2] = a.z; cs[j + 3] = a.w;
                sn[j] = b.x; sn[j + 1] = b.y; sn[j + 2] = b.z; sn[j + 3] = b.w;
            }
        } else {
#pragma unroll
            for (int j = 0; j < D / 2; ++j) { cs[j] = 1.f; sn[j] = 0.f; }
        }
        const int slot = (row_ok && p.write_kv) ? p.slots[t] : -1;
        const bool ok = __all_sync(0xffffffffu, mbar_wait(done, 0, abort_flag, p.error_flag, 23));
        if (ok) {
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
#pragma unroll 1   // (the two heads run the same code: half as much to fetch, and the second time it is there)
            for (int h = 0; h < BN / D; ++h) {
                const int head = n0 / D + h;
                uint32_t v[D];
                __syncwarp();  // the loads below are the whole warp's, whatever each lane's row did with the head before
#pragma unroll
                for (int j = 0; j < D; j += 16) tmem_ld16(lane_base + h * D + j, v + j);
                asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
                if (!row_ok || head >= heads) continue;
                float x[D];
#pragma unroll
                for (int j = 0; j < D; ++j) x[j] = __uint_as_float(v[j]);
                if (p.bias) {
#pragma unroll
                    for (int j = 0; j < D; j += 4) {
                        const float4 b = *reinterpret_cast<const float4*>(p.bias + (size_t)head * D + j);
                        x[j] += b.x; x[j + 1] += b.y; x[j + 2] += b.z; x[j + 3] += b.w;
                    }
                }
                if (head < p.nq + p.nkv) {  // queries and keys are rotated: pairs (j, j + D / 2)
#pragma unroll
                    for (int j = 0; j < D / 2; ++j) {
                        const float x1 = x[j], x2 = x[j + D / 2];
                        x[j] = x1 * cs[j] - x2 * sn[j];
                        x[j + D / 2] = x2 * cs[j] + x1 * sn[j];
                    }
                }
                uint4 packed[D / 8];
#pragma unroll
                for (int j = 0; j < D / 8; ++j)
                    packed[j] = make_uint4(pack2(x[8 * j], x[8 * j + 1]), pack2(x[8 * j + 2], x[8 * j + 3]), pack2(x[8 * j + 4], x[8 * j + 5]),
                                           pack2(x[8 * j + 6], x[8 * j + 7]));
                uint4* dst = reinterpret_cast<uint4*>(p.out + (size_t)t * heads * D + (size_t)head * D);
#pragma unroll
                for (int j = 0; j < D / 8; ++j) dst[j] = packed[j];
                if (head >= p.nq && slot >= 0) {
                    const bool is_key = head < p.nq + p.nkv;
                    const int kvh = is_key ? head - p.nq : head - p.nq - p.nkv;
                    const int page = slot / p.page_size, off = slot % p.page_size;
                    uint4* cell = reinterpret_cast<uint4*>((is_key ? p.k_pool : p.v_pool) + (((size_t)page * p.nkv + kvh) * p.page_size + off) * D);
#pragma unroll
                    for (int j = 0; j < D / 8; ++j) cell[j] = packed[j];
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (*abort_flag && tid == 0) {
        // gave up somewhere: let the copies that were started land before the block's shared memory goes away
        const int n_issued = *issued;
        for (int c = max(0, n_issued - STAGES); c < n_issued; ++c) {
            for (uint32_t i = 0; i < SPIN_LIMIT; ++i) {
                if (mbar_try_wait(full + c % STAGES, (c / STAGES) & 1)) break;
                __nanosleep(40);
            }
        }
    }
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "n"(TMEM_COLS) : "memory");
}

}  // namespace

// out [M][heads * 64] = rotate(x [M][K] w^T + bias), heads = nq + 2 nkv, w [heads * 64][K], both bfloat16 and row-major; the
// key and value heads of token t also go to the cache slot slots[t] (if write_kv and the slot is not negative). K must be a
// multiple of 8 (rows start on 16-byte boundaries), x, w and out 16-byte aligned; the error flag receives a wait's code.
LLMIE_API int llmie_qkv_rope_tc(const bf16* x, int M, int K, const bf16* w, const float* bias, const float* cos_t, const float* sin_t,
                                const int* slots, bf16* out, bf16* k_pool, bf16* v_pool, int nq, int nkv, int d, int page_size, int write_kv,
                                int* error_flag, cudaStream_t s) {
    if (M <= 0) return 0;
    const long long heads = (long long)nq + 2 * nkv;
    if (d != D || K <= 0 || K % 8 || nq <= 0 || nkv <= 0 || page_size <= 0 || !x || !w || !cos_t || !sin_t || !out || !error_flag ||
        ((uintptr_t)x & 15) || ((uintptr_t)w & 15) || ((uintptr_t)out & 15) || ((uintptr_t)cos_t & 15) || ((uintptr_t)sin_t & 15) ||
        ((uintptr_t)bias & 15) || (write_kv && (!slots || !k_pool || !v_pool || ((uintptr_t)k_pool & 15) || ((uintptr_t)v_pool & 15))) ||
        heads * D > 0x7fffffffLL)
        return LLMIE_ERR_BAD_ARGUMENT;
    QkvParams p;
    p.bias = bias; p.cos_t = cos_t; p.sin_t = sin_t; p.slots = slots; p.out = out; p.k_pool = k_pool; p.v_pool = v_pool;
    p.error_flag = error_flag; p.M = M; p.K = K; p.nq = nq; p.nkv = nkv; p.page_size = page_size; p.write_kv = write_kv;
    CUtensorMap mx, mw;
    int rc = tensor_map(x, M, K, BM, &mx);
    if (rc) return rc;
    rc = tensor_map(w, (int)(heads * D), K, BN, &mw);
    if (rc) return rc;
    constexpr size_t smem = (size_t)STAGES * (A_BYTES + B_BYTES) + 1024 + 256;
    static bool set = false;
    if (!set) {
        cudaError_t e = cudaFuncSetAttribute(qkv_rope_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        set = true;
    }
    const dim3 grid((unsigned)((heads * D + BN - 1) / BN), (unsigned)((M + BM - 1) / BM));
    if (grid.y > 65535) return LLMIE_ERR_BAD_ARGUMENT;
    return launch_kernel(qkv_rope_tc_kernel, grid, dim3(THREADS), smem, s, mx, mw, p);
}
