// Paged attention for prompt portions on the 5th-generation tensor cores of sm_100a (head size 64, bfloat16).
//
// One block owns a tile of up to 128 query rows: 128 / G consecutive tokens of one request times the G query
// heads that share one key/value head. Row i of the tile is lane i of tensor memory and thread i of the block.
// The keys go by in chunks of 64:
//
//   S  = Q K^T        tcgen05.mma, A = Q tile (shared memory, K-major), B = key chunk (K-major), D = S in tensor
//                     memory [128 lanes x 64 columns, float32]; two S buffers, so the product for chunk c + 1 runs
//                     while the threads are busy with chunk c
//   P  = softmax step every thread reads ITS row of S with tcgen05.ld (no shuffles: one thread, one row), masks, keeps
//                     the running maximum and sum in 32-bit, and writes its row of P as bfloat16 into shared memory
//                     in the swizzled K-major layout an A operand has
//   O_c = P V         tcgen05.mma, A = P, B = value chunk as it lies in the cache ([key][dim]: MN-major), D = O_c in
//                     tensor memory; every thread reads its row of O_c and adds it to its 64 running outputs in
//                     registers, scaled by exp2(old maximum - new maximum). P and O_c have two buffers each: the
//                     threads go on to the scores of chunk c + 1 and pick up O_c after that
//
//   warps 0-3  the 128 row threads
//   warp 4     producer: looks up the pages of a chunk in the block table and fetches them by TMA (one box per page
//              and pool, 128-byte swizzle, no multicast) into two rings of STAGES buffers (keys, values) guarded by mbarriers
//   warp 5     one lane issues the MMAs and commits them to the barriers the other warps wait on
//
// Keys and values arrive exactly as the cache holds them, so a page's slots behind the sequence's last key may
// hold anything (another request's old values, NaN). Scores there are replaced (not multiplied) by -inf; the
// value rows there are set to zero in shared memory before the P V product reads them, because 0 * NaN is NaN.
//
// Every wait on an mbarrier is bounded: after SPIN_LIMIT polls the block records an error, every role leaves its
// loop, the copies in flight are given (bounded) time to land, tensor memory is freed and the block returns.
#include "common.cuh"
#include "attention_merge.cuh"
#include "tcgen05.cuh"

namespace {

constexpr int D = 64, BM = 128, BN = 64, STAGES = 3, THREADS = 192;  // STAGES: depth of the key ring and of the value ring
constexpr int Q_BYTES = BM * D * 2, P_BYTES = BM * BN * 2, K_BYTES = BN * D * 2;
constexpr int TMEM_COLS = 256;  // S0 [0, 64), S1 [64, 128), O0 [128, 192), O1 [192, 256)
constexpr float LOG2E = 1.4426950408889634f;

struct TcParams {
    const bf16* q;          // [tokens][q_stride], query heads first
    const int* block_table; // [table rows][max_blocks]
    const int* token_seq;   // [tokens] row of the block table
    const int* positions;   // [tokens]
    const int* tile_info;   // [tiles][2] = (first token, tokens)
    bf16* out;              // [tokens][nq * D]
    float* part_o;          // [tiles][nkv][splits][BM][D]   scratch for tiles whose keys are cut into slices
    float* part_ml;         // [tiles][nkv][splits][BM][2]
    int* counters;          // [tiles * nkv], zero between launches
    int num_splits;
    int* error_flag;
    int q_stride, max_blocks, nq, nkv, page_size, window;
    int box_rows;           // rows per TMA box: min(page_size, BN)
    int num_tiles, first_round;  // first_round: blocks that get an SM of their own (the number of SMs, or all blocks if fewer)
    float scale_log2;       // softmax scale * log2(e)
};

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

// MN-major operand: [k][64 elements of 2 bytes] rows of 128 bytes, 128-byte swizzle, groups of 8 k-rows 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc_mn(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)(1024 >> 4) << 16;  // leading byte offset: between 64-element column blocks (one block here: not used)
    d |= (uint64_t)(1024 >> 4) << 32;  // stride byte offset: between groups of 8 k-rows
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}

__global__ void __launch_bounds__(THREADS, 2) attn_tc_prefill_kernel(const __grid_constant__ CUtensorMap tmap_k,
                                                                     const __grid_constant__ CUtensorMap tmap_v, const TcParams p) {
    extern __shared__ unsigned char raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~(uintptr_t)1023);
    unsigned char* q_s = base;
    unsigned char* p_s = base + Q_BYTES;
    unsigned char* k_s = p_s + 2 * P_BYTES;      // [STAGES] key chunks; P has two buffers
    unsigned char* v_s = k_s + STAGES * K_BYTES;  // [STAGES] value chunks
    // Keys and values have rings of their own: a key chunk is free again as soon as its scores are made, long before the
    // values of the same chunk have been used, so the next keys are on their way that much earlier.
    uint64_t* k_full = reinterpret_cast<uint64_t*>(v_s + STAGES * K_BYTES);
    uint64_t* k_empty = k_full + STAGES;
    uint64_t* v_full = k_empty + STAGES;
    uint64_t* v_empty = v_full + STAGES;
    uint64_t* s_ready = v_empty + STAGES;  // [2]
    uint64_t* p_ready = s_ready + 2;     // [2]: the row threads may finish chunk c + 1 before the P V product of chunk c has begun
    uint64_t* o_ready = p_ready + 2;     // [2]
    uint64_t* q_ready = o_ready + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(q_ready + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile int* issued = abort_flag + 1;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // Which (tile, key/value head) this block takes. Later tiles of a prompt see more keys, so the list runs from the last
    // tile down; all blocks are resident at once (two to an SM), the first `first_round` one to an SM, the others beside
    // them in the same order of SMs: those take the list from its short end, so that every SM's two blocks add up alike.
    const int total = gridDim.x, b = blockIdx.x;
    const int work = b < p.first_round ? b : total - 1 - (b - p.first_round);
    const int split = work % p.num_splits, item = work / p.num_splits;
    const int tile = p.num_tiles - 1 - item / p.nkv;
    const int kvh = item % p.nkv;

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(k_full + s, 1); mbar_init(k_empty + s, 1); mbar_init(v_full + s, 1); mbar_init(v_empty + s, 1); }
        mbar_init(s_ready, 1);
        mbar_init(s_ready + 1, 1);
        mbar_init(p_ready, BM / 32);  // one arrival per row warp
        mbar_init(p_ready + 1, BM / 32);
        mbar_init(o_ready, 1);
        mbar_init(o_ready + 1, 1);
        mbar_init(q_ready, BM / 32);
        *abort_flag = 0;
        issued[0] = issued[1] = 0;  // key chunks, value chunks whose copies were started
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(tmem_slot)), "n"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    if (warp == 4 && lane == 0) {
        asm volatile("prefetch.tensormap [%0];\n" ::"l"(&tmap_k) : "memory");
        asm volatile("prefetch.tensormap [%0];\n" ::"l"(&tmap_v) : "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem = *tmem_slot;

    pdl_trigger();
    pdl_wait();  // queries, keys, values and the step's tables all come from kernels before this one

    const int n0 = p.tile_info[2 * tile];
    const int ntok = p.tile_info[2 * tile + 1];
    const int G = p.nq / p.nkv;
    const int nrows = ntok * G;  // <= BM
    const int pos0 = ntok > 0 ? p.positions[n0] : 0;
    const int hi = pos0 + ntok;  // one past the last visible key
    const int lo = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
    const int lo_al = lo / p.box_rows * p.box_rows;  // chunks start where a TMA box starts
    // this block's slice of the tile's chunks: [chunk0, chunk0 + chunks), empty for the later slices of a short tile
    const int all_chunks = ntok > 0 ? (hi - lo_al + BN - 1) / BN : 0;
    const int per_split = (all_chunks + p.num_splits - 1) / p.num_splits;
    const int chunk0 = split * per_split;
    const int chunks = max(0, min(all_chunks, chunk0 + per_split) - chunk0);
    const int* table = p.block_table + (size_t)(ntok > 0 ? p.token_seq[n0] : 0) * p.max_blocks;

    if (warp == 4) {
        // ---------------------------------------------------------------- producer
        const int boxes = BN / p.box_rows;  // per chunk and pool
        // Where box i of chunk c lies in the pool (a row of the [pages * heads * page_size, D] matrix): lane i finds out.
        auto box_row = [&](int c) {
            int row = 0;
            if (lane < boxes) {
                const int key = lo_al + (chunk0 + c) * BN + lane * p.box_rows;
                const int page = key < hi ? table[key / p.page_size] : 0;  // behind the sequence: any page, its keys are masked
                row = (page * p.nkv + kvh) * p.page_size + key % p.page_size;
            }
            return row;
        };
        // The keys of chunk c are wanted a chunk earlier than its values (for the scores, made ahead of time) and their
        // stage is free earlier too (after the scores of chunk c - STAGES): step c of this loop fetches the keys of chunk c
        // and the values of chunk c - 1. Lanes 0 .. boxes-1 issue one key box each, the next `boxes` lanes one value box
        // each, all at once: issuing a TMA copy occupies a thread for hundreds of cycles, and a chunk of small pages has
        // many. The block table is read one step ahead of its use.
        bool ok = true;
        int row_now = box_row(0), row_before = 0;
        for (int c = 0; c <= chunks && ok; ++c) {
            const int row_next = c + 1 < chunks ? box_row(c + 1) : 0;
            const bool keys = c < chunks, values = c > 0;
            const int kst = c % STAGES, vst = (c + STAGES - 1) % STAGES;  // stage of chunk c, of chunk c - 1
            if (lane == 0 && keys && c >= STAGES) ok = mbar_wait(k_empty + kst, ((c / STAGES) & 1) ^ 1, abort_flag, p.error_flag, 11);
            if (lane == boxes && values && c - 1 >= STAGES) ok = mbar_wait(v_empty + vst, (((c - 1) / STAGES) & 1) ^ 1, abort_flag, p.error_flag, 11);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            if (lane == 0 && keys) mbar_expect_tx(k_full + kst, K_BYTES);
            if (lane == boxes && values) mbar_expect_tx(v_full + vst, K_BYTES);
            const int row_v = __shfl_sync(0xffffffffu, row_before, (lane - boxes) & 31);
            __syncwarp();
            if (lane < boxes) {
                if (keys) tma_load_2d(k_s + kst * K_BYTES + lane * p.box_rows * 128, &tmap_k, 0, row_now, k_full + kst);
            } else if (lane < 2 * boxes) {
                if (values) tma_load_2d(v_s + vst * K_BYTES + (lane - boxes) * p.box_rows * 128, &tmap_v, 0, row_v, v_full + vst);
            }
            __syncwarp();
            if (lane == 0) { if (keys) issued[0] = c + 1; if (values) issued[1] = c; }
            row_before = row_now;
            row_now = row_next;
        }
    } else if (warp == 5) {
        // ---------------------------------------------------------------- MMA issuer
        if (lane == 0 && chunks > 0) {
            // D float32, A and B bfloat16, M = 128, N = 64; for P V the B operand (values) is MN-major
            constexpr uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
            constexpr uint32_t idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(D >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
            const uint64_t q_desc = umma_desc(smem_u32(q_s));
            auto issue_s = [&](int c) {
                const uint64_t k_desc = umma_desc(smem_u32(k_s + (c % STAGES) * K_BYTES));
#pragma unroll
                for (int k = 0; k < D / 16; ++k) umma_bf16(tmem + (c & 1) * BN, q_desc + 2 * k, k_desc + 2 * k, idesc_s, k > 0 ? 1u : 0u);
                umma_commit(s_ready + (c & 1));
                umma_commit(k_empty + c % STAGES);
            };
            bool ok = mbar_wait(q_ready, 0, abort_flag, p.error_flag, 12) && mbar_wait(k_full, 0, abort_flag, p.error_flag, 13);
            if (ok) {
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                issue_s(0);
            }
            int s_next = 1;  // the next chunk whose scores are to be made
            for (int c = 0; c < chunks && ok; ++c) {
                if (s_next == c) {
                    // the keys of this chunk had not come while the chunk before was waited for: now nothing else can go on
                    ok = mbar_wait(k_full + c % STAGES, (c / STAGES) & 1, abort_flag, p.error_flag, 13);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                    issue_s(s_next++);
                }
                // Until P of this chunk is there, make the scores of the next chunk as soon as its keys have landed, whichever
                // comes first. (S buffer (c + 1) & 1 held chunk c - 1, whose rows every thread had read before p_ready of c - 1.)
                bool p_there = false;
                for (uint32_t i = 0; i < SPIN_LIMIT && !p_there; ++i) {
                    if (s_next == c + 1 && s_next < chunks && mbar_try_wait(k_full + s_next % STAGES, (s_next / STAGES) & 1)) {
                        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                        issue_s(s_next++);
                    }
                    p_there = mbar_try_wait(p_ready + (c & 1), (c >> 1) & 1) && mbar_try_wait(v_full + c % STAGES, (c / STAGES) & 1);
                    if (*abort_flag) break;
                    if (!p_there && i > 64) __nanosleep(40);
                }
                if (!p_there) {
                    if (!*abort_flag) { *abort_flag = 1; atomicExch(p.error_flag, 14); }
                    ok = false;
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const uint32_t v_addr = smem_u32(v_s + (c % STAGES) * K_BYTES);
                const uint64_t p_desc = umma_desc(smem_u32(p_s + (c & 1) * P_BYTES));
#pragma unroll
                for (int k = 0; k < BN / 16; ++k)  // 16 keys per step: 32 bytes along a row of P, 2048 bytes down the values
                    umma_bf16(tmem + 2 * BN + (c & 1) * D, p_desc + 2 * k, umma_desc_mn(v_addr + k * 2048), idesc_o, k > 0 ? 1u : 0u);
                umma_commit(o_ready + (c & 1));
                umma_commit(v_empty + c % STAGES);
            }
        }
    } else {
        // ---------------------------------------------------------------- the 128 row threads
        const int row = tid;
        const bool row_ok = row < nrows;
        const int tok = row_ok ? row / G : 0;
        const int pos = pos0 + tok;
        {
            // this thread's query row into the swizzled tile (zeros for rows beyond the tile)
            const uint4* src = reinterpret_cast<const uint4*>(p.q + (size_t)(n0 + tok) * p.q_stride + (size_t)(kvh * G + (row_ok ? row % G : 0)) * D);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const uint4 v = row_ok ? src[j] : make_uint4(0, 0, 0, 0);
                *reinterpret_cast<uint4*>(q_s + row * 128 + ((j ^ (row & 7)) << 4)) = v;
            }
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(q_ready);
        }
        float o[D];
#pragma unroll
        for (int i = 0; i < D; ++i) o[i] = 0.f;
        float m = -INFINITY, l = 0.f;
        const uint32_t lane_base = tmem + ((uint32_t)(warp * 32) << 16);
        bool ok = true;
        float corr_before = 0.f;
        auto take_outputs = [&](int c, float corr) {
            if (!__all_sync(0xffffffffu, mbar_wait(o_ready + (c & 1), (c >> 1) & 1, abort_flag, p.error_flag, 16))) return false;
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            uint32_t v[D];
#pragma unroll
            for (int j = 0; j < D; j += 16) tmem_ld16(lane_base + 2 * BN + (c & 1) * D + j, v + j);
            asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
            for (int i = 0; i < D; ++i) o[i] = fmaf(o[i], corr, __uint_as_float(v[i]));
            return true;
        };
        for (int c = 0; c < chunks; ++c) {
            ok = __all_sync(0xffffffffu, mbar_wait(s_ready + (c & 1), (c >> 1) & 1, abort_flag, p.error_flag, 15));
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            uint32_t s[BN];
#pragma unroll
            for (int j = 0; j < BN; j += 16) tmem_ld16(lane_base + (c & 1) * BN + j, s + j);
            asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
            const int key0 = lo_al + (chunk0 + c) * BN;
            // A chunk that every row of the tile sees in full needs no mask arithmetic (rows beyond the tile have zero
            // queries and collect numbers nobody reads). The scale is positive: the maximum is taken over the raw scores.
            const bool interior = key0 >= lo && key0 + BN - 1 <= pos0 && (p.window <= 0 || key0 > hi - 1 - p.window);
            // four running maxima and sums each: a single chain of 64 dependent operations would cost its latency 64 times
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
            if (interior) {
#pragma unroll
                for (int j = 0; j < BN; ++j) mx4[j & 3] = fmaxf(mx4[j & 3], __uint_as_float(s[j]));
            } else {
#pragma unroll
                for (int j = 0; j < BN; ++j) {
                    const int key = key0 + j;
                    const bool seen = row_ok && key <= pos && (p.window <= 0 || key > pos - p.window);
                    const float x = seen ? __uint_as_float(s[j]) : -INFINITY;  // replaced, not multiplied: the score may be NaN
                    s[j] = __float_as_uint(x);
                    mx4[j & 3] = fmaxf(mx4[j & 3], x);
                }
            }
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            const float m_new = fmaxf(m, mx * p.scale_log2);
            const float use = m_new == -INFINITY ? 0.f : m_new;
            const float corr = fast_exp2(m - use);
            m = m_new;
            // all 64 exponentials first, in place and independent of each other (the special-function unit is the narrow
            // place of this loop and must not wait for the sums and stores that follow)
#pragma unroll
            for (int j = 0; j < BN; ++j) s[j] = __float_as_uint(fast_exp2(fmaf(__uint_as_float(s[j]), p.scale_log2, -use)));
            float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int j = 0; j < BN; j += 8) {
                float e[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) { e[i] = __uint_as_float(s[j + i]); sum4[i & 3] += e[i]; }
                uint4 packed;
                packed.x = pack_bf16x2(e[0], e[1]); packed.y = pack_bf16x2(e[2], e[3]);
                packed.z = pack_bf16x2(e[4], e[5]); packed.w = pack_bf16x2(e[6], e[7]);
                *reinterpret_cast<uint4*>(p_s + (c & 1) * P_BYTES + row * 128 + (((j >> 3) ^ (row & 7)) << 4)) = packed;
            }
            l = l * corr + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
            if (key0 + BN > hi) {
                // the chunk reaches behind the last key: those value rows may hold anything; they become zeros
                unsigned char* v_c = v_s + (c % STAGES) * K_BYTES;
                const int first_bad = hi - key0;
                ok = __all_sync(0xffffffffu, mbar_wait(v_full + c % STAGES, (c / STAGES) & 1, abort_flag, p.error_flag, 18));  // the values have landed
                if (!ok) break;
                for (int i = tid; i < (BN - first_bad) * 8; i += BM)
                    *reinterpret_cast<uint4*>(v_c + (first_bad + (i >> 3)) * 128 + ((i & 7) << 4)) = make_uint4(0, 0, 0, 0);
            }
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");  // the tensor core reads shared memory through the async proxy
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            __syncwarp();  // every lane's writes (and reads of S) are done and fenced: one arrival speaks for the warp
            if (lane == 0) mbar_arrive(p_ready + (c & 1));
            // The outputs of the chunk before are picked up now, while the tensor core is busy with this chunk's P V:
            // o = o * corr(c - 1) + O(c - 1), in the order of the chunks.
            if (c > 0) {
                ok = take_outputs(c - 1, corr_before);
                if (!ok) break;
            }
            corr_before = corr;
        }
        if (ok && chunks > 0) ok = take_outputs(chunks - 1, corr_before);
        if (ok && p.num_splits == 1) {
            if (row_ok) {
                const float inv = l > 0.f ? 1.f / l : 0.f;
                uint4* dst = reinterpret_cast<uint4*>(p.out + (size_t)(n0 + tok) * p.nq * D + (size_t)(kvh * G + row % G) * D);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    uint4 packed;
                    packed.x = pack_bf16x2(o[8 * j] * inv, o[8 * j + 1] * inv); packed.y = pack_bf16x2(o[8 * j + 2] * inv, o[8 * j + 3] * inv);
                    packed.z = pack_bf16x2(o[8 * j + 4] * inv, o[8 * j + 5] * inv); packed.w = pack_bf16x2(o[8 * j + 6] * inv, o[8 * j + 7] * inv);
                    dst[j] = packed;
                }
            }
        } else if (ok) {
            // one slice of several: (max, sum, outputs) of the row go to shared memory (every product has been waited for and
            // no copy is in flight: the tiles' space is free), from where the whole block hands them on below
            float* fm = reinterpret_cast<float*>(p_s);
            float* fl = fm + BM;
            float* fo = fl + BM;
            fm[row] = m;
            fl[row] = l;
#pragma unroll
            for (int i = 0; i < D; i += 4) *reinterpret_cast<float4*>(fo + row * D + i) = make_float4(o[i], o[i + 1], o[i + 2], o[i + 3]);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (*abort_flag && tid == 0) {
        // gave up somewhere: let the copies that were started land before the block's shared memory goes away
        for (int ring = 0; ring < 2; ++ring) {
            uint64_t* bars = ring == 0 ? k_full : v_full;
            const int n_issued = issued[ring];
            for (int c = max(0, n_issued - STAGES); c < n_issued; ++c) {
                for (uint32_t i = 0; i < SPIN_LIMIT; ++i) {
                    if (mbar_try_wait(bars + c % STAGES, (c / STAGES) & 1)) break;
                    __nanosleep(40);
                }
            }
        }
    }
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "n"(TMEM_COLS) : "memory");
    if (p.num_splits > 1 && !*abort_flag) {
        float* fm = reinterpret_cast<float*>(p_s);
        __shared__ int last_flag;
        finish_tile<D, BM, THREADS>(p, fm, fm + BM, fm + 2 * BM, tile, kvh, split, n0, nrows, G, &last_flag);
    }
}

}  // namespace

// Attention of prompt portions over the paged cache on the tcgen05 tensor cores: head size 64, bfloat16, up to 128 rows
// (tokens x heads of a group) per tile as listed in tile_info. page_size must be a multiple of 8 that divides 64 or is a
// multiple of 64. Pools: [pages][nkv][page_size][64]. With num_splits > 1 the keys of every tile are cut into that many slices,
// one block each, which meet in scratch_o [tiles * nkv * splits * 128 * 64] and scratch_ml [tiles * nkv * splits * 128 * 2]
// floats; the block that finishes a tile last (counters [tiles * nkv], zero before and after) merges them.
LLMIE_API int llmie_paged_attention_tc(const bf16* q, int q_stride, const bf16* k_pool, const bf16* v_pool, long long pool_pages,
                                       const int* block_table, int max_blocks, const int* token_seq, const int* positions,
                                       const int* tile_info, int num_tiles, bf16* out, float* scratch_o, float* scratch_ml, int* counters,
                                       int nq, int nkv, int d, int page_size, float scale, int window, int num_splits, int* error_flag,
                                       cudaStream_t s) {
    if (num_tiles <= 0) return 0;
    if (d != D || nkv <= 0 || nq % nkv || nq / nkv > BM || page_size <= 0 || page_size % 8 || q_stride % 8 ||
        !(BN % page_size == 0 || page_size % BN == 0) || !tile_info || !error_flag || pool_pages <= 0 || ((uintptr_t)q & 15) ||
        ((uintptr_t)out & 15) || pool_pages * nkv * page_size > 0x7fffffffLL || num_splits < 1 || num_splits > 16 ||
        (num_splits > 1 && (!scratch_o || !scratch_ml || !counters)))
        return LLMIE_ERR_BAD_ARGUMENT;
    TcParams p;
    p.q = q; p.block_table = block_table; p.token_seq = token_seq; p.positions = positions; p.tile_info = tile_info; p.out = out;
    p.error_flag = error_flag; p.part_o = scratch_o; p.part_ml = scratch_ml; p.counters = counters; p.num_splits = num_splits; p.q_stride = q_stride; p.max_blocks = max_blocks; p.nq = nq; p.nkv = nkv; p.page_size = page_size;
    p.window = window; p.box_rows = page_size < BN ? page_size : BN; p.scale_log2 = scale * LOG2E;
    CUtensorMap mk, mv;
    const int rows = (int)(pool_pages * nkv * page_size);
    int rc = tensor_map(k_pool, rows, D, p.box_rows, &mk);
    if (rc) return rc;
    rc = tensor_map(v_pool, rows, D, p.box_rows, &mv);
    if (rc) return rc;
    constexpr size_t smem = Q_BYTES + 2 * P_BYTES + 2 * STAGES * K_BYTES + 1024 + 256;
    static bool set = false;
    if (!set) {
        cudaError_t e = cudaFuncSetAttribute(attn_tc_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        set = true;
    }
    static int num_sms = 0;
    if (!num_sms) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return LLMIE_ERR_BAD_ARGUMENT;
    }
    const long long blocks = (long long)num_tiles * nkv * num_splits;
    if (blocks > 0x7fffffffLL) return LLMIE_ERR_BAD_ARGUMENT;
    p.num_tiles = num_tiles;
    p.first_round = blocks < num_sms ? (int)blocks : num_sms;
    return launch_kernel(attn_tc_prefill_kernel, dim3((unsigned)blocks), dim3(THREADS), smem, s, mk, mv, p);
}
