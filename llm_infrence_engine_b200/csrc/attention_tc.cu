// Paged attention for prompt portions on the 5th-generation tensor cores of sm_100a (head sizes 64 and 128, bfloat16).
//
// One block owns a tile of up to 128 query rows: 128 / G consecutive tokens of one request times the G query
// heads that share one key/value head. Row i of the tile is lane i of tensor memory and thread i of the block.
// The keys go by in chunks of 64:
//
//   S  = Q K^T        tcgen05.mma, A = Q tile (shared memory, K-major), B = key chunk (K-major), D = S in tensor
//                     memory [128 lanes x 64 columns, float32]; three S buffers (two for heads of 128), so the scores run
//                     ahead of the threads and never keep them waiting
//   P  = softmax step every thread reads ITS row of S with tcgen05.ld (no shuffles: one thread, one row), masks, keeps
//                     the running maximum and sum in 32-bit, and writes its row of P as bfloat16 back into tensor memory
//                     with tcgen05.st, over the scores it was made from (two values per column: 32 columns)
//   O += P V          tcgen05.mma with A = P FROM TENSOR MEMORY, B = value chunk as it lies in the cache ([key][dim]:
//                     MN-major), D = O in tensor memory, accumulated over all chunks. P is exp2(score - reference) with a
//                     reference that follows the row's running maximum lazily: only when the maximum has grown by more than
//                     2^8 over the reference does the thread scale its row of O (and its sum) down in tensor memory, between
//                     two P V products. Softmax does not depend on the reference, P stays below 2^8, and after the
//                     first chunks a row is hardly ever rescaled; O is read once, at the end. The MMAs of one thread run in
//                     the order they were issued, so the scores that overwrite a buffer cannot overtake the P V product
//                     that still reads P there
//
//   warps 0-3  the 128 row threads
//   warp 4     producer: looks up the pages of a chunk in the block table and fetches them by TMA (one box per page,
//              pool and block of 64 dims, 128-byte swizzle, no multicast) into two rings of STAGES buffers (keys, values)
//              guarded by mbarriers
//   warp 5     one lane issues the MMAs and commits them to the barriers the other warps wait on
//
// A launch follows a plan made once per step on the device (attn_tc_plan_kernel): which pieces of work there are (a tile,
// or one slice of a long tile's keys, whose partial result the last slice merges), long pieces first.
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

constexpr int BM = 128, BN = 64, THREADS = 192;
// What depends on the head size D (64 or 128). Operands lie in shared memory in blocks of 64 elements (128 bytes, the width
// of the swizzle) along D: a tile of Q or of keys is D / 64 such blocks one behind the other, a chunk of values likewise
// (its blocks are the MMA's N there). Two blocks share a multiprocessor: each has half of its tensor memory (256 columns:
// the score buffers, in which P takes the place of the scores it was made from, and the outputs) and up to 113 KB of its
// shared memory (the tile of Q and the two rings).
template <int D> struct Sizes {
    static constexpr int ATOMS = D / 64;
    static constexpr int STAGES = D == 64 ? 4 : 2;          // depth of the key ring and of the value ring
    static constexpr int S_BUFS = D == 64 ? 3 : 2;          // score buffers: the scores run S_BUFS - 1 chunks ahead of the softmax
    static constexpr int Q_BYTES = BM * D * 2, K_BYTES = BN * D * 2;
    static constexpr int TMEM_COLS = 256;                   // S buffers of 64 columns, then O [S_BUFS * 64, S_BUFS * 64 + D)
    static constexpr size_t SMEM = Q_BYTES + 2 * STAGES * K_BYTES + 1024 + 256;
};
constexpr float RESCALE_AFTER = 8.f;  // log2: a row's reference lags its running maximum by at most this much
constexpr float LOG2E = 1.4426950408889634f;

struct TcParams {
    const bf16* q;          // [tokens][q_stride], query heads first
    const int* block_table; // [table rows][max_blocks]
    const int* work;        // [items][8] = (tile, slice, slices of the tile, item of the tile's first slice, first token, tokens,
                            //               position of the first token, row of the block table); then the item count
    bf16* out;              // [tokens][nq * D]
    float* part_o;          // [items][nkv][BM][D]   scratch for tiles whose keys are cut into slices
    float* part_ml;         // [items][nkv][BM][2]
    int* counters;          // [tiles * nkv], zero between launches
    int max_items;
    int* error_flag;
    int q_stride, max_blocks, nq, nkv, page_size, window;
    int box_rows;           // rows per TMA box: min(page_size, BN)
    int num_tiles;
    float scale_log2;       // softmax scale * log2(e)
};

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

// Three-input maximum and the packed 32-bit forms of sm_100a (two independent float32 operations per instruction): the
// softmax step is bound by issue slots, and these halve the slots of its maxima, scalings and sums.
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;\n" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
__device__ __forceinline__ uint64_t pair_of(float lo, float hi) {
    uint64_t v;
    asm("mov.b64 %0, {%1, %2};\n" : "=l"(v) : "f"(lo), "f"(hi));
    return v;
}
__device__ __forceinline__ void unpair(uint64_t v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;\n" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;\n" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;\n" : "=l"(d) : "l"(a), "l"(b));
    return d;
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

// MN-major operand: [k][64 elements of 2 bytes] rows of 128 bytes, 128-byte swizzle, groups of 8 k-rows 1024 bytes apart;
// blocks of 64 columns `block_bytes` apart.
__device__ __forceinline__ uint64_t umma_desc_mn(uint32_t smem_addr, uint32_t block_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)(block_bytes >> 4) << 16;  // leading byte offset: between 64-element column blocks
    d |= (uint64_t)(1024 >> 4) << 32;  // stride byte offset: between groups of 8 k-rows
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// D += A B with A in tensor memory (128 lanes x K 16-bit elements, two per column) and B in shared memory.
__device__ __forceinline__ void umma_bf16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n" ::"r"(d_tmem),
                 "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}

template <int D>
__global__ void __launch_bounds__(THREADS, 2) attn_tc_prefill_kernel(const __grid_constant__ CUtensorMap tmap_k,
                                                                                          const __grid_constant__ CUtensorMap tmap_v, const TcParams p) {
    constexpr int ATOMS = Sizes<D>::ATOMS, STAGES = Sizes<D>::STAGES, Q_BYTES = Sizes<D>::Q_BYTES, K_BYTES = Sizes<D>::K_BYTES;
    constexpr int TMEM_COLS = Sizes<D>::TMEM_COLS, S_BUFS = Sizes<D>::S_BUFS;
    extern __shared__ unsigned char raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~(uintptr_t)1023);
    unsigned char* q_s = base;
    unsigned char* k_s = base + Q_BYTES;           // [STAGES] key chunks
    unsigned char* v_s = k_s + STAGES * K_BYTES;  // [STAGES] value chunks
    // Keys and values have rings of their own: a key chunk is free again as soon as its scores are made, long before the
    // values of the same chunk have been used, so the next keys are on their way that much earlier.
    uint64_t* k_full = reinterpret_cast<uint64_t*>(v_s + STAGES * K_BYTES);
    uint64_t* k_empty = k_full + STAGES;
    uint64_t* v_full = k_empty + STAGES;
    uint64_t* v_empty = v_full + STAGES;
    uint64_t* s_ready = v_empty + STAGES;  // [S_BUFS]
    uint64_t* p_ready = s_ready + S_BUFS;     // [2], taken in turn: the row threads may hand over P(c + 1) before the MMA thread has looked at P(c)'s barrier
    uint64_t* o_ready = p_ready + 2;     // completes once per chunk, after its P V product
    uint64_t* o_done = o_ready + 1;      // completes once, after the last chunk's P V product
    uint64_t* q_ready = o_done + 1;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(q_ready + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile int* issued = abort_flag + 1;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // Which piece of work this block takes: item blockIdx.x / nkv of the plan (a tile, or one slice of a tile's keys), for
    // key/value head blockIdx.x % nkv. The plan lists long pieces first; blocks beyond its end have nothing to do.
    const int item = blockIdx.x / p.nkv, kvh = blockIdx.x % p.nkv;

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(k_full + s, 1); mbar_init(k_empty + s, 1); mbar_init(v_full + s, 1); mbar_init(v_empty + s, 1); }
        for (int i = 0; i < S_BUFS; ++i) mbar_init(s_ready + i, 1);
        mbar_init(p_ready, BM / 32);  // one arrival per row warp
        mbar_init(p_ready + 1, BM / 32);
        mbar_init(o_ready, 1);
        mbar_init(o_done, 1);
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

    // everything about the piece comes in one trip to memory: the plan has looked up the tile, its position and its request
    const int4 job = *reinterpret_cast<const int4*>(p.work + 8 * item);
    const int4 where = *reinterpret_cast<const int4*>(p.work + 8 * item + 4);
    const bool idle = item >= p.work[8 * p.max_items];
    const int tile = idle ? 0 : job.x, split = idle ? 0 : job.y, num_splits = idle ? 1 : job.z;
    const int n0 = idle ? 0 : where.x;
    const int ntok = idle ? 0 : where.y;
    const int G = p.nq / p.nkv;
    const int nrows = ntok * G;  // <= BM
    const int pos0 = ntok > 0 ? where.z : 0;
    const int hi = pos0 + ntok;  // one past the last visible key
    const int lo = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
    const int lo_al = lo / p.box_rows * p.box_rows;  // chunks start where a TMA box starts
    // this block's slice of the tile's chunks: [chunk0, chunk0 + chunks), empty for the later slices of a short tile
    const int all_chunks = ntok > 0 ? (hi - lo_al + BN - 1) / BN : 0;
    const int per_split = (all_chunks + num_splits - 1) / num_splits;
    const int chunk0 = split * per_split;
    const int chunks = max(0, min(all_chunks, chunk0 + per_split) - chunk0);
    const int* table = p.block_table + (size_t)(ntok > 0 ? where.w : 0) * p.max_blocks;

    if (warp == 4) {
        // ---------------------------------------------------------------- producer
        const int boxes = BN / p.box_rows;  // per chunk and pool: 1, 2, 4 or 8
        // Where the boxes lie in the pool (rows of the [pages * heads * page_size, D] matrix). A look-up in the block table is a
        // trip to memory, and one per step would set the pace of the whole block. So the warp reads the table for 32 / boxes
        // chunks at once: lane i learns the row of box i % boxes of the (i / boxes)-th chunk of a group of chunks, one group
        // ahead of its use, and every step takes its rows from the lanes that hold them.
        const int box_shift = 31 - __clz(boxes), group_shift = 5 - box_shift;  // boxes and the group are powers of two
        const int group = 1 << group_shift, my_box = lane & (boxes - 1);
        auto group_rows = [&](int g) {
            const int cc = (g << group_shift) + (lane >> box_shift);
            const int key = lo_al + (chunk0 + cc) * BN + my_box * p.box_rows;
            const int page = (cc < chunks && key < hi) ? table[key / p.page_size] : 0;  // behind the sequence: any page, its keys are masked
            return (page * p.nkv + kvh) * p.page_size + key % p.page_size;
        };
        // The keys of chunk c are wanted a chunk earlier than its values (for the scores, made ahead of time) and their
        // stage is free earlier too (after the scores of chunk c - STAGES): step c of this loop fetches the keys of chunk c
        // and the values of chunk c - 1. Lanes 0 .. boxes-1 issue one key box each, the next `boxes` lanes one value box
        // each, all at once: issuing a TMA copy occupies a thread for hundreds of cycles, and a chunk of small pages has
        // many.
        bool ok = true;
        int rows_before = 0, rows_now = group_rows(0), rows_next = group_rows(1);
        for (int c = 0; c <= chunks && ok; ++c) {
            if (c > 0 && (c & (group - 1)) == 0) {
                rows_before = rows_now;
                rows_now = rows_next;
                rows_next = group_rows((c >> group_shift) + 1);
            }
            const bool keys = c < chunks, values = c > 0;
            const int kst = c % STAGES, vst = (c + STAGES - 1) % STAGES;  // stage of chunk c, of chunk c - 1
            const int row_k = __shfl_sync(0xffffffffu, rows_now, (((c & (group - 1)) << box_shift) + my_box) & 31);
            const int cv = c > 0 ? c - 1 : 0;
            const int row_v = __shfl_sync(0xffffffffu, (cv >> group_shift) == (c >> group_shift) ? rows_now : rows_before,
                                          (((cv & (group - 1)) << box_shift) + my_box) & 31);
            if (lane == 0) {
                // one lane speaks to the barriers: both stages must be free, then both are told what is coming
                if (keys && c >= STAGES) ok = mbar_wait(k_empty + kst, ((c / STAGES) & 1) ^ 1, abort_flag, p.error_flag, 11);
                if (ok && values && c - 1 >= STAGES) ok = mbar_wait(v_empty + vst, (((c - 1) / STAGES) & 1) ^ 1, abort_flag, p.error_flag, 11);
                if (ok && keys) mbar_expect_tx(k_full + kst, K_BYTES);
                if (ok && values) mbar_expect_tx(v_full + vst, K_BYTES);
            }
            ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
            if (!ok) break;
            // lane = (block of 64 dims) * boxes + box for the keys, the same again behind them for the values
            const int atom = (lane >> box_shift) % ATOMS;
            if (lane < boxes * ATOMS) {
                if (keys) tma_load_2d(k_s + kst * K_BYTES + atom * (BN * 128) + my_box * p.box_rows * 128, &tmap_k, atom * 64, row_k, k_full + kst);
            } else if (lane < 2 * boxes * ATOMS) {
                if (values) tma_load_2d(v_s + vst * K_BYTES + atom * (BN * 128) + my_box * p.box_rows * 128, &tmap_v, atom * 64, row_v, v_full + vst);
            }
            __syncwarp();
            if (lane == 0) { if (keys) issued[0] = c + 1; if (values) issued[1] = c; }
        }
    } else if (warp == 5) {
        // ---------------------------------------------------------------- MMA issuer
        if (lane == 0 && chunks > 0) {
            // D float32, A and B bfloat16, M = 128, N = 64; for P V the B operand (values) is MN-major
            constexpr uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
            constexpr uint32_t idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(D >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
            auto issue_s = [&](int c) {
                const uint32_t k_addr = smem_u32(k_s + (c % STAGES) * K_BYTES);
#pragma unroll
                for (int k = 0; k < D / 16; ++k)  // 16 dims per step: 32 bytes along a row, four steps per block of 64 dims
                    umma_bf16(tmem + (c % S_BUFS) * BN, umma_desc(smem_u32(q_s) + (k / 4) * (BM * 128)) + 2 * (k % 4),
                              umma_desc(k_addr + (k / 4) * (BN * 128)) + 2 * (k % 4), idesc_s, k > 0 ? 1u : 0u);
                umma_commit(s_ready + c % S_BUFS);
                umma_commit(k_empty + c % STAGES);
            };
            // Scores are made as early as their keys and a buffer allow: S(n) goes into the buffer in which P(n - S_BUFS) took the
            // place of S(n - S_BUFS); the product that reads that P was issued by this thread before, and a thread's MMAs run in
            // the order of their issue. After the last chunk comes one commit without a product: the rows wait for "S(c + 1)"
            // in every chunk (it tells them that the P V products up to chunk c - S_BUFS + 1 are over: a commit completes only
            // after everything this thread issued before it).
            int s_next = 0;
            auto more_scores = [&](int upto, bool wait) {
                while (s_next <= upto && s_next <= chunks) {
                    if (s_next < chunks) {
                        uint64_t* bar = k_full + s_next % STAGES;
                        const uint32_t parity = (s_next / STAGES) & 1;
                        if (wait) {
                            if (!mbar_wait(bar, parity, abort_flag, p.error_flag, 13)) return false;
                        } else if (!mbar_try_wait(bar, parity)) {
                            break;
                        }
                        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                        issue_s(s_next);
                    } else {
                        umma_commit(s_ready + s_next % S_BUFS);
                    }
                    ++s_next;
                    wait = false;
                }
                return true;
            };
            bool ok = mbar_wait(q_ready, 0, abort_flag, p.error_flag, 12) && more_scores(S_BUFS - 1, true);
            for (int c = 0; c < chunks && ok; ++c) {
                // Until P of this chunk is there: the scores of the chunks up to c + 2, as their keys land (the rows have handed
                // over P(c - 1), so the buffer of S(c - 1) is free). The rows wait for S(c + 1) before they hand over P(c), and
                // this loop is where it gets made. (Sleeping on one barrier after the other instead of polling all of them was
                // measured slower.)
                bool p_there = false;
                for (uint32_t i = 0; i < SPIN_LIMIT && !p_there; ++i) {
                    more_scores(c + S_BUFS - 1, false);
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
#pragma unroll
                for (int k = 0; k < BN / 16; ++k) {  // 16 keys per step: 32 bytes along a row of P, 2048 bytes down the values
                    // P lies where the chunk's scores lay: two bfloat16 per column, 8 columns per step
                    umma_bf16_ts(tmem + S_BUFS * BN, tmem + (c % S_BUFS) * BN + 8 * k, umma_desc_mn(v_addr + k * 2048, BN * 128), idesc_o, (c > 0 || k > 0) ? 1u : 0u);
                }
                umma_commit(o_ready);
                if (c == chunks - 1) umma_commit(o_done);
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
            for (int j = 0; j < D / 8; ++j) {
                const uint4 v = row_ok ? src[j] : make_uint4(0, 0, 0, 0);
                *reinterpret_cast<uint4*>(q_s + (j / 8) * (BM * 128) + row * 128 + (((j % 8) ^ (row & 7)) << 4)) = v;
            }
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(q_ready);
        }
        // m: the row's running maximum (log2 units); ref: what P is taken relative to (-inf until the row has seen a key);
        // l: the row's sum of P relative to ref
        float m = -INFINITY, ref = -INFINITY, l = 0.f;
        const uint32_t lane_base = tmem + ((uint32_t)(warp * 32) << 16);
        const uint32_t o_addr = lane_base + S_BUFS * BN;
        // the scores of chunk c are waited for during chunk c - 1 (see below): only the first ones here
        bool ok = chunks == 0 || __all_sync(0xffffffffu, mbar_wait(s_ready, 0, abort_flag, p.error_flag, 15));
        // The row's scores of a chunk are asked for at the end of the chunk before it (they are ready by then, see below), so
        // that their way from tensor memory lies under that chunk's fences, arrival and loop instead of at the head of the
        // next one; only the first chunk's are asked for here.
        uint32_t s[BN];
        if (ok && chunks > 0) {
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
#pragma unroll
            for (int j = 0; j < BN; j += 16) tmem_ld16(lane_base + j, s + j);
        }
        for (int c = 0; c < chunks && ok; ++c) {
            asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
            const int key0 = lo_al + (chunk0 + c) * BN;
            // A chunk that every row of the tile sees in full needs no mask arithmetic (rows beyond the tile have zero
            // queries and collect numbers nobody reads). The scale is positive: the maximum is taken over the raw scores.
            const bool interior = key0 >= lo && key0 + BN - 1 <= pos0 && (p.window <= 0 || key0 > hi - 1 - p.window);
            if (__builtin_expect(!interior, 0)) {
                // The columns this row sees are a run [first, last] of the chunk's 64: two words of bits say which, and a
                // column outside is replaced (not multiplied: the score may be NaN) by -inf. Written small (three
                // instructions a column) and marked unlikely: this code sits in the middle of the loop that every chunk runs,
                // and what the loop's instructions occupy of the instruction cache shows in its time.
                const int last = row_ok ? min(pos - key0, BN - 1) : -1;
                const int first = p.window > 0 ? max(pos - p.window + 1 - key0, 0) : 0;
                const uint64_t upto = last < 0 ? 0ull : (last >= 63 ? ~0ull : ((1ull << (last + 1)) - 1ull));
                const uint64_t seen = first >= 64 ? 0ull : upto & ~((1ull << first) - 1ull);
                const uint32_t seen_lo = (uint32_t)seen, seen_hi = (uint32_t)(seen >> 32);
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    if (!((seen_lo >> j) & 1u)) s[j] = 0xff800000u;
                    if (!((seen_hi >> j) & 1u)) s[32 + j] = 0xff800000u;
                }
            }
            // four running maxima and sums each: a single chain of 64 dependent operations would cost its latency 64 times
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int j = 0; j < BN; j += 8) {
#pragma unroll
                for (int k = 0; k < 4; ++k) mx4[k] = max3(mx4[k], __uint_as_float(s[j + k]), __uint_as_float(s[j + 4 + k]));
            }
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            m = fmaxf(m, mx * p.scale_log2);
            // The reference follows the maximum only when it lags too far behind: then this row of O and the row's sum are
            // scaled down. The first keys a row sees set its reference for free (everything so far was zero).
            float corr = 1.f;
            bool rescale = false;
            if (ref == -INFINITY) {
                ref = m;
            } else if (m - ref > RESCALE_AFTER) {
                corr = fast_exp2(ref - m);
                ref = m;
                rescale = true;
            }
            const float use = ref == -INFINITY ? 0.f : ref;
            // The scores of the next chunk (after the last chunk: a commit that stands for them): they are asked for at the end
            // of this chunk. They were issued after the P V product of chunk c - 2 (c - 1 with two score buffers), and a commit
            // completes only after everything issued before it: from here on the barrier of the P V products is at most one
            // phase behind, which the wait before a rescaling relies on. The scores themselves were made a chunk ago; this
            // wait hardly ever waits.
            ok = __all_sync(0xffffffffu, mbar_wait(s_ready + (c + 1) % S_BUFS, ((c + 1) / S_BUFS) & 1, abort_flag, p.error_flag, 15));
            if (!ok) break;
            if (__builtin_expect(__any_sync(0xffffffffu, rescale), 0)) {
                // O holds the products up to chunk c - 1 (there is one: a row's first chunk never gets here). The product
                // of chunk c waits for this chunk's P, so nothing else touches O meanwhile. (Sixteen columns at a time in a
                // loop that is not unrolled: after the first chunks this hardly ever runs, and it should take little room
                // in the loop that always does.)
                ok = __all_sync(0xffffffffu, mbar_wait(o_ready, (c - 1) & 1, abort_flag, p.error_flag, 16));
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
#pragma unroll 1
                for (int part = 0; part < D; part += 16) {
                    uint32_t v[16];
                    tmem_ld16(o_addr + part, v);
                    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
                    for (int i = 0; i < 16; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * corr);
                    tmem_st16(o_addr + part, v);
                }
                asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
            }
            // all 64 exponentials first, in place and independent of each other (the special-function unit is the narrow
            // place of this loop and must not wait for the sums and stores that follow)
            const uint64_t scale2 = pair_of(p.scale_log2, p.scale_log2), shift2 = pair_of(-use, -use);
#pragma unroll
            for (int j = 0; j < BN; j += 2) {
                float x0, x1;
                unpair(fma2(pair_of(__uint_as_float(s[j]), __uint_as_float(s[j + 1])), scale2, shift2), x0, x1);
                s[j] = __float_as_uint(fast_exp2(x0));
                s[j + 1] = __float_as_uint(fast_exp2(x1));
            }
            uint64_t sum2[2] = {pair_of(0.f, 0.f), pair_of(0.f, 0.f)};
#pragma unroll
            for (int j = 0; j < BN; j += 8) {
                float e[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) e[i] = __uint_as_float(s[j + i]);
                sum2[0] = add2(add2(sum2[0], pair_of(e[0], e[1])), pair_of(e[4], e[5]));
                sum2[1] = add2(add2(sum2[1], pair_of(e[2], e[3])), pair_of(e[6], e[7]));
                uint4 packed;
                packed.x = pack_bf16x2(e[0], e[1]); packed.y = pack_bf16x2(e[2], e[3]);
                packed.z = pack_bf16x2(e[4], e[5]); packed.w = pack_bf16x2(e[6], e[7]);
                // (s[0 .. j + 7] are spent: the packed P of columns j .. j + 7 moves into s[j / 2 .. j / 2 + 3])
                s[j / 2] = packed.x; s[j / 2 + 1] = packed.y; s[j / 2 + 2] = packed.z; s[j / 2 + 3] = packed.w;
            }
            // P into tensor memory, over the scores it was made from (this thread has read them all): 32 columns of two
            // bfloat16 each, the A operand of the P V product
            tmem_st16(lane_base + (c % S_BUFS) * BN, s);
            tmem_st16(lane_base + (c % S_BUFS) * BN + 16, s + 16);
            asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
            float sum4[4];
            unpair(sum2[0], sum4[0], sum4[1]);
            unpair(sum2[1], sum4[2], sum4[3]);
            l = l * corr + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
            if (key0 + BN > hi) {
                // the chunk reaches behind the last key: those value rows may hold anything; they become zeros
                unsigned char* v_c = v_s + (c % STAGES) * K_BYTES;
                const int first_bad = hi - key0;
                ok = __all_sync(0xffffffffu, mbar_wait(v_full + c % STAGES, (c / STAGES) & 1, abort_flag, p.error_flag, 18));  // the values have landed
                if (!ok) break;
                for (int i = tid; i < (BN - first_bad) * 8 * ATOMS; i += BM) {
                    const int in_block = i % ((BN - first_bad) * 8);  // which 16 bytes of the bad rows of a block of 64 dims
                    *reinterpret_cast<uint4*>(v_c + (i / ((BN - first_bad) * 8)) * (BN * 128) + (first_bad + (in_block >> 3)) * 128 + ((in_block & 7) << 4)) =
                        make_uint4(0, 0, 0, 0);
                }
            }
            if (key0 + BN > hi)
                asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");  // the zeros above: the tensor core reads shared memory through the async proxy
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            __syncwarp();  // every lane's writes (and reads of S) are done and fenced: one arrival speaks for the warp
            if (lane == 0) mbar_arrive(p_ready + (c & 1));
            if (c + 1 < chunks) {
                // S(c + 1) is complete (waited for above) and stays until S(c + 4) is made, which waits for P(c + 1)
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
#pragma unroll
                for (int j = 0; j < BN; j += 16) tmem_ld16(lane_base + ((c + 1) % S_BUFS) * BN + j, s + j);
            }
        }
        asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");  // (a loop left early may have a read in flight)
        // the row's outputs, once: everything the tensor core has added up, relative to ref like the sum; 64 at a time
        if (ok && chunks > 0) {
            ok = __all_sync(0xffffffffu, mbar_wait(o_done, 0, abort_flag, p.error_flag, 16));
            if (ok) asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        }
        // one slice of several: (max, sum, outputs) of the row go to shared memory (every product has been waited for and no
        // copy is in flight: the tiles' space is free), from where the whole block hands them on below
        float* fm = reinterpret_cast<float*>(q_s);
        float* fl = fm + BM;
        float* fo = fl + BM;
        if (ok && num_splits > 1) {
            fm[row] = ref;  // what the sum and the outputs are relative to
            fl[row] = l;
        }
        const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll 1
        for (int part = 0; part < D && ok; part += 64) {
            float o[64];
#pragma unroll
            for (int i = 0; i < 64; ++i) o[i] = 0.f;
            if (chunks > 0) {
                uint32_t v[64];
#pragma unroll
                for (int j = 0; j < 64; j += 16) tmem_ld16(o_addr + part + j, v + j);
                asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
                for (int i = 0; i < 64; ++i) o[i] = __uint_as_float(v[i]);
            }
            if (num_splits == 1) {
                if (row_ok) {
                    uint4* dst = reinterpret_cast<uint4*>(p.out + (size_t)(n0 + tok) * p.nq * D + (size_t)(kvh * G + row % G) * D + part);
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        uint4 packed;
                        packed.x = pack_bf16x2(o[8 * j] * inv, o[8 * j + 1] * inv); packed.y = pack_bf16x2(o[8 * j + 2] * inv, o[8 * j + 3] * inv);
                        packed.z = pack_bf16x2(o[8 * j + 4] * inv, o[8 * j + 5] * inv); packed.w = pack_bf16x2(o[8 * j + 6] * inv, o[8 * j + 7] * inv);
                        dst[j] = packed;
                    }
                }
            } else {
#pragma unroll
                for (int i = 0; i < 64; i += 4) *reinterpret_cast<float4*>(fo + row * D + part + i) = make_float4(o[i], o[i + 1], o[i + 2], o[i + 3]);
            }
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
    if (num_splits > 1 && !*abort_flag) {
        float* fm = reinterpret_cast<float*>(q_s);
        __shared__ int last_flag;
        finish_tile<D, BM, THREADS>(p, fm, fm + BM, fm + 2 * BM, num_splits, (size_t)job.w * p.nkv + kvh, (size_t)p.nkv, tile * p.nkv + kvh, kvh,
                                    split, n0, nrows, G, &last_flag, fm + 2 * BM + BM * D);
    }
}

// The plan of a launch: which tiles' keys are cut into how many slices, and in which order the pieces start.
//
// A tile's chunks run one after the other (about a microsecond each), so the longest tile sets the time of the launch while
// most SMs have long finished: a prompt's last tiles see all its keys, its first ones almost none. `capacity` pieces can be
// on the device at once (two blocks per SM, divided by the key/value heads that every piece is run for). The plan finds the
// smallest piece length L >= MIN_SLICE chunks for which cutting every tile into pieces of at most L chunks gives no more
// than `capacity` pieces. A slice costs about SLICE_COST chunks' time on top of its chunks (its partial result goes through
// memory and the last slice merges them), so tiles are only cut if L + SLICE_COST is less than the longest tile. The
// pieces are listed long tiles first, so that whatever does not fit at once starts in the order of its length.
// With fixed_splits > 0 every tile is cut into that many slices instead (empty ones included).
constexpr int MIN_SLICE = 8, SLICE_COST = 8, MAX_SLICES = 16, PLAN_THREADS = 256;

__global__ void __launch_bounds__(PLAN_THREADS) attn_tc_plan_kernel(const int* __restrict__ tile_info, int num_tiles, const int* __restrict__ positions,
                                                                    const int* __restrict__ token_seq, int window, int box_rows, int capacity, int fixed_splits, int max_items,
                                                                    int* __restrict__ work, int* __restrict__ tmp) {
    pdl_trigger();
    pdl_wait();
    __shared__ int red[PLAN_THREADS];
    __shared__ int piece;
    const int tid = threadIdx.x;
    int* chunks = tmp;               // [tiles]
    int* order = tmp + num_tiles;    // [tiles] tiles by falling length
    int* first = order + num_tiles;  // [tiles] item of the tile's first slice
    int longest = 0;
    for (int t = tid; t < num_tiles; t += PLAN_THREADS) {
        const int n0 = tile_info[2 * t], ntok = tile_info[2 * t + 1];
        int c = 0;
        if (ntok > 0) {
            const int pos0 = positions[n0], hi = pos0 + ntok;
            const int lo = window > 0 ? max(0, pos0 - window + 1) : 0;
            c = (hi - lo / box_rows * box_rows + BN - 1) / BN;
        }
        chunks[t] = c;
        longest = max(longest, c);
    }
    red[tid] = longest;
    __syncthreads();
    for (int w = PLAN_THREADS / 2; w > 0; w >>= 1) { if (tid < w) red[tid] = max(red[tid], red[tid + w]); __syncthreads(); }
    longest = red[0];
    __syncthreads();
    auto slices_of = [&](int c, int L) { return fixed_splits > 0 ? fixed_splits : max(1, min(MAX_SLICES, (c + L - 1) / L)); };
    auto pieces = [&](int L) {  // how many pieces a piece length of L gives (the same value in every thread)
        int n = 0;
        for (int t = tid; t < num_tiles; t += PLAN_THREADS) n += slices_of(chunks[t], L);
        red[tid] = n;
        __syncthreads();
        for (int w = PLAN_THREADS / 2; w > 0; w >>= 1) { if (tid < w) red[tid] += red[tid + w]; __syncthreads(); }
        n = red[0];
        __syncthreads();
        return n;
    };
    int lo_len = MIN_SLICE, hi_len = max(MIN_SLICE, longest);  // pieces(hi_len) is the number of tiles: the least there is
    if (fixed_splits <= 0 && pieces(hi_len) <= min(capacity, max_items)) {
        while (lo_len < hi_len) {
            const int mid = (lo_len + hi_len) / 2;
            if (pieces(mid) <= min(capacity, max_items)) hi_len = mid; else lo_len = mid + 1;
        }
    }
    if (tid == 0) piece = hi_len + SLICE_COST < longest ? hi_len : max(MIN_SLICE, longest);
    __syncthreads();
    const int L = piece;
    // Order: by falling number of chunks (ties by tile number; later tiles of a prompt are the longer ones). Every thread
    // ranks its tiles against all others; beyond a few thousand tiles the list stays in reverse tile order.
    const bool sort = fixed_splits <= 0 && num_tiles <= 2048;
    for (int t = tid; t < num_tiles; t += PLAN_THREADS) {
        int rank = num_tiles - 1 - t;
        if (sort) {
            rank = 0;
            const int c = chunks[t];
            for (int u = 0; u < num_tiles; ++u) rank += chunks[u] > c || (chunks[u] == c && u > t);
        }
        order[rank] = t;
    }
    __syncthreads();
    if (tid == 0) {
        int item = 0;
        for (int r = 0; r < num_tiles; ++r) {
            const int t = order[r];
            first[t] = item;
            item += slices_of(chunks[t], L);
        }
        work[8 * max_items] = min(item, max_items);
    }
    __syncthreads();
    for (int t = tid; t < num_tiles; t += PLAN_THREADS) {
        const int n = slices_of(chunks[t], L);
        const int n0 = tile_info[2 * t], ntok = tile_info[2 * t + 1];
        const int4 where = make_int4(n0, ntok, ntok > 0 ? positions[n0] : 0, ntok > 0 ? token_seq[n0] : 0);
        for (int k = 0; k < n; ++k) {
            const int item = first[t] + k;
            if (item < max_items) {
                *reinterpret_cast<int4*>(work + 8 * item) = make_int4(t, k, n, first[t]);
                *reinterpret_cast<int4*>(work + 8 * item + 4) = where;
            }
        }
    }
}

}  // namespace

// The plan for llmie_paged_attention_tc (see attn_tc_plan_kernel): work [8 * max_items + 1] receives the pieces and their number,
// tmp [3 * num_tiles] is scratch. capacity: pieces that can run at once. max_items >= num_tiles * max(1, fixed_splits).
LLMIE_API int llmie_attn_tc_plan(const int* tile_info, int num_tiles, const int* positions, const int* token_seq, int window, int page_size,
                                 int capacity, int fixed_splits, int max_items, int* work, int* tmp, cudaStream_t s) {
    if (num_tiles <= 0) return 0;
    if (!tile_info || !positions || !token_seq || !work || !tmp || page_size <= 0 || capacity <= 0 || fixed_splits < 0 || fixed_splits > MAX_SLICES ||
        max_items < (long long)num_tiles * (fixed_splits > 0 ? fixed_splits : 1) || ((uintptr_t)work & 15))
        return LLMIE_ERR_BAD_ARGUMENT;
    return launch_kernel(attn_tc_plan_kernel, dim3(1), dim3(PLAN_THREADS), 0, s, tile_info, num_tiles, positions, token_seq, window,
                         page_size < BN ? page_size : BN, capacity, fixed_splits, max_items, work, tmp);
}

// Attention of prompt portions over the paged cache on the tcgen05 tensor cores: head size d = 64 or 128, bfloat16, up to 128
// rows (tokens x heads of a group) per tile. page_size must be a multiple of 8 that divides 64 or is a multiple of 64. Pools:
// [pages][nkv][page_size][d]. `work` is the plan that llmie_attn_tc_plan made for the step's num_tiles tiles, its positions,
// this window and page size, with the same max_items. The slices of a tile meet in scratch_o [max_items * nkv * 128 * d]
// and scratch_ml [max_items * nkv * 128 * 2] floats; the block that finishes a tile last (counters [tiles * nkv], zero before and
// after) merges them.
LLMIE_API int llmie_paged_attention_tc(const bf16* q, int q_stride, const bf16* k_pool, const bf16* v_pool, long long pool_pages,
                                       const int* block_table, int max_blocks, int num_tiles, const int* work, int max_items, bf16* out, float* scratch_o,
                                       float* scratch_ml, int* counters, int nq, int nkv, int d, int page_size, float scale, int window,
                                       int* error_flag, cudaStream_t s) {
    if (num_tiles <= 0) return 0;
    if ((d != 64 && d != 128) || nkv <= 0 || nq % nkv || nq / nkv > BM || page_size <= 0 || page_size % 8 || q_stride % 8 ||
        !(BN % page_size == 0 || page_size % BN == 0) || !error_flag || pool_pages <= 0 || ((uintptr_t)q & 15) ||
        ((uintptr_t)out & 15) || pool_pages * nkv * page_size > 0x7fffffffLL || !work || ((uintptr_t)work & 15) || max_items < num_tiles ||
        !scratch_o || !scratch_ml || !counters)
        return LLMIE_ERR_BAD_ARGUMENT;
    TcParams p;
    p.q = q; p.block_table = block_table; p.work = work;
    p.out = out; p.error_flag = error_flag; p.part_o = scratch_o; p.part_ml = scratch_ml; p.counters = counters; p.max_items = max_items;
    p.q_stride = q_stride; p.max_blocks = max_blocks; p.nq = nq; p.nkv = nkv; p.page_size = page_size; p.num_tiles = num_tiles;
    p.window = window; p.box_rows = page_size < BN ? page_size : BN; p.scale_log2 = scale * LOG2E;
    CUtensorMap mk, mv;
    const int rows = (int)(pool_pages * nkv * page_size);
    int rc = tensor_map(k_pool, rows, d, p.box_rows, &mk);
    if (rc) return rc;
    rc = tensor_map(v_pool, rows, d, p.box_rows, &mv);
    if (rc) return rc;
    const long long blocks = (long long)max_items * nkv;
    if (blocks > 0x7fffffffLL) return LLMIE_ERR_BAD_ARGUMENT;
    static bool set[2] = {false, false};
    auto launch = [&](auto kernel, size_t smem, int which) -> int {
        if (!set[which]) {
            cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return (int)e;
            set[which] = true;
        }
        return launch_kernel(kernel, dim3((unsigned)blocks), dim3(THREADS), smem, s, mk, mv, p);
    };
    return d == 64 ? launch(attn_tc_prefill_kernel<64>, Sizes<64>::SMEM, 0) : launch(attn_tc_prefill_kernel<128>, Sizes<128>::SMEM, 1);
}
