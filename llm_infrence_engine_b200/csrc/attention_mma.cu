// Paged grouped-query attention in bfloat16 on the tensor cores (mma.sync m16n8k16, 32-bit
// accumulators and a 32-bit online softmax), for head sizes 64 and 128.
//
// The rows of a tile are (token, query head of the group) pairs of ONE key/value head, token-major:
// row r is token n0 + r / G, head kvh * G + r % G (G = query heads per key/value head). All rows of
// a tile read the same keys and values, so a page is fetched once for the whole group.
//
//   decode kernel   one tile = up to 16 rows (one token of up to 16 heads, or a few tokens). The eight
//                   warps of a block split the KEYS: each warp streams its own 32-key (or 16-key)
//                   chunks through a private cp.async ring, keeps its own running (max, sum, output)
//                   and the warps are merged in shared memory at the end.
//   prefill kernel  one tile = up to 64 rows (64 / G consecutive tokens of one request). The four warps
//                   split the ROWS, 16 each; the block loads 64-key chunks together, double buffered.
//
// Both cut a tile's key range into `num_splits` slices (blockIdx.z). With more than one slice every
// block writes its partial (max, sum, output) to scratch; the block that arrives last at the tile's
// counter merges the slices and writes the output row, so no second kernel is needed. Keys are found
// through the request's block-table row, chunk by chunk; a query at position p sees keys
// max(0, p - window + 1) .. p, the mask is computed from positions, never stored.
#include <math.h>

#include "common.cuh"
#include "attention_merge.cuh"

namespace {

constexpr int WARPS = 4;
constexpr float LOG2E = 1.4426950408889634f;

struct Params {
    const bf16* q;          // [tokens][q_stride], query heads first
    const bf16* k_pool;     // [pages][nkv][page_size][D]
    const bf16* v_pool;
    const int* block_table; // [table rows][max_blocks]
    const int* token_seq;   // [tokens] row of the block table
    const int* positions;   // [tokens]
    const int* tile_info;   // [tiles][2] = (first token, tokens) or null: tile i is token i alone
    bf16* out;              // [tokens][nq * D]
    float* part_o;          // [tiles][nkv][splits][ROWS][D]
    float* part_ml;         // [tiles][nkv][splits][ROWS][2]
    int* counters;          // [tiles * nkv], zero between launches
    int q_stride, max_blocks, nq, nkv, page_size, window, num_splits;
    int page_shift;         // log2(page_size), or -1 if that is no power of two
    int cluster;            // 1: the slices of a tile are one thread-block cluster and merge through distributed shared memory
    float scale_log2;       // softmax scale * log2(e)
    // Decode steps may hand over the fused q/k/v projection as it leaves a split-K product: float32 sums that still lack the
    // bias and the rotation (`q` is then unused). The kernel finishes the queries in its own registers, and the one warp whose
    // keys include the token's own position finishes that key and value, puts them into its chunk and into the cache.
    const float* qkv_acc;   // [tokens][acc_stride]: query heads, key heads, value heads; or null
    const float* bias;      // [(nq + 2 nkv) * D] or null
    const float* cos_t;     // [tokens][D / 2]
    const float* sin_t;
    const int* slots;       // [tokens] cache slot (page * page_size + offset) of the token's own key and value; null: already cached
    bf16* k_pool_w;         // the pools again, to write into
    bf16* v_pool_w;
    int acc_stride;
};

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem) {
    const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem) {
    const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
__device__ __forceinline__ float ld_cluster(const float* local, int rank) {  // the same shared-memory word in block `rank` of the cluster
    uint32_t remote;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(remote) : "r"((uint32_t)__cvta_generic_to_shared(local)), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];\n" : "=f"(v) : "r"(remote));  // no memory clobber: loads may be in flight together
    return v;
}

// 2^x by the hardware's approximation unit (about two units in the last place; -inf gives 0): the softmax stays 32-bit.
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

// Element (row, col) of a [rows][D] bfloat16 tile in shared memory; 16-byte chunks of a row are
// permuted by the row's low bits so that the 8 rows one ldmatrix phase reads fall on different banks.
template <int D> __device__ __forceinline__ int swz(int row, int col) { return row * D + ((((col >> 3) ^ (row & 7)) << 3) | (col & 7)); }

// One warp copies NKEYS consecutive cache rows (keys key_abs0 .., clamped to last_key) into rows tile_row0 .. of a
// swizzled K tile and V tile. Every lane looks up the page of at most two keys; the row numbers then travel by
// shuffle to the lanes that copy that row's 16-byte pieces, 8 (or 16) neighbouring lanes per row.
template <int NKEYS>
struct PoolRows {
    int idx[(NKEYS + 31) / 32];  // lane l: row of key l (l + 32, ...) of the chunk in the [pages * heads * page_size, D] pool
};

// First half of a load: where the chunk's keys lie. A read of the block table that the copies depend on; a caller that can
// issues it well before `copy_rows_warp`, so that its latency passes while it does something else.
template <int NKEYS>
__device__ __forceinline__ PoolRows<NKEYS> find_rows_warp(const Params& p, const int* table, int kvh, int key_abs0, int last_key, int lane) {
    PoolRows<NKEYS> rows;
#pragma unroll
    for (int h = 0; h < (NKEYS + 31) / 32; ++h) {
        const int ka = min(key_abs0 + h * 32 + lane, last_key);
        const int pg = p.page_shift >= 0 ? ka >> p.page_shift : ka / p.page_size;  // page sizes are powers of two as a rule
        rows.idx[h] = (table[pg] * p.nkv + kvh) * p.page_size + (ka - pg * p.page_size);
    }
    return rows;
}

// Second half: the row numbers travel by shuffle to the lanes that copy that row's 16-byte pieces, 8 (or 16) neighbouring
// lanes per row, into the swizzled K tile and V tile.
template <int D, int NKEYS>
__device__ __forceinline__ void copy_rows_warp(const Params& p, const PoolRows<NKEYS>& rows, int tile_row0, bf16* ks, bf16* vs, int lane) {
    constexpr int CH = D / 8, KPI = 32 / CH;
    const int ch = lane % CH, sub = lane / CH;
#pragma unroll
    for (int i = 0; i < NKEYS / KPI; ++i) {
        const int key = i * KPI + sub;
        const int r = __shfl_sync(0xffffffffu, rows.idx[(i * KPI) >> 5], key & 31);
        const int trow = tile_row0 + key;
        const int dst = trow * D + ((ch ^ (trow & 7)) << 3);
        const size_t src = (size_t)r * D + ch * 8;
        cp_async16(ks + dst, p.k_pool + src);
        cp_async16(vs + dst, p.v_pool + src);
    }
}

template <int D, int NKEYS>
__device__ __forceinline__ void load_rows_warp(const Params& p, const int* table, int kvh, int key_abs0, int last_key, int tile_row0,
                                               bf16* ks, bf16* vs, int lane) {
    copy_rows_warp<D, NKEYS>(p, find_rows_warp<NKEYS>(p, table, kvh, key_abs0, last_key, lane), tile_row0, ks, vs, lane);
}

// One chunk of BN keys for one warp's 16 rows: S = Q K^T, masked online softmax, O += P V.
template <int D, int BN, bool MASKED = true>
__device__ __forceinline__ void attend_chunk(const uint32_t (&qa)[D / 16][4], const bf16* ks, const bf16* vs, float (&o)[D / 8][4],
                                             float (&m)[2], float (&l)[2], int key0, const int (&row_pos)[2], const bool (&row_ok)[2],
                                             int window, float scale_log2, int lane) {
    float s[BN / 8][4];
#pragma unroll
    for (int i = 0; i < BN / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
#pragma unroll
        for (int nt = 0; nt < BN / 16; ++nt) {
            uint32_t b[4];
            const int key = nt * 16 + (lane & 7) + ((lane >> 4) << 3);
            const int col = kk * 16 + (((lane >> 3) & 1) << 3);
            ldmatrix_x4(b, ks + swz<D>(key, col));
            mma_bf16(s[2 * nt], qa[kk], b[0], b[1]);
            mma_bf16(s[2 * nt + 1], qa[kk], b[2], b[3]);
        }
    }
    // mask and running maximum, in units of log2: x = s * scale * log2(e)
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < BN / 8; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int r = e >> 1;
            const int key = key0 + nt * 8 + ((lane & 3) << 1) + (e & 1);
            const bool ok = !MASKED || (row_ok[r] && key <= row_pos[r] && (window <= 0 || key > row_pos[r] - window));
            const float x = ok ? s[nt][e] * scale_log2 : -INFINITY;
            s[nt][e] = x;
            mx[r] = fmaxf(mx[r], x);
        }
    }
    float corr[2], use[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        const float m_new = fmaxf(m[r], mx[r]);
        use[r] = m_new == -INFINITY ? 0.f : m_new;
        corr[r] = fast_exp2(m[r] - use[r]);
        m[r] = m_new;
        l[r] *= corr[r];
    }
#pragma unroll
    for (int dt = 0; dt < D / 8; ++dt) {
        o[dt][0] *= corr[0]; o[dt][1] *= corr[0];
        o[dt][2] *= corr[1]; o[dt][3] *= corr[1];
    }
    uint32_t pa[BN / 16][4];
#pragma unroll
    for (int nt = 0; nt < BN / 8; ++nt) {
        const float p0 = fast_exp2(s[nt][0] - use[0]), p1 = fast_exp2(s[nt][1] - use[0]);
        const float p2 = fast_exp2(s[nt][2] - use[1]), p3 = fast_exp2(s[nt][3] - use[1]);
        l[0] += p0 + p1;
        l[1] += p2 + p3;
        pa[nt >> 1][(nt & 1) * 2] = pack_bf16(p0, p1);
        pa[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16(p2, p3);
    }
#pragma unroll
    for (int kk = 0; kk < BN / 16; ++kk) {
#pragma unroll
        for (int dt = 0; dt < D / 16; ++dt) {
            uint32_t b[4];
            const int key = kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
            const int col = dt * 16 + ((lane >> 4) << 3);
            ldmatrix_x4_trans(b, vs + swz<D>(key, col));
            mma_bf16(o[2 * dt], pa[kk], b[0], b[1]);
            mma_bf16(o[2 * dt + 1], pa[kk], b[2], b[3]);
        }
    }
}


// The same for tiles of at most 8 rows (a decoded token's heads of one group), computed TRANSPOSED so that no tensor-core work
// goes to padding rows: S^T = K Q^T (m16n8k16 with the 16 KEYS as M, the 8 rows as N) and O^T = V^T P^T (16 dims as M).
// Per lane: scores of keys lane / 4 (+ 8) and rows 2 (lane % 4), + 1; P^T goes from accumulator to B-operand layout by
// transposing 8 x 8 blocks across the warp (movmatrix). Half the MMAs, exponentials and registers of attend_chunk.
//   qb[kk][h]   Q^T as B operand: row lane / 4, dims kk * 16 + 2 (lane % 4) + {0, 1} (+ 8 h)
//   ot[dt][e]   O^T: dim dt * 16 + lane / 4 + 8 (e >> 1), row 2 (lane % 4) + (e & 1)
//   m[j], l[j]  of row 2 (lane % 4) + j; l holds this lane's keys only until the caller sums it over lanes 4, 8, 16 apart
__device__ __forceinline__ uint32_t transpose_8x8(uint32_t a) {
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(d) : "r"(a));
    return d;
}

template <int D, int BN, bool MASKED>
__device__ __forceinline__ void attend_chunk_t8(const uint32_t (&qb)[D / 16][2], const bf16* ks, const bf16* vs, float (&ot)[D / 16][4],
                                                float (&m)[2], float (&l)[2], int key0, int pos, int nrows, int window, float scale_log2,
                                                int lane) {
    float st[BN / 16][4];
#pragma unroll
    for (int kt = 0; kt < BN / 16; ++kt) {
        st[kt][0] = st[kt][1] = st[kt][2] = st[kt][3] = 0.f;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
            uint32_t b[4];
            const int key = kt * 16 + (lane & 7) + ((lane >> 4) << 3);
            const int col = kk * 16 + (((lane >> 3) & 1) << 3);
            ldmatrix_x4(b, ks + swz<D>(key, col));  // (keys 0-7, dims 0-7), (0-7, 8-15), (8-15, 0-7), (8-15, 8-15)
            const uint32_t a[4] = {b[0], b[2], b[1], b[3]};
            mma_bf16(st[kt], a, qb[kk][0], qb[kk][1]);
        }
    }
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int kt = 0; kt < BN / 16; ++kt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int key = key0 + kt * 16 + (lane >> 2) + ((e >> 1) << 3);
            const bool ok = !MASKED || (((lane & 3) << 1) + (e & 1) < nrows && key <= pos && (window <= 0 || key > pos - window));
            const float x = ok ? st[kt][e] * scale_log2 : -INFINITY;
            st[kt][e] = x;
            mx[e & 1] = fmaxf(mx[e & 1], x);
        }
    }
    float corr[2], use[2];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        mx[j] = fmaxf(mx[j], __shfl_xor_sync(0xffffffffu, mx[j], 4));
        mx[j] = fmaxf(mx[j], __shfl_xor_sync(0xffffffffu, mx[j], 8));
        mx[j] = fmaxf(mx[j], __shfl_xor_sync(0xffffffffu, mx[j], 16));
        const float m_new = fmaxf(m[j], mx[j]);
        use[j] = m_new == -INFINITY ? 0.f : m_new;
        corr[j] = fast_exp2(m[j] - use[j]);
        m[j] = m_new;
        l[j] *= corr[j];
    }
#pragma unroll
    for (int dt = 0; dt < D / 16; ++dt) {
        ot[dt][0] *= corr[0]; ot[dt][1] *= corr[1];
        ot[dt][2] *= corr[0]; ot[dt][3] *= corr[1];
    }
    uint32_t pb[BN / 16][2];
#pragma unroll
    for (int kt = 0; kt < BN / 16; ++kt) {
        const float p0 = fast_exp2(st[kt][0] - use[0]), p1 = fast_exp2(st[kt][1] - use[1]);
        const float p2 = fast_exp2(st[kt][2] - use[0]), p3 = fast_exp2(st[kt][3] - use[1]);
        l[0] += p0 + p2;
        l[1] += p1 + p3;
        pb[kt][0] = transpose_8x8(pack_bf16(p0, p1));  // keys 0-7 of the tile: [key][row] -> [row][key]
        pb[kt][1] = transpose_8x8(pack_bf16(p2, p3));  // keys 8-15
    }
#pragma unroll
    for (int dt = 0; dt < D / 16; ++dt) {
#pragma unroll
        for (int kt = 0; kt < BN / 16; ++kt) {
            uint32_t b[4];
            const int key = kt * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
            const int col = dt * 16 + ((lane >> 4) << 3);
            ldmatrix_x4_trans(b, vs + swz<D>(key, col));  // transposed: (dims 0-7, keys 0-7), (0-7, 8-15), (8-15, 0-7), (8-15, 8-15)
            const uint32_t a[4] = {b[0], b[2], b[1], b[3]};
            mma_bf16(ot[dt], a, pb[kt][0], pb[kt][1]);
        }
    }
}

// ---------------------------------------------------------------------------------------------- decode
// T8: every tile has at most 8 rows and one token (a decode step of a model with up to 8 heads per group): the transposed form.
template <int D, int BN, int STAGES, int DW, bool T8>
__global__ void __launch_bounds__(DW * 32) attn_mma_decode_kernel(const Params p) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    constexpr int TILE = BN * D;                       // elements of one K or V chunk
    bf16* my = reinterpret_cast<bf16*>(smem_raw) + (size_t)warp * STAGES * 2 * TILE;
    __shared__ int flag;

    const int tile = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
    pdl_trigger();
    // What this block needs of the step's own integers (positions, table rows, block tables) was copied to the device
    // before the step's first kernel, and keys and values of earlier positions were written by earlier steps: none of it
    // depends on the kernels just before this one. So when tile i is simply token i, the block finds its key range and
    // starts fetching its first chunks BEFORE the wait; only chunks that reach the new positions, and the queries, which
    // the rotation kernel has just written, come after it.
    const bool early = p.tile_info == nullptr;
    if (!early) pdl_wait();
    const int n0 = p.tile_info ? p.tile_info[2 * tile] : tile;
    const int ntok = p.tile_info ? p.tile_info[2 * tile + 1] : 1;
    const int G = p.nq / p.nkv;
    const int nrows = ntok * G;  // <= 16
    const int pos0 = p.positions[n0];
    const int* table = p.block_table + (size_t)p.token_seq[n0] * p.max_blocks;
    const int hi = pos0 + ntok;  // one past the last visible key
    const int lo = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
    const int chunks = (hi - lo + BN - 1) / BN;
    const int per = (chunks + p.num_splits - 1) / p.num_splits;
    const int c_begin = split * per, c_end = min(chunks, c_begin + per);

    // this warp's chunks: c_begin + warp, + DW, ...
    const int first = c_begin + warp;
    const int mine = first < c_end ? (c_end - first + DW - 1) / DW : 0;
    // All STAGES slots of the ring are filled up front; a slot is filled again right AFTER its chunk has been used, so the
    // instructions that issue a copy never stand between a landed chunk and its arithmetic.
    bool fetched[STAGES];
#pragma unroll
    for (int s = 0; s < STAGES; ++s) {
        const int key0 = lo + (first + s * DW) * BN;
        fetched[s] = early && s < mine && key0 + BN <= pos0;  // wholly before the first new position
        if (fetched[s]) load_rows_warp<D, BN>(p, table, kvh, key0, hi - 1, 0, my + s * 2 * TILE, my + s * 2 * TILE + TILE, lane);
    }
    if (early) pdl_wait();

    int row_pos[2];
    bool row_ok[2];
    uint32_t qa[T8 ? 1 : D / 16][4];   // the queries as A operand (rows lane / 4 and + 8), or ...
    uint32_t qb[T8 ? D / 16 : 1][2];   // ... transposed, as B operand (row lane / 4 only)
    float o[T8 ? D / 16 : D / 8][4];
    // (from the projection's sums) the token's own key and value, finished by the warp that owns its position: pairs
    // (j, j + D / 2) for j = lane, lane + 32, ...
    constexpr int NP = D / 64;
    int own_it = -1;
    uint32_t own_k[NP], own_v[NP];   // (element j, element j + D / 2) as two bfloat16
    if constexpr (T8) {
        const int row = lane >> 2;
        const bool ok = row < nrows;
        if (p.qkv_acc) {
            const int head = kvh * G + (ok ? row : 0);
            const float* src = p.qkv_acc + (size_t)n0 * p.acc_stride + (size_t)head * D;
            const float* ct = p.cos_t + (size_t)n0 * (D / 2);
            const float* sn = p.sin_t + (size_t)n0 * (D / 2);
            float x[D / 16][4];
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
                const int col = kk * 16 + ((lane & 3) << 1);
                const float2 a = __ldcg(reinterpret_cast<const float2*>(src + col)), c = __ldcg(reinterpret_cast<const float2*>(src + col + 8));
                x[kk][0] = a.x; x[kk][1] = a.y; x[kk][2] = c.x; x[kk][3] = c.y;
                if (p.bias) {
                    const float2 ba = *reinterpret_cast<const float2*>(p.bias + (size_t)head * D + col);
                    const float2 bc = *reinterpret_cast<const float2*>(p.bias + (size_t)head * D + col + 8);
                    x[kk][0] += ba.x; x[kk][1] += ba.y; x[kk][2] += bc.x; x[kk][3] += bc.y;
                }
            }
#pragma unroll
            for (int kk = 0; kk < D / 32; ++kk) {   // dims of the first half and their partners D / 2 further on, both in this lane
                const int col = kk * 16 + ((lane & 3) << 1);
                const float2 c0 = *reinterpret_cast<const float2*>(ct + col), c1 = *reinterpret_cast<const float2*>(ct + col + 8);
                const float2 s0 = *reinterpret_cast<const float2*>(sn + col), s1 = *reinterpret_cast<const float2*>(sn + col + 8);
                const float cs[4] = {c0.x, c0.y, c1.x, c1.y}, ss[4] = {s0.x, s0.y, s1.x, s1.y};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float x1 = x[kk][e], x2 = x[kk + D / 32][e];
                    x[kk][e] = x1 * cs[e] - x2 * ss[e];
                    x[kk + D / 32][e] = x2 * cs[e] + x1 * ss[e];
                }
            }
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
                qb[kk][0] = ok ? pack_bf16(x[kk][0], x[kk][1]) : 0u;
                qb[kk][1] = ok ? pack_bf16(x[kk][2], x[kk][3]) : 0u;
            }
            if (p.slots) {
                const int c_p = (pos0 - lo) / BN;   // the chunk that holds the token's own position
                if (c_p >= c_begin && c_p < c_end && (c_p - c_begin) % DW == warp) own_it = (c_p - first) / DW;
            }
            if (own_it >= 0) {
                const float* ks_ = p.qkv_acc + (size_t)n0 * p.acc_stride + (size_t)(p.nq + kvh) * D;
                const float* vs_ = p.qkv_acc + (size_t)n0 * p.acc_stride + (size_t)(p.nq + p.nkv + kvh) * D;
                const float* kb = p.bias ? p.bias + (size_t)(p.nq + kvh) * D : nullptr;
                const float* vb = p.bias ? p.bias + (size_t)(p.nq + p.nkv + kvh) * D : nullptr;
                const int slot = p.slots[n0];
                const int page = slot >= 0 ? slot / p.page_size : 0, off = slot >= 0 ? slot - page * p.page_size : 0;
                const size_t dst = (((size_t)page * p.nkv + kvh) * p.page_size + off) * D;
#pragma unroll
                for (int i = 0; i < NP; ++i) {
                    const int j = lane + 32 * i;
                    float k1 = __ldcg(ks_ + j), k2 = __ldcg(ks_ + j + D / 2), v1 = __ldcg(vs_ + j), v2 = __ldcg(vs_ + j + D / 2);
                    if (p.bias) { k1 += kb[j]; k2 += kb[j + D / 2]; v1 += vb[j]; v2 += vb[j + D / 2]; }
                    const float c = ct[j], sv = sn[j];
                    const __nv_bfloat16 r1 = __float2bfloat16_rn(k1 * c - k2 * sv), r2 = __float2bfloat16_rn(k2 * c + k1 * sv);
                    const __nv_bfloat16 w1 = __float2bfloat16_rn(v1), w2 = __float2bfloat16_rn(v2);
                    own_k[i] = (uint32_t)__bfloat16_as_ushort(r1) | ((uint32_t)__bfloat16_as_ushort(r2) << 16);
                    own_v[i] = (uint32_t)__bfloat16_as_ushort(w1) | ((uint32_t)__bfloat16_as_ushort(w2) << 16);
                    if (slot >= 0) {
                        p.k_pool_w[dst + j] = r1; p.k_pool_w[dst + j + D / 2] = r2;
                        p.v_pool_w[dst + j] = w1; p.v_pool_w[dst + j + D / 2] = w2;
                    }
                }
            }
        } else {
            const bf16* qp = p.q + (size_t)n0 * p.q_stride + (size_t)(kvh * G + (ok ? row : 0)) * D;
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
                const int col = kk * 16 + ((lane & 3) << 1);
                qb[kk][0] = ok ? *reinterpret_cast<const uint32_t*>(qp + col) : 0u;
                qb[kk][1] = ok ? *reinterpret_cast<const uint32_t*>(qp + col + 8) : 0u;
            }
        }
#pragma unroll
        for (int i = 0; i < D / 16; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    } else {
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int row = (lane >> 2) + 8 * r;
            row_ok[r] = row < nrows;
            row_pos[r] = pos0 + row / G;
            const bf16* qp = p.q + (size_t)(n0 + (row_ok[r] ? row / G : 0)) * p.q_stride + (size_t)(kvh * G + (row_ok[r] ? row % G : 0)) * D;
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
                const int col = kk * 16 + ((lane & 3) << 1);
                qa[kk][r] = row_ok[r] ? *reinterpret_cast<const uint32_t*>(qp + col) : 0u;
                qa[kk][r + 2] = row_ok[r] ? *reinterpret_cast<const uint32_t*>(qp + col + 8) : 0u;
            }
        }
#pragma unroll
        for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    }
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

#pragma unroll
    for (int s = 0; s < STAGES; ++s) {
        if (s < mine && !fetched[s]) load_rows_warp<D, BN>(p, table, kvh, lo + (first + s * DW) * BN, hi - 1, 0, my + s * 2 * TILE, my + s * 2 * TILE + TILE, lane);
        cp_async_commit();  // stage 0's group may also hold later stages' early fetches: it then completes a little later, never too early
    }
    // where the chunk lies that refills the first slot: the block table is read now, not between a chunk's arithmetic and the
    // copies that refill its slot
    PoolRows<BN> refill;
    if (STAGES < mine) refill = find_rows_warp<BN>(p, table, kvh, lo + (first + STAGES * DW) * BN, hi - 1, lane);
    for (int it = 0; it < mine; ++it) {
        // groups so far: STAGES from above and one per iteration before this one; chunk `it` is in group `it` (and the early
        // fetches in group 0): everything but the STAGES - 1 youngest groups must have landed
        cp_async_wait<STAGES - 1>();
        __syncwarp();
        bf16* cur = my + (it % STAGES) * 2 * TILE;
        const int key0 = lo + (first + it * DW) * BN;
        if (it == own_it) {
            // The token's own position lies in this chunk, and the cache did not hold its key and value when the chunk was
            // fetched: the row (and the rows behind it, which were fetched from the same place and which the mask hides, but
            // whose values would still be multiplied by zero) gets what this warp has just made.
#pragma unroll 1
            for (int r = pos0 - key0; r < BN; ++r) {
#pragma unroll
                for (int i = 0; i < NP; ++i) {
                    const int j = lane + 32 * i;
                    cur[swz<D>(r, j)] = __ushort_as_bfloat16((unsigned short)(own_k[i] & 0xffffu));
                    cur[swz<D>(r, j + D / 2)] = __ushort_as_bfloat16((unsigned short)(own_k[i] >> 16));
                    cur[TILE + swz<D>(r, j)] = __ushort_as_bfloat16((unsigned short)(own_v[i] & 0xffffu));
                    cur[TILE + swz<D>(r, j + D / 2)] = __ushort_as_bfloat16((unsigned short)(own_v[i] >> 16));
                }
            }
            __syncwarp();
        }
        // a chunk that lies wholly before the first token's position (and inside every window) needs no mask arithmetic;
        // rows beyond the tile then collect numbers nobody reads
        const bool interior = key0 + BN - 1 <= pos0 && (p.window <= 0 || key0 > hi - 1 - p.window);
        if constexpr (T8) {
            if (interior) attend_chunk_t8<D, BN, false>(qb, cur, cur + TILE, o, m, l, key0, pos0, nrows, p.window, p.scale_log2, lane);
            else attend_chunk_t8<D, BN, true>(qb, cur, cur + TILE, o, m, l, key0, pos0, nrows, p.window, p.scale_log2, lane);
        } else {
            if (interior) attend_chunk<D, BN, false>(qa, cur, cur + TILE, o, m, l, key0, row_pos, row_ok, p.window, p.scale_log2, lane);
            else attend_chunk<D, BN, true>(qa, cur, cur + TILE, o, m, l, key0, row_pos, row_ok, p.window, p.scale_log2, lane);
        }
        __syncwarp();  // every lane is done with the slot
        const int nxt = it + STAGES;
        if (nxt < mine) {
            bf16* dst = my + (it % STAGES) * 2 * TILE;
            copy_rows_warp<D, BN>(p, refill, 0, dst, dst + TILE, lane);
            if (nxt + 1 < mine) refill = find_rows_warp<BN>(p, table, kvh, lo + (first + (nxt + 1) * DW) * BN, hi - 1, lane);
        }
        cp_async_commit();
    }
    cp_async_wait<0>();
#pragma unroll
    for (int r = 0; r < 2; ++r) {  // a row's sum over the lanes that hold its keys
        if constexpr (T8) {
            l[r] += __shfl_xor_sync(0xffffffffu, l[r], 4);
            l[r] += __shfl_xor_sync(0xffffffffu, l[r], 8);
            l[r] += __shfl_xor_sync(0xffffffffu, l[r], 16);
        } else {
            l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
            l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
        }
    }
    __syncthreads();  // every warp is done with its ring; the space is reused for the merge
    constexpr int MR = T8 ? 8 : 16;                     // rows that are merged
    constexpr int WS = D + 8;                           // row stride of the warps' outputs: eight rows written at once spread over the banks
    float* wm = reinterpret_cast<float*>(smem_raw);        // [DW][16] each warp's row maxima
    float* wl = wm + DW * 16;                           // [DW][16] row sums
    float* wf = wl + DW * 16;                           // [DW][16] the weight of each warp's row in the merged row
    float* wo = wf + DW * 16;                           // [DW][16][WS] outputs
    float* fm = wo + DW * 16 * WS;                      // merged [16], [16], [16][D]
    float* fl = fm + 16;
    float* fo = fl + 16;
    if constexpr (T8) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int row = ((lane & 3) << 1) + j;
            if ((lane >> 2) == 0) { wm[warp * 16 + row] = m[j]; wl[warp * 16 + row] = l[j]; }
#pragma unroll
            for (int dt = 0; dt < D / 16; ++dt) {
                wo[(warp * 16 + row) * WS + dt * 16 + (lane >> 2)] = o[dt][j];
                wo[(warp * 16 + row) * WS + dt * 16 + (lane >> 2) + 8] = o[dt][2 + j];
            }
        }
    } else {
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int row = (lane >> 2) + 8 * r;
            if ((lane & 3) == 0) { wm[warp * 16 + row] = m[r]; wl[warp * 16 + row] = l[r]; }
#pragma unroll
            for (int dt = 0; dt < D / 8; ++dt) {
                const int col = dt * 8 + ((lane & 3) << 1);
                *reinterpret_cast<float2*>(wo + (warp * 16 + row) * WS + col) = make_float2(o[dt][2 * r], o[dt][2 * r + 1]);
            }
        }
    }
    __syncthreads();
    // a row's weights once (not once per output element): exp2(warp's maximum - overall maximum); the row's merged maximum and sum
    for (int i = tid; i < DW * MR; i += DW * 32) {
        const int w = i / MR, r = i % MR;
        float M = -INFINITY;
#pragma unroll
        for (int w2 = 0; w2 < DW; ++w2) M = fmaxf(M, wm[w2 * 16 + r]);
        wf[w * 16 + r] = M > -INFINITY ? fast_exp2(wm[w * 16 + r] - M) : 0.f;
        if (w == 0) fm[r] = M;
    }
    __syncthreads();
    for (int i = tid; i < MR * D; i += DW * 32) {
        const int r = i / D, dim = i % D;
        float O = 0.f;
#pragma unroll
        for (int w = 0; w < DW; ++w) O = fmaf(wo[(w * 16 + r) * WS + dim], wf[w * 16 + r], O);
        fo[i] = O;
        if (dim == 0) {
            float L = 0.f;
#pragma unroll
            for (int w = 0; w < DW; ++w) L = fmaf(wl[w * 16 + r], wf[w * 16 + r], L);
            fl[r] = L;
        }
    }
    __syncthreads();
    if (p.cluster && p.num_splits > 1) {
        // The slices of this tile are the blocks of one cluster: block 0 reads every block's (max, sum, output) out of
        // its shared memory and writes the rows. Nothing goes through global memory and nobody waits on a counter.
        cluster_sync_all();
        if (split == 0) {
            // (max[16], sum[16], output[16][D]) of every block lie in one run of shared memory starting at fm: bring all of
            // them here with loads that do not wait for each other, then merge locally.
            constexpr int RUN = 32 + 16 * D;
            float* stage = fo + 16 * D;  // behind the block's own run; the rings' space is free now
            const int total = p.num_splits * RUN;
#pragma unroll 8
            for (int idx = tid; idx < total; idx += DW * 32) stage[idx] = ld_cluster(fm + idx % RUN, idx / RUN);
            __syncthreads();
            float* wgt = wm;      // [splits][16] weights, reusing the warps' merge space
            float* linv = wl;     // [16]
            for (int r = tid; r < nrows; r += DW * 32) {
                float M = -INFINITY;
                for (int s2 = 0; s2 < p.num_splits; ++s2) M = fmaxf(M, stage[s2 * RUN + r]);
                float L = 0.f;
                for (int s2 = 0; s2 < p.num_splits; ++s2) {
                    const float f = M > -INFINITY ? exp2f(stage[s2 * RUN + r] - M) : 0.f;
                    wgt[s2 * 16 + r] = f;
                    L = fmaf(stage[s2 * RUN + 16 + r], f, L);
                }
                linv[r] = L > 0.f ? 1.f / L : 0.f;
            }
            __syncthreads();
            for (int i = tid; i < nrows * D; i += DW * 32) {
                const int r = i / D, dim = i % D;
                float O = 0.f;
                for (int s2 = 0; s2 < p.num_splits; ++s2) O = fmaf(stage[s2 * RUN + 32 + i], wgt[s2 * 16 + r], O);
                p.out[(size_t)(n0 + r / G) * p.nq * D + (size_t)(kvh * G + r % G) * D + dim] = __float2bfloat16_rn(O * linv[r]);
            }
        }
        cluster_sync_all();  // the other blocks' shared memory stays until block 0 has read it
        return;
    }
    finish_tile<D, 16, DW * 32>(p, fm, fl, fo, p.num_splits, ((size_t)tile * p.nkv + kvh) * p.num_splits, 1, tile * p.nkv + kvh, kvh, split, n0, nrows, G, &flag, wo);
}

// ---------------------------------------------------------------------------------------------- prefill
template <int D>
__global__ void __launch_bounds__(WARPS * 32) attn_mma_prefill_kernel(const Params p) {
    constexpr int BM = 64, BN = 64, TILE = BN * D;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    bf16* qs = reinterpret_cast<bf16*>(smem_raw);   // [BM][D]
    bf16* kv = qs + BM * D;                         // [3 stages][K, V][BN][D]
    __shared__ int flag;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int tile = gridDim.x - 1 - blockIdx.x;  // later tiles of a prompt see more keys: start them first
    const int kvh = blockIdx.y, split = blockIdx.z;
    pdl_trigger();
    pdl_wait();
    const int n0 = p.tile_info ? p.tile_info[2 * tile] : tile;
    const int ntok = p.tile_info ? p.tile_info[2 * tile + 1] : 1;
    const int G = p.nq / p.nkv;
    const int nrows = ntok * G;  // <= 64
    const int pos0 = p.positions[n0];
    const int* table = p.block_table + (size_t)p.token_seq[n0] * p.max_blocks;
    const int hi = pos0 + ntok;
    const int lo = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
    const int chunks = (hi - lo + BN - 1) / BN;
    const int per = (chunks + p.num_splits - 1) / p.num_splits;
    const int c_begin = split * per, c_end = min(chunks, c_begin + per);

    // queries of the tile into shared memory (zeros for rows beyond the tile), first key chunk behind them
    constexpr int CH = D / 8;
    for (int idx = tid; idx < BM * CH; idx += WARPS * 32) {
        const int row = idx / CH, ch = idx % CH;
        bf16* dst = qs + row * D + ((ch ^ (row & 7)) << 3);
        if (row < nrows) cp_async16(dst, p.q + (size_t)(n0 + row / G) * p.q_stride + (size_t)(kvh * G + row % G) * D + ch * 8);
        else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
    }
    // a ring of three key chunks: chunk c + 2 is on its way while chunk c is computed, with one block-wide barrier per chunk
    if (c_begin < c_end) load_rows_warp<D, BN / WARPS>(p, table, kvh, lo + c_begin * BN + warp * (BN / WARPS), hi - 1, warp * (BN / WARPS), kv, kv + TILE, lane);
    cp_async_commit();
    if (c_begin + 1 < c_end) load_rows_warp<D, BN / WARPS>(p, table, kvh, lo + (c_begin + 1) * BN + warp * (BN / WARPS), hi - 1, warp * (BN / WARPS), kv + 2 * TILE, kv + 3 * TILE, lane);
    cp_async_commit();

    int row_pos[2];
    bool row_ok[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = warp * 16 + (lane >> 2) + 8 * r;
        row_ok[r] = row < nrows;
        row_pos[r] = pos0 + row / G;
    }
    const int warp_last_pos = pos0 + min(ntok - 1, (warp * 16 + 15) / G);  // the furthest key any row of this warp sees
    const int warp_first_pos = pos0 + min(ntok - 1, (warp * 16) / G);
    const bool warp_has_rows = warp * 16 < nrows;

    uint32_t qa[D / 16][4];
    float o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

    const int warp_min_pos = warp_first_pos;  // every row of the warp sees keys up to at least here
    for (int c = c_begin; c < c_end; ++c) {
        const int stage = (c - c_begin) % 3;
        cp_async_wait<1>();   // chunk c has landed (chunk c + 1 may still be in flight)
        __syncthreads();      // ... for every warp; and every warp is done with chunk c - 1, whose buffer is filled next
        if (c + 2 < c_end) {
            bf16* dst = kv + ((c + 2 - c_begin) % 3) * 2 * TILE;
            load_rows_warp<D, BN / WARPS>(p, table, kvh, lo + (c + 2) * BN + warp * (BN / WARPS), hi - 1, warp * (BN / WARPS), dst, dst + TILE, lane);
        }
        cp_async_commit();
        if (c == c_begin) {
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
                const int row = warp * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
                const int col = kk * 16 + ((lane >> 4) << 3);
                ldmatrix_x4(qa[kk], qs + swz<D>(row, col));
            }
        }
        const int key0 = lo + c * BN;
        const bool visible = warp_has_rows && key0 <= warp_last_pos && (p.window <= 0 || key0 + BN - 1 > warp_first_pos - p.window);
        if (visible) {
            const bf16* cur = kv + stage * 2 * TILE;
            // a chunk that every row of the warp sees in full needs no mask arithmetic
            const bool interior = key0 + BN - 1 <= warp_min_pos && warp * 16 + 15 < nrows && (p.window <= 0 || key0 > warp_last_pos - p.window);
            if (interior) attend_chunk<D, BN, false>(qa, cur, cur + TILE, o, m, l, key0, row_pos, row_ok, p.window, p.scale_log2, lane);
            else attend_chunk<D, BN, true>(qa, cur, cur + TILE, o, m, l, key0, row_pos, row_ok, p.window, p.scale_log2, lane);
        }
    }
    cp_async_wait<0>();
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
    }
    __syncthreads();
    float* fm = reinterpret_cast<float*>(smem_raw);  // [64], [64], [64][D]: reuses the tiles' space
    float* fl = fm + BM;
    float* fo = fl + BM;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = warp * 16 + (lane >> 2) + 8 * r;
        if ((lane & 3) == 0) { fm[row] = m[r]; fl[row] = l[r]; }
#pragma unroll
        for (int dt = 0; dt < D / 8; ++dt) {
            const int col = dt * 8 + ((lane & 3) << 1);
            fo[row * D + col] = o[dt][2 * r];
            fo[row * D + col + 1] = o[dt][2 * r + 1];
        }
    }
    __syncthreads();
    finish_tile<D, BM, WARPS * 32>(p, fm, fl, fo, p.num_splits, ((size_t)tile * p.nkv + kvh) * p.num_splits, 1, tile * p.nkv + kvh, kvh, split, n0, nrows, G, &flag, fo + BM * D);
}

// tile list of a step: request r brings tokens [starts[r], starts[r + 1]); tiles hold up to `per_tile` tokens of one request
__global__ void attn_plan_kernel(const int* __restrict__ starts, int num_seqs, int per_tile, int* __restrict__ tile_info, int max_tiles) {
    pdl_trigger();
    pdl_wait();
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    int t = 0;
    for (int r = 0; r < num_seqs; ++r) {
        for (int a = starts[r]; a < starts[r + 1] && t < max_tiles; a += per_tile, ++t) {
            tile_info[2 * t] = a;
            tile_info[2 * t + 1] = min(per_tile, starts[r + 1] - a);
        }
    }
    for (; t < max_tiles; ++t) { tile_info[2 * t] = 0; tile_info[2 * t + 1] = 0; }
}

template <int D, bool T8, int DW>
int launch_decode(const Params& p, dim3 grid, cudaStream_t s) {
    constexpr int BN = D == 64 ? 32 : 16, STAGES = 3;  // DW warps, each with its own ring of 4 KB + 4 KB chunks
    constexpr size_t ring = (size_t)DW * STAGES * 2 * BN * D * sizeof(bf16);
    constexpr size_t merge = (size_t)(DW * 16 * (D + 8 + 3) + 16 * (D + 2)) * sizeof(float);
    constexpr size_t smem = ring > merge ? ring : merge;
    static bool set = false;
    if (!set) {
        cudaError_t e = cudaFuncSetAttribute(attn_mma_decode_kernel<D, BN, STAGES, DW, T8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        set = true;
    }
    if (p.cluster && p.num_splits > 1) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = grid;
        cfg.blockDim = dim3(DW * 32);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = s;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 1;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = p.num_splits;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = llmie_pdl_flag ? 2 : 1;
        return (int)cudaLaunchKernelEx(&cfg, attn_mma_decode_kernel<D, BN, STAGES, DW, T8>, p);
    }
    return launch_kernel(attn_mma_decode_kernel<D, BN, STAGES, DW, T8>, grid, dim3(DW * 32), smem, s, p);
}

template <int D>
int launch(const Params& p, int num_tiles, int decode_mode, cudaStream_t s) {
    const dim3 grid(num_tiles, p.nkv, p.num_splits);
    if (decode_mode) {
        // tiles of one token with up to 8 heads per group: the transposed form, which spends nothing on padding rows
        const bool t8 = p.tile_info == nullptr && p.nq / p.nkv <= 8;
        // Eight warps (192 KB of rings: one block per multiprocessor) walk a block's keys fastest. When there are more
        // blocks than multiprocessors and nothing is cut into slices, the caller may ask for blocks of four warps (96 KB:
        // two per multiprocessor), which then run in fewer, fuller rounds (96 requests of 8,192 keys: 94 us in two rounds of
        // eight-warp blocks, the second half empty; 74.5 us at once).
        if (decode_mode == 2 && p.num_splits == 1) return t8 ? launch_decode<D, true, 4>(p, grid, s) : launch_decode<D, false, 4>(p, grid, s);
        return t8 ? launch_decode<D, true, 8>(p, grid, s) : launch_decode<D, false, 8>(p, grid, s);
    } else {
        constexpr size_t tiles = (size_t)(64 * D + 3 * 2 * 64 * D) * sizeof(bf16);
        constexpr size_t merge = (size_t)(64 * (D + 2)) * sizeof(float);
        constexpr size_t smem = tiles > merge ? tiles : merge;
        static bool set = false;
        if (!set) {
            cudaError_t e = cudaFuncSetAttribute(attn_mma_prefill_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return (int)e;
            set = true;
        }
        return launch_kernel(attn_mma_prefill_kernel<D>, grid, dim3(WARPS * 32), smem, s, p);
    }
}

}  // namespace

LLMIE_API int llmie_attn_plan(const int* seq_starts, int num_seqs, int tokens_per_tile, int* tile_info, int max_tiles, cudaStream_t s) {
    if (num_seqs <= 0 || max_tiles <= 0) return 0;
    if (tokens_per_tile <= 0) return LLMIE_ERR_BAD_ARGUMENT;
    return launch_kernel(attn_plan_kernel, dim3(1), dim3(32), 0, s, seq_starts, num_seqs, tokens_per_tile, tile_info, max_tiles);
}

// decode_mode 1 or 2: every tile has at most 16 rows (tokens * group); 2 asks for blocks of four warps instead of eight when
// nothing is cut into slices. 0: at most 64 rows.
// scratch_o / scratch_ml / counters are needed for num_splits > 1 (counters zeroed once; the kernel leaves them zero), unless
// `cluster` is set (decode mode, at most 8 slices): the slices then form one thread-block cluster and merge in shared memory.
static int run_mma(const bf16* q, int q_stride, const bf16* k_pool, const bf16* v_pool, const int* block_table,
                   int max_blocks, const int* token_seq, const int* positions, const int* tile_info, int num_tiles,
                   bf16* out, float* scratch_o, float* scratch_ml, int* counters, int nq, int nkv, int d,
                   int page_size, float scale, int window, int num_splits, int decode_mode, int cluster, const float* qkv_acc,
                   int acc_stride, const float* bias, const float* cos_t, const float* sin_t, const int* slots, cudaStream_t s) {
    if (num_tiles <= 0) return 0;
    if (qkv_acc && (!decode_mode || tile_info || nq / (nkv > 0 ? nkv : 1) > 8 || !cos_t || !sin_t || acc_stride < (nq + 2 * nkv) * d ||
                    (acc_stride & 1) || ((uintptr_t)qkv_acc & 7) || ((uintptr_t)bias & 7) || ((uintptr_t)cos_t & 7) || ((uintptr_t)sin_t & 7)))
        return LLMIE_ERR_BAD_ARGUMENT;
    if (cluster && (!decode_mode || num_splits > 8)) return LLMIE_ERR_BAD_ARGUMENT;
    if ((d != 64 && d != 128) || nkv <= 0 || nq % nkv || page_size <= 0 || num_splits < 1 || q_stride % 8 || nkv > 65535 ||
        num_splits > 64 || (num_splits > 1 && !cluster && (!scratch_o || !scratch_ml || !counters)))
        return LLMIE_ERR_BAD_ARGUMENT;
    const int G = nq / nkv;
    if (G > (decode_mode ? 16 : 64)) return LLMIE_ERR_BAD_ARGUMENT;
    Params p;
    p.q = q; p.k_pool = k_pool; p.v_pool = v_pool; p.block_table = block_table; p.token_seq = token_seq; p.positions = positions;
    p.tile_info = tile_info; p.out = out; p.part_o = scratch_o; p.part_ml = scratch_ml; p.counters = counters;
    p.q_stride = q_stride; p.max_blocks = max_blocks; p.nq = nq; p.nkv = nkv; p.page_size = page_size; p.window = window;
    p.page_shift = (page_size & (page_size - 1)) == 0 ? __builtin_ctz((unsigned)page_size) : -1;
    p.num_splits = num_splits; p.scale_log2 = scale * LOG2E; p.cluster = cluster;
    p.qkv_acc = qkv_acc; p.acc_stride = acc_stride; p.bias = bias; p.cos_t = cos_t; p.sin_t = sin_t; p.slots = slots;
    p.k_pool_w = const_cast<bf16*>(k_pool); p.v_pool_w = const_cast<bf16*>(v_pool);
    return d == 64 ? launch<64>(p, num_tiles, decode_mode, s) : launch<128>(p, num_tiles, decode_mode, s);
}

LLMIE_API int llmie_paged_attention_mma(const bf16* q, int q_stride, const bf16* k_pool, const bf16* v_pool, const int* block_table,
                                        int max_blocks, const int* token_seq, const int* positions, const int* tile_info, int num_tiles,
                                        bf16* out, float* scratch_o, float* scratch_ml, int* counters, int nq, int nkv, int d,
                                        int page_size, float scale, int window, int num_splits, int decode_mode, int cluster, cudaStream_t s) {
    return run_mma(q, q_stride, k_pool, v_pool, block_table, max_blocks, token_seq, positions, tile_info, num_tiles, out, scratch_o, scratch_ml,
                   counters, nq, nkv, d, page_size, scale, window, num_splits, decode_mode, cluster, nullptr, 0, nullptr, nullptr, nullptr,
                   nullptr, s);
}

// Decode steps (every tile one token, at most 8 query heads per key/value head): the same attention, with the queries, keys and
// values of the step's tokens taken from `qkv_acc`, the float32 sums [tokens][acc_stride] of the fused q/k/v projection
// before bias and rotation (nothing clears them here). The kernel adds `bias` (or none), rotates queries and keys by
// cos_t / sin_t [tokens][d / 2] and, where `slots` is given, writes each token's key and value into its cache slot.
LLMIE_API int llmie_paged_attention_mma_acc(const float* qkv_acc, int acc_stride, const float* bias, const float* cos_t, const float* sin_t,
                                            const int* slots, bf16* k_pool, bf16* v_pool, const int* block_table, int max_blocks,
                                            const int* token_seq, const int* positions, int num_tokens, bf16* out, float* scratch_o,
                                            float* scratch_ml, int* counters, int nq, int nkv, int d, int page_size, float scale, int window,
                                            int num_splits, int cluster, int four_warps, cudaStream_t s) {
    if (!qkv_acc) return LLMIE_ERR_BAD_ARGUMENT;
    return run_mma(nullptr, 8, k_pool, v_pool, block_table, max_blocks, token_seq, positions, nullptr, num_tokens, out, scratch_o, scratch_ml,
                   counters, nq, nkv, d, page_size, scale, window, num_splits, four_warps ? 2 : 1, cluster, qkv_acc, acc_stride, bias, cos_t, sin_t, slots, s);
}
