// Embedding, rotary tables, residual add + RMS norm, QKV bias + rotation + cache write, SiLU * up.
// Every kernel takes its sizes as arguments; T is the compute dtype (float or bfloat16). The
// residual stream, the norms' reductions, the rotation angles and the activation are 32-bit.
#include <type_traits>

#include "common.cuh"

int llmie_pdl_flag = 0;

// 1: kernels of a step overlap their set-up with the tail of the kernel before them (see common.cuh); 0: plain launches.
LLMIE_API int llmie_set_pdl(int on) {
    llmie_pdl_flag = on ? 1 : 0;
    return 0;
}

// ------------------------------------------------------------------------------------------------
// x[n, :] = table[ids[n], :]  widened to float (the residual stream)
template <typename T>
__global__ void embed_kernel(const int* __restrict__ ids, const T* __restrict__ table, float* __restrict__ out, int H) {
    pdl_trigger();
    pdl_wait();
    const int n = blockIdx.x;
    const T* row = table + (size_t)ids[n] * H;
    float* o = out + (size_t)n * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = to_f32(row[i]);
}

LLMIE_API int llmie_embed(const int* ids, const void* table, float* out, int N, int H, int dtype, cudaStream_t s) {
    if (N <= 0) return 0;
    const int threads = H >= 1024 ? 256 : 128;
    if (dtype == DT_F32) return launch_kernel(embed_kernel<float>, dim3(N), dim3(threads), 0, s, ids, (const float*)table, out, H);
    return launch_kernel(embed_kernel<bf16>, dim3(N), dim3(threads), 0, s, ids, (const bf16*)table, out, H);
}

// ------------------------------------------------------------------------------------------------
// ids[i] = previous[src[i]] where src[i] >= 0: a request's next token taken from the tokens the step before chose, which
// are still on the device (the host has not read them yet)
__global__ void feed_tokens_kernel(int* __restrict__ ids, const int* __restrict__ src, const int* __restrict__ previous, int N) {
    pdl_trigger();
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < N && src[i] >= 0) ids[i] = previous[src[i]];
}

LLMIE_API int llmie_feed_tokens(int* ids, const int* src, const int* previous, int N, cudaStream_t s) {
    if (N <= 0) return 0;
    return launch_kernel(feed_tokens_kernel, dim3((N + 127) / 128), dim3(128), 0, s, ids, (const int*)src, previous, N);
}

// ------------------------------------------------------------------------------------------------
// Fixed-size per-request state starts at zero: state[slots[r], :] = 0 for every request r of the step whose first token of
// this step is the first of the request (position 0). Decided on the device from the step's own arrays, so the step can be
// replayed from a graph. One block per request.
__global__ void zero_fresh_state_kernel(float* __restrict__ state, long long row_floats, const int* __restrict__ slots,
                                        const int* __restrict__ starts, const int* __restrict__ positions) {
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.x;
    if (positions[starts[r]] != 0) return;
    float* row = state + (long long)slots[r] * row_floats;
    for (long long i = threadIdx.x; i < row_floats; i += blockDim.x) row[i] = 0.f;
}

LLMIE_API int llmie_zero_fresh_state(float* state, long long row_floats, const int* slots, const int* starts, const int* positions,
                                     int num_seqs, cudaStream_t s) {
    if (num_seqs <= 0 || row_floats <= 0) return 0;
    return launch_kernel(zero_fresh_state_kernel, dim3(num_seqs), dim3(128), 0, s, state, row_floats, slots, starts, positions);
}

// ------------------------------------------------------------------------------------------------
// cos/sin[n, j] of the angle float(position[n]) * inv_freq[j], all in 32-bit
__global__ void rope_tables_kernel(const int* __restrict__ pos, const float* __restrict__ inv_freq, float* __restrict__ cos_out,
                                   float* __restrict__ sin_out, int N, int half) {
    pdl_trigger();
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= N * half) return;
    const int n = i / half, j = i % half;
    const float ang = __int2float_rn(pos[n]) * inv_freq[j];
    cos_out[i] = cosf(ang);
    sin_out[i] = sinf(ang);
}

LLMIE_API int llmie_rope_tables(const int* pos, const float* inv_freq, float* cos_out, float* sin_out, int N, int half,
                                cudaStream_t s) {
    if (N <= 0) return 0;
    const int total = N * half;
    return launch_kernel(rope_tables_kernel, dim3((total + 127) / 128), dim3(128), 0, s, pos, inv_freq, cos_out, sin_out, N, half);
}

// ------------------------------------------------------------------------------------------------
// One block per output row.
//   rows == nullptr: r = blockIdx.x; residual[r] += delta[r] (stored); out[r] = norm(residual[r])
//   rows != nullptr: r = rows[blockIdx.x]; out[blockIdx.x] = norm(residual[r] + delta[r]); residual untouched
// norm(x) = weight * T(x / sqrt(mean(x^2) + eps)), the mean and the scaling in 32-bit.
// The row is kept in shared memory between the two passes; VEC = 4 moves four elements per access when H allows.
template <typename T, int VEC>
__global__ void add_rmsnorm_kernel(float* __restrict__ residual, const T* __restrict__ delta, const float* __restrict__ weight,
                                   T* __restrict__ out, const int* __restrict__ rows, int H, float eps) {
    extern __shared__ __align__(16) float row_buf[];  // H floats, 33 for the reduction, H floats of weights
    float* scratch = row_buf + H;
    float* w_buf = scratch + 36;  // the norm's weights, H floats: fetched before the wait, they do not depend on the kernel before
    pdl_trigger();
    for (int i = threadIdx.x * VEC; i < H; i += blockDim.x * VEC) {
        if constexpr (VEC == 4) *reinterpret_cast<float4*>(w_buf + i) = *reinterpret_cast<const float4*>(weight + i);
        else w_buf[i] = weight[i];
    }
    pdl_wait();
    const int r = rows ? rows[blockIdx.x] : blockIdx.x;
    float* x = residual + (size_t)r * H;
    const T* d = delta ? delta + (size_t)r * H : nullptr;
    float ss = 0.f;
    for (int i = threadIdx.x * VEC; i < H; i += blockDim.x * VEC) {
        float v[VEC];
        if constexpr (VEC == 4) load4(x + i, v); else v[0] = x[i];
        if (d) {
            float dv[VEC];
            if constexpr (VEC == 4) load4(d + i, dv); else dv[0] = to_f32(d[i]);
#pragma unroll
            for (int j = 0; j < VEC; ++j) v[j] += dv[j];
            if (!rows) { if constexpr (VEC == 4) store4(x + i, v); else x[i] = v[0]; }
        }
#pragma unroll
        for (int j = 0; j < VEC; ++j) { row_buf[i + j] = v[j]; ss += v[j] * v[j]; }
    }
    ss = block_sum(ss, scratch);
    const float rstd = 1.0f / sqrtf(ss / (float)H + eps);
    T* o = out + (size_t)blockIdx.x * H;
    for (int i = threadIdx.x * VEC; i < H; i += blockDim.x * VEC) {
        float y[VEC];
#pragma unroll
        for (int j = 0; j < VEC; ++j) y[j] = w_buf[i + j] * round_through<T>(row_buf[i + j] * rstd);
        if constexpr (VEC == 4) store4(o + i, y); else o[i] = from_f32<T>(y[0]);
    }
}

template <typename T>
static int launch_add_rmsnorm(float* residual, const T* delta, const float* weight, T* out, const int* rows, int n_out, int H, float eps,
                              cudaStream_t s) {
    const size_t smem = (size_t)(2 * H + 36) * sizeof(float);
    const bool vec = H % 4 == 0 && ((uintptr_t)residual % 16 == 0) && ((uintptr_t)out % 8 == 0) && ((uintptr_t)delta % 8 == 0) &&
                     ((uintptr_t)weight % 16 == 0);
    const int per = vec ? 4 : 1;
    int threads = 32;
    while (threads < 512 && threads * per * 2 <= H) threads *= 2;
    if (vec) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(add_rmsnorm_kernel<T, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        return launch_kernel(add_rmsnorm_kernel<T, 4>, dim3(n_out), dim3(threads), smem, s, residual, delta, weight, out, rows, H, eps);
    } else {
        if (smem > 48 * 1024) cudaFuncSetAttribute(add_rmsnorm_kernel<T, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        return launch_kernel(add_rmsnorm_kernel<T, 1>, dim3(n_out), dim3(threads), smem, s, residual, delta, weight, out, rows, H, eps);
    }
}

LLMIE_API int llmie_add_rmsnorm(float* residual, const void* delta, const float* weight, void* out, const int* rows,
                                int n_out, int H, float eps, int dtype, cudaStream_t s) {
    if (n_out <= 0) return 0;
    if ((size_t)(2 * H + 36) * sizeof(float) > 200 * 1024) return LLMIE_ERR_BAD_ARGUMENT;
    if (dtype == DT_F32) return launch_add_rmsnorm<float>(residual, (const float*)delta, weight, (float*)out, rows, n_out, H, eps, s);
    return launch_add_rmsnorm<bf16>(residual, (const bf16*)delta, weight, (bf16*)out, rows, n_out, H, eps, s);
}

// ------------------------------------------------------------------------------------------------
// in[n] is [num_heads + 2 num_kv_heads][d]. Adds the bias, rotates the query and key heads by the
// token's angle (pairs (j, j + d/2)), writes everything to out[n] (which may be `in` itself) and, if asked,
// copies the key and value heads into the token's cache slot: pool[page][kv head][offset][d],
// slot = page * page_size + offset. With `clear_in` the input is set to zero after it was read: it is
// then a float32 accumulation buffer that the next split-K product adds into.
template <typename TI, typename TO, int VEC>
__global__ void rope_kv_write_kernel(TI* __restrict__ in, TO* __restrict__ out, const float* __restrict__ bias,
                                     const float* __restrict__ cos_t, const float* __restrict__ sin_t, const int* __restrict__ slots,
                                     TO* __restrict__ k_pool, TO* __restrict__ v_pool, int nq, int nkv, int d, int page_size, int write_kv,
                                     int clear_in) {
    pdl_trigger();
    pdl_wait();
    const int n = blockIdx.x;
    const int half = d >> 1;
    const int heads = nq + 2 * nkv;
    TI* src = in + (size_t)n * heads * d;
    TO* row = out + (size_t)n * heads * d;
    const float* c = cos_t + (size_t)n * half;
    const float* sn = sin_t + (size_t)n * half;
    const int slot = write_kv ? slots[n] : -1;
    const int page = slot >= 0 ? slot / page_size : 0, off = slot >= 0 ? slot % page_size : 0;
    // a thread takes VEC neighbouring pairs (j, j + d/2) of one head
    for (int i = threadIdx.x * VEC; i < heads * half; i += blockDim.x * VEC) {
        const int h = i / half, j = i % half;
        const int a = h * d + j, b = a + half;
        float x1[VEC], x2[VEC], y1[VEC], y2[VEC];
        if constexpr (VEC == 4) { load4(src + a, x1); load4(src + b, x2); } else { x1[0] = to_f32(src[a]); x2[0] = to_f32(src[b]); }
        if (clear_in) {
            const float zero[4] = {0.f, 0.f, 0.f, 0.f};
            if constexpr (VEC == 4) { store4(src + a, zero); store4(src + b, zero); } else { src[a] = from_f32<TI>(0.f); src[b] = from_f32<TI>(0.f); }
        }
        if (bias) {
#pragma unroll
            for (int v = 0; v < VEC; ++v) { x1[v] += bias[a + v]; x2[v] += bias[b + v]; }
        }
#pragma unroll
        for (int v = 0; v < VEC; ++v) {
            if (h < nq + nkv) {
                y1[v] = x1[v] * c[j + v] - x2[v] * sn[j + v];
                y2[v] = x2[v] * c[j + v] + x1[v] * sn[j + v];
            } else {
                y1[v] = x1[v];
                y2[v] = x2[v];
            }
        }
        if constexpr (VEC == 4) { store4(row + a, y1); store4(row + b, y2); } else { row[a] = from_f32<TO>(y1[0]); row[b] = from_f32<TO>(y2[0]); }
        if (slot >= 0 && h >= nq) {
            const int kvh = h < nq + nkv ? h - nq : h - nq - nkv;
            TO* pool = h < nq + nkv ? k_pool : v_pool;
            TO* dst = pool + (((size_t)page * nkv + kvh) * page_size + off) * d;
            if constexpr (VEC == 4) { store4(dst + j, y1); store4(dst + j + half, y2); } else { dst[j] = from_f32<TO>(y1[0]); dst[j + half] = from_f32<TO>(y2[0]); }
        }
    }
}

// The same for many tokens in bfloat16 (prompt portions after a library product): 16-byte accesses, eight pairs (j, j + d/2)
// per thread and step, bias and angles as float4, and 128 threads per token so that twice as many tokens are in flight per
// multiprocessor (the kernel is one trip to memory and back per block: what counts is how many blocks are there at once).
__global__ void __launch_bounds__(128) rope_kv_write_bf16x8_kernel(const bf16* in, bf16* out, const float* __restrict__ bias,   // (out may be in)
                                                                    const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                                                    const int* __restrict__ slots, bf16* __restrict__ k_pool, bf16* __restrict__ v_pool,
                                                                    int nq, int nkv, int d, int page_size, int write_kv) {
    pdl_trigger();
    pdl_wait();
    const int n = blockIdx.x;
    const int half = d >> 1;
    const int heads = nq + 2 * nkv;
    const bf16* src = in + (size_t)n * heads * d;
    bf16* row = out + (size_t)n * heads * d;
    const float* c = cos_t + (size_t)n * half;
    const float* sn = sin_t + (size_t)n * half;
    const int slot = write_kv ? slots[n] : -1;
    const int page = slot >= 0 ? slot / page_size : 0, off = slot >= 0 ? slot % page_size : 0;
    for (int i = threadIdx.x * 8; i < heads * half; i += blockDim.x * 8) {
        const int h = i / half, j = i % half;
        const int a = h * d + j, b = a + half;
        float x1[8], x2[8];
        load4(src + a, x1); load4(src + a + 4, x1 + 4);
        load4(src + b, x2); load4(src + b + 4, x2 + 4);
        if (bias) {
            float t[8];
            load4(bias + a, t); load4(bias + a + 4, t + 4);
#pragma unroll
            for (int v = 0; v < 8; ++v) x1[v] += t[v];
            load4(bias + b, t); load4(bias + b + 4, t + 4);
#pragma unroll
            for (int v = 0; v < 8; ++v) x2[v] += t[v];
        }
        if (h < nq + nkv) {
            float cs[8], ss[8];
            load4(c + j, cs); load4(c + j + 4, cs + 4);
            load4(sn + j, ss); load4(sn + j + 4, ss + 4);
#pragma unroll
            for (int v = 0; v < 8; ++v) {
                const float y1 = x1[v] * cs[v] - x2[v] * ss[v], y2 = x2[v] * cs[v] + x1[v] * ss[v];
                x1[v] = y1; x2[v] = y2;
            }
        }
        store4(row + a, x1); store4(row + a + 4, x1 + 4);
        store4(row + b, x2); store4(row + b + 4, x2 + 4);
        if (slot >= 0 && h >= nq) {
            const int kvh = h < nq + nkv ? h - nq : h - nq - nkv;
            bf16* dst = (h < nq + nkv ? k_pool : v_pool) + (((size_t)page * nkv + kvh) * page_size + off) * d;
            store4(dst + j, x1); store4(dst + j + 4, x1 + 4);
            store4(dst + j + half, x2); store4(dst + j + half + 4, x2 + 4);
        }
    }
}

template <typename TI, typename TO>
static int launch_rope(TI* in, TO* out, const float* bias, const float* cos_t, const float* sin_t, const int* slots, TO* k_pool, TO* v_pool,
                       int N, int nq, int nkv, int d, int page_size, int write_kv, int clear_in, cudaStream_t s) {
    const int work = (nq + 2 * nkv) * (d / 2);
    const bool vec = d % 8 == 0 && ((uintptr_t)in % 16 == 0) && ((uintptr_t)out % 16 == 0) && ((uintptr_t)k_pool % 16 == 0) &&
                     ((uintptr_t)v_pool % 16 == 0);
    if constexpr (std::is_same<TI, bf16>::value && std::is_same<TO, bf16>::value) {
        // (8-byte halves of 16-byte pieces: the same alignment rule as below, d a multiple of 16)
        if (vec && d % 16 == 0 && N >= 64 && !clear_in && ((uintptr_t)bias % 16 == 0) && ((uintptr_t)cos_t % 16 == 0) && ((uintptr_t)sin_t % 16 == 0))
            return launch_kernel(rope_kv_write_bf16x8_kernel, dim3(N), dim3(128), 0, s, (const bf16*)in, out, bias, cos_t, sin_t, slots, k_pool, v_pool,
                                 nq, nkv, d, page_size, write_kv);
    }
    if (vec) {
        const int threads = work / 4 >= 256 ? 256 : 128;
        return launch_kernel(rope_kv_write_kernel<TI, TO, 4>, dim3(N), dim3(threads), 0, s, in, out, bias, cos_t, sin_t, slots, k_pool, v_pool,
                             nq, nkv, d, page_size, write_kv, clear_in);
    }
    const int threads = work >= 512 ? 256 : 128;
    return launch_kernel(rope_kv_write_kernel<TI, TO, 1>, dim3(N), dim3(threads), 0, s, in, out, bias, cos_t, sin_t, slots, k_pool, v_pool, nq,
                         nkv, d, page_size, write_kv, clear_in);
}

// in_dtype / out_dtype: 0 float32, 1 bfloat16; allowed pairs: equal types (out may alias in), or float32 in and bfloat16 out.
LLMIE_API int llmie_rope_kv_write(void* in, void* out, const float* bias, const float* cos_t, const float* sin_t, const int* slots,
                                  void* k_pool, void* v_pool, int N, int nq, int nkv, int d, int page_size, int write_kv,
                                  int clear_in, int in_dtype, int out_dtype, cudaStream_t s) {
    if (N <= 0) return 0;
    if (d <= 0 || (d & 1) || page_size <= 0 || (clear_in && in == out)) return LLMIE_ERR_BAD_ARGUMENT;
    if (in_dtype == DT_F32 && out_dtype == DT_F32)
        return launch_rope<float, float>((float*)in, (float*)out, bias, cos_t, sin_t, slots, (float*)k_pool, (float*)v_pool, N, nq, nkv, d, page_size,
                                         write_kv, clear_in, s);
    if (in_dtype == DT_BF16 && out_dtype == DT_BF16)
        return launch_rope<bf16, bf16>((bf16*)in, (bf16*)out, bias, cos_t, sin_t, slots, (bf16*)k_pool, (bf16*)v_pool, N, nq, nkv, d, page_size,
                                       write_kv, clear_in, s);
    if (in_dtype == DT_F32 && out_dtype == DT_BF16)
        return launch_rope<float, bf16>((float*)in, (bf16*)out, bias, cos_t, sin_t, slots, (bf16*)k_pool, (bf16*)v_pool, N, nq, nkv, d, page_size,
                                        write_kv, clear_in, s);
    return LLMIE_ERR_BAD_ARGUMENT;
}

// ------------------------------------------------------------------------------------------------
// out[n, i] = silu(gu[n, i]) * gu[n, I + i], silu(z) = z / (1 + exp(-z)) in 32-bit; `clear_in` zeroes what was read.
// grid = (column blocks, rows); VEC = 4 moves four columns per thread.
// `also_zero` (with `zero_n4` groups of four floats): another float32 accumulation buffer that this kernel clears on its way,
// one that an earlier kernel of the step read but could not clear itself because several of its blocks read it.
template <typename TI, typename TO, int VEC>
__global__ void silu_mul_kernel(TI* __restrict__ gu, TO* __restrict__ out, int I, int clear_in, float* __restrict__ also_zero, int zero_n4) {
    pdl_trigger();
    pdl_wait();
    if (also_zero) {
        const int threads = gridDim.x * gridDim.y * blockDim.x;
        for (int i = (blockIdx.y * gridDim.x + blockIdx.x) * blockDim.x + threadIdx.x; i < zero_n4; i += threads)
            reinterpret_cast<float4*>(also_zero)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    constexpr int PER = VEC == 4 ? 2 : 1;  // vectors per thread: two loads of gate and two of up are in flight together
    const int i0 = (blockIdx.x * blockDim.x + threadIdx.x) * VEC * PER;
    TI* row = gu + (size_t)blockIdx.y * 2 * I;
    float g[PER][VEC], u[PER][VEC];
#pragma unroll
    for (int v = 0; v < PER; ++v) {
        const int i = i0 + v * VEC;
        if (i < I) {
            if constexpr (VEC == 4) { load4(row + i, g[v]); load4(row + I + i, u[v]); } else { g[v][0] = to_f32(row[i]); u[v][0] = to_f32(row[I + i]); }
        }
    }
#pragma unroll
    for (int v = 0; v < PER; ++v) {
        const int i = i0 + v * VEC;
        if (i >= I) continue;
        if (clear_in) {
            const float zero[4] = {0.f, 0.f, 0.f, 0.f};
            if constexpr (VEC == 4) { store4(row + i, zero); store4(row + I + i, zero); } else { row[i] = from_f32<TI>(0.f); row[I + i] = from_f32<TI>(0.f); }
        }
        float y[VEC];
#pragma unroll
        for (int j = 0; j < VEC; ++j) y[j] = g[v][j] / (1.0f + expf(-g[v][j])) * u[v][j];
        TO* o = out + (size_t)blockIdx.y * I + i;
        if constexpr (VEC == 4) store4(o, y); else *o = from_f32<TO>(y[0]);
    }
}

// bfloat16 in and out, widths that are multiples of 8: 16-byte loads and stores; a thread takes 8 outputs of one row and the
// same 8 half the matrix further on, so that four loads are in flight. The result is rounded to bfloat16 (8 bits), so the
// exponential and the division are the fast 32-bit forms (errors of about 1e-7): the exact ones were half this kernel's time.
__global__ void __launch_bounds__(256) silu_mul_bf16x8_kernel(const bf16* __restrict__ gu, bf16* __restrict__ out, int I, long long items) {
    pdl_trigger();
    pdl_wait();
    const long long half = (items + 1) / 2;
    const long long first = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (first >= half) return;
    const int per_row = I / 8;
    float g[2][8], u[2][8];
    long long row[2];
    int col[2];
    bool live[2];
#pragma unroll
    for (int k = 0; k < 2; ++k) {
        const long long item = first + k * half;
        live[k] = item < items;
        row[k] = live[k] ? item / per_row : 0;
        col[k] = live[k] ? (int)(item % per_row) * 8 : 0;
        Vec16<bf16>::load(gu + row[k] * 2 * I + col[k], g[k]);
        Vec16<bf16>::load(gu + row[k] * 2 * I + I + col[k], u[k]);
    }
#pragma unroll
    for (int k = 0; k < 2; ++k) {
        if (!live[k]) continue;
        uint4 packed;
        uint32_t* w = reinterpret_cast<uint32_t*>(&packed);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float a = __fdividef(g[k][2 * j], 1.0f + __expf(-g[k][2 * j])) * u[k][2 * j];
            const float b = __fdividef(g[k][2 * j + 1], 1.0f + __expf(-g[k][2 * j + 1])) * u[k][2 * j + 1];
            const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
            w[j] = *reinterpret_cast<const uint32_t*>(&v);
        }
        *reinterpret_cast<uint4*>(out + row[k] * I + col[k]) = packed;
    }
}

template <typename TI, typename TO>
static int launch_silu_mul(TI* gu, TO* out, int N, int I, int clear_in, float* also_zero, int zero_n4, cudaStream_t s) {
    if (N > 65535) {  // rows ride in grid.y; more rows than that go in slabs
        for (int n0 = 0; n0 < N; n0 += 65535) {
            const int rc = launch_silu_mul<TI, TO>(gu + (size_t)n0 * 2 * I, out + (size_t)n0 * I, min(65535, N - n0), I, clear_in,
                                                   n0 == 0 ? also_zero : nullptr, zero_n4, s);
            if (rc) return rc;
        }
        return 0;
    }
    const bool vec = I % 4 == 0 && ((uintptr_t)gu % 16 == 0) && ((uintptr_t)out % 16 == 0);
    if (vec) return launch_kernel(silu_mul_kernel<TI, TO, 4>, dim3(((I + 7) / 8 + 127) / 128, N), dim3(128), 0, s, gu, out, I, clear_in, also_zero, zero_n4);
    return launch_kernel(silu_mul_kernel<TI, TO, 1>, dim3((I + 127) / 128, N), dim3(128), 0, s, gu, out, I, clear_in, also_zero, zero_n4);
}

// also_zero / zero_floats: a float32 buffer (16-byte aligned, a multiple of 4 floats) that is cleared as well, or null.
LLMIE_API int llmie_silu_mul(void* gu, void* out, int N, int I, int clear_in, int in_dtype, int out_dtype, float* also_zero,
                             long long zero_floats, cudaStream_t s) {
    if (N <= 0) return 0;
    if (also_zero && (((uintptr_t)also_zero & 15) || (zero_floats & 3) || zero_floats > (1ll << 32))) return LLMIE_ERR_BAD_ARGUMENT;
    const int n4 = also_zero ? (int)(zero_floats / 4) : 0;
    if (in_dtype == DT_F32 && out_dtype == DT_F32) return launch_silu_mul<float, float>((float*)gu, (float*)out, N, I, clear_in, also_zero, n4, s);
    if (in_dtype == DT_BF16 && out_dtype == DT_BF16) {
        if (!clear_in && !also_zero && I % 8 == 0 && ((uintptr_t)gu % 16 == 0) && ((uintptr_t)out % 16 == 0)) {
            const long long items = (long long)N * (I / 8);
            return launch_kernel(silu_mul_bf16x8_kernel, dim3((unsigned)(((items + 1) / 2 + 255) / 256)), dim3(256), 0, s, (const bf16*)gu, (bf16*)out, I, items);
        }
        return launch_silu_mul<bf16, bf16>((bf16*)gu, (bf16*)out, N, I, clear_in, also_zero, n4, s);
    }
    if (in_dtype == DT_F32 && out_dtype == DT_BF16) return launch_silu_mul<float, bf16>((float*)gu, (bf16*)out, N, I, clear_in, also_zero, n4, s);
    return LLMIE_ERR_BAD_ARGUMENT;
}

// ------------------------------------------------------------------------------------------------
// residual[i] += delta[i] (the residual stream is float32)
template <typename T, int VEC>
__global__ void add_into_kernel(float* __restrict__ residual, const T* __restrict__ delta, size_t total) {
    const size_t idx = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * VEC;
    if (idx >= total) return;
    if constexpr (VEC == 4) {
        float r[4], d[4];
        load4(residual + idx, r);
        load4(delta + idx, d);
#pragma unroll
        for (int j = 0; j < 4; ++j) r[j] += d[j];
        store4(residual + idx, r);
    } else {
        residual[idx] += to_f32(delta[idx]);
    }
}

LLMIE_API int llmie_add_into(float* residual, const void* delta, long long total, int dtype, cudaStream_t s) {
    if (total <= 0) return 0;
    const bool vec = total % 4 == 0 && ((uintptr_t)residual % 16 == 0) && ((uintptr_t)delta % 16 == 0);
    const long long work = vec ? total / 4 : total;
    const int blocks = (int)((work + 255) / 256);
    if (dtype == DT_F32) {
        if (vec) add_into_kernel<float, 4><<<blocks, 256, 0, s>>>(residual, (const float*)delta, (size_t)total);
        else add_into_kernel<float, 1><<<blocks, 256, 0, s>>>(residual, (const float*)delta, (size_t)total);
    } else {
        if (vec) add_into_kernel<bf16, 4><<<blocks, 256, 0, s>>>(residual, (const bf16*)delta, (size_t)total);
        else add_into_kernel<bf16, 1><<<blocks, 256, 0, s>>>(residual, (const bf16*)delta, (size_t)total);
    }
    return launch_status();
}
