// C[M, N] = A[M, K] * W[N, K]^T on the CUDA cores, 32-bit multiply-add, one fixed order over K.
//
// This is the matrix product of the true 32-bit path (no tensor cores, no reduced-precision mode),
// and it also takes bfloat16 inputs (32-bit accumulate) for shapes the tensor-core kernels refuse.
// Every output element is the sum over k = 0 .. K-1 in that order by fused multiply-add, whatever
// M is and wherever the row lies in the batch: a token's result does not depend on its neighbours.
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;  // 16 x 16 threads, 4 x 4 outputs each

template <typename T>
__device__ __forceinline__ void load4(const T* __restrict__ base, int row, int rows, int k, int K, bool vec, float* out) {
    out[0] = out[1] = out[2] = out[3] = 0.f;
    if (row >= rows) return;
    const T* p = base + (size_t)row * K + k;
    if (vec && k + 3 < K) {
        if constexpr (sizeof(T) == 4) {
            const float4 v = *reinterpret_cast<const float4*>(p);
            out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
        } else {
            const uint2 v = *reinterpret_cast<const uint2*>(p);
            out[0] = __uint_as_float(v.x << 16); out[1] = __uint_as_float(v.x & 0xffff0000u);
            out[2] = __uint_as_float(v.y << 16); out[3] = __uint_as_float(v.y & 0xffff0000u);
        }
    } else {
#pragma unroll
        for (int i = 0; i < 4; ++i)
            if (k + i < K) out[i] = to_f32(p[i]);
    }
}

template <typename TI, typename TO>
__global__ void __launch_bounds__(256) gemm_simt_kernel(const TI* __restrict__ A, const TI* __restrict__ W, TO* __restrict__ C,
                                                       int M, int N, int K, int vec, int accumulate) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int lrow = tid >> 2, lk = (tid & 3) * 4;  // each thread stages 4 consecutive k of one row of each tile
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        float a[4], w[4];
        load4<TI>(A, m0 + lrow, M, k0 + lk, K, vec, a);
        load4<TI>(W, n0 + lrow, N, k0 + lk, K, vec, w);
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            As[lk + i][lrow] = a[i];
            Ws[lk + i][lrow] = w[i];
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float av[TM], wv[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) av[i] = As[kk][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) wv[j] = Ws[kk][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
        }
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int m = m0 + ty * TM + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int n = n0 + tx * TN + j;
            if (n < N) {
                TO* dst = C + (size_t)m * N + n;  // with `accumulate` the product is added to what C holds (its only writer is this thread)
                *dst = from_f32<TO>(accumulate ? to_f32(*dst) + acc[i][j] : acc[i][j]);
            }
        }
    }
}

}  // namespace

// in_dtype / out_dtype: 0 float32, 1 bfloat16. Beyond K the tiles are padded with zeros, which add nothing.
LLMIE_API int llmie_gemm_simt(const void* A, const void* W, void* C, int M, int N, int K, int in_dtype, int out_dtype,
                              int accumulate, cudaStream_t s) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0) return LLMIE_ERR_BAD_ARGUMENT;
    const dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    const int vec = (K % 4 == 0) && ((uintptr_t)A % 16 == 0) && ((uintptr_t)W % 16 == 0);
    if (in_dtype == DT_F32 && out_dtype == DT_F32)
        gemm_simt_kernel<float, float><<<grid, 256, 0, s>>>((const float*)A, (const float*)W, (float*)C, M, N, K, vec, accumulate);
    else if (in_dtype == DT_BF16 && out_dtype == DT_F32)
        gemm_simt_kernel<bf16, float><<<grid, 256, 0, s>>>((const bf16*)A, (const bf16*)W, (float*)C, M, N, K, vec, accumulate);
    else if (in_dtype == DT_BF16 && out_dtype == DT_BF16)
        gemm_simt_kernel<bf16, bf16><<<grid, 256, 0, s>>>((const bf16*)A, (const bf16*)W, (bf16*)C, M, N, K, vec, accumulate);
    else
        return LLMIE_ERR_BAD_ARGUMENT;
    return launch_status();
}
