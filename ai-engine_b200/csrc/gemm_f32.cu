// True float32 matrix product on the CUDA cores (FMA; no tensor cores, no TF32):
//   C[M, N] = A[M, K] . W[N, K]^T        (weights as stored by HF: [out, in])
// It is the 32-bit path of every projection and of the LM head.  Each output
// element is one thread's running sum over k = 0 .. K-1 in that order, so a
// row's result does not depend on M: the same token gives the same bits
// whatever else is in the batch.
// The reference multiplies x[B,S,in] by a weight kept as [in,out]
// (crates/ai-engine-runtime/src/arch/linear.rs:106-123); the product is the same.
#include "common.cuh"

#define BM 64
#define BN 64
#define BK 16

template <typename WT>
__global__ void __launch_bounds__(256)
gemm_f32_kernel(const float* __restrict__ A, const WT* __restrict__ W, float* __restrict__ C,
                const int* __restrict__ a_rows, int M, int N, int K, int ldc) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int tm = (tid / 16) * 4, tn = (tid % 16) * 4;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    // loader mapping: 64 rows x 16 k per tile, 256 threads -> 4 consecutive k each
    const int lr = tid / 4, lk = (tid % 4) * 4;
    const int am = m0 + lr, wn = n0 + lr;
    const float* arow = nullptr;
    if (am < M) arow = A + (size_t)(a_rows ? a_rows[am] : am) * K;
    const WT* wrow = wn < N ? W + (size_t)wn * K : nullptr;

    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int k = k0 + lk + j;
            As[lk + j][lr] = (arow && k < K) ? arow[k] : 0.f;
            Ws[lk + j][lr] = (wrow && k < K) ? to_f32<WT>(wrow[k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[k][tm + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) w[j] = Ws[k][tn + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + tm + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tn + j;
            if (n < N) C[(size_t)m * ldc + n] = acc[i][j];
        }
    }
}

// a_rows (optional): row m of the product reads A[a_rows[m]] (the LM head runs
// only on the rows whose logits are wanted).
extern "C" int aie_gemm_f32(const float* A, const void* W, int w_dtype, float* C, const int* a_rows,
                            int M, int N, int K, int ldc, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0) return AIE_BAD_ARG;
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    if (grid.y > 65535) return AIE_UNSUPPORTED;
    if (w_dtype == AIE_F32)
        gemm_f32_kernel<float><<<grid, 256, 0, stream>>>(A, (const float*)W, C, a_rows, M, N, K, ldc);
    else if (w_dtype == AIE_BF16)
        gemm_f32_kernel<bf16><<<grid, 256, 0, stream>>>(A, (const bf16*)W, C, a_rows, M, N, K, ldc);
    else
        return AIE_BAD_ARG;
    AIE_LAUNCH_CHECK();
}
