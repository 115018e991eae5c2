// Plain matrix product on the CUDA cores in true 32-bit:
//   C[M, N] = A[M, K] . W[N, K]^T      (W in checkpoint layout [out, in])
// Every output element is one chain of fused multiply-adds over k = 0..K-1 in
// ascending order, so a row of C does not depend on M, on the other rows, or
// on how the rows were batched.  Operands may be bf16 (widened exactly); the
// products and sums are 32-bit; no tensor-core or reduced-precision mode.
// It stands where the reference calls cuBLAS with 32-bit compute
// (infernum-cuda/src/inner/cuda/ops/matmul.rs:68-116) on its f32 path.
#include "common.cuh"

using namespace ib;

namespace {
constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;
}

template <typename TA, typename TW, typename TC>
__global__ void __launch_bounds__(256)
gemm_plain_kernel(const TA* __restrict__ A, int lda, const TW* __restrict__ W, int ldw,
                  TC* __restrict__ C, int ldc, int M, int N, int K) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    const int tid = threadIdx.x;
    const int tx = tid % 16, ty = tid / 16;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int lrow = tid / 4, lk = (tid % 4) * 4;

    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        {
            const int gm = m0 + lrow;
            const TA* src = A + (size_t)gm * lda + k0 + lk;
#pragma unroll
            for (int u = 0; u < 4; ++u)
                As[lk + u][lrow] = (gm < M && k0 + lk + u < K) ? to_f32(src[u]) : 0.f;
            const int gn = n0 + lrow;
            const TW* wsrc = W + (size_t)gn * ldw + k0 + lk;
#pragma unroll
            for (int u = 0; u < 4; ++u)
                Ws[lk + u][lrow] = (gn < N && k0 + lk + u < K) ? to_f32(wsrc[u]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[TM], w[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) w[j] = Ws[kk][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int gm = m0 + ty * TM + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int gn = n0 + tx * TN + j;
            if (gn < N) C[(size_t)gm * ldc + gn] = from_f32<TC>(acc[i][j]);
        }
    }
}

template <typename TA, typename TW, typename TC>
static int launch(const void* A, int lda, const void* W, int ldw, void* C, int ldc, int M, int N,
                  int K, cudaStream_t s) {
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    gemm_plain_kernel<TA, TW, TC><<<grid, 256, 0, s>>>((const TA*)A, lda, (const TW*)W, ldw,
                                                        (TC*)C, ldc, M, N, K);
    IB_LAUNCH_CHECK();
    return IB_OK;
}

// dtypes: 0 = f32, 1 = bf16.  Leading dimensions are in elements.
IB_EXPORT int ib_gemm_plain(const void* A, int a_dtype, int lda, const void* W, int w_dtype,
                            int ldw, void* C, int c_dtype, int ldc, int M, int N, int K,
                            void* stream) {
    if (M <= 0 || N <= 0) return IB_OK;
    if (!A || !W || !C || K <= 0 || lda < K || ldw < K || ldc < N) return IB_ERR_BAD_ARG;
    if ((M + BM - 1) / BM > 65535) return IB_ERR_TOO_LARGE;
    cudaStream_t s = (cudaStream_t)stream;
    const int key = a_dtype * 100 + w_dtype * 10 + c_dtype;
    switch (key) {
        case 0: return launch<float, float, float>(A, lda, W, ldw, C, ldc, M, N, K, s);
        case 10: return launch<float, bf16, float>(A, lda, W, ldw, C, ldc, M, N, K, s);
        case 100: return launch<bf16, float, float>(A, lda, W, ldw, C, ldc, M, N, K, s);
        case 101: return launch<bf16, float, bf16>(A, lda, W, ldw, C, ldc, M, N, K, s);
        case 110: return launch<bf16, bf16, float>(A, lda, W, ldw, C, ldc, M, N, K, s);
        case 111: return launch<bf16, bf16, bf16>(A, lda, W, ldw, C, ldc, M, N, K, s);
        default: return IB_ERR_UNSUPPORTED;
    }
}
