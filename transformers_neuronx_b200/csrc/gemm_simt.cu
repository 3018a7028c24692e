// Matrix product on CUDA cores with 32-bit FMA accumulation: the true 32-bit path (no tensor
// cores, no reduced-precision mode), and the path for sizes that the tensor-core kernel refuses.
//
//   C[m, n] = epilogue( sum_k A[m, k] * W[n, k] )           A: [M, K], W: [N, K] (both row-major)
//   epilogue: + bias[n]; activation (by code, common.cuh); + residual[m, n] (32-bit); stored as float or in the 16-bit type.
//
// Every output element adds its products in ascending k with one accumulator, so a row's result
// does not depend on which other rows are in the call.
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

template <typename TA, typename TW, typename TO>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const TA* __restrict__ A, const TW* __restrict__ W, const float* __restrict__ bias,
                 const float* residual, TO* C, int M, int N, int K, int lda, int ldw, int ldc,
                 int act) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    pdl_launch_dependents();
    pdl_wait();
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int tx = tid % 16, ty = tid / 16;          // thread's 4x4 patch: rows ty*4.., cols tx*4..
    const int lrow = tid / 4, lk = (tid % 4) * 4;     // loader: one row, four consecutive k
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int k = k0 + lk + e;
            const int am = m0 + lrow, wn = n0 + lrow;
            As[lk + e][lrow] = (am < M && k < K) ? to_float(A[(size_t)am * lda + k]) : 0.f;
            Ws[lk + e][lrow] = (wn < N && k < K) ? to_float(W[(size_t)wn * ldw + k]) : 0.f;
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
        const int m = m0 + ty * TM + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int n = n0 + tx * TN + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (bias) v += bias[n];
            v = apply_activation(v, act);
            if (residual) v += residual[(size_t)m * ldc + n];
            C[(size_t)m * ldc + n] = from_float<TO>(v);
        }
    }
}

template <typename TA, typename TW, typename TO>
int launch(const void* A, const void* W, const float* bias, const float* residual, void* C, int M,
           int N, int K, int lda, int ldw, int ldc, int act, cudaStream_t stream) {
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    return tnx_launch_in_order(gemm_simt_kernel<TA, TW, TO>, grid, dim3(256), 0, stream, (const TA*)A, (const TW*)W, bias,
                          residual, (TO*)C, M, N, K, lda, ldw, ldc, act);
}

}  // namespace

// a_h16 / w_h16 / c_h16: element types (1 = bfloat16, 0 = float).  residual (32-bit, same
// leading dimension as C) may alias C when C is float.
TNX_EXPORT int tnx_gemm_simt(const void* A, const void* W, const float* bias, const float* residual,
                             void* C, int M, int N, int K, int lda, int ldw, int ldc, int act,
                             int a_h16, int w_h16, int c_h16, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || lda < K || ldw < K || ldc < N) return TNX_ERR_BAD_ARG;
    if (residual && c_h16) return TNX_ERR_BAD_ARG;
    if (act < 0 || act >= TNX_ACT_COUNT) return TNX_ERR_BAD_ARG;
    const int code = (a_h16 ? 4 : 0) | (w_h16 ? 2 : 0) | (c_h16 ? 1 : 0);
    switch (code) {
        case 0: return launch<float, float, float>(A, W, bias, residual, C, M, N, K, lda, ldw, ldc, act, stream);
        case 2: return launch<float, h16, float>(A, W, bias, residual, C, M, N, K, lda, ldw, ldc, act, stream);
        case 4: return launch<h16, float, float>(A, W, bias, residual, C, M, N, K, lda, ldw, ldc, act, stream);
        case 5: return launch<h16, float, h16>(A, W, bias, residual, C, M, N, K, lda, ldw, ldc, act, stream);
        case 6: return launch<h16, h16, float>(A, W, bias, residual, C, M, N, K, lda, ldw, ldc, act, stream);
        case 7: return launch<h16, h16, h16>(A, W, bias, residual, C, M, N, K, lda, ldw, ldc, act, stream);
        default: return TNX_ERR_UNSUPPORTED;
    }
}
