// C[M,N] = A[M,K] * W[N,K]^T + bias[N] with float32 FMAs on the SIMT cores.
//
// This is the true 32-bit matrix product of the engine (no tensor cores, no reduced
// precision mode) and the fallback for operand types the tensor-core kernels do not take.
// Every output element is one chain acc = fmaf(a[k], w[k], acc) over k = 0..K-1 in rising
// order, then + bias: the result of a row does not depend on M, on the row's place in the
// batch, or on the tile it falls in.
#include "zi_common.cuh"

ZI_DEFINE_LAST_ERROR(gemm_simt)

#define BM 64
#define BN 64
#define BK 16
#define TM 4
#define TN 4

template <typename TA, typename TW, typename TB, typename TC>
__global__ void __launch_bounds__(256)
gemm_nt_kernel(const TA* __restrict__ A, const TW* __restrict__ W, const TB* __restrict__ bias,
               TC* __restrict__ C, int M, int N, int K, long long lda, long long ldw, long long ldc) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;            // 16 x 16 threads, 4x4 outputs each
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;

    // each thread loads 4 elements of each tile: row = tid/4 (0..63), k = (tid%4)*4 .. +3
    const int lr = tid >> 2, lk = (tid & 3) * 4;
    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int k = k0 + lk + q;
            const int am = m0 + lr, wn = n0 + lr;
            As[lk + q][lr] = (am < M && k < K) ? to_f32<TA>(A[(size_t)am * lda + k]) : 0.0f;
            Ws[lk + q][lr] = (wn < N && k < K) ? to_f32<TW>(W[(size_t)wn * ldw + k]) : 0.0f;
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
            if (bias) v += to_f32<TB>(bias[n]);
            C[(size_t)m * ldc + n] = from_f32<TC>(v);
        }
    }
}

// Zero padding inside a K tile adds fmaf(0, 0, acc) = acc, so the chain over the real k is unchanged.

ZI_EXPORT int zi_gemm_nt(const void* A, int a_dtype, const void* W, int w_dtype, const void* bias, int bias_dtype,
                         void* C, int c_dtype, int M, int N, int K, long long lda, long long ldw, long long ldc,
                         cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0) return zi_fail("gemm: K=%d must be positive", K);
    if (lda < K || ldw < K || ldc < N) return zi_fail("gemm: leading dimensions (%lld, %lld, %lld) too small for K=%d N=%d", lda, ldw, ldc, K, N);
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    if (grid.y > 65535) return zi_fail("gemm: M=%d is too large for one launch", M);
    ZI_DISPATCH(a_dtype, TA, ZI_DISPATCH(w_dtype, TW, ZI_DISPATCH(bias_dtype, TB, ZI_DISPATCH(c_dtype, TC, {
        gemm_nt_kernel<TA, TW, TB, TC><<<grid, 256, 0, stream>>>((const TA*)A, (const TW*)W, (const TB*)bias, (TC*)C,
                                                                 M, N, K, lda, ldw, ldc);
    }););););
    return zi_check_launch("gemm_nt");
}
