// C[M, N] = A[M, K] * W[N, K]^T with fp32 multiply-add on the CUDA cores.
//
// This is the matrix product of the true 32-bit path (no tensor cores, no reduced-precision
// mode) and the fallback for operand types or sizes the tensor-core kernels refuse (for
// instance a weight the checkpoint stores in 32-bit while activations are bfloat16).
// Every output element is the sum over k in ascending order in one fp32 accumulator, whatever M
// is and wherever the element lies in a tile: rows do not depend on what else is in the batch.
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16;

template <typename TA, typename TW, typename TC>
__global__ void __launch_bounds__(256) gemm_simt_kernel(const TA* __restrict__ A, const TW* __restrict__ W,
                                                        TC* __restrict__ C, int M, int N, int K, int64_t lda,
                                                        int64_t ldw, int64_t ldc) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    int tid = threadIdx.x;
    int tx = tid & 15, ty = tid >> 4;
    int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.f;

    int lrow = tid >> 2;        // 0..63
    int lk = (tid & 3) * 4;     // 0,4,8,12
    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int i = 0; i < 4; i++) {
            int k = k0 + lk + i;
            int m = m0 + lrow, n = n0 + lrow;
            As[lk + i][lrow] = (m < M && k < K) ? to_f32<TA>(A[(int64_t)m * lda + k]) : 0.f;
            Ws[lk + i][lrow] = (n < N && k < K) ? to_f32<TW>(W[(int64_t)n * ldw + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; kk++) {
            float a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; i++) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; j++) w[j] = Ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            int n = n0 + tx * 4 + j;
            if (n < N) C[(int64_t)m * ldc + n] = from_f32<TC>(acc[i][j]);
        }
    }
}

template <typename TA, typename TW, typename TC>
int launch(const void* A, const void* W, void* C, int M, int N, int K, int64_t lda, int64_t ldw, int64_t ldc,
           cudaStream_t stream) {
    dim3 grid(ceil_div(N, BN), ceil_div(M, BM));
    if (grid.y > 65535) GB_REFUSE("gemm_simt: %d rows exceed one launch (%d); the step splits larger batches", M, 65535 * BM);
    gemm_simt_kernel<TA, TW, TC><<<grid, 256, 0, stream>>>((const TA*)A, (const TW*)W, (TC*)C, M, N, K, lda, ldw, ldc);
    GB_CHECK_LAUNCH("gemm_simt");
    return 0;
}

}  // namespace

GB_API int gb_gemm_simt(const void* A, int a_dtype, const void* W, int w_dtype, void* C, int c_dtype, int M, int N,
                        int K, int64_t lda, int64_t ldw, int64_t ldc, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0) GB_REFUSE("gemm_simt: K = %d", K);
    if (lda < K || ldw < K || ldc < N) GB_REFUSE("gemm_simt: strides (%lld, %lld, %lld) are shorter than the rows (K %d, N %d)",
                                                 (long long)lda, (long long)ldw, (long long)ldc, K, N);
    if ((a_dtype | w_dtype | c_dtype) & ~1) GB_REFUSE("gemm_simt: unknown dtypes (%d, %d, %d)", a_dtype, w_dtype, c_dtype);
    typedef __nv_bfloat16 bf;
    int key = a_dtype * 4 + w_dtype * 2 + c_dtype;
    switch (key) {
        case 0: return launch<float, float, float>(A, W, C, M, N, K, lda, ldw, ldc, stream);
        case 1: return launch<float, float, bf>(A, W, C, M, N, K, lda, ldw, ldc, stream);
        case 2: return launch<float, bf, float>(A, W, C, M, N, K, lda, ldw, ldc, stream);
        case 3: return launch<float, bf, bf>(A, W, C, M, N, K, lda, ldw, ldc, stream);
        case 4: return launch<bf, float, float>(A, W, C, M, N, K, lda, ldw, ldc, stream);
        case 5: return launch<bf, float, bf>(A, W, C, M, N, K, lda, ldw, ldc, stream);
        case 6: return launch<bf, bf, float>(A, W, C, M, N, K, lda, ldw, ldc, stream);
        case 7: return launch<bf, bf, bf>(A, W, C, M, N, K, lda, ldw, ldc, stream);
    }
    GB_REFUSE("gemm_simt: unknown dtypes (%d, %d, %d)", a_dtype, w_dtype, c_dtype);
}
