// C[M, N] = A[M, K] * W[N, K]^T, bfloat16 operands, fp32 accumulation, on mma.sync tensor cores.
//
// The general tiled kernel of the bfloat16 path: it takes every M and N (edges are predicated)
// and every K that is a multiple of 8 (16-byte rows), so it is the kernel behind shapes the
// tcgen05 kernel refuses.  CTA tile 128 x 128 x 32, eight warps of 64 x 32, a four-stage
// cp.async pipeline into XOR-swizzled shared memory, ldmatrix fragments.  An output element is
// accumulated over k in ascending order of 16-wide steps whatever M is, so a row does not
// depend on what else is in the batch.
#include "mma.cuh"

namespace {

constexpr int BM = 128, BN = 128, BK = 32, STAGES = 4, THREADS = 256;
constexpr int TILE_BYTES = BM * BK * 2;  // one operand, one stage

// element (row, 16-byte chunk) of a [128][32] bf16 tile; chunks are XOR-swizzled by row pair
__device__ __forceinline__ int swz(int row, int chunk) { return row * 64 + ((chunk ^ ((row >> 1) & 3)) << 4); }

template <typename TC>
__global__ void __launch_bounds__(THREADS) gemm_mma_kernel(const __nv_bfloat16* __restrict__ A, const __nv_bfloat16* __restrict__ W,
                                                          TC* __restrict__ C, int M, int N, int K, int64_t lda, int64_t ldc) {
    extern __shared__ __align__(128) unsigned char smem[];
    unsigned char* sA = smem;
    unsigned char* sB = smem + STAGES * TILE_BYTES;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int wm = warp >> 2, wn = warp & 3;  // 2 x 4 warps
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int KT = (K + BK - 1) / BK;

    float acc[4][4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++)
#pragma unroll
            for (int e = 0; e < 4; e++) acc[i][j][e] = 0.f;

    auto load_tile = [&](int kt, int stage) {
        const int k0 = kt * BK;
#pragma unroll
        for (int it = 0; it < 2; it++) {
            int idx = tid + it * THREADS;  // 0..511
            int row = idx >> 2, chunk = idx & 3;
            int k = k0 + chunk * 8;
            bool kin = k < K;
            {
                int m = m0 + row;
                bool ok = kin && m < M;
                const __nv_bfloat16* src = ok ? A + (int64_t)m * lda + k : A;
                cp_async16(sA + stage * TILE_BYTES + swz(row, chunk), src, ok ? 16 : 0);
            }
            {
                int n = n0 + row;
                bool ok = kin && n < N;
                const __nv_bfloat16* src = ok ? W + (int64_t)n * K + k : W;
                cp_async16(sB + stage * TILE_BYTES + swz(row, chunk), src, ok ? 16 : 0);
            }
        }
    };

#pragma unroll
    for (int s = 0; s < STAGES - 1; s++) {
        if (s < KT) load_tile(s, s);
        cp_async_commit();
    }
    for (int kt = 0; kt < KT; kt++) {
        cp_async_wait<STAGES - 2>();
        __syncthreads();
        {
            int nk = kt + STAGES - 1;
            if (nk < KT) load_tile(nk, nk % STAGES);
            cp_async_commit();
        }
        const unsigned char* a_s = sA + (kt % STAGES) * TILE_BYTES;
        const unsigned char* b_s = sB + (kt % STAGES) * TILE_BYTES;
#pragma unroll
        for (int ks = 0; ks < 2; ks++) {
            uint32_t af[4][4], bfr[4][2];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                int row = wm * 64 + i * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
                int chunk = ks * 2 + (lane >> 4);
                ldmatrix_x4(af[i], a_s + swz(row, chunk));
            }
#pragma unroll
            for (int jp = 0; jp < 2; jp++) {
                int row = wn * 32 + jp * 16 + (lane & 7) + (lane >> 4) * 8;
                int chunk = ks * 2 + ((lane >> 3) & 1);
                uint32_t r[4];
                ldmatrix_x4(r, b_s + swz(row, chunk));
                bfr[jp * 2][0] = r[0];
                bfr[jp * 2][1] = r[1];
                bfr[jp * 2 + 1][0] = r[2];
                bfr[jp * 2 + 1][1] = r[3];
            }
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) mma_bf16_16816(acc[i][j], af[i][0], af[i][1], af[i][2], af[i][3], bfr[j][0], bfr[j][1]);
        }
    }
    cp_async_wait<0>();

    const int g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int i = 0; i < 4; i++) {
#pragma unroll
        for (int half = 0; half < 2; half++) {
            int m = m0 + wm * 64 + i * 16 + g + half * 8;
            if (m >= M) continue;
            TC* crow = C + (int64_t)m * ldc;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                int n = n0 + wn * 32 + j * 8 + t * 2;
                if (n < N) crow[n] = from_f32<TC>(acc[i][j][half * 2]);
                if (n + 1 < N) crow[n + 1] = from_f32<TC>(acc[i][j][half * 2 + 1]);
            }
        }
    }
}

template <typename TC>
int launch(const void* A, const void* W, void* C, int M, int N, int K, int64_t lda, int64_t ldc, cudaStream_t stream) {
    static bool configured = false;
    const int smem = 2 * STAGES * TILE_BYTES;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_mma_kernel<TC>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) GB_REFUSE("gemm_mma: cannot reserve %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
        configured = true;
    }
    dim3 grid(ceil_div(N, BN), ceil_div(M, BM));
    if (grid.y > 65535) GB_REFUSE("gemm_mma: %d rows exceed one launch", M);
    gemm_mma_kernel<TC><<<grid, THREADS, smem, stream>>>((const __nv_bfloat16*)A, (const __nv_bfloat16*)W, (TC*)C, M, N, K, lda, ldc);
    GB_CHECK_LAUNCH("gemm_mma");
    return 0;
}

}  // namespace

GB_API int gb_gemm_mma(const void* A, const void* W, void* C, int c_dtype, int M, int N, int K, int64_t lda, int64_t ldc,
                       cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || (K & 7)) GB_REFUSE("gemm_mma: K = %d must be a positive multiple of 8", K);
    if ((lda & 7) || lda < K) GB_REFUSE("gemm_mma: row stride %lld of A must be a multiple of 8 and at least K", (long long)lda);
    if (ldc < N) GB_REFUSE("gemm_mma: row stride %lld of C is shorter than N = %d", (long long)ldc, N);
    if (((uintptr_t)A & 15) || ((uintptr_t)W & 15)) GB_REFUSE("gemm_mma: operands must be 16-byte aligned");
    if (c_dtype == GB_F32) return launch<float>(A, W, C, M, N, K, lda, ldc, stream);
    if (c_dtype == GB_BF16) return launch<__nv_bfloat16>(A, W, C, M, N, K, lda, ldc, stream);
    GB_REFUSE("gemm_mma: unknown output dtype %d", c_dtype);
}
