// Y[M, N] = X[M, K] * W[N, K]^T for a few rows (M <= 64): the decode-step matrix product.
//
// The step is bound by reading W once from HBM, so the kernel is built around that stream.  The
// weight rows take the M side of the tensor-core instruction and the batch takes the N side
// (Y^T = W X^T): a warp owns 16 weight rows and walks a K range; each lane reads 16 contiguous
// bytes of its two rows straight from global memory into the A fragment, with no shared-memory
// staging.  That is possible because a dot product does not care in which order k is visited:
// within a 32-wide K step, lane (g, t) holds k = 8t .. 8t+7, used as the fragment's logical
// columns (2t, 2t+1, 2t+8, 2t+9) in a first instruction and again in a second one, and the
// activations are read with the same assignment.  Warps of a CTA split K and are summed in a
// fixed order through shared memory, so results do not depend on the batch around a row.
#include "mma.cuh"

namespace {

constexpr int MIN_STEPS = 4;  // fewest 32-wide K steps a warp should own

template <int MT>  // MT tiles of 8 batch rows
__global__ void __launch_bounds__(512) gemm_skinny_kernel(const __nv_bfloat16* __restrict__ X, const __nv_bfloat16* __restrict__ W,
                                                         void* __restrict__ Yv, int y_is_bf16, int M, int N, int K, int64_t ldx,
                                                         int64_t ldy, int k_per_warp, int epi) {
    extern __shared__ float red[];  // [KW][16][MT * 8]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, KW = blockDim.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int n0 = blockIdx.x * 16;
    int r_lo = n0 + g, r_hi = n0 + g + 8;
    if (r_lo >= N) r_lo = N - 1;  // clamped rows are computed and dropped
    if (r_hi >= N) r_hi = N - 1;
    const __nv_bfloat16* w_lo = W + (int64_t)r_lo * K + t * 8;
    const __nv_bfloat16* w_hi = W + (int64_t)r_hi * K + t * 8;
    const __nv_bfloat16* xp[MT];
#pragma unroll
    for (int j = 0; j < MT; j++) {
        int b = j * 8 + g;
        if (b >= M) b = M - 1;
        xp[j] = X + (int64_t)b * ldx + t * 8;
    }
    float acc[MT][4];
#pragma unroll
    for (int j = 0; j < MT; j++)
#pragma unroll
        for (int e = 0; e < 4; e++) acc[j][e] = 0.f;

    const int k_begin = warp * k_per_warp;
    int k_end = k_begin + k_per_warp;
    if (k_end > K) k_end = K;
    const int k_full = k_begin + ((k_end - k_begin) / 32) * 32;

    // The weights do not depend on the kernel before this one: start this warp's first weight
    // loads while that kernel may still be running (programmatic dependent launch), then wait for
    // it, let the kernel after this one start its own prologue, and only then read activations.
    int k = k_begin;
    constexpr int PRE = 4;
    const bool pre = k + PRE * 32 <= k_full;
    uint4 a_lo[PRE], a_hi[PRE];
    if (pre) {
#pragma unroll
        for (int u = 0; u < PRE; u++) {
            a_lo[u] = ld_stream16(w_lo + k + u * 32);
            a_hi[u] = ld_stream16(w_hi + k + u * 32);
        }
    }
    pdl_wait_cta();
    pdl_trigger();
    if (pre) {
#pragma unroll
        for (int u = 0; u < PRE; u++) {
#pragma unroll
            for (int j = 0; j < MT; j++) {
                uint4 xb = *reinterpret_cast<const uint4*>(xp[j] + k + u * 32);
                mma_bf16_16816(acc[j], a_lo[u].x, a_hi[u].x, a_lo[u].y, a_hi[u].y, xb.x, xb.y);
                mma_bf16_16816(acc[j], a_lo[u].z, a_hi[u].z, a_lo[u].w, a_hi[u].w, xb.z, xb.w);
            }
        }
        k += PRE * 32;
    }
#pragma unroll 4
    for (; k < k_full; k += 32) {
        uint4 a_lo = ld_stream16(w_lo + k);
        uint4 a_hi = ld_stream16(w_hi + k);
#pragma unroll
        for (int j = 0; j < MT; j++) {
            uint4 xb = *reinterpret_cast<const uint4*>(xp[j] + k);
            mma_bf16_16816(acc[j], a_lo.x, a_hi.x, a_lo.y, a_hi.y, xb.x, xb.y);
            mma_bf16_16816(acc[j], a_lo.z, a_hi.z, a_lo.w, a_hi.w, xb.z, xb.w);
        }
    }
    if (k < k_end) {  // K is a multiple of 8: a lane's chunk is wholly inside or wholly outside
        const bool in = k + t * 8 < k_end;
        uint4 z = make_uint4(0, 0, 0, 0);
        uint4 a_lo = in ? ld_stream16(w_lo + k) : z;
        uint4 a_hi = in ? ld_stream16(w_hi + k) : z;
#pragma unroll
        for (int j = 0; j < MT; j++) {
            uint4 xb = in ? *reinterpret_cast<const uint4*>(xp[j] + k) : z;
            mma_bf16_16816(acc[j], a_lo.x, a_hi.x, a_lo.y, a_hi.y, xb.x, xb.y);
            mma_bf16_16816(acc[j], a_lo.z, a_hi.z, a_lo.w, a_hi.w, xb.z, xb.w);
        }
    }

    // fragment (rows g, g + 8 of the weight tile; batch columns 2t, 2t + 1) -> red[warp][row][batch]
    constexpr int MB = MT * 8;
    float* mine = red + (size_t)warp * 16 * MB;
#pragma unroll
    for (int j = 0; j < MT; j++) {
        mine[g * MB + j * 8 + 2 * t] = acc[j][0];
        mine[g * MB + j * 8 + 2 * t + 1] = acc[j][1];
        mine[(g + 8) * MB + j * 8 + 2 * t] = acc[j][2];
        mine[(g + 8) * MB + j * 8 + 2 * t + 1] = acc[j][3];
    }
    __syncthreads();
    if (epi == 1) {
        // rows 0-7 of the tile are gate rows and rows 8-15 the up rows of the same eight outputs:
        // out[b, n0 / 2 + i] = silu(gate) * up            (internal/qwen3lm/gpu.metal:130-137)
        for (int idx = threadIdx.x; idx < 8 * MB; idx += blockDim.x) {
            int b = idx >> 3, i = idx & 7;
            if (b >= M || n0 + 8 + i >= N) continue;
            float gsum = 0.f, usum = 0.f;
            for (int w = 0; w < KW; w++) {
                gsum += red[(size_t)w * 16 * MB + i * MB + b];
                usum += red[(size_t)w * 16 * MB + (i + 8) * MB + b];
            }
            float act = gsum >= 0.f ? gsum / (1.f + expf(-gsum)) : gsum * expf(gsum) / (1.f + expf(gsum));
            act *= usum;
            int64_t o = (int64_t)b * ldy + (n0 >> 1) + i;
            if (y_is_bf16)
                ((__nv_bfloat16*)Yv)[o] = __float2bfloat16_rn(act);
            else
                ((float*)Yv)[o] = act;
        }
        return;
    }
    for (int idx = threadIdx.x; idx < 16 * MB; idx += blockDim.x) {
        int b = idx >> 4, i = idx & 15;  // 16 consecutive outputs of one batch row
        if (b >= M || n0 + i >= N) continue;
        float s = 0.f;
        for (int w = 0; w < KW; w++) s += red[(size_t)w * 16 * MB + i * MB + b];
        if (y_is_bf16)
            ((__nv_bfloat16*)Yv)[(int64_t)b * ldy + n0 + i] = __float2bfloat16_rn(s);
        else
            ((float*)Yv)[(int64_t)b * ldy + n0 + i] = s;
    }
}

template <int MT>
int launch(const void* X, const void* W, void* Y, int c_dtype, int M, int N, int K, int64_t ldx, int64_t ldy, int epi,
           cudaStream_t stream) {
    int steps = ceil_div(K, 32);
    // Few weight tiles (narrow outputs) leave SMs short of loads in flight: give each CTA more warps.
    // See skinny_warps() in mma.cuh.
    int max_kw = skinny_warps(ceil_div(N, 16));
    if (MT > 4 && max_kw > 8) max_kw = 8;  // many batch rows: the accumulators take the registers of the second CTA
    int kw = 1;
    while (kw < max_kw && steps / (kw * 2) >= MIN_STEPS) kw *= 2;
    int k_per_warp = ceil_div(steps, kw) * 32;
    size_t smem = (size_t)kw * 16 * MT * 8 * sizeof(float);
    // as a programmatic dependent launch the kernel requests its first weights before it waits for the
    // kernel ahead of it; see skinny_dependent() for when it is one
    const bool dependent = skinny_dependent(ceil_div(N, 16));
    cudaError_t e = launch_maybe_pdl(dependent, gemm_skinny_kernel<MT>, dim3(ceil_div(N, 16)), dim3(kw * 32), smem, stream, (const __nv_bfloat16*)X,
                               (const __nv_bfloat16*)W, Y, (int)(c_dtype == GB_BF16), M, N, K, ldx, ldy, k_per_warp, epi);
    if (e != cudaSuccess) GB_REFUSE("gemm_skinny: launch failed: %s", cudaGetErrorString(e));
    return 0;
}

}  // namespace

static int skinny(const void* X, const void* W, void* Y, int c_dtype, int M, int N, int K, int64_t ldx, int64_t ldy, int epi,
                  cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > 64) GB_REFUSE("gemm_skinny: %d rows; this kernel takes at most 64", M);
    if (K <= 0 || (K & 7)) GB_REFUSE("gemm_skinny: K = %d must be a positive multiple of 8", K);
    if ((ldx & 7) || ldx < K) GB_REFUSE("gemm_skinny: row stride %lld of X must be a multiple of 8 and at least K", (long long)ldx);
    if (epi == 0 && ldy < N) GB_REFUSE("gemm_skinny: row stride %lld of Y is shorter than N = %d", (long long)ldy, N);
    if (epi == 1 && ((N & 15) || ldy < N / 2))
        GB_REFUSE("gemm_skinny: the SwiGLU epilogue needs N = %d to be a multiple of 16 and Y rows of at least N / 2 (stride %lld)", N, (long long)ldy);
    if (((uintptr_t)X & 15) || ((uintptr_t)W & 15)) GB_REFUSE("gemm_skinny: operands must be 16-byte aligned");
    if (c_dtype != GB_F32 && c_dtype != GB_BF16) GB_REFUSE("gemm_skinny: unknown output dtype %d", c_dtype);
    if (M <= 8) return launch<1>(X, W, Y, c_dtype, M, N, K, ldx, ldy, epi, stream);
    if (M <= 16) return launch<2>(X, W, Y, c_dtype, M, N, K, ldx, ldy, epi, stream);
    if (M <= 32) return launch<4>(X, W, Y, c_dtype, M, N, K, ldx, ldy, epi, stream);
    return launch<8>(X, W, Y, c_dtype, M, N, K, ldx, ldy, epi, stream);
}

GB_API int gb_gemm_skinny(const void* X, const void* W, void* Y, int c_dtype, int M, int N, int K, int64_t ldx, int64_t ldy,
                          cudaStream_t stream) {
    return skinny(X, W, Y, c_dtype, M, N, K, ldx, ldy, 0, stream);
}

// Y[M, N / 2] = silu(X Wg^T) * (X Wu^T) where W holds gate and up rows interleaved in blocks of
// eight (rows 16j .. 16j+7 are gate rows 8j .. 8j+7, rows 16j+8 .. 16j+15 the matching up rows).
GB_API int gb_gemm_skinny_swiglu(const void* X, const void* W, void* Y, int c_dtype, int M, int N, int K, int64_t ldx,
                                 int64_t ldy, cudaStream_t stream) {
    return skinny(X, W, Y, c_dtype, M, N, K, ldx, ldy, 1, stream);
}
