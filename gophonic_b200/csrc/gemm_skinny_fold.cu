// The few-row product (gemm_skinny.cu: up to 8 rows, weights streamed from global memory straight
// into tensor-core fragments, K split over the warps of a CTA) with the residual stream's two
// row-wise kernels folded into it, so that a decode layer runs without its two norm kernels
// (the reference's decode layer folds its norms the same way: the producer's epilogue adds into
// the residual and publishes partial sums of squares, the consumer applies the RMSNorm factor from
// them: internal/qwen3lm/gpu.metal:70-162).
//
// RMSNorm is y = h * rs * w with rs = 1 / sqrt(sum(h^2) / n + eps) a constant of the row.  The
// producer, which has just made 16 new residual values of each row, knows h and the norm's weight
// but not yet the row's sum; the consumer knows the sum but would pay for h and w in its inner
// loop.  So the work is cut where it is free on both sides:
//
//   EPI 2 (producer):  Y is the fp32 residual itself: Y += product, one thread per element and one
//           fp32 addition each, as the separate add gave; stats_out[row][blockIdx.x] = the sum of
//           squares of this CTA's 16 new values of the row, taken in a fixed order; and, if the next
//           norm's weight is given, xn_out = bf16(Y * w_next): the next product's activations but for
//           their row factor.
//   SCALED (consumer): the activations X lack their row factor; the finished fp32 sums are
//           multiplied by rs in the epilogue, with sum(h^2) added up in a fixed order from the
//           `count` partial sums stats_in[row][0 .. count) (the warps' shares, then the warps in
//           order).  This is the product of the normed row with the activations rounded to bfloat16
//           before instead of after the factor: the same relative rounding.
//   EPI 0:  Y = product (bfloat16 or fp32).   EPI 1:  Y = silu(gate) * up for gate/up rows
//           interleaved in blocks of eight.
//
// A row's result depends on nothing else in the batch.
#include "mma.cuh"

namespace {

constexpr int MIN_STEPS = 4;
constexpr int STAT_ROWS = 8;  // rows of a statistics buffer: [STAT_ROWS][count]

// 1 / sqrt(mean of squares + eps) of batch row bb from the warps' shares, added in warp order
__device__ __forceinline__ float row_factor(const float (*stat_part)[STAT_ROWS], int KW, int bb, int n, float eps) {
    float total = 0.f;
    for (int w = 0; w < KW; w++) total += stat_part[w][bb];
    return 1.0f / sqrtf(total / (float)n + eps);
}

template <bool SCALED, int EPI>
__global__ void __launch_bounds__(512, 2) gemm_skinny_fold_kernel(const __nv_bfloat16* __restrict__ X, int64_t ldx,
                                                                  const float* __restrict__ stats_in, int stats_count,
                                                                  int64_t stats_in_stride, float eps, const __nv_bfloat16* __restrict__ W,
                                                                  void* __restrict__ Yv, int y_is_bf16, int64_t ldy,
                                                                  float* __restrict__ stats_out, int64_t stats_out_stride,
                                                                  const float* __restrict__ next_w, __nv_bfloat16* __restrict__ xn_out,
                                                                  int64_t ldxn, int M, int N, int K, int k_per_warp) {
    extern __shared__ float red[];  // [KW][16][8]
    __shared__ float stat_part[16][STAT_ROWS];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, KW = blockDim.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int n0 = blockIdx.x * 16;
    int r_lo = n0 + g, r_hi = n0 + g + 8;
    if (r_lo >= N) r_lo = N - 1;  // clamped rows are computed and dropped
    if (r_hi >= N) r_hi = N - 1;
    const __nv_bfloat16* w_lo = W + (int64_t)r_lo * K + t * 8;
    const __nv_bfloat16* w_hi = W + (int64_t)r_hi * K + t * 8;
    const int b = g < M ? g : M - 1;  // this lane's batch row
    const __nv_bfloat16* xp = X + (int64_t)b * ldx + t * 8;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};

    const int k_begin = warp * k_per_warp;
    int k_end = k_begin + k_per_warp;
    if (k_end > K) k_end = K;
    const int k_full = k_begin + ((k_end - k_begin) / 32) * 32;

    // the weights do not depend on the kernel ahead: request this warp's first ones before waiting for it
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

    if (SCALED) {
        // this warp's share of the partial sums of squares of row g, four lanes a row, for the epilogue;
        // fetched here, while the first weights are on their way (fetched behind the products instead,
        // the wait showed: 40.1 against 37.6 us for the gate/up product of an 8B layer at eight rows)
        const int per = (stats_count + KW - 1) / KW;
        const int c_lo = warp * per, c_hi = min(stats_count, c_lo + per);
        const float* sp = stats_in + (int64_t)b * stats_in_stride;
        float s = 0.f;
        for (int c = c_lo + t; c < c_hi; c += 4) s += sp[c];
        s += __shfl_xor_sync(0xffffffffu, s, 1);
        s += __shfl_xor_sync(0xffffffffu, s, 2);
        if (t == 0) stat_part[warp][g] = s;
    }
    if (pre) {
#pragma unroll
        for (int u = 0; u < PRE; u++) {
            const uint4 xb = *reinterpret_cast<const uint4*>(xp + k + u * 32);
            mma_bf16_16816(acc, a_lo[u].x, a_hi[u].x, a_lo[u].y, a_hi[u].y, xb.x, xb.y);
            mma_bf16_16816(acc, a_lo[u].z, a_hi[u].z, a_lo[u].w, a_hi[u].w, xb.z, xb.w);
        }
        k += PRE * 32;
    }
#pragma unroll 4
    for (; k < k_full; k += 32) {
        const uint4 lo = ld_stream16(w_lo + k);
        const uint4 hi = ld_stream16(w_hi + k);
        const uint4 xb = *reinterpret_cast<const uint4*>(xp + k);
        mma_bf16_16816(acc, lo.x, hi.x, lo.y, hi.y, xb.x, xb.y);
        mma_bf16_16816(acc, lo.z, hi.z, lo.w, hi.w, xb.z, xb.w);
    }
    if (k < k_end) {  // K is a multiple of 8: a lane's chunk is wholly inside or wholly outside
        const bool in = k + t * 8 < k_end;
        const uint4 z = make_uint4(0, 0, 0, 0);
        const uint4 lo = in ? ld_stream16(w_lo + k) : z;
        const uint4 hi = in ? ld_stream16(w_hi + k) : z;
        const uint4 xb = in ? *reinterpret_cast<const uint4*>(xp + k) : z;
        mma_bf16_16816(acc, lo.x, hi.x, lo.y, hi.y, xb.x, xb.y);
        mma_bf16_16816(acc, lo.z, hi.z, lo.w, hi.w, xb.z, xb.w);
    }

    // fragment (rows g, g + 8 of the weight tile; batch columns 2t, 2t + 1) -> red[warp][row][batch]
    constexpr int MB = 8;
    float* mine = red + (size_t)warp * 16 * MB;
    mine[g * MB + 2 * t] = acc[0];
    mine[g * MB + 2 * t + 1] = acc[1];
    mine[(g + 8) * MB + 2 * t] = acc[2];
    mine[(g + 8) * MB + 2 * t + 1] = acc[3];
    __syncthreads();
    if (EPI == 1) {
        // rows 0-7 of the tile are gate rows and rows 8-15 the up rows of the same eight outputs
        for (int idx = threadIdx.x; idx < 8 * MB; idx += blockDim.x) {
            const int bb = idx >> 3, i = idx & 7;
            if (bb >= M || n0 + 8 + i >= N) continue;
            float gsum = 0.f, usum = 0.f;
            for (int w = 0; w < KW; w++) {
                gsum += red[(size_t)w * 16 * MB + i * MB + bb];
                usum += red[(size_t)w * 16 * MB + (i + 8) * MB + bb];
            }
            if (SCALED) {
                const float rs = row_factor(stat_part, KW, bb, K, eps);
                gsum *= rs;
                usum *= rs;
            }
            float act = gsum >= 0.f ? gsum / (1.f + expf(-gsum)) : gsum * expf(gsum) / (1.f + expf(gsum));
            act *= usum;
            const int64_t o = (int64_t)bb * ldy + (n0 >> 1) + i;
            if (y_is_bf16)
                ((__nv_bfloat16*)Yv)[o] = __float2bfloat16_rn(act);
            else
                ((float*)Yv)[o] = act;
        }
        return;
    }
    // 16 consecutive threads hold the 16 outputs of one batch row; whole warps take part or stay out
    for (int base = 0; base + warp * 32 < 16 * MB; base += blockDim.x) {
        const int idx = base + threadIdx.x;
        const int bb = idx >> 4, i = idx & 15;
        const bool valid = bb < M && n0 + i < N;
        float s = 0.f;
        for (int w = 0; w < KW; w++) s += red[(size_t)w * 16 * MB + i * MB + bb];
        if (EPI == 2) {
            float sq = 0.f;
            if (valid) {
                float* hq = (float*)Yv + (int64_t)bb * ldy + n0 + i;
                const float hn = *hq + s;
                *hq = hn;
                sq = hn * hn;
                if (next_w != nullptr) xn_out[(int64_t)bb * ldxn + n0 + i] = __float2bfloat16_rn(hn * next_w[n0 + i]);
            }
            sq += __shfl_xor_sync(0xffffffffu, sq, 8);
            sq += __shfl_xor_sync(0xffffffffu, sq, 4);
            sq += __shfl_xor_sync(0xffffffffu, sq, 2);
            sq += __shfl_xor_sync(0xffffffffu, sq, 1);
            if (i == 0 && bb < M) stats_out[(int64_t)bb * stats_out_stride + blockIdx.x] = sq;
        } else if (valid) {
            if (SCALED) s *= row_factor(stat_part, KW, bb, K, eps);
            if (y_is_bf16)
                ((__nv_bfloat16*)Yv)[(int64_t)bb * ldy + n0 + i] = __float2bfloat16_rn(s);
            else
                ((float*)Yv)[(int64_t)bb * ldy + n0 + i] = s;
        }
    }
}

struct FoldArgs {
    const void* X;
    int64_t ldx;
    const float* stats_in;
    int stats_count;
    int64_t stats_in_stride;
    float eps;
    const void* W;
    void* Y;
    int y_dtype;
    int64_t ldy;
    float* stats_out;
    int64_t stats_out_stride;
    const float* next_w;
    void* xn_out;
    int64_t ldxn;
    int M, N, K;
    bool ordinary = false;  // never a dependent launch
};

template <bool SCALED, int EPI>
int launch(const FoldArgs& a, cudaStream_t stream) {
    const int steps = ceil_div(a.K, 32);
    const int max_kw = skinny_warps(ceil_div(a.N, 16));
    int kw = 1;
    while (kw < max_kw && steps / (kw * 2) >= MIN_STEPS) kw *= 2;
    const int k_per_warp = ceil_div(steps, kw) * 32;
    const size_t smem = (size_t)kw * 16 * 8 * sizeof(float);
    const bool dependent = skinny_dependent(ceil_div(a.N, 16)) && !a.ordinary;
    cudaError_t e = launch_maybe_pdl(dependent, gemm_skinny_fold_kernel<SCALED, EPI>, dim3(ceil_div(a.N, 16)), dim3(kw * 32), smem, stream,
                               (const __nv_bfloat16*)a.X, a.ldx, a.stats_in, a.stats_count, a.stats_in_stride, a.eps,
                               (const __nv_bfloat16*)a.W, a.Y, (int)(a.y_dtype == GB_BF16), a.ldy, a.stats_out, a.stats_out_stride,
                               a.next_w, (__nv_bfloat16*)a.xn_out, a.ldxn, a.M, a.N, a.K, k_per_warp);
    if (e != cudaSuccess) GB_REFUSE("gemm_skinny_fold: launch failed: %s", cudaGetErrorString(e));
    return 0;
}

int check_common(const char* who, const FoldArgs& a) {
    if (a.M > STAT_ROWS) GB_REFUSE("%s: %d rows; this kernel takes at most %d", who, a.M, STAT_ROWS);
    if (a.K <= 0 || (a.K & 7)) GB_REFUSE("%s: K = %d must be a positive multiple of 8", who, a.K);
    if (((uintptr_t)a.W & 15) || ((uintptr_t)a.X & 15) || (a.ldx & 7) || a.ldx < a.K)
        GB_REFUSE("%s: weights and activation rows must be 16-byte aligned, activation rows at least K long", who);
    return 0;
}

}  // namespace

// Y[M, N] (or, with swiglu, Y[M, N / 2] = silu(gate) * up) = rs[row] * (X W^T): X holds the rows of
// bf16(h * w_norm), whose factor rs = 1 / sqrt(sum(h^2) / K + eps) comes from the partial sums
// stats_in[row][0 .. stats_count) (row stride stats_in_stride floats).
GB_API int gb_gemm_skinny_scaled(const void* X, int64_t ldx, float eps, const float* stats_in, int stats_count,
                                 int64_t stats_in_stride, const void* W, void* Y, int y_dtype, int64_t ldy, int M, int N, int K,
                                 int swiglu, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    const char* who = "gemm_skinny_scaled";
    FoldArgs a = {X, ldx, stats_in, stats_count, stats_in_stride, eps, W, Y, y_dtype, ldy, nullptr, 0, nullptr, nullptr, 0, M, N, K};
    if (int rc = check_common(who, a)) return rc;
    if (stats_count <= 0 || stats_in_stride < stats_count) GB_REFUSE("%s: %d partial sums a row with a row stride of %lld", who, stats_count, (long long)stats_in_stride);
    if (y_dtype != GB_F32 && y_dtype != GB_BF16) GB_REFUSE("%s: unknown output dtype %d", who, y_dtype);
    if (swiglu) {
        if ((N & 15) || ldy < N / 2) GB_REFUSE("%s: the SwiGLU epilogue needs N = %d to be a multiple of 16 and Y rows of at least N / 2", who, N);
        return launch<true, 1>(a, stream);
    }
    if (ldy < N) GB_REFUSE("%s: row stride %lld of Y is shorter than N = %d", who, (long long)ldy, N);
    return launch<true, 0>(a, stream);
}

// Hres[M, N] += X[M, K] W^T (fp32 residual, in place); stats_out[row][c] = sum of squares of the 16
// new values of the row in columns 16 c .. 16 c + 15; and, if next_w is given, xn_out[row][n] =
// bf16(Hres[row][n] * next_w[n]), the next norm's output but for the row factor.
// `ordinary`: launch as an ordinary kernel, never as a dependent one (for a product that follows a kernel
// whose CTAs hold most of an SM's shared memory: see gb_gemm_scaled_algo).
GB_API int gb_gemm_skinny_residual(const void* X, int64_t ldx, const void* W, float* Hres, int64_t ldh, float* stats_out,
                                   int64_t stats_out_stride, const float* next_w, void* xn_out, int64_t ldxn, int M, int N, int K,
                                   int ordinary, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    const char* who = "gemm_skinny_residual";
    FoldArgs a = {X, ldx, nullptr, 0, 0, 0.f, W, Hres, GB_F32, ldh, stats_out, stats_out_stride, next_w, xn_out, ldxn, M, N, K};
    a.ordinary = ordinary != 0;
    if (int rc = check_common(who, a)) return rc;
    if (ldh < N) GB_REFUSE("%s: row stride %lld of the residual is shorter than N = %d", who, (long long)ldh, N);
    if (!stats_out || stats_out_stride < ceil_div(N, 16)) GB_REFUSE("%s: the statistics buffer needs %d floats a row", who, ceil_div(N, 16));
    if (next_w && (!xn_out || ldxn < N)) GB_REFUSE("%s: the next norm's weight is given without room for its %d-wide rows", who, N);
    return launch<false, 2>(a, stream);
}
