// Y[M, N] = X[M, K] * W[N, K]^T for 9 to 256 rows on tcgen05: the product of a decode step, or of
// a short prompt, when there are too many rows for the fragment-streaming kernel and too few for
// the tiled kernels to give every SM a share of the weights.  (Also for fewer rows where the
// dispatch rule finds it the faster stream: head-sized outputs, and products long on both sides.)
//
// The weights take the M side of the instruction: a CTA owns 128 rows of W and a slice of K, and
// computes Y^T[128, batch] with UMMA M = 128, N = 16 / 32 / 64 / 128 / 256 (the batch rounded up;
// TMA fills the missing rows of X with zeros).  Per K step of 64 a stage holds 16 KB of W from HBM
// and 2 to 32 KB of X from L2; up to 64 rows four stages deep, above that three; two CTAs to an SM
// (one at 256 columns), so every SM keeps tens of KB of weights in flight.  K is cut into slices so
// that about that many CTAs exist even for narrow outputs.  The CTAs that share a tile (1, 2, 4 or 8
// slices of K) form a thread-block cluster:
// each leaves its partial tile in its own shared memory, and after a cluster barrier each CTA adds
// the slices, in slice order, for its share of the batch rows (a warp a row), reading the other CTAs'
// shared memory directly (distributed shared memory).  No scratch in global memory, and the sum does not
// depend on timing.  With the gate/up rows of a SwiGLU interleaved in blocks of eight the
// activation is applied in the same epilogue.
//
// Up to 64 rows the residual's row-wise work can be folded into the product as in the few-row
// kernel (gemm_skinny_fold.cu).  As producer (epi 2) Y is the fp32 residual: Y += product, one
// thread and one fp32 addition per element; one partial sum of squares per row and tile of 128
// columns goes to stats_out[row][tile]; and the new rows times the next norm's weight go out as
// bfloat16.  As consumer (stats_in given) the activations are such rows and the finished sums are
// multiplied by the rows' norm factors, the partial sums added up in index order.
//
// Roles by warp as in the tiled kernel: warp 0 loads by TMA, warp 1 issues tcgen05.mma, warps
// 2-5 read tensor memory (lane = weight row, column = batch row) and store.  Barrier waits are
// bounded; a wait that gives up is recorded and read with gb_gemm_tc5_decode_status().
#include "api.h"
#include "tc5.cuh"

namespace {

__device__ int g_status;

constexpr int BMW = 128, BK = 64, THREADS = 192;
constexpr int W_BYTES = BMW * BK * 2;

// the folded variants' extra operands (all null / 0 for the plain product)
struct DecodeFold {
    const float* stats_in;   // [rows][stats_count] partial sums of squares of the rows X was made from
    int stats_count;
    int64_t stats_in_stride;
    float eps;
    int norm_n;              // width of the normed rows
    float* stats_out;        // epi 2: [rows][tiles]
    int64_t stats_out_stride;
    const float* next_w;     // epi 2, optional: weight of the norm that reads the residual next
    __nv_bfloat16* xn_out;   // [rows][N] = bf16(Y * next_w)
    int64_t ldxn;
};
constexpr int FOLD_ROWS = GB_FOLD_MAX_ROWS;

__device__ __forceinline__ float silu_f(float x) {
    if (x >= 0.f) return x / (1.f + expf(-x));
    float e = expf(x);
    return x * e / (1.f + e);
}

// value v of (weight row n, batch row b) -> Y, plain or through the SwiGLU epilogue; `other` is the
// value of weight row n + 8 (the up row of a gate row), fetched by the caller with a shuffle
template <typename TC>
__device__ __forceinline__ void store_out(TC* __restrict__ Y, int64_t ldy, int b, int n, int N, float v, float other, int epi) {
    if (epi == 0) {
        if (n < N) Y[(int64_t)b * ldy + n] = from_f32<TC>(v);
    } else {
        if ((n & 15) < 8 && n + 8 < N) Y[(int64_t)b * ldy + ((n >> 4) << 3) + (n & 7)] = from_f32<TC>(silu_f(v) * other);
    }
}

template <typename TC, int NB, int STAGES>  // NB = batch columns of the instruction: 16 to 256; STAGES deep
__global__ void __launch_bounds__(THREADS) gemm_tc5_decode_kernel(const __grid_constant__ CUtensorMap map_w,
                                                                 const __grid_constant__ CUtensorMap map_x, TC* __restrict__ Y,
                                                                 int M, int N, int K, int64_t ldy, int splits, int kb_per_split,
                                                                 int epi, DecodeFold fold) {
    constexpr int X_BYTES = NB * BK * 2, STAGE_BYTES = W_BYTES + X_BYTES;
    constexpr int TMEM_COLS = NB < 32 ? 32 : NB;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* tiles = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    __shared__ uint64_t full_bar[STAGES], empty_bar[STAGES], accum_bar;
    __shared__ uint32_t tmem_base_s;
    __shared__ int abort_s;
    __shared__ float rs_s[FOLD_ROWS];          // the rows' norm factors (consumer)
    __shared__ float sq_part[4][FOLD_ROWS];    // sums of squares of the four epilogue warps' rows (producer)

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * BMW, split = blockIdx.y;
    const int KB = (K + BK - 1) / BK;
    const int kb0 = split * kb_per_split;
    const int kb1 = kb0 + kb_per_split < KB ? kb0 + kb_per_split : KB;
    const int KT = kb1 > kb0 ? kb1 - kb0 : 0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        mbar_init(&accum_bar, 1);
        abort_s = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(s32(&tmem_base_s)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem_base = tmem_base_s;
    // Barriers and tensor memory were set up while the kernel ahead was still running.  The weights
    // do not depend on that kernel either: the loading thread requests the first stages' weights
    // before it waits, and only their activations after.
    const int early = KT < STAGES ? KT : STAGES;
    if (warp == 0 && lane == 0) {
        for (int kt = 0; kt < early; kt++) {
            mbar_expect_tx(&full_bar[kt], STAGE_BYTES);
            tma_load_2d(tiles + (size_t)kt * STAGE_BYTES, &map_w, (kb0 + kt) * BK, n0, &full_bar[kt]);
        }
    }
    pdl_wait();
    pdl_trigger();

    if (warp == 0) {
        if (lane == 0) {
            int issued = early;
            for (int kt = 0; kt < early; kt++)
                tma_load_2d(tiles + (size_t)kt * STAGE_BYTES + W_BYTES, &map_x, (kb0 + kt) * BK, 0, &full_bar[kt]);
            for (int kt = early; kt < KT; kt++) {
                const int s = kt % STAGES;
                const uint32_t phase = (uint32_t)(kt / STAGES) & 1u;
                if (!mbar_wait(&empty_bar[s], phase ^ 1u)) {
                    atomicCAS(&g_status, 0, 1);
                    abort_s = 1;
                    break;
                }
                if (*(volatile int*)&abort_s) break;
                mbar_expect_tx(&full_bar[s], STAGE_BYTES);
                unsigned char* st = tiles + (size_t)s * STAGE_BYTES;
                tma_load_2d(st, &map_w, (kb0 + kt) * BK, n0, &full_bar[s]);
                tma_load_2d(st + W_BYTES, &map_x, (kb0 + kt) * BK, 0, &full_bar[s]);
                issued = kt + 1;
            }
            if (*(volatile int*)&abort_s) {
                for (int kt = issued > STAGES ? issued - STAGES : 0; kt < issued; kt++)
                    mbar_wait(&full_bar[kt % STAGES], (uint32_t)(kt / STAGES) & 1u);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = instr_desc(BMW, NB);
            bool ok = true;
            for (int kt = 0; kt < KT; kt++) {
                const int s = kt % STAGES;
                const uint32_t phase = (uint32_t)(kt / STAGES) & 1u;
                if (!mbar_wait(&full_bar[s], phase)) {
                    atomicCAS(&g_status, 0, 2);
                    abort_s = 1;
                    ok = false;
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const uint32_t w_addr = s32(tiles + (size_t)s * STAGE_BYTES);
                const uint64_t adesc = smem_desc(w_addr), bdesc = smem_desc(w_addr + W_BYTES);
#pragma unroll
                for (int k = 0; k < BK / 16; k++)
                    umma(tmem_base, adesc + (uint64_t)(k * 2), bdesc + (uint64_t)(k * 2), idesc, (kt > 0 || k > 0) ? 1u : 0u);
                umma_commit(&empty_bar[s]);
            }
            if (ok) umma_commit(&accum_bar);
        }
    } else {
        const int quad = warp & 3;
        const int n = n0 + quad * 32 + lane;  // this thread's weight row
        if (fold.stats_in != nullptr) {
            // The norm factors.  Warp q of the four takes batch rows q, q + 4, ..., eight at a time
            // so that their loads are in flight together; its lanes add every 32nd partial sum of a
            // row and a tree adds the lanes: an order that does not depend on the other rows.
            for (int b0 = quad; b0 < M; b0 += 32) {
                float t[8];
#pragma unroll
                for (int u = 0; u < 8; u++) t[u] = 0.f;
#pragma unroll 2
                for (int c = lane; c < fold.stats_count; c += 32) {
#pragma unroll
                    for (int u = 0; u < 8; u++) {
                        const int b = b0 + 4 * u;
                        if (b < M) t[u] += fold.stats_in[(int64_t)b * fold.stats_in_stride + c];
                    }
                }
#pragma unroll
                for (int u = 0; u < 8; u++) {
                    const int b = b0 + 4 * u;
                    const float total = warp_sum(t[u]);
                    if (lane == 0 && b < M) rs_s[b] = 1.0f / sqrtf(total / (float)fold.norm_n + fold.eps);
                }
            }
            asm volatile("bar.sync 1, 128;\n" ::: "memory");  // the four epilogue warps
        }
        bool have = KT > 0;
        if (have && !mbar_wait(&accum_bar, 0)) {
            atomicCAS(&g_status, 0, 3);
            have = false;
        }
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
#pragma unroll 1
        for (int c0 = 0; c0 < NB; c0 += 16) {
            if (c0 >= M) break;
            uint32_t r[16];
            if (have) {
                tmem_ld16(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)c0, r);
            } else {
#pragma unroll
                for (int i = 0; i < 16; i++) r[i] = 0u;
            }
            if (splits == 1 && epi == 2) {
#pragma unroll
                for (int i = 0; i < 16; i++) {
                    const int b = c0 + i;
                    float sq = 0.f;
                    if (b < M && n < N) {
                        float* hq = reinterpret_cast<float*>(Y) + (int64_t)b * ldy + n;
                        const float hn = *hq + __uint_as_float(r[i]);
                        *hq = hn;
                        sq = hn * hn;
                        if (fold.next_w != nullptr) fold.xn_out[(int64_t)b * fold.ldxn + n] = __float2bfloat16_rn(hn * fold.next_w[n]);
                    }
                    sq = warp_sum(sq);
                    if (lane == 0 && b < M) sq_part[quad][b] = sq;
                }
            } else if (splits == 1) {
#pragma unroll
                for (int i = 0; i < 16; i++) {
                    float v = __uint_as_float(r[i]);
                    if (fold.stats_in != nullptr && c0 + i < M) v *= rs_s[c0 + i];
                    float other = __shfl_down_sync(0xffffffffu, v, 8);
                    if (c0 + i < M) store_out<TC>(Y, ldy, c0 + i, n, N, v, other, epi);
                }
            } else {
                // partial tile in this CTA's shared memory: part[b][row of the tile]; the operand
                // stages are free, every product that read them has completed
                float* part = reinterpret_cast<float*>(tiles);
#pragma unroll
                for (int i = 0; i < 16; i++) part[(c0 + i) * BMW + quad * 32 + lane] = __uint_as_float(r[i]);
            }
        }
        if (splits == 1 && epi == 2) {
            // the four warps' sums of each batch row, added in warp order
            asm volatile("bar.sync 1, 128;\n" ::: "memory");
            const int b = (int)threadIdx.x - 64;
            if (b < M) fold.stats_out[(int64_t)b * fold.stats_out_stride + blockIdx.x] = (sq_part[0][b] + sq_part[1][b]) + (sq_part[2][b] + sq_part[3][b]);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
    if (splits == 1) return;

    // All slices of the tile have left their partial tiles: add them.  CTA r of the cluster takes
    // batch rows r, r + slices, ...: a warp a row, a lane four neighbouring rows of the tile.  What the
    // residual variant reads from global memory is requested while the cluster gathers.
    uint32_t rank;
    asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(rank));
    const int nl = lane * 4;
    const int row_step = splits * (THREADS / 32);
    const int row0 = (int)rank + splits * warp;
    float pre_h[2][4], next_w[4];
    asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
    if (epi == 2) {
#pragma unroll
        for (int e = 0; e < 4; e++) next_w[e] = (fold.next_w != nullptr && n0 + nl + e < N) ? fold.next_w[n0 + nl + e] : 0.f;
#pragma unroll
        for (int j = 0; j < 2; j++) {
            const int bj = row0 + j * row_step;
#pragma unroll
            for (int e = 0; e < 4; e++)
                pre_h[j][e] = (bj < M && n0 + nl + e < N) ? reinterpret_cast<const float*>(Y)[(int64_t)bj * ldy + n0 + nl + e] : 0.f;
        }
    }
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
    const uint32_t part_addr = s32(tiles);
    int j = 0;
    for (int bb = row0; bb < M; bb += row_step, j++) {
        float v[4] = {0.f, 0.f, 0.f, 0.f};
        for (int sl = 0; sl < splits; sl++) {
            uint32_t remote;
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(remote) : "r"(part_addr + (uint32_t)((bb * BMW + nl) * 4)), "r"(sl));
            float x0, x1, x2, x3;
            asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];\n" : "=f"(x0), "=f"(x1), "=f"(x2), "=f"(x3) : "r"(remote) : "memory");
            v[0] += x0;
            v[1] += x1;
            v[2] += x2;
            v[3] += x3;
        }
        if (epi == 2) {
            float* hq = reinterpret_cast<float*>(Y) + (int64_t)bb * ldy + n0 + nl;
            float sq = 0.f;
#pragma unroll
            for (int e = 0; e < 4; e++) {
                if (n0 + nl + e < N) {
                    const float before = j == 0 ? pre_h[0][e] : (j == 1 ? pre_h[1][e] : hq[e]);
                    const float hn = before + v[e];
                    hq[e] = hn;
                    sq += hn * hn;
                    if (fold.next_w != nullptr) fold.xn_out[(int64_t)bb * fold.ldxn + n0 + nl + e] = __float2bfloat16_rn(hn * next_w[e]);
                }
            }
            // the lanes of the warp hold the whole tile's share of this batch row
            sq = warp_sum(sq);
            if (lane == 0) fold.stats_out[(int64_t)bb * fold.stats_out_stride + blockIdx.x] = sq;
            continue;
        }
        if (fold.stats_in != nullptr) {
            const float rs = rs_s[bb];
#pragma unroll
            for (int e = 0; e < 4; e++) v[e] *= rs;
        }
        // the up rows of these four gate rows are eight rows on: two lanes on
#pragma unroll
        for (int e = 0; e < 4; e++) {
            float other = __shfl_down_sync(0xffffffffu, v[e], 2);
            store_out<TC>(Y, ldy, bb, n0 + nl + e, N, v[e], other, epi);
        }
    }
    // no CTA may leave while another still reads its shared memory
    asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}

constexpr int MAX_TILES = 8192;
constexpr int UNEVEN_TILES = 148;  // more tiles than this many SMs: see dispatch()

template <typename TC, int NB, int STAGES>
int launch(const void* X, const void* W, void* Y, int M, int N, int K, int64_t ldx, int64_t ldy, int epi, int splits,
           const DecodeFold& fold, cudaStream_t stream) {
    constexpr int X_BYTES = NB * BK * 2;
    int smem = STAGES * (W_BYTES + X_BYTES) + 1024;
    const int part = NB * BMW * 4 + 1024;
    if (part > smem) smem = part;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc5_decode_kernel<TC, NB, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) GB_REFUSE("gemm_tc5_decode: cannot reserve %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
        configured = true;
    }
    CUtensorMap map_w, map_x;
    if (int rc = tc5_make_map(&map_w, W, N, K, K, BMW)) return rc;
    if (int rc = tc5_make_map(&map_x, X, M, K, ldx, NB)) return rc;
    const int tiles = ceil_div(N, BMW);
    const int KB = ceil_div(K, BK);
    while (splits > 1 && KB < splits) splits >>= 1;
    const int kb_per_split = ceil_div(KB, splits);
    if (tiles > MAX_TILES) GB_REFUSE("gemm_tc5_decode: N = %d exceeds %d tiles", N, MAX_TILES);
    cudaError_t e = launch_pdl_cluster(gemm_tc5_decode_kernel<TC, NB, STAGES>, dim3(tiles, splits), dim3(THREADS), (size_t)smem, stream, 1,
                                       (unsigned)splits, map_w, map_x, (TC*)Y, M, N, K, ldy, splits, kb_per_split, epi, fold);
    if (e != cudaSuccess) GB_REFUSE("gemm_tc5_decode: launch failed: %s", cudaGetErrorString(e));
    return 0;
}

template <typename TC>
int dispatch(const void* X, const void* W, void* Y, int M, int N, int K, int64_t ldx, int64_t ldy, int epi, int splits,
             const DecodeFold& fold, cudaStream_t stream) {
    if (M <= 16) return launch<TC, 16, 4>(X, W, Y, M, N, K, ldx, ldy, epi, splits, fold, stream);
    // More tiles than SMs but fewer than two to an SM (the gate/up product of an 8B layer: 192 tiles on
    // 148 SMs): some SMs would stream two tiles while most stream one.  Such a product runs in two K
    // slices with three stages, so that three CTAs fit an SM and every SM gets two or three of the
    // smaller pieces (64 rows: 50.7 -> 43.3 us; 33 rows: 43.5 -> 38.4 us).
    const bool uneven = splits == 2 && ceil_div(N, BMW) > UNEVEN_TILES;
    if (M <= 32) {
        if (uneven) return launch<TC, 32, 3>(X, W, Y, M, N, K, ldx, ldy, epi, splits, fold, stream);
        return launch<TC, 32, 4>(X, W, Y, M, N, K, ldx, ldy, epi, splits, fold, stream);
    }
    if (M <= 64) {
        if (uneven) return launch<TC, 64, 3>(X, W, Y, M, N, K, ldx, ldy, epi, splits, fold, stream);
        return launch<TC, 64, 4>(X, W, Y, M, N, K, ldx, ldy, epi, splits, fold, stream);
    }
    if (M <= 128) return launch<TC, 128, 3>(X, W, Y, M, N, K, ldx, ldy, epi, splits, fold, stream);
    return launch<TC, 256, 3>(X, W, Y, M, N, K, ldx, ldy, epi, splits, fold, stream);
}

}  // namespace

// How many slices of K (1, 2, 4 or 8, the size of the cluster) the kernel would like for M rows of
// this shape on a device with `sms` SMs, two CTAs to an SM.
//   More than 16 rows: the most slices that keep at most about 2 * sms CTAs and at least eight K
//   steps of 64 a slice; CTAs that queue behind a full machine cost more than they gain (24576 x 4096
//   at 64 rows: 40.8 us whole, 57.6 us in two slices).
//   Up to 16 rows a CTA is lighter and a short queue pays: a CTA's time is its K steps plus about
//   eight steps of fixed cost, and the choice minimises queue depth x CTA time (24576 x 4096 at 16
//   rows: 36.5 us in two slices, 38.0 whole, 39.3 in four).
GB_API int gb_gemm_tc5_decode_splits(int M, int N, int K, int sms) {
    const int tiles = ceil_div(N, BMW), KB = ceil_div(K, BK);
    if (sms <= 0) sms = 1;
    if (M > 16) {
        int per_sm = M > 128 ? 1 : 2;  // CTAs that fit on an SM with the operand stages of this many rows
        if (M <= 64 && tiles > UNEVEN_TILES && tiles > sms && tiles < 2 * sms) per_sm = 3;  // see dispatch(): three stages
        int want = (per_sm * sms) / (tiles > 0 ? tiles : 1);
        if (want > KB / 8) want = KB / 8;
        int s = 1;
        while (s * 2 <= want && s < 8) s *= 2;
        return s;
    }
    int best = 1;
    double best_cost = 0.0;
    for (int s = 1; s <= 8; s *= 2) {
        if (s > 1 && KB / s < 1) break;
        const double queue = tiles * (double)s / (2.0 * sms);
        const double cost = (queue > 1.0 ? queue : 1.0) * ((double)ceil_div(KB, s) + 8.0);
        if (s == 1 || cost < best_cost) {
            best = s;
            best_cost = cost;
        }
    }
    return best;
}

static int decode_checks(const char* who, const void* X, const void* W, int M, int N, int K, int64_t ldx, int splits) {
    if (M > 256) GB_REFUSE("%s: %d rows; this kernel takes at most 256", who, M);
    if (K <= 0 || (K & 7)) GB_REFUSE("%s: K = %d must be a positive multiple of 8", who, K);
    if ((ldx & 7) || ldx < K) GB_REFUSE("%s: row stride %lld of X must be a multiple of 8 and at least K", who, (long long)ldx);
    if (((uintptr_t)X & 15) || ((uintptr_t)W & 15)) GB_REFUSE("%s: operands must be 16-byte aligned", who);
    if (splits != 1 && splits != 2 && splits != 4 && splits != 8) GB_REFUSE("%s: %d slices; 1, 2, 4 or 8", who, splits);
    return 0;
}

// epi = 0: Y[M, N].  epi = 1: Y[M, N / 2] = silu(gate) * up with gate/up rows of W interleaved in
// blocks of eight.  splits: 1, 2, 4 or 8 slices of K (the size of the cluster).
GB_API int gb_gemm_tc5_decode(const void* X, const void* W, void* Y, int c_dtype, int M, int N, int K, int64_t ldx, int64_t ldy,
                              int epi, int splits, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    const char* who = "gemm_tc5_decode";
    if (int rc = decode_checks(who, X, W, M, N, K, ldx, splits)) return rc;
    if (epi == 0 && ldy < N) GB_REFUSE("%s: row stride %lld of Y is shorter than N = %d", who, (long long)ldy, N);
    if (epi == 1 && ((N & 15) || ldy < N / 2)) GB_REFUSE("%s: the SwiGLU epilogue needs N = %d to be a multiple of 16", who, N);
    if (epi != 0 && epi != 1) GB_REFUSE("%s: unknown epilogue %d", who, epi);
    const DecodeFold none = {};
    if (c_dtype == GB_F32) return dispatch<float>(X, W, Y, M, N, K, ldx, ldy, epi, splits, none, stream);
    if (c_dtype == GB_BF16) return dispatch<__nv_bfloat16>(X, W, Y, M, N, K, ldx, ldy, epi, splits, none, stream);
    GB_REFUSE("%s: unknown output dtype %d", who, c_dtype);
}

// The consumer of prescaled rows (see gemm_skinny_fold.cu) for 9 to 64 rows: Y = rs[row] * (X W^T),
// plain (swiglu 0) or through the SwiGLU epilogue, rs from stats_in[row][0 .. stats_count).
GB_API int gb_gemm_tc5_decode_scaled(const void* X, int64_t ldx, float eps, const float* stats_in, int stats_count,
                                     int64_t stats_in_stride, const void* W, void* Y, int c_dtype, int64_t ldy, int M, int N, int K,
                                     int swiglu, int splits, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    const char* who = "gemm_tc5_decode_scaled";
    if (int rc = decode_checks(who, X, W, M, N, K, ldx, splits)) return rc;
    if (M > FOLD_ROWS) GB_REFUSE("%s: %d rows; the folded variants take at most %d", who, M, FOLD_ROWS);
    if (!stats_in || stats_count <= 0 || stats_in_stride < stats_count) GB_REFUSE("%s: %d partial sums a row with a row stride of %lld", who, stats_count, (long long)stats_in_stride);
    if (!swiglu && ldy < N) GB_REFUSE("%s: row stride %lld of Y is shorter than N = %d", who, (long long)ldy, N);
    if (swiglu && ((N & 15) || ldy < N / 2)) GB_REFUSE("%s: the SwiGLU epilogue needs N = %d to be a multiple of 16", who, N);
    DecodeFold fold = {};
    fold.stats_in = stats_in;
    fold.stats_count = stats_count;
    fold.stats_in_stride = stats_in_stride;
    fold.eps = eps;
    fold.norm_n = K;
    if (c_dtype == GB_F32) return dispatch<float>(X, W, Y, M, N, K, ldx, ldy, swiglu ? 1 : 0, splits, fold, stream);
    if (c_dtype == GB_BF16) return dispatch<__nv_bfloat16>(X, W, Y, M, N, K, ldx, ldy, swiglu ? 1 : 0, splits, fold, stream);
    GB_REFUSE("%s: unknown output dtype %d", who, c_dtype);
}

// The producer for 9 to 64 rows: Hres[M, N] += X W^T (fp32 residual, in place); stats_out[row][c] =
// the sum of squares of the new values of the row in columns 128 c .. 128 c + 127; and, if next_w is
// given, xn_out = bf16(Hres * next_w).  *stats_count receives the number of such tiles.
GB_API int gb_gemm_tc5_decode_residual(const void* X, int64_t ldx, const void* W, float* Hres, int64_t ldh, float* stats_out,
                                       int64_t stats_out_stride, int* stats_count, const float* next_w, void* xn_out, int64_t ldxn,
                                       int M, int N, int K, int splits, cudaStream_t stream) {
    const int count = ceil_div(N, BMW);
    if (stats_count) *stats_count = count;
    if (M <= 0 || N <= 0) return 0;
    const char* who = "gemm_tc5_decode_residual";
    if (int rc = decode_checks(who, X, W, M, N, K, ldx, splits)) return rc;
    if (M > FOLD_ROWS) GB_REFUSE("%s: %d rows; the folded variants take at most %d", who, M, FOLD_ROWS);
    if (ldh < N) GB_REFUSE("%s: row stride %lld of the residual is shorter than N = %d", who, (long long)ldh, N);
    if (!stats_out || stats_out_stride < count) GB_REFUSE("%s: the statistics buffer needs %d floats a row", who, count);
    if (next_w && (!xn_out || ldxn < N)) GB_REFUSE("%s: the next norm's weight is given without room for its %d-wide rows", who, N);
    DecodeFold fold = {};
    fold.stats_out = stats_out;
    fold.stats_out_stride = stats_out_stride;
    fold.next_w = next_w;
    fold.xn_out = (__nv_bfloat16*)xn_out;
    fold.ldxn = ldxn;
    return dispatch<float>(X, W, Hres, M, N, K, ldx, ldh, 2, splits, fold, stream);
}

GB_API int gb_gemm_tc5_decode_status() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_status, sizeof(int)) != cudaSuccess) return -1;
    if (v != 0) cudaMemcpyToSymbol(g_status, &zero, sizeof(int));
    return v;
}
