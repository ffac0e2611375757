// C[M, N] = A[M, K] * W[N, K]^T, bfloat16 operands, on the fifth-generation tensor cores:
// tcgen05.mma with the accumulator in tensor memory, operands brought into shared memory by TMA.
//
// Tiles are 128 x 256; one CTA per SM walks them (M tile fastest).  Tensor memory holds two
// accumulators, so the epilogue of a tile runs while the products of the next tile are issued.
// Roles, by warp:
//   warp 0   one lane issues the TMA loads (cp.async.bulk.tensor.2d) of a 128 x 64 slab of A and a
//            256 x 64 slab of W per stage into 128-byte-swizzled shared memory, four stages deep;
//   warp 1   allocates all 512 columns of tensor memory; one lane issues four tcgen05.mma
//            (M 128, N 256, K 16) per stage and commits the stage's barrier when they are done,
//            and the accumulator's barrier after a tile's last step;
//   warps 2-5  wait for an accumulator, read it with tcgen05.ld (each warp the 32 lanes of its
//            quadrant), convert and store 32 columns at a time, then hand the accumulator back.
// Tiles that run together share their W slabs, so W crosses HBM once.  Edges: TMA fills rows and columns outside the operands with zeros and
// the stores are bounded, so M, N and K need no padding (K and the row strides must be multiples
// of 8 elements, the 16-byte rule of TMA).
//
// Every wait on a barrier gives up after a bounded number of polls; the CTA then records a status
// word, lets its roles run out, frees its tensor memory and returns.  The status is read with
// gb_gemm_tc5_status().
#include "tc5.cuh"

#include <string.h>

__device__ int g_tc5_status;

namespace {

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int TMEM_COLS = 512;  // two accumulators of 256 columns
constexpr int THREADS = 192;


__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(s32(bar)) : "memory");
}

// Stores 32 accumulator columns (n0c .. n0c + 31 of the product) of row `row`: plain, or through the
// SwiGLU epilogue, where columns alternate in blocks of eight between gate and up outputs.
template <typename TC>
__device__ __forceinline__ void store_cols32(TC* __restrict__ C, int64_t ldc, int row, int M, int N, int n0c, const uint32_t (&r)[32],
                                             int epi, bool vec_ok) {
    if (epi == 1) {
        // columns alternate in blocks of eight between gate and up outputs of a SwiGLU:
        // sixteen activations per 32 columns, out[row, (n0c) / 2 + ...]
        if (row < M) {
            float act[16];
#pragma unroll
            for (int j = 0; j < 2; j++)
#pragma unroll
                for (int e = 0; e < 8; e++) {
                    float g = __uint_as_float(r[16 * j + e]), u = __uint_as_float(r[16 * j + 8 + e]);
                    // g / (1 + e^-g): for very negative g the exponential overflows to +inf and
                    // the quotient is -0, the limit of the function
                    act[8 * j + e] = __fdividef(g, 1.f + __expf(-g)) * u;
                }
            TC* dst = C + (int64_t)row * ldc + ((n0c) >> 1);
            const int left = (N - (n0c)) >> 1;  // outputs that exist from here on
            if (vec_ok && left >= 16 && sizeof(TC) == 2) {
                uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
                for (int e = 0; e < 2; e++) {
                    uint4 v;
                    __nv_bfloat162 t0 = __floats2bfloat162_rn(act[e * 8 + 0], act[e * 8 + 1]);
                    __nv_bfloat162 t1 = __floats2bfloat162_rn(act[e * 8 + 2], act[e * 8 + 3]);
                    __nv_bfloat162 t2 = __floats2bfloat162_rn(act[e * 8 + 4], act[e * 8 + 5]);
                    __nv_bfloat162 t3 = __floats2bfloat162_rn(act[e * 8 + 6], act[e * 8 + 7]);
                    v.x = *reinterpret_cast<uint32_t*>(&t0);
                    v.y = *reinterpret_cast<uint32_t*>(&t1);
                    v.z = *reinterpret_cast<uint32_t*>(&t2);
                    v.w = *reinterpret_cast<uint32_t*>(&t3);
                    d4[e] = v;
                }
            } else {
#pragma unroll
                for (int e = 0; e < 16; e++)
                    if (e < left) dst[e] = from_f32<TC>(act[e]);
            }
        }
        return;
    }
    if (epi == 2) {
        // C is the fp32 residual stream: the product is added to it in place
        if (row < M && sizeof(TC) == 4) {
            float* dst = reinterpret_cast<float*>(C) + (int64_t)row * ldc + n0c;
            if ((ldc & 3) == 0 && (((uintptr_t)C & 15) == 0) && n0c + 32 <= N) {
                float4* d4 = reinterpret_cast<float4*>(dst);
#pragma unroll
                for (int e = 0; e < 8; e++) {
                    float4 v = d4[e];
                    v.x += __uint_as_float(r[e * 4]);
                    v.y += __uint_as_float(r[e * 4 + 1]);
                    v.z += __uint_as_float(r[e * 4 + 2]);
                    v.w += __uint_as_float(r[e * 4 + 3]);
                    d4[e] = v;
                }
            } else {
#pragma unroll
                for (int e = 0; e < 32; e++)
                    if (n0c + e < N) dst[e] += __uint_as_float(r[e]);
            }
        }
        return;
    }
    if (row < M) {
        TC* dst = C + (int64_t)row * ldc + n0c;
        if (vec_ok && n0c + 32 <= N) {
            if (sizeof(TC) == 2) {
                uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    uint4 v;
                    __nv_bfloat162 t0 = __floats2bfloat162_rn(__uint_as_float(r[e * 8 + 0]), __uint_as_float(r[e * 8 + 1]));
                    __nv_bfloat162 t1 = __floats2bfloat162_rn(__uint_as_float(r[e * 8 + 2]), __uint_as_float(r[e * 8 + 3]));
                    __nv_bfloat162 t2 = __floats2bfloat162_rn(__uint_as_float(r[e * 8 + 4]), __uint_as_float(r[e * 8 + 5]));
                    __nv_bfloat162 t3 = __floats2bfloat162_rn(__uint_as_float(r[e * 8 + 6]), __uint_as_float(r[e * 8 + 7]));
                    v.x = *reinterpret_cast<uint32_t*>(&t0);
                    v.y = *reinterpret_cast<uint32_t*>(&t1);
                    v.z = *reinterpret_cast<uint32_t*>(&t2);
                    v.w = *reinterpret_cast<uint32_t*>(&t3);
                    d4[e] = v;
                }
            } else {
                uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
                for (int e = 0; e < 8; e++) d4[e] = make_uint4(r[e * 4], r[e * 4 + 1], r[e * 4 + 2], r[e * 4 + 3]);
            }
        } else {
#pragma unroll
            for (int e = 0; e < 32; e++)
                if (n0c + e < N) dst[e] = from_f32<TC>(__uint_as_float(r[e]));
        }
    }
}

template <typename TC>
__global__ void __launch_bounds__(THREADS) gemm_tc5_kernel(const __grid_constant__ CUtensorMap map_a,
                                                          const __grid_constant__ CUtensorMap map_w, TC* __restrict__ C, int M, int N,
                                                          int K, int64_t ldc, int epi) {
    extern __shared__ unsigned char smem_raw[];
    // operand stages need 1024-byte alignment for the 128-byte swizzle
    unsigned char* tiles = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    __shared__ uint64_t full_bar[STAGES], empty_bar[STAGES], acc_full[2], acc_empty[2];
    __shared__ uint32_t tmem_base_s;
    __shared__ int abort_s;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int KT = (K + BK - 1) / BK;
    const int tiles_m = (M + BM - 1) / BM, tiles_n = (N + BN - 1) / BN;
    const int total = tiles_m * tiles_n;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], 4);  // one arrival per epilogue warp
        }
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
    pdl_wait();  // barriers and tensor memory were set up while the kernel ahead was still running
    pdl_trigger();

    // A CTA walks tiles blockIdx.x, blockIdx.x + gridDim.x, ...; tiles are numbered with the M tile
    // fastest, so CTAs that run together share their W slabs.
    if (warp == 0) {
        if (lane == 0) {
            int it = 0;  // K steps issued so far, over all tiles
            bool stop = false;
            for (int tile = blockIdx.x; tile < total && !stop; tile += gridDim.x) {
                const int m0 = (tile % tiles_m) * BM, n0 = (tile / tiles_m) * BN;
                for (int kt = 0; kt < KT; kt++, it++) {
                    const int s = it % STAGES;
                    const uint32_t phase = (uint32_t)(it / STAGES) & 1u;
                    if (!mbar_wait(&empty_bar[s], phase ^ 1u)) {
                        atomicCAS(&g_tc5_status, 0, 1);
                        abort_s = 1;
                    }
                    if (*(volatile int*)&abort_s) {
                        stop = true;
                        break;
                    }
                    mbar_expect_tx(&full_bar[s], STAGE_BYTES);
                    unsigned char* st = tiles + (size_t)s * STAGE_BYTES;
                    tma_load_2d(st, &map_a, kt * BK, m0, &full_bar[s]);
                    tma_load_2d(st + A_BYTES, &map_w, kt * BK, n0, &full_bar[s]);
                }
            }
            if (stop) {
                // let the copies that are still in flight land before the CTA leaves
                for (int j = it > STAGES ? it - STAGES : 0; j < it; j++) mbar_wait(&full_bar[j % STAGES], (uint32_t)(j / STAGES) & 1u);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = instr_desc(BM, BN);
            int it = 0, i = 0;
            bool stop = false;
            for (int tile = blockIdx.x; tile < total && !stop; tile += gridDim.x, i++) {
                const int buf = i & 1;
                const uint32_t use = (uint32_t)(i >> 1) & 1u;
                // the epilogue must have drained this accumulator (passes at once on its first use)
                if (!mbar_wait(&acc_empty[buf], use ^ 1u)) {
                    atomicCAS(&g_tc5_status, 0, 4);
                    abort_s = 1;
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const uint32_t d_tmem = tmem_base + (uint32_t)(buf * BN);
                for (int kt = 0; kt < KT; kt++, it++) {
                    const int s = it % STAGES;
                    const uint32_t phase = (uint32_t)(it / STAGES) & 1u;
                    if (!mbar_wait(&full_bar[s], phase)) {
                        atomicCAS(&g_tc5_status, 0, 2);
                        abort_s = 1;
                        stop = true;
                        break;
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                    const uint32_t a_addr = s32(tiles + (size_t)s * STAGE_BYTES);
                    const uint64_t adesc = smem_desc(a_addr), bdesc = smem_desc(a_addr + A_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / 16; k++) {
                        // 16 elements of K = 32 bytes = 2 units of the descriptor's address field
                        umma(d_tmem, adesc + (uint64_t)(k * 2), bdesc + (uint64_t)(k * 2), idesc, (kt > 0 || k > 0) ? 1u : 0u);
                    }
                    umma_commit(&empty_bar[s]);  // the stage is free once these products have read it
                }
                if (!stop) umma_commit(&acc_full[buf]);
            }
        }
    } else {
        // epilogue: warp w reads the tensor-memory lanes of quadrant w % 4, while the next tile's
        // products already run into the other accumulator
        const int quad = warp & 3;
        const bool vec_ok = (ldc % 8 == 0) && (((uintptr_t)C & 15) == 0);
        int i = 0;
        for (int tile = blockIdx.x; tile < total; tile += gridDim.x, i++) {
            const int m0 = (tile % tiles_m) * BM, n0 = (tile / tiles_m) * BN;
            const int buf = i & 1;
            const uint32_t use = (uint32_t)(i >> 1) & 1u;
            const int row = m0 + quad * 32 + lane;
            if (!mbar_wait(&acc_full[buf], use)) {
                atomicCAS(&g_tc5_status, 0, 3);
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const uint32_t t_addr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(buf * BN);
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                if (n0 + c0 >= N) break;  // uniform across the warp
                uint32_t r[32];
                tmem_ld32(t_addr + (uint32_t)c0, r);
                store_cols32<TC>(C, ldc, row, M, N, n0 + c0, r, epi, vec_ok);
            }
            // this warp has read its part of the accumulator: hand the buffer back
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buf]);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// ---- the same product on pairs of SMs --------------------------------------------------------
// Two CTAs of a cluster (the two SMs of a TPC) share tiles of 256 x 256: each loads its own 128
// rows of A and its own half (128 rows) of the W slab, 32 KB a stage instead of 48, six stages
// deep, and the first CTA's issuing thread drives both tensor cores with tcgen05.mma.cta_group::2
// (M 256, N 256, K 16).  Each CTA's tensor memory receives its own 128 rows of the tile and each
// CTA's epilogue warps store them.  Barriers: the TMA loads of both CTAs count bytes on the first
// CTA's stage barrier; a commit with a cluster mask frees the stage in both CTAs and announces a
// full accumulator to both; the epilogue warps of both CTAs arrive on the first CTA's
// accumulator-free barrier.
constexpr int PAIR_STAGES = 3, PAIR_BK = 128;  // a stage holds two 64-wide panels of each operand
constexpr int PAIR_PANEL = 128 * 64 * 2;
constexpr int PAIR_A_BYTES = 2 * PAIR_PANEL, PAIR_B_BYTES = 2 * PAIR_PANEL, PAIR_STAGE_BYTES = PAIR_A_BYTES + PAIR_B_BYTES;
constexpr int PAIR_STAGING_BYTES = 4 * 2 * 4096;  // epilogue staging for TMA reductions into C
constexpr uint32_t PEER_BIT_MASK = 0xFEFFFFFFu;  // a shared-memory address of either CTA of a pair -> the first CTA's

__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, int x, int y, uint32_t leader_bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n" ::"r"(
            s32(smem_dst)),
        "l"(map), "r"(x), "r"(y), "r"(leader_bar)
        : "memory");
}
__device__ __forceinline__ void umma_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// arrives, once the products issued so far have completed, on the barrier at this offset in both CTAs
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n" ::"r"(s32(bar)),
                 "h"((uint16_t)3)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive_leader(uint64_t* bar) {
    asm volatile(
        "{\n"
        ".reg .b32 ra;\n"
        "mapa.shared::cluster.u32 ra, %0, 0;\n"
        "mbarrier.arrive.release.cluster.shared::cluster.b64 _, [ra];\n"
        "}\n" ::"r"(s32(bar))
        : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}

template <typename TC>
__global__ void __launch_bounds__(THREADS) gemm_tc5_pair_kernel(const __grid_constant__ CUtensorMap map_a,
                                                               const __grid_constant__ CUtensorMap map_w,
                                                               const __grid_constant__ CUtensorMap map_c, TC* __restrict__ C, int M, int N,
                                                               int K, int64_t ldc, int epi) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* tiles = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* staging = tiles + (size_t)PAIR_STAGES * PAIR_STAGE_BYTES;  // [4 epilogue warps][2][32 x 32 floats]
    __shared__ uint64_t full_bar[PAIR_STAGES], empty_bar[PAIR_STAGES], acc_full[2], acc_empty[2];
    __shared__ uint32_t tmem_base_s;
    __shared__ int abort_s;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint32_t rank;
    asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(rank));
    const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
    const int KT = (K + PAIR_BK - 1) / PAIR_BK;
    const int tiles_m = (M + 255) / 256, tiles_n = (N + 255) / 256;
    const int total = tiles_m * tiles_n;

    if (threadIdx.x == 0) {
        for (int s = 0; s < PAIR_STAGES; s++) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], 8);  // one arrival per epilogue warp of both CTAs (used in the first CTA)
        }
        abort_s = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(s32(&tmem_base_s)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    cluster_sync_all();  // the other CTA's barriers are initialised before anything signals them
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem_base = tmem_base_s;
    pdl_wait();  // barriers and tensor memory were set up while the kernel ahead was still running
    pdl_trigger();

    if (warp == 0) {
        if (lane == 0) {
            int it = 0;
            bool stop = false;
            for (int tile = pair; tile < total && !stop; tile += pairs) {
                const int m0 = (tile % tiles_m) * 256 + (int)rank * 128, n0 = (tile / tiles_m) * 256 + (int)rank * 128;
                for (int kt = 0; kt < KT; kt++, it++) {
                    const int s = it % PAIR_STAGES;
                    const uint32_t phase = (uint32_t)(it / PAIR_STAGES) & 1u;
                    if (!mbar_wait(&empty_bar[s], phase ^ 1u)) {
                        atomicCAS(&g_tc5_status, 0, 1);
                        abort_s = 1;
                    }
                    if (*(volatile int*)&abort_s) {
                        stop = true;
                        break;
                    }
                    if (rank == 0) mbar_expect_tx(&full_bar[s], 2 * PAIR_STAGE_BYTES);  // this CTA's bytes and the other's
                    const uint32_t leader_bar = s32(&full_bar[s]) & PEER_BIT_MASK;
                    unsigned char* st = tiles + (size_t)s * PAIR_STAGE_BYTES;
                    tma_load_2d_pair(st, &map_a, kt * PAIR_BK, m0, leader_bar);
                    tma_load_2d_pair(st + PAIR_PANEL, &map_a, kt * PAIR_BK + 64, m0, leader_bar);
                    tma_load_2d_pair(st + PAIR_A_BYTES, &map_w, kt * PAIR_BK, n0, leader_bar);
                    tma_load_2d_pair(st + PAIR_A_BYTES + PAIR_PANEL, &map_w, kt * PAIR_BK + 64, n0, leader_bar);
                }
            }
            if (stop) {
                // let the copies that are still in flight land before the CTA leaves: the first CTA
                // sees them on its stage barriers, the second can only give them time
                if (rank == 0) {
                    for (int j = it > PAIR_STAGES ? it - PAIR_STAGES : 0; j < it; j++)
                        mbar_wait(&full_bar[j % PAIR_STAGES], (uint32_t)(j / PAIR_STAGES) & 1u);
                } else {
                    for (int j = 0; j < 1000; j++) __nanosleep(1000);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            const uint32_t idesc = instr_desc(256, 256);
            int it = 0, i = 0;
            bool stop = false;
            for (int tile = pair; tile < total && !stop; tile += pairs, i++) {
                const int buf = i & 1;
                const uint32_t use = (uint32_t)(i >> 1) & 1u;
                if (!mbar_wait(&acc_empty[buf], use ^ 1u)) {
                    atomicCAS(&g_tc5_status, 0, 4);
                    abort_s = 1;
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const uint32_t d_tmem = tmem_base + (uint32_t)(buf * 256);
                for (int kt = 0; kt < KT; kt++, it++) {
                    const int s = it % PAIR_STAGES;
                    const uint32_t phase = (uint32_t)(it / PAIR_STAGES) & 1u;
                    if (!mbar_wait(&full_bar[s], phase)) {
                        atomicCAS(&g_tc5_status, 0, 2);
                        abort_s = 1;
                        stop = true;
                        break;
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                    const uint32_t a_addr = s32(tiles + (size_t)s * PAIR_STAGE_BYTES);
                    const uint64_t adesc = smem_desc(a_addr), bdesc = smem_desc(a_addr + PAIR_A_BYTES);
#pragma unroll
                    for (int k = 0; k < PAIR_BK / 16; k++) {
                        // four steps of 16 (32 bytes each) to a panel
                        const uint64_t off = (uint64_t)((k >> 2) * (PAIR_PANEL >> 4) + (k & 3) * 2);
                        umma_pair(d_tmem, adesc + off, bdesc + off, idesc, (kt > 0 || k > 0) ? 1u : 0u);
                    }
                    umma_commit_pair(&empty_bar[s]);  // frees the stage in both CTAs
                }
                if (!stop) umma_commit_pair(&acc_full[buf]);
            }
        }
    } else {
        const int quad = warp & 3;
        const bool vec_ok = (ldc % 8 == 0) && (((uintptr_t)C & 15) == 0);
        int i = 0;
        for (int tile = pair; tile < total; tile += pairs, i++) {
            const int m0 = (tile % tiles_m) * 256 + (int)rank * 128, n0 = (tile / tiles_m) * 256;
            const int buf = i & 1;
            const uint32_t use = (uint32_t)(i >> 1) & 1u;
            const int row = m0 + quad * 32 + lane;
            if (!mbar_wait(&acc_full[buf], use)) {
                atomicCAS(&g_tc5_status, 0, 3);
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const uint32_t t_addr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(buf * 256);
#pragma unroll 1
            for (int c0 = 0; c0 < 256; c0 += 32) {
                if (n0 + c0 >= N) break;  // uniform across the warp
                uint32_t r[32];
                tmem_ld32(t_addr + (uint32_t)c0, r);
                if (epi == 2) {
                    // C += tile: the warp lays its 32 x 32 floats out in shared memory (128-byte rows,
                    // 16-byte pieces swizzled as the tensor map says) and one lane hands them to a TMA
                    // reduction, which adds them to C in memory; nothing is read back here.  Two
                    // staging buffers a warp: the reduction issued two chunks ago has read its buffer.
                    const int sb = (c0 >> 5) & 1;
                    if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;\n" ::: "memory");
                    __syncwarp();
                    unsigned char* stg = staging + (size_t)((quad * 2 + sb) * 4096);
#pragma unroll
                    for (int e = 0; e < 8; e++)
                        *reinterpret_cast<uint4*>(stg + lane * 128 + ((e ^ (lane & 7)) << 4)) =
                            make_uint4(r[e * 4], r[e * 4 + 1], r[e * 4 + 2], r[e * 4 + 3]);
                    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
                    __syncwarp();
                    if (lane == 0) {
                        asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.bulk_group [%0, {%2, %3}], [%1];\n" ::"l"(&map_c),
                                     "r"(s32(stg)), "r"(n0 + c0), "r"(m0 + quad * 32)
                                     : "memory");
                        asm volatile("cp.async.bulk.commit_group;\n" ::: "memory");
                    }
                    continue;
                }
                store_cols32<TC>(C, ldc, row, M, N, n0 + c0, r, epi, vec_ok);
            }
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive_leader(&acc_empty[buf]);
        }
    }
    if (epi == 2 && warp >= 2 && lane == 0) asm volatile("cp.async.bulk.wait_group 0;\n" ::: "memory");  // this warp's reductions are done
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    cluster_sync_all();  // neither CTA leaves while the other may still read its memory or signal its barriers
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

template <typename TC>
int launch_pair(const void* A, const void* W, void* C, int M, int N, int K, int64_t lda, int64_t ldc, int epi, cudaStream_t stream) {
    const int smem = PAIR_STAGES * PAIR_STAGE_BYTES + PAIR_STAGING_BYTES + 1024;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc5_pair_kernel<TC>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) GB_REFUSE("gemm_tc5_pair: cannot reserve %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
        configured = true;
    }
    CUtensorMap map_a, map_w, map_c;
    if (int rc = tc5_make_map(&map_a, A, M, K, lda, 128)) return rc;
    if (int rc = tc5_make_map(&map_w, W, N, K, K, 128)) return rc;
    memset(&map_c, 0, sizeof(map_c));
    if (epi == 2) {
        // float32 C in boxes of 32 x 32, 128-byte swizzle, for the epilogue's TMA reductions
        Tc5EncodeTiledFn fn = tc5_encode_fn();
        if (!fn) GB_REFUSE("tcgen05 kernels: the driver offers no cuTensorMapEncodeTiled");
        if ((ldc & 3) || ((uintptr_t)C & 15)) GB_REFUSE("gemm_tc5: adding into C needs 16-byte aligned rows (stride %lld)", (long long)ldc);
        cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)M};
        cuuint64_t strides[1] = {(cuuint64_t)ldc * 4};
        cuuint32_t box[2] = {32u, 32u};
        cuuint32_t estr[2] = {1, 1};
        CUresult r = fn(&map_c, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, C, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) GB_REFUSE("gemm_tc5: cuTensorMapEncodeTiled for C failed with code %d", (int)r);
    }
    static int sms = 0;
    if (sms == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
    }
    const int64_t total = (int64_t)ceil_div(M, 256) * ceil_div(N, 256);
    if (total > 0x7fffffff) GB_REFUSE("gemm_tc5_pair: %lld tiles are too many", (long long)total);
    const int pairs = total < sms / 2 ? (int)total : sms / 2;  // one pair of CTAs per pair of SMs walks the tiles
    cudaError_t e = launch_pdl_cluster(gemm_tc5_pair_kernel<TC>, dim3(2 * pairs), dim3(THREADS), (size_t)smem, stream, 2, 1, map_a, map_w,
                                       map_c, (TC*)C, M, N, K, ldc, epi);
    if (e != cudaSuccess) GB_REFUSE("gemm_tc5_pair: launch failed: %s", cudaGetErrorString(e));
    return 0;
}

template <typename TC>
int launch(const void* A, const void* W, void* C, int M, int N, int K, int64_t lda, int64_t ldc, int epi, cudaStream_t stream) {
    const int smem = STAGES * STAGE_BYTES + 1024;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc5_kernel<TC>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) GB_REFUSE("gemm_tc5: cannot reserve %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
        configured = true;
    }
    CUtensorMap map_a, map_w;
    if (int rc = tc5_make_map(&map_a, A, M, K, lda, BM)) return rc;
    if (int rc = tc5_make_map(&map_w, W, N, K, K, BN)) return rc;
    static int sms = 0;
    if (sms == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
    }
    const int64_t total = (int64_t)ceil_div(M, BM) * ceil_div(N, BN);
    if (total > 0x7fffffff) GB_REFUSE("gemm_tc5: %lld tiles are too many", (long long)total);
    const int grid = total < sms ? (int)total : sms;  // one CTA per SM walks the tiles
    cudaError_t e = launch_pdl(gemm_tc5_kernel<TC>, dim3(grid), dim3(THREADS), (size_t)smem, stream, map_a, map_w, (TC*)C, M, N, K, ldc, epi);
    if (e != cudaSuccess) GB_REFUSE("gemm_tc5: launch failed: %s", cudaGetErrorString(e));
    return 0;
}

}  // namespace

static int tc5(const void* A, const void* W, void* C, int c_dtype, int M, int N, int K, int64_t lda, int64_t ldc, int epi, int pair,
               cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || (K & 7)) GB_REFUSE("gemm_tc5: K = %d must be a positive multiple of 8", K);
    if ((lda & 7) || lda < K) GB_REFUSE("gemm_tc5: row stride %lld of A must be a multiple of 8 and at least K", (long long)lda);
    if ((epi == 0 || epi == 2) && ldc < N) GB_REFUSE("gemm_tc5: row stride %lld of C is shorter than N = %d", (long long)ldc, N);
    if (epi == 2 && c_dtype != GB_F32) GB_REFUSE("gemm_tc5: adding into C needs a float32 C");
    if (epi == 1 && ((N & 15) || ldc < N / 2)) GB_REFUSE("gemm_tc5: the SwiGLU epilogue needs N = %d to be a multiple of 16", N);
    if (((uintptr_t)A & 15) || ((uintptr_t)W & 15)) GB_REFUSE("gemm_tc5: operands must be 16-byte aligned");
    if (pair) {
        if (c_dtype == GB_F32) return launch_pair<float>(A, W, C, M, N, K, lda, ldc, epi, stream);
        if (c_dtype == GB_BF16) return launch_pair<__nv_bfloat16>(A, W, C, M, N, K, lda, ldc, epi, stream);
    } else {
        if (c_dtype == GB_F32) return launch<float>(A, W, C, M, N, K, lda, ldc, epi, stream);
        if (c_dtype == GB_BF16) return launch<__nv_bfloat16>(A, W, C, M, N, K, lda, ldc, epi, stream);
    }
    GB_REFUSE("gemm_tc5: unknown output dtype %d", c_dtype);
}

GB_API int gb_gemm_tc5(const void* A, const void* W, void* C, int c_dtype, int M, int N, int K, int64_t lda, int64_t ldc,
                       cudaStream_t stream) {
    return tc5(A, W, C, c_dtype, M, N, K, lda, ldc, 0, 0, stream);
}

// The same product with tiles of 256 x 256 on pairs of SMs (tcgen05.mma.cta_group::2).
GB_API int gb_gemm_tc5_pair(const void* A, const void* W, void* C, int c_dtype, int M, int N, int K, int64_t lda, int64_t ldc,
                            cudaStream_t stream) {
    return tc5(A, W, C, c_dtype, M, N, K, lda, ldc, 0, 1, stream);
}
GB_API int gb_gemm_tc5_pair_swiglu(const void* A, const void* W, void* C, int c_dtype, int M, int N, int K, int64_t lda, int64_t ldc,
                                   cudaStream_t stream) {
    return tc5(A, W, C, c_dtype, M, N, K, lda, ldc, 1, 1, stream);
}

// C[M, N] += A W^T for a float32 C (the residual stream), on the paired-SM kernel.
GB_API int gb_gemm_tc5_pair_add(const void* A, const void* W, void* C, int M, int N, int K, int64_t lda, int64_t ldc, cudaStream_t stream) {
    return tc5(A, W, C, GB_F32, M, N, K, lda, ldc, 2, 1, stream);
}

// C[M, N / 2] = silu(A Wg^T) * (A Wu^T); W holds gate and up rows interleaved in blocks of eight.
GB_API int gb_gemm_tc5_swiglu(const void* A, const void* W, void* C, int c_dtype, int M, int N, int K, int64_t lda, int64_t ldc,
                              cudaStream_t stream) {
    return tc5(A, W, C, c_dtype, M, N, K, lda, ldc, 1, 0, stream);
}

// 0 if no tcgen05 kernel has given up on a barrier since the last call; else the role that did
// (1 loader, 2 multiplier, 3 epilogue).  Synchronises the device.
GB_API int gb_gemm_tc5_status() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_tc5_status, sizeof(int)) != cudaSuccess) return -1;
    if (v != 0) cudaMemcpyToSymbol(g_tc5_status, &zero, sizeof(int));
    return v;
}
