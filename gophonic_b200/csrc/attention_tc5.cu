// Flash attention for prompts on the fifth-generation tensor cores (bfloat16, head_dim 128).
//
// A CTA owns 256 query rows of one head of one sequence, as two groups of 128, and walks the
// sequence's keys one cache page (64 keys) at a time.  Both products of a step run as tcgen05.mma
// with the accumulators in tensor memory:
//     S_g = Q_g K^T   (M 128, N 64 keys, K 128)   -> two S buffers of 64 columns per group
//     O_g += P_g V    (M 128, N 128, K 64 keys)    -> one O buffer of 128 columns per group
// Roles by warp: warp 0 loads the query tiles once and per page two boxes of keys, the last warp per
// page two boxes of values, by TMA straight from the paged cache, five pages deep each; one thread each of warps 1-2 issues the
// scores products of group A and B and one each of warps 3-4 their values products; warps 5-8 and
// 9-12 are the softmax of group A and B: each thread owns one query row, reads its row of S
// from tensor memory, keeps the running maximum and sum, and writes the probabilities as bfloat16
// back into tensor memory, over the scores it has read, where the second product takes them as its
// A operand (no shared memory, no proxy fence on the way).  O stays in tensor memory and is
// rescaled only when a row's maximum has grown by more than 2^8 since the scale in use was chosen
// (the final division by the row sum makes the choice of scale immaterial).  The scores of the
// next page are issued before the probabilities of the current one are ready, and the two groups
// alternate, so the tensor core works while the softmax runs.
//
// Values sit in the cache as [key][d]; they enter the second product as an MN-major operand, so
// nothing is transposed.  Causal and window masks come from absolute positions; a prompt that
// continues a cached prefix needs nothing special.  All barrier waits are bounded; a wait that
// gives up sets a status word (gb_attention_tc5_status) and the CTA runs out.
#include "tc5.cuh"
#include "api.h"

#include <math.h>


namespace {

__device__ int g_status;

typedef __nv_bfloat16 bf16;
constexpr int HD = 128, BQ = 128, GROUPS = 2, BKV = 64, STAGES = 5, THREADS = 448;
constexpr int FIRST_SOFTMAX_WARP = 1 + 2 * GROUPS;  // warp 0 loads queries and keys, then a scores issuer and a values issuer per group
constexpr int VALUE_LOADER_WARP = FIRST_SOFTMAX_WARP + 4 * GROUPS;  // the last warp loads the values
constexpr int QPANEL = 128 * 128;               // 128 rows of 128 bytes (64 head elements)
constexpr int KPANEL = 64 * 128;                // 64 keys of 128 bytes
constexpr int Q_BYTES = 2 * QPANEL;             // one group's query tile
constexpr int K_BYTES = 2 * KPANEL, V_BYTES = 2 * KPANEL, STAGE_BYTES = K_BYTES + V_BYTES;
constexpr int TMEM_COLS = 512;                  // S: 2 groups x 2 buffers x 64; O: 2 groups x 128
constexpr float LOG2E = 1.4426950408889634f;
constexpr int POLY_PAIRS = 1;                   // of every four pairs of scores, how many take the polynomial exponential (measured: 0 -> 55.5 us, 1 -> 52.9, 2 -> 56.8 at 2048 tokens)
constexpr float RESCALE_AT = 8.0f;              // rescale O when the row maximum outgrew the scale by 2^8

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(s32(bar)) : "memory");
}

// MN-major operand (values: rows are keys, 128-byte rows of 64 head elements, the second half of
// the head one panel further): leading byte offset = panel, stride byte offset = 8 rows.
__device__ __forceinline__ uint64_t smem_desc_mn(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFF) >> 4);
    d |= (uint64_t)(KPANEL >> 4) << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// D (+)= A B with A in tensor memory (128 lanes, two bfloat16 a column) and B from shared memory
__device__ __forceinline__ void umma_ta(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
        "}\n" ::"r"(d_tmem),
        "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

// Packed pairs of fp32 (one instruction works on two values) and the three-input maximum: the
// softmax warps set the pace of the kernel, so their instruction count matters.
__device__ __forceinline__ uint64_t pack2(float a, float b) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};\n" : "=l"(r) : "f"(a), "f"(b));
    return r;
}
__device__ __forceinline__ void unpack2(uint64_t r, float& a, float& b) { asm("mov.b64 {%0, %1}, %2;\n" : "=f"(a), "=f"(b) : "l"(r)); }
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;\n" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;\n" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ uint64_t add2_down(uint64_t a, uint64_t b) {  // rounded towards minus infinity
    uint64_t d;
    asm("add.rm.f32x2 %0, %1, %2;\n" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;\n" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// 2^x of two values on the FMA pipe alone, for the share of the exponentials that the
// special-function unit (16 a clock and SM) has no time for: x = n + f with n = floor(x) taken by
// adding 1.5 * 2^23 rounded down, 2^f by a cubic (relative error 1.9e-4, a twentieth of the
// bfloat16 step the probabilities are rounded to), and n added into the exponent field.
__device__ __forceinline__ void exp2_poly_x2(float x0, float x1, float& y0, float& y1) {
    x0 = fmaxf(x0, -126.f);
    x1 = fmaxf(x1, -126.f);
    const uint64_t x = pack2(x0, x1);
    const uint64_t r = add2_down(x, pack2(12582912.f, 12582912.f));
    const uint64_t n = add2(r, pack2(-12582912.f, -12582912.f));
    const uint64_t f = fma2(n, pack2(-1.f, -1.f), x);
    uint64_t q = fma2(f, pack2(0.0790199414f, 0.0790199414f), pack2(0.2241264433f, 0.2241264433f));
    q = fma2(q, f, pack2(0.6968385577f, 0.6968385577f));
    q = fma2(q, f, pack2(0.9998119473f, 0.9998119473f));
    float q0, q1, r0, r1;
    unpack2(q, q0, q1);
    unpack2(r, r0, r1);
    y0 = __int_as_float(__float_as_int(q0) + (__float_as_int(r0) << 23));
    y1 = __int_as_float(__float_as_int(q1) + (__float_as_int(r1) << 23));
}

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};\n" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
        "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]),
        "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]),
        "r"(r[31])
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
}

// 32 columns of this thread's lane without waiting for them (pair with tmem_wait_ld)
__device__ __forceinline__ void tmem_ld32_nowait(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }

__global__ void __launch_bounds__(THREADS) attn_prefill_tc5_kernel(const __grid_constant__ CUtensorMap map_q,
                                                                   const __grid_constant__ CUtensorMap map_k,
                                                                   const __grid_constant__ CUtensorMap map_v, AttnParams p,
                                                                   int by_kv_head) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* base = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* Qs = base;                          // [GROUPS][Q_BYTES]
    unsigned char* KVs = Qs + GROUPS * Q_BYTES;        // [STAGES][K | V]
    __shared__ uint64_t q_full, k_full[STAGES], v_full[STAGES], k_empty[STAGES], v_empty[STAGES];
    __shared__ uint64_t s_full[GROUPS][2], p_full[GROUPS][2], o_done[GROUPS][2];
    __shared__ uint32_t tmem_base_s;
    __shared__ int abort_s;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    pdl_wait();  // the tile's extent comes from the step's metadata
    pdl_trigger();
    // The order in which CTAs start.  Short prompts: heads vary fastest and the longest tiles of all
    // heads come first, so the SMs that finish a long tile early pick up the short ones (tiles of a
    // causal prompt differ manyfold in work).  Long prompts, whose keys and values do not fit L2
    // together: one kv head after the other (the query heads that share it side by side, longest
    // tiles first), so that what runs together reads the same keys and values.
    const int seq = blockIdx.z;
    int head = blockIdx.x, qt = (int)gridDim.y - 1 - (int)blockIdx.y;
    if (by_kv_head) {
        const int G = p.heads / p.kv_heads, tiles = (int)gridDim.y;
        const int id = (int)blockIdx.x + (int)gridDim.x * (int)blockIdx.y;
        const int per = G * tiles, rem = id % per;
        head = (id / per) * G + rem % G;
        qt = tiles - 1 - rem / G;
    }
    const int q_len = p.seq_q_len[seq], kv_len = p.seq_kv_len[seq];
    const int q0 = qt * (GROUPS * BQ);
    if (q0 >= q_len) return;  // the whole CTA leaves before anything is allocated
    const int past = kv_len - q_len;
    const int q_start = p.seq_q_start[seq];
    const int G = p.heads / p.kv_heads, kvh = head / G;
    const int* bt = block_table_row(p.block_table, p.bt_stride, p.seq_slot[seq], p.max_slots);

    // pages each group walks: from the first page any of its rows may see to the page of its last row
    int lo_pos = 0;
    if (p.window > 0) {
        lo_pos = past + q0 - p.window + 1;
        if (lo_pos < 0) lo_pos = 0;
    }
    const int t_lo = lo_pos / BKV;
    int n_g[GROUPS];
#pragma unroll
    for (int g = 0; g < GROUPS; g++) {
        const int first = q0 + g * BQ;
        if (first >= q_len) {
            n_g[g] = 0;
        } else {
            const int last = (first + BQ < q_len ? first + BQ : q_len) - 1;
            n_g[g] = (past + last) / BKV - t_lo + 1;
        }
    }
    const int n = n_g[0] > n_g[1] ? n_g[0] : n_g[1];

    if (threadIdx.x == 0) {
        mbar_init(&q_full, 1);
        for (int s = 0; s < STAGES; s++) {
            mbar_init(&k_full[s], 1);
            mbar_init(&v_full[s], 1);
            mbar_init(&k_empty[s], GROUPS);  // one arrival from each group's scores issuer
            mbar_init(&v_empty[s], GROUPS);  // one arrival from each group's values issuer
        }
        for (int g = 0; g < GROUPS; g++) {
            for (int b = 0; b < 2; b++) {
                mbar_init(&s_full[g][b], 1);
                mbar_init(&p_full[g][b], 4);
                mbar_init(&o_done[g][b], 1);
            }
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
    // columns: S of group g, buffer b at g * 128 + b * 64; O of group g at 256 + g * 128

    if (warp == 0) {
        if (lane == 0) {
            mbar_expect_tx(&q_full, GROUPS * Q_BYTES);
#pragma unroll
            for (int g = 0; g < GROUPS; g++) {
                tma_load_2d(Qs + g * Q_BYTES, &map_q, head * HD, q_start + q0 + g * BQ, &q_full);
                tma_load_2d(Qs + g * Q_BYTES + QPANEL, &map_q, head * HD + 64, q_start + q0 + g * BQ, &q_full);
            }
            // Keys and values travel separately: the keys of a page are free as soon as its scores are
            // done, long before its values are, so the key loads run further ahead than a shared
            // ring would let them, and the scores issuer never waits for them.
            int issued = 0;
            for (int j = 0; j < n; j++) {
                const int s = j % STAGES;
                const uint32_t phase = (uint32_t)(j / STAGES) & 1u;
                if (!mbar_wait_relaxed(&k_empty[s], phase ^ 1u)) {
                    atomicCAS(&g_status, 0, 1);
                    abort_s = 1;
                }
                if (*(volatile int*)&abort_s) break;
                mbar_expect_tx(&k_full[s], K_BYTES);
                unsigned char* ks = KVs + (size_t)s * STAGE_BYTES;
                int lp = t_lo + j;
                if (!gb_check(lp, p.bt_stride, GB_CHECK_LOGICAL_PAGE) || lp >= p.bt_stride) lp = p.bt_stride - 1;
                const int row = ((int)page_of(bt, lp * BKV, p.bt_stride, p.pages) * p.kv_heads + kvh) * 64;
#pragma unroll
                for (int h = 0; h < 2; h++) tma_load_2d(ks + h * KPANEL, &map_k, h * 64, row, &k_full[s]);
                issued = j + 1;
            }
            if (*(volatile int*)&abort_s) {
                for (int j = issued > STAGES ? issued - STAGES : 0; j < issued; j++)
                    mbar_wait(&k_full[j % STAGES], (uint32_t)(j / STAGES) & 1u);
                mbar_wait(&q_full, 0);
            }
        }
    } else if (warp == VALUE_LOADER_WARP) {
        if (lane == 0) {
            int issued = 0;
            for (int j = 0; j < n; j++) {
                const int s = j % STAGES;
                const uint32_t phase = (uint32_t)(j / STAGES) & 1u;
                if (!mbar_wait_relaxed(&v_empty[s], phase ^ 1u)) {
                    atomicCAS(&g_status, 0, 1);
                    abort_s = 1;
                }
                if (*(volatile int*)&abort_s) break;
                mbar_expect_tx(&v_full[s], V_BYTES);
                unsigned char* vs = KVs + (size_t)s * STAGE_BYTES + K_BYTES;
                int lp = t_lo + j;
                if (!gb_check(lp, p.bt_stride, GB_CHECK_LOGICAL_PAGE) || lp >= p.bt_stride) lp = p.bt_stride - 1;
                const int row = ((int)page_of(bt, lp * BKV, p.bt_stride, p.pages) * p.kv_heads + kvh) * 64;
#pragma unroll
                for (int h = 0; h < 2; h++) tma_load_2d(vs + h * KPANEL, &map_v, h * 64, row, &v_full[s]);
                issued = j + 1;
            }
            if (*(volatile int*)&abort_s) {
                for (int j = issued > STAGES ? issued - STAGES : 0; j < issued; j++)
                    mbar_wait(&v_full[j % STAGES], (uint32_t)(j / STAGES) & 1u);
            }
        }
    } else if (warp < FIRST_SOFTMAX_WARP) {
        // Two issuing threads per group, in warps of their own: one issues the scores products, one
        // the values products.  On an issuing thread a barrier wait that blocks and a commit cost a
        // few hundred cycles each and a product about fifty, so a single thread doing both kinds
        // (two or three waits, twelve products, three commits a page) set the pace of the kernel.
        if (lane == 0) {
            const int g = (warp - 1) % GROUPS;
            const bool scores_role = warp - 1 < GROUPS;
            const int my_n = n_g[g];
            bool ok = true;
            int kv_seen = -1;  // last page whose arrival this thread has waited for
            auto need_page = [&](int j) -> bool {
                while (kv_seen < j) {
                    kv_seen++;
                    uint64_t* full = scores_role ? &k_full[kv_seen % STAGES] : &v_full[kv_seen % STAGES];
                    if (!mbar_wait_relaxed(full, (uint32_t)(kv_seen / STAGES) & 1u)) return false;
                }
                return true;
            };
            if (scores_role) {
                // S_g[j & 1] = Q_g K_j^T, then the keys of page j are free
                const uint32_t idesc_qk = instr_desc(BQ, BKV);
                ok = mbar_wait(&q_full, 0);
                const uint64_t q_desc = smem_desc(s32(Qs + g * Q_BYTES));
                uint64_t k_desc[STAGES];
#pragma unroll
                for (int s = 0; s < STAGES; s++) k_desc[s] = smem_desc(s32(KVs + (size_t)s * STAGE_BYTES));
                for (int j = 0; j < n && ok; j++) {
                    // a group with fewer pages only keeps the count, but never ahead of the loads, or it
                    // would arrive twice in one phase
                    ok = need_page(j);
                    if (ok && j < my_n) {
                        const int b = j & 1;
                        // the probabilities of page j - 2 lie in this buffer's columns until their product has read them
                        if (j >= 2) ok = mbar_wait_relaxed(&o_done[g][b], (uint32_t)((j - 2) >> 1) & 1u);
                        if (!ok) break;
                        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                        const uint64_t kd = k_desc[j % STAGES];
                        const uint32_t d_tmem = tmem_base + (uint32_t)(g * 128 + b * 64);
#pragma unroll
                        for (int ks = 0; ks < HD / 16; ks++) {
                            // 64 head elements to a panel; 16 elements = 32 bytes = 2 address units inside it
                            umma(d_tmem, q_desc + (uint64_t)((ks >> 2) * (QPANEL >> 4) + (ks & 3) * 2),
                                 kd + (uint64_t)((ks >> 2) * (KPANEL >> 4) + (ks & 3) * 2), idesc_qk, ks > 0 ? 1u : 0u);
                        }
                        umma_commit(&s_full[g][b]);
                    }
                    if (ok) umma_commit(&k_empty[j % STAGES]);
                }
            } else {
                // O_g (+)= P_g[j & 1] V_j, then the values of page j are free
                const uint32_t idesc_pv = instr_desc(BQ, HD) | (1u << 16);  // values enter MN-major
                uint64_t v_desc[STAGES];
#pragma unroll
                for (int s = 0; s < STAGES; s++) v_desc[s] = smem_desc_mn(s32(KVs + (size_t)s * STAGE_BYTES + K_BYTES));
                for (int j = 0; j < n && ok; j++) {
                    ok = need_page(j);
                    if (ok && j < my_n) {
                        const int b = j & 1;
                        ok = mbar_wait(&p_full[g][b], (uint32_t)(j >> 1) & 1u);
                        if (!ok) break;
                        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                        const uint64_t vd = v_desc[j % STAGES];
                        const uint32_t d_tmem = tmem_base + (uint32_t)(256 + g * 128);
#pragma unroll
                        // 16 keys = 8 columns of the probabilities (written over the page's scores) and 16 rows of
                        // 128 bytes further into the values
                        for (int kk = 0; kk < BKV / 16; kk++)
                            umma_ta(d_tmem, tmem_base + (uint32_t)(g * 128 + b * 64 + kk * 8), vd + (uint64_t)(kk * ((16 * 128) >> 4)), idesc_pv,
                                    (j > 0 || kk > 0) ? 1u : 0u);
                        umma_commit(&o_done[g][b]);
                    }
                    if (ok) umma_commit(&v_empty[j % STAGES]);
                }
            }
            if (!ok) {
                atomicCAS(&g_status, 0, 3);
                abort_s = 1;
            }
        }
    } else {
        // softmax: group g, thread = query row
        const int g = (warp - FIRST_SOFTMAX_WARP) >> 2;
        const int quad = warp & 3;
        const int r = quad * 32 + lane;               // row within the group
        const int qrow = q0 + g * BQ + r;             // row within the sequence's new rows
        const int pos = past + qrow;                  // absolute position
        const bool row_ok = qrow < q_len;
        const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
        const uint32_t o_addr = tmem_base + lane_addr + (uint32_t)(256 + g * 128);
        const float sc = p.scale * LOG2E;
        const int my_n = n_g[g];
        float m_run = -INFINITY;   // true running maximum (scaled, base 2)
        float m_used = -INFINITY;  // the maximum the probabilities and O are currently scaled by
        float l = 0.f;
        bool ok = true;
        for (int j = 0; j < my_n && ok; j++) {
            const int b = j & 1, key0 = (t_lo + j) * BKV;
            if (!mbar_wait(&s_full[g][b], (uint32_t)(j >> 1) & 1u)) {
                ok = false;
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const uint32_t s_addr = tmem_base + lane_addr + (uint32_t)(g * 128 + b * 64);
            uint32_t v0[32], v1[32];
            tmem_ld32_nowait(s_addr, v0);
            tmem_ld32_nowait(s_addr + 32u, v1);
            tmem_wait_ld();

            const bool need_mask = key0 + BKV - 1 > pos || (p.window > 0 && key0 <= pos - p.window);
            if (need_mask) {
#pragma unroll
                for (int i = 0; i < 32; i++) {
                    const int ka = key0 + i, kb = key0 + 32 + i;
                    if (ka > pos || (p.window > 0 && ka <= pos - p.window)) v0[i] = 0xff800000u;  // -inf
                    if (kb > pos || (p.window > 0 && kb <= pos - p.window)) v1[i] = 0xff800000u;
                }
            }
            float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
#pragma unroll
                for (int e = 0; e < 4; e++) mx[e] = max3(mx[e], __uint_as_float(v0[i + e]), __uint_as_float(v1[i + e]));
            }
            const float tile_max = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * sc;  // sc > 0
            m_run = fmaxf(m_run, tile_max);
            // rescale only when the maximum has outgrown the scale in use (or there is none yet)
            const bool grow = m_run > m_used + RESCALE_AT || (m_used == -INFINITY && m_run != -INFINITY);
            // this page's probability buffer was read by the product of two pages ago
            if (!mbar_wait(&o_done[g][b], ((uint32_t)(j >> 1) & 1u) ^ 1u)) {
                ok = false;
                break;
            }

            if (__any_sync(0xffffffffu, grow && j > 0)) {
                // O_g may only be touched between products: wait for the previous page's
                if (!mbar_wait(&o_done[g][(j - 1) & 1], (uint32_t)((j - 1) >> 1) & 1u)) {
                    ok = false;
                    break;
                }
                // the whole warp takes part (tensor-memory access is warp-wide); rows that keep their scale multiply by 1
                const float f = (grow && j > 0) ? fast_exp2(m_used - m_run) : 1.f;  // m_used = -inf gives 0: O is all zeros then
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
#pragma unroll 1
                for (int c0 = 0; c0 < HD; c0 += 32) {
                    uint32_t o[32];
                    tmem_ld32(o_addr + (uint32_t)c0, o);
#pragma unroll
                    for (int i = 0; i < 32; i++) o[i] = __float_as_uint(__uint_as_float(o[i]) * f);
                    tmem_st32(o_addr + (uint32_t)c0, o);
                }
                l *= f;
            }
            if (grow) m_used = m_run;
            const float mbase = m_used == -INFINITY ? 0.f : m_used;
            const uint64_t sc2 = pack2(sc, sc), nmb2 = pack2(-mbase, -mbase);
            uint64_t sum2[2] = {pack2(0.f, 0.f), pack2(0.f, 0.f)};
            uint32_t pw[32];  // the row's 64 probabilities, two a word
#pragma unroll
            for (int c = 0; c < 8; c++) {  // eight 16-byte chunks of eight keys
                uint32_t pk[4];
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const int i = (c & 3) * 8 + e * 2;
                    const uint32_t a = c < 4 ? v0[i] : v1[i], bb = c < 4 ? v0[i + 1] : v1[i + 1];
                    float t0, t1, p0, p1;
                    unpack2(fma2(pack2(__uint_as_float(a), __uint_as_float(bb)), sc2, nmb2), t0, t1);
                    if (e < POLY_PAIRS) {
                        exp2_poly_x2(t0, t1, p0, p1);
                    } else {
                        p0 = fast_exp2(t0);
                        p1 = fast_exp2(t1);
                    }
                    sum2[e & 1] = add2(sum2[e & 1], pack2(p0, p1));
                    __nv_bfloat162 h2 = __floats2bfloat162_rn(p0, p1);
                    pk[e] = *reinterpret_cast<uint32_t*>(&h2);
                }
#pragma unroll
                for (int e = 0; e < 4; e++) pw[c * 4 + e] = pk[e];
            }
            // The probabilities stay in tensor memory, as the A operand of the second product (128 lanes = rows,
            // two bfloat16 a column): over the first 32 columns of this page's scores, which this thread has read out.
            tmem_st32(s_addr, pw);
            float sum[4];
            unpack2(sum2[0], sum[0], sum[1]);
            unpack2(sum2[1], sum[2], sum[3]);
            l += (sum[0] + sum[1]) + (sum[2] + sum[3]);
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_full[g][b]);
        }
        if (ok && my_n > 0 && !mbar_wait(&o_done[g][(my_n - 1) & 1], (uint32_t)((my_n - 1) >> 1) & 1u)) ok = false;
        if (!ok) {
            atomicCAS(&g_status, 0, 4);
            abort_s = 1;
        } else if (my_n > 0) {
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const float inv = 1.f / l;
            bf16* op = (bf16*)p.out + (int64_t)(q_start + qrow) * p.out_row_stride + (int64_t)head * HD;
#pragma unroll 1
            for (int c0 = 0; c0 < HD; c0 += 32) {
                uint32_t o[32];
                tmem_ld32(o_addr + (uint32_t)c0, o);
                if (row_ok) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        uint4 o4;
                        __nv_bfloat162 a0 = __floats2bfloat162_rn(__uint_as_float(o[i]) * inv, __uint_as_float(o[i + 1]) * inv);
                        __nv_bfloat162 a1 = __floats2bfloat162_rn(__uint_as_float(o[i + 2]) * inv, __uint_as_float(o[i + 3]) * inv);
                        __nv_bfloat162 a2 = __floats2bfloat162_rn(__uint_as_float(o[i + 4]) * inv, __uint_as_float(o[i + 5]) * inv);
                        __nv_bfloat162 a3 = __floats2bfloat162_rn(__uint_as_float(o[i + 6]) * inv, __uint_as_float(o[i + 7]) * inv);
                        o4.x = *reinterpret_cast<uint32_t*>(&a0);
                        o4.y = *reinterpret_cast<uint32_t*>(&a1);
                        o4.z = *reinterpret_cast<uint32_t*>(&a2);
                        o4.w = *reinterpret_cast<uint32_t*>(&a3);
                        *reinterpret_cast<uint4*>(op + c0 + i) = o4;
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// 2-D map over `rows` rows of `cols` bfloat16 with a row stride of ld elements; boxes of box_rows x 64
int make_map(CUtensorMap* map, const void* base, int64_t rows, int cols, int64_t ld, int box_rows) {
    Tc5EncodeTiledFn fn = tc5_encode_fn();
    if (!fn) GB_REFUSE("attention_tc5: the driver offers no cuTensorMapEncodeTiled");
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) GB_REFUSE("attention_tc5: cuTensorMapEncodeTiled failed with code %d", (int)r);
    return 0;
}

}  // namespace

// rows: packed query rows in the q buffer; pages: pages in each cache plane
GB_API int gb_attention_prefill_tc5(const AttnParams* pp, int rows, int pages, cudaStream_t stream) {
    AttnParams p = *pp;
    if (p.nseq <= 0 || p.max_q_len <= 0) return 0;
    const char* who = "attention_prefill_tc5";
    if (p.d != HD) GB_REFUSE("%s: head_dim %d; this kernel takes 128", who, p.d);
    if (p.heads <= 0 || p.kv_heads <= 0 || p.heads % p.kv_heads) GB_REFUSE("%s: %d heads over %d kv heads", who, p.heads, p.kv_heads);
    if (p.num_splits != 1) GB_REFUSE("%s: key splits are for single-token rows", who);
    if (p.window < 0) GB_REFUSE("%s: window %d", who, p.window);
    if (((uintptr_t)p.q & 15) || (p.q_row_stride & 7)) GB_REFUSE("%s: query rows must be 16-byte aligned", who);
    if (((uintptr_t)p.out & 15) || (p.out_row_stride & 7)) GB_REFUSE("%s: output rows must be 16-byte aligned", who);
    if (((uintptr_t)p.k_plane & 15) || ((uintptr_t)p.v_plane & 15)) GB_REFUSE("%s: cache planes must be 16-byte aligned", who);
    if (rows <= 0 || pages <= 0) GB_REFUSE("%s: %d rows, %d pages", who, rows, pages);
    if ((int64_t)pages * p.kv_heads * 64 > 0x7fffffff) GB_REFUSE("%s: the cache plane has too many rows for one tensor map", who);
    const int smem = GROUPS * Q_BYTES + STAGES * STAGE_BYTES + 1024;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc5_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) GB_REFUSE("%s: cannot reserve %d bytes of shared memory: %s", who, smem, cudaGetErrorString(e));
        configured = true;
    }
    CUtensorMap map_q, map_k, map_v;
    if (int rc = make_map(&map_q, p.q, rows, p.heads * HD, p.q_row_stride, BQ)) return rc;
    if (int rc = make_map(&map_k, p.k_plane, (int64_t)pages * p.kv_heads * 64, HD, HD, 64)) return rc;
    if (int rc = make_map(&map_v, p.v_plane, (int64_t)pages * p.kv_heads * 64, HD, HD, 64)) return rc;
    dim3 grid(p.heads, ceil_div(p.max_q_len, GROUPS * BQ), p.nseq);
    if (grid.y > 65535 || grid.z > 65535) GB_REFUSE("%s: grid (%u, %u, %u) exceeds one launch", who, grid.x, grid.y, grid.z);
    // keys and values of the longest prompt, all kv heads: more than 48 MB do not stay in L2 beside the rest
    const int by_kv_head = (int64_t)p.max_q_len * p.kv_heads * (4 * HD) > ((int64_t)48 << 20) ? 1 : 0;
    cudaError_t e = launch_pdl(attn_prefill_tc5_kernel, grid, dim3(THREADS), (size_t)smem, stream, map_q, map_k, map_v, p, by_kv_head);
    if (e != cudaSuccess) GB_REFUSE("%s: launch failed: %s", who, cudaGetErrorString(e));
    return 0;
}

GB_API int gb_attention_tc5_status() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_status, sizeof(int)) != cudaSuccess) return -1;
    if (v != 0) cudaMemcpyToSymbol(g_status, &zero, sizeof(int));
    return v;
}

// the checked build's record of the first index this file's kernels found out of bounds
GB_CHECK_READER(gb_checked_status_attention_tc5)
