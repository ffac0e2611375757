// Causal grouped-query attention over the paged cache on the CUDA cores, all arithmetic fp32.
//
// It is the attention of the true 32-bit path for prompts and for single tokens, and the
// fallback of the bfloat16 path for head sizes the tensor-core kernels do not take.  A CTA owns
// one (sequence, kv head, tile of query rows); its 16 rows are (query position, head of the
// group) pairs, so the heads of a group share every key/value tile that is read
// (internal/qwen3lm/gpu.metal:1102-1234 shares tiles the same way).  Keys are visited in tiles of
// 32 that start at absolute positions 0, 32, 64, ..., with a streaming softmax
// (internal/qwen3lm/ops.go:259-293): a row's result does not depend on how its sequence was cut
// into steps or on what else is in the batch.
#include "common.cuh"
#include "api.h"

#include <math.h>


namespace {

constexpr int RW = 4;       // rows per warp
constexpr int ROWS = 16;    // rows per CTA (4 warps)
constexpr int KT = 32;      // keys per tile

template <typename T, int NE>
__global__ void __launch_bounds__(128) attn_simt_kernel(AttnParams p) {
    extern __shared__ float sm[];
    const int d = p.d, ks = d + 1;
    float* Qs = sm;                // [16][d], pre-scaled
    float* Ks = Qs + ROWS * d;     // [32][d + 1]
    float* Vs = Ks + KT * ks;      // [32][d + 1]

    const int G = p.heads / p.kv_heads;
    const int GC = G < ROWS ? G : ROWS;
    const int hchunks = (G + GC - 1) / GC;
    const int QT = ROWS / GC;

    const int seq = blockIdx.z / p.num_splits, split = blockIdx.z % p.num_splits;
    const int kvh = blockIdx.y / hchunks, chunk = blockIdx.y % hchunks;
    const int q_len = p.seq_q_len[seq], kv_len = p.seq_kv_len[seq];
    const int q0 = blockIdx.x * QT;
    if (q0 >= q_len) return;
    const int past = kv_len - q_len;
    const int q_start = p.seq_q_start[seq];
    const int* bt = block_table_row(p.block_table, p.bt_stride, p.seq_slot[seq], p.max_slots);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    // stage the query rows, scaled
    for (int idx = tid; idx < ROWS * d; idx += 128) {
        int r = idx / d, c = idx - r * d;
        int qi = r / GC, hg = chunk * GC + r % GC;
        bool ok = qi < QT && q0 + qi < q_len && hg < G;
        float v = 0.f;
        if (ok) {
            const T* qp = (const T*)p.q + (int64_t)(q_start + q0 + qi) * p.q_row_stride + (int64_t)(kvh * G + hg) * d;
            v = to_f32<T>(qp[c]) * p.scale;
        }
        Qs[idx] = v;
    }

    int row_pos[RW], row_head[RW], row_q[RW];
    bool row_ok[RW];
#pragma unroll
    for (int rr = 0; rr < RW; rr++) {
        int r = warp * RW + rr;
        int qi = r / GC, hg = chunk * GC + r % GC;
        row_ok[rr] = qi < QT && q0 + qi < q_len && hg < G;
        row_q[rr] = q0 + qi;
        row_head[rr] = kvh * G + hg;
        row_pos[rr] = past + q0 + qi;
    }

    int last_q = (q0 + QT < q_len ? q0 + QT : q_len) - 1;
    const int hi_pos = past + last_q;
    int lo_pos = 0;
    if (p.window > 0) {
        lo_pos = past + q0 - p.window + 1;
        if (lo_pos < 0) lo_pos = 0;
    }
    const int t_lo = lo_pos / KT, t_hi = hi_pos / KT + 1;
    const int per = (t_hi - t_lo + p.num_splits - 1) / p.num_splits;
    const int my_lo = t_lo + split * per;
    const int my_hi = my_lo + per < t_hi ? my_lo + per : t_hi;

    float m[RW], l[RW], acc[RW][NE];
#pragma unroll
    for (int rr = 0; rr < RW; rr++) {
        m[rr] = -INFINITY;
        l[rr] = 0.f;
#pragma unroll
        for (int e = 0; e < NE; e++) acc[rr][e] = 0.f;
    }

    for (int t = my_lo; t < my_hi; t++) {
        __syncthreads();
        // each warp stages 8 keys of the tile
        for (int jj = 0; jj < 8; jj++) {
            int j = warp * 8 + jj;
            int key = t * KT + j;
            if (key <= hi_pos) {
                int64_t page = page_of(bt, key, p.bt_stride, p.pages);
                int64_t off = ((page * p.kv_heads + kvh) * GB_PAGE + (key % GB_PAGE)) * (int64_t)d;
                const T* kp = (const T*)p.k_plane + off;
                const T* vp = (const T*)p.v_plane + off;
                for (int c = lane; c < d; c += 32) {
                    Ks[j * ks + c] = to_f32<T>(kp[c]);
                    Vs[j * ks + c] = to_f32<T>(vp[c]);
                }
            } else {
                for (int c = lane; c < d; c += 32) {
                    Ks[j * ks + c] = 0.f;
                    Vs[j * ks + c] = 0.f;
                }
            }
        }
        __syncthreads();

        float s[RW];
#pragma unroll
        for (int rr = 0; rr < RW; rr++) s[rr] = 0.f;
        const float* krow = Ks + lane * ks;
        const float* qrow = Qs + warp * RW * d;
        for (int c = 0; c < d; c++) {
            float kv = krow[c];
#pragma unroll
            for (int rr = 0; rr < RW; rr++) s[rr] = fmaf(qrow[rr * d + c], kv, s[rr]);
        }
        const int key = t * KT + lane;
        float pr[RW];
#pragma unroll
        for (int rr = 0; rr < RW; rr++) {
            bool valid = row_ok[rr] && key <= row_pos[rr] && (p.window <= 0 || key > row_pos[rr] - p.window);
            float sv = valid ? s[rr] : -INFINITY;
            float m_new = fmaxf(m[rr], warp_max(sv));
            if (m_new == -INFINITY) {
                pr[rr] = 0.f;
                continue;
            }
            float corr = expf(m[rr] - m_new);
            float pv = valid ? expf(sv - m_new) : 0.f;
            l[rr] = l[rr] * corr + warp_sum(pv);
#pragma unroll
            for (int e = 0; e < NE; e++) acc[rr][e] *= corr;
            m[rr] = m_new;
            pr[rr] = pv;
        }
        for (int jj = 0; jj < KT; jj++) {
            const float* vrow = Vs + jj * ks;
#pragma unroll
            for (int rr = 0; rr < RW; rr++) {
                float pj = __shfl_sync(0xffffffffu, pr[rr], jj);
#pragma unroll
                for (int e = 0; e < NE; e++) {
                    int c = lane + 32 * e;
                    if (c < d) acc[rr][e] = fmaf(pj, vrow[c], acc[rr][e]);
                }
            }
        }
    }

#pragma unroll
    for (int rr = 0; rr < RW; rr++) {
        if (!row_ok[rr]) continue;
        if (p.num_splits == 1) {
            T* op = (T*)p.out + (int64_t)(q_start + row_q[rr]) * p.out_row_stride + (int64_t)row_head[rr] * d;
            float inv = 1.f / l[rr];
#pragma unroll
            for (int e = 0; e < NE; e++) {
                int c = lane + 32 * e;
                if (c < d) op[c] = from_f32<T>(acc[rr][e] * inv);
            }
        } else {
            float* sp = p.scratch + (((int64_t)seq * p.heads + row_head[rr]) * p.num_splits + split) * (d + 2);
            if (lane == 0) {
                sp[0] = m[rr];
                sp[1] = l[rr];
            }
#pragma unroll
            for (int e = 0; e < NE; e++) {
                int c = lane + 32 * e;
                if (c < d) sp[2 + c] = acc[rr][e];
            }
        }
    }
}

// out[seq, head, :] = sum_s exp(m_s - M) acc_s / sum_s exp(m_s - M) l_s over the key splits.
// One CTA of 128 threads per (sequence, head).  The first warp reads every split's maximum and sum
// at once and leaves the weights exp(m_s - M) in shared memory (maximum and normaliser by shuffle
// trees, a fixed order); then thread c adds column c of the splits in split order.
constexpr int MERGE_MAX_SPLITS = 256;

template <typename T>
__global__ void __launch_bounds__(128) attn_merge_kernel(const float* __restrict__ scratch, T* __restrict__ out, int64_t out_row_stride,
                                                         const int* __restrict__ seq_q_start, int heads, int d, int num_splits) {
    __shared__ float w_s[MERGE_MAX_SPLITS];
    __shared__ float l_s;
    pdl_trigger();  // the product that follows may start fetching its weights
    const int head = blockIdx.x, seq = blockIdx.y;
    const float* sp = scratch + ((int64_t)seq * heads + head) * num_splits * (d + 2);
    if (threadIdx.x < 32) {
        const int lane = threadIdx.x;
        float M = -INFINITY;
        for (int s = lane; s < num_splits; s += 32) M = fmaxf(M, sp[(int64_t)s * (d + 2)]);
        M = warp_max(M);
        float L = 0.f;
        for (int s = lane; s < num_splits; s += 32) {
            const float ms = sp[(int64_t)s * (d + 2)];
            const float w = ms != -INFINITY ? expf(ms - M) : 0.f;
            w_s[s] = w;
            L += w * sp[(int64_t)s * (d + 2) + 1];
        }
        L = warp_sum(L);
        if (lane == 0) l_s = L;
    }
    __syncthreads();
    const float L = l_s;
    T* op = out + (int64_t)seq_q_start[seq] * out_row_stride + (int64_t)head * d;
    for (int c = threadIdx.x; c < d; c += blockDim.x) {
        float a = 0.f;
        // sixteen loads in flight at a time; the sum itself stays in split order
        for (int s0 = 0; s0 < num_splits; s0 += 16) {
            float v[16];
#pragma unroll
            for (int j = 0; j < 16; j++) v[j] = s0 + j < num_splits ? sp[(int64_t)(s0 + j) * (d + 2) + 2 + c] : 0.f;
#pragma unroll
            for (int j = 0; j < 16; j++)
                if (s0 + j < num_splits) a += w_s[s0 + j] * v[j];
        }
        op[c] = from_f32<T>(a / L);
    }
}

template <typename T, int NE>
int launch_ne(const AttnParams& p, dim3 grid, size_t smem, cudaStream_t stream) {
    static bool configured = false;
    if (!configured && smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(attn_simt_kernel<T, NE>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) GB_REFUSE("attention_simt: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
        configured = true;
    }
    attn_simt_kernel<T, NE><<<grid, 128, smem, stream>>>(p);
    GB_CHECK_LAUNCH("attention_simt");
    return 0;
}

template <typename T>
int launch(const AttnParams& p, cudaStream_t stream) {
    const int G = p.heads / p.kv_heads;
    const int GC = G < ROWS ? G : ROWS;
    const int hchunks = (G + GC - 1) / GC;
    const int QT = ROWS / GC;
    dim3 grid(ceil_div(p.max_q_len, QT), p.kv_heads * hchunks, p.nseq * p.num_splits);
    if (grid.y > 65535 || grid.z > 65535)
        GB_REFUSE("attention_simt: grid (%u, %u, %u) exceeds one launch", grid.x, grid.y, grid.z);
    size_t smem = ((size_t)ROWS * p.d + 2 * (size_t)KT * (p.d + 1)) * sizeof(float);
    int ne = ceil_div(p.d, 32);
    int rc;
    switch (ne) {
        case 1: rc = launch_ne<T, 1>(p, grid, smem, stream); break;
        case 2: rc = launch_ne<T, 2>(p, grid, smem, stream); break;
        case 3: rc = launch_ne<T, 3>(p, grid, smem, stream); break;
        case 4: rc = launch_ne<T, 4>(p, grid, smem, stream); break;
        case 5: rc = launch_ne<T, 5>(p, grid, smem, stream); break;
        case 6: rc = launch_ne<T, 6>(p, grid, smem, stream); break;
        case 7: rc = launch_ne<T, 7>(p, grid, smem, stream); break;
        case 8: rc = launch_ne<T, 8>(p, grid, smem, stream); break;
        default: GB_REFUSE("attention_simt: head_dim %d is larger than 256", p.d);
    }
    if (rc) return rc;
    if (p.num_splits > 1) {
        attn_merge_kernel<T><<<dim3(p.heads, p.nseq), 128, 0, stream>>>(p.scratch, (T*)p.out, p.out_row_stride,
                                                                        p.seq_q_start, p.heads, p.d, p.num_splits);
        GB_CHECK_LAUNCH("attention_merge");
    }
    return 0;
}

}  // namespace

// Merge of per-split partial results, shared with the tensor-core single-token kernel.
int gb_attention_merge_launch(const float* scratch, void* out, int dtype, int64_t out_row_stride, const int* seq_q_start,
                              int nseq, int heads, int d, int num_splits, cudaStream_t stream) {
    if (num_splits > MERGE_MAX_SPLITS) GB_REFUSE("attention: %d key splits; at most %d", num_splits, MERGE_MAX_SPLITS);
    if (dtype == GB_F32)
        attn_merge_kernel<float><<<dim3(heads, nseq), 128, 0, stream>>>(scratch, (float*)out, out_row_stride, seq_q_start, heads, d, num_splits);
    else
        attn_merge_kernel<__nv_bfloat16><<<dim3(heads, nseq), 128, 0, stream>>>(scratch, (__nv_bfloat16*)out, out_row_stride,
                                                                                seq_q_start, heads, d, num_splits);
    GB_CHECK_LAUNCH("attention_merge");
    return 0;
}

GB_API int gb_attention_simt(const AttnParams* pp, int dtype, cudaStream_t stream) {
    AttnParams p = *pp;
    if (p.nseq <= 0 || p.max_q_len <= 0) return 0;
    if (p.heads <= 0 || p.kv_heads <= 0 || p.heads % p.kv_heads) GB_REFUSE("attention: %d heads over %d kv heads", p.heads, p.kv_heads);
    if (p.d <= 0 || p.d > 256) GB_REFUSE("attention_simt: head_dim %d is outside [1, 256]", p.d);
    if (p.num_splits < 1 || p.num_splits > MERGE_MAX_SPLITS) GB_REFUSE("attention: %d key splits; 1 to %d", p.num_splits, MERGE_MAX_SPLITS);
    if (p.num_splits > 1 && p.max_q_len != 1) GB_REFUSE("attention: key splits need single-token rows, got rows of up to %d", p.max_q_len);
    if (p.num_splits > 1 && !p.scratch) GB_REFUSE("attention: %d key splits without scratch memory", p.num_splits);
    if (p.window < 0) GB_REFUSE("attention: window %d", p.window);
    if (dtype == GB_F32) return launch<float>(p, stream);
    if (dtype == GB_BF16) return launch<__nv_bfloat16>(p, stream);
    GB_REFUSE("attention: unknown dtype %d", dtype);
}

// the checked build's record of the first index this file's kernels found out of bounds
GB_CHECK_READER(gb_checked_status_attention_simt)
