// bfloat16 attention over the paged cache on mma.sync tensor cores.
//
//  * prompts: a flash-attention kernel.  A CTA owns 64 query rows of one head of one sequence
//    (16 rows a warp) and walks the sequence's cache pages; a page of 64 keys of one kv head is
//    one contiguous block, fetched with cp.async one page ahead of the arithmetic.  Causal and
//    window masks are taken from absolute positions, so a prompt that continues a cached prefix
//    (or arrives in pieces) needs nothing special.
//  * single tokens: a split-key kernel.  A CTA owns one (sequence, kv head, split of the keys);
//    the 16 rows of its tiles are the query heads of the group, so the group's heads share
//    every key and value that is read (internal/qwen3lm/gpu.metal:389-466 shares them the same
//    way).  The four warps take 16 keys each of every page, keep their own running softmax, and
//    are merged in shared memory; splits are merged by a second small kernel through scratch.
//
// Scores, the softmax and the output accumulators are fp32; probabilities are rounded to
// bfloat16 for the second product, as the values are bfloat16.
#include "mma.cuh"
#include "api.h"

#include <math.h>


int gb_attention_merge_launch(const float* scratch, void* out, int dtype, int64_t out_row_stride, const int* seq_q_start,
                              int nseq, int heads, int d, int num_splits, cudaStream_t stream);

namespace {

typedef __nv_bfloat16 bf16;
constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;

// copy 64 rows of HD bf16 (contiguous in global memory) into padded shared rows
template <int HD>
__device__ __forceinline__ void load_page(bf16* dst, const bf16* src, int tid, int nthreads) {
    constexpr int SD = HD + 8, CH = HD / 8;
    for (int idx = tid; idx < 64 * CH; idx += nthreads) {
        int row = idx / CH, c = idx - row * CH;
        cp_async16(dst + row * SD + c * 8, src + row * HD + c * 8, 16);
    }
}

// ------------------------------------------------------------------------------------------
template <int HD, bool QREG>
__global__ void __launch_bounds__(128) attn_prefill_mma_kernel(AttnParams p) {
    constexpr int SD = HD + 8, KS = HD / 16, NF = HD / 8;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* Qs = reinterpret_cast<bf16*>(smem_raw);
    bf16* Ks = Qs + 64 * SD;
    bf16* Vs = Ks + 2 * 64 * SD;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
    const int seq = blockIdx.z, head = blockIdx.y;
    const int q_len = p.seq_q_len[seq], kv_len = p.seq_kv_len[seq];
    const int qt = (int)gridDim.x - 1 - (int)blockIdx.x;  // late (long) tiles first
    const int q0 = qt * 64;
    if (q0 >= q_len) return;
    const int past = kv_len - q_len;
    const int q_start = p.seq_q_start[seq];
    const int G = p.heads / p.kv_heads, kvh = head / G;
    const int* bt = block_table_row(p.block_table, p.bt_stride, p.seq_slot[seq], p.max_slots);
    const bf16* kbase = (const bf16*)p.k_plane;
    const bf16* vbase = (const bf16*)p.v_plane;

    // query tile
    {
        constexpr int CH = HD / 8;
        const bf16* qsrc = (const bf16*)p.q + (int64_t)(q_start + q0) * p.q_row_stride + (int64_t)head * HD;
        for (int idx = tid; idx < 64 * CH; idx += 128) {
            int row = idx / CH, c = idx - row * CH;
            bool ok = q0 + row < q_len;
            cp_async16(Qs + row * SD + c * 8, ok ? qsrc + (int64_t)row * p.q_row_stride + c * 8 : qsrc, ok ? 16 : 0);
        }
    }
    const int last_q = (q0 + 64 < q_len ? q0 + 64 : q_len) - 1;
    const int hi_pos = past + last_q;
    int lo_pos = 0;
    if (p.window > 0) {
        lo_pos = past + q0 - p.window + 1;
        if (lo_pos < 0) lo_pos = 0;
    }
    const int t_lo = lo_pos / 64, t_hi = hi_pos / 64;

    auto load_tile = [&](int t, int buf) {
        int64_t page = page_of(bt, t * 64, p.bt_stride, p.pages);
        int64_t off = ((page * p.kv_heads + kvh) * 64) * (int64_t)HD;
        load_page<HD>(Ks + buf * 64 * SD, kbase + off, tid, 128);
        load_page<HD>(Vs + buf * 64 * SD, vbase + off, tid, 128);
    };
    load_tile(t_lo, 0);
    cp_async_commit();

    const float sc = p.scale * LOG2E;
    const int row0 = past + q0 + warp * 16 + g;  // absolute position of this thread's first row
    const int row1 = row0 + 8;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    float o[NF][4];
#pragma unroll
    for (int j = 0; j < NF; j++)
#pragma unroll
        for (int e = 0; e < 4; e++) o[j][e] = 0.f;
    uint32_t qf[QREG ? KS : 1][4];

    for (int t = t_lo; t <= t_hi; t++) {
        const int buf = (t - t_lo) & 1;
        cp_async_wait<0>();
        __syncthreads();
        if (t + 1 <= t_hi) load_tile(t + 1, buf ^ 1);
        cp_async_commit();
        if (QREG && t == t_lo) {
#pragma unroll
            for (int ks = 0; ks < KS; ks++)
                ldmatrix_x4(qf[QREG ? ks : 0], Qs + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * SD + ks * 16 + (lane >> 4) * 8);
        }
        const bf16* kt = Ks + buf * 64 * SD;
        const bf16* vt = Vs + buf * 64 * SD;
        float s[8][4];
#pragma unroll
        for (int j = 0; j < 8; j++)
#pragma unroll
            for (int e = 0; e < 4; e++) s[j][e] = 0.f;
#pragma unroll
        for (int ks = 0; ks < KS; ks++) {
            uint32_t a[4];
            if (QREG) {
#pragma unroll
                for (int e = 0; e < 4; e++) a[e] = qf[QREG ? ks : 0][e];
            } else {
                ldmatrix_x4(a, Qs + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * SD + ks * 16 + (lane >> 4) * 8);
            }
#pragma unroll
            for (int jp = 0; jp < 4; jp++) {
                uint32_t b[4];
                ldmatrix_x4(b, kt + (jp * 16 + (lane & 7) + (lane >> 4) * 8) * SD + ks * 16 + ((lane >> 3) & 1) * 8);
                mma_bf16_16816(s[jp * 2], a[0], a[1], a[2], a[3], b[0], b[1]);
                mma_bf16_16816(s[jp * 2 + 1], a[0], a[1], a[2], a[3], b[2], b[3]);
            }
        }
        // scale, mask by absolute position, running maximum
        float mx0 = m0, mx1 = m1;
#pragma unroll
        for (int j = 0; j < 8; j++) {
#pragma unroll
            for (int e = 0; e < 4; e++) {
                int key = t * 64 + j * 8 + t4 * 2 + (e & 1);
                int row = (e & 2) ? row1 : row0;
                bool ok = key <= row && (p.window <= 0 || key > row - p.window);
                float v = ok ? s[j][e] * sc : -INFINITY;
                s[j][e] = v;
                if (e & 2) mx1 = fmaxf(mx1, v); else mx0 = fmaxf(mx0, v);
            }
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float base0 = mx0 == -INFINITY ? 0.f : mx0, base1 = mx1 == -INFINITY ? 0.f : mx1;
        const float c0 = exp2f(m0 - base0), c1 = exp2f(m1 - base1);  // m = -inf gives 0
        m0 = mx0;
        m1 = mx1;
        l0 *= c0;
        l1 *= c1;
#pragma unroll
        for (int j = 0; j < NF; j++) {
            o[j][0] *= c0;
            o[j][1] *= c0;
            o[j][2] *= c1;
            o[j][3] *= c1;
        }
        uint32_t pa[4][4];
#pragma unroll
        for (int j = 0; j < 8; j++) {
            float p0 = exp2f(s[j][0] - base0), p1 = exp2f(s[j][1] - base0);
            float p2 = exp2f(s[j][2] - base1), p3 = exp2f(s[j][3] - base1);
            l0 += p0 + p1;
            l1 += p2 + p3;
            pa[j >> 1][(j & 1) * 2] = pack_bf16(p0, p1);
            pa[j >> 1][(j & 1) * 2 + 1] = pack_bf16(p2, p3);
        }
#pragma unroll
        for (int kk = 0; kk < 4; kk++) {
#pragma unroll
            for (int c = 0; c < KS; c++) {
                uint32_t b[4];
                ldmatrix_x4_trans(b, vt + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * SD + c * 16 + (lane >> 4) * 8);
                mma_bf16_16816(o[c * 2], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], b[0], b[1]);
                mma_bf16_16816(o[c * 2 + 1], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], b[2], b[3]);
            }
        }
    }
    cp_async_wait<0>();
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const int r0 = q0 + warp * 16 + g, r1 = r0 + 8;
    bf16* ob = (bf16*)p.out + (int64_t)head * HD;
    if (r0 < q_len) {
        float inv = 1.f / l0;
        bf16* op = ob + (int64_t)(q_start + r0) * p.out_row_stride;
#pragma unroll
        for (int j = 0; j < NF; j++) *reinterpret_cast<uint32_t*>(op + j * 8 + t4 * 2) = pack_bf16(o[j][0] * inv, o[j][1] * inv);
    }
    if (r1 < q_len) {
        float inv = 1.f / l1;
        bf16* op = ob + (int64_t)(q_start + r1) * p.out_row_stride;
#pragma unroll
        for (int j = 0; j < NF; j++) *reinterpret_cast<uint32_t*>(op + j * 8 + t4 * 2) = pack_bf16(o[j][2] * inv, o[j][3] * inv);
    }
}

// ------------------------------------------------------------------------------------------
constexpr int DSTAGES = 3;

// What the single-token kernel needs to do the work of the row-wise q/k norm + rotation + cache write
// kernel (elementwise.cu) itself: the queries then arrive as the q/k/v product left them, and the
// token's own key and value are not in the cache yet.
struct RopeFuse {
    int on;
    const float* q_w;   // per-head norm weights, or null
    const float* k_w;
    float eps;
    const float* cos_t;  // [table_positions][rot / 2]
    const float* sin_t;
    int rot;
    int table_positions;
    int write_kv;        // store the token's key and value in the cache planes
    int consecutive;     // head_dim 128 rotated in full: the lane layout and order of sums of the row-wise kernel's fast path
};

// One head row of HD bfloat16 in shared memory, normed (if w) and rotated in place by one warp, with
// the arithmetic and the order of sums of the row-wise kernel for the same geometry, so that a key
// written by either is the same bits.  y: HD floats of scratch for this warp.
template <int HD>
__device__ __forceinline__ void norm_rope_row(bf16* x, float* y, const float* __restrict__ w, float eps, const float* __restrict__ c,
                                              const float* __restrict__ s, int rot, int lane, bool consecutive) {
    if (HD == 128 && consecutive) {
        const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(x + lane * 4), hi = *reinterpret_cast<const __nv_bfloat162*>(x + lane * 4 + 2);
        float v[4] = {__low2float(lo), __high2float(lo), __low2float(hi), __high2float(hi)};
        if (w) {
            const float4 ww = *reinterpret_cast<const float4*>(w + lane * 4);
            float ss = warp_sum(v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3]);
            const float inv = 1.0f / sqrtf(ss / 128.f + eps);
            v[0] = v[0] * inv * ww.x;
            v[1] = v[1] * inv * ww.y;
            v[2] = v[2] * inv * ww.z;
            v[3] = v[3] * inv * ww.w;
        }
        const int ci = (lane & 15) * 4;
        const float4 c4 = *reinterpret_cast<const float4*>(c + ci), s4 = *reinterpret_cast<const float4*>(s + ci);
        const float cs[4] = {c4.x, c4.y, c4.z, c4.w}, sv[4] = {s4.x, s4.y, s4.z, s4.w};
        float o[4];
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const float partner = __shfl_xor_sync(0xffffffffu, v[e], 16);
            o[e] = lane < 16 ? v[e] * cs[e] - partner * sv[e] : v[e] * cs[e] + partner * sv[e];
        }
        *reinterpret_cast<__nv_bfloat162*>(x + lane * 4) = __floats2bfloat162_rn(o[0], o[1]);
        *reinterpret_cast<__nv_bfloat162*>(x + lane * 4 + 2) = __floats2bfloat162_rn(o[2], o[3]);
        return;
    }
    float ss = 0.f;
    for (int i = lane; i < HD; i += 32) {
        float v = __bfloat162float(x[i]);
        y[i] = v;
        ss += v * v;
    }
    float inv = 1.f;
    if (w) {
        ss = warp_sum(ss);
        inv = 1.0f / sqrtf(ss / (float)HD + eps);
    }
    __syncwarp();
    if (w)
        for (int i = lane; i < HD; i += 32) y[i] = y[i] * inv * w[i];
    __syncwarp();
    const int half = rot / 2;
    for (int i = lane; i < HD; i += 32) {
        float v;
        if (i < half)
            v = y[i] * c[i] - y[i + half] * s[i];
        else if (i < rot)
            v = y[i] * c[i - half] + y[i - half] * s[i - half];
        else
            v = y[i];
        x[i] = __float2bfloat16_rn(v);
    }
    __syncwarp();
}

template <int HD, bool QREG>
__global__ void __launch_bounds__(128) attn_decode_mma_kernel(AttnParams p, RopeFuse f) {
    constexpr int SD = HD + 8, KS = HD / 16, NF = HD / 8;
    constexpr int STAGE = 2 * 64 * SD;  // elements: keys then values
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* Qs = reinterpret_cast<bf16*>(smem_raw);     // [16][SD]
    bf16* KV = Qs + 16 * SD;                          // [DSTAGES][2][64][SD]
    float* Ys = reinterpret_cast<float*>(KV + DSTAGES * STAGE);  // [4 warps][HD]: scratch of norm_rope_row
    bf16* fresh = reinterpret_cast<bf16*>(Ys + 4 * HD);          // [2][HD]: the token's own key and value

    // Ahead of the dependency wait: the step's metadata and the pages of earlier steps, none of which
    // the kernel before this one writes (the step's metadata is uploaded before its first kernel,
    // and every kernel waits for its predecessor before it lets its successor start).  With
    // `f.on` that includes the page the token's own key will go to: only this kernel writes there.
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
    const int G = p.heads / p.kv_heads;
    const int GC = G < 16 ? G : 16;
    const int hchunks = (G + GC - 1) / GC;
    const int split = blockIdx.x, seq = blockIdx.z;
    const int kvh = blockIdx.y / hchunks, chunk = blockIdx.y % hchunks;
    const int kv_len = p.seq_kv_len[seq];
    const int q_row = p.seq_q_start[seq];
    const int pos = kv_len - 1;
    const int* bt = block_table_row(p.block_table, p.bt_stride, p.seq_slot[seq], p.max_slots);
    const bf16* kbase = (const bf16*)p.k_plane;
    const bf16* vbase = (const bf16*)p.v_plane;
    const int h0 = kvh * G + chunk * GC;            // first head of this CTA
    const int nh = (G - chunk * GC) < GC ? (G - chunk * GC) : GC;  // heads of this CTA
    int lo_pos = 0;
    if (p.window > 0) {
        lo_pos = pos - p.window + 1;
        if (lo_pos < 0) lo_pos = 0;
    }
    const int t_lo = lo_pos / 64, t_hi = pos / 64 + 1;  // [t_lo, t_hi)
    const int per = (t_hi - t_lo + p.num_splits - 1) / p.num_splits;
    const int my_lo = t_lo + split * per;
    const int my_hi = my_lo + per < t_hi ? my_lo + per : t_hi;
    const int n = my_hi > my_lo ? my_hi - my_lo : 0;

    auto load_tile = [&](int i) {
        int t = my_lo + i;
        int64_t page = page_of(bt, t * 64, p.bt_stride, p.pages);
        int64_t off = ((page * p.kv_heads + kvh) * 64) * (int64_t)HD;
        bf16* st = KV + (i % DSTAGES) * STAGE;
        load_page<HD>(st, kbase + off, tid, 128);
        load_page<HD>(st + 64 * SD, vbase + off, tid, 128);
    };
    // Without `f.on` the keys of this step were written by the kernel just ahead: nothing is fetched early.
    if (!f.on) pdl_wait();
#pragma unroll
    for (int s = 0; s < DSTAGES - 1; s++) {
        if (s < n) load_tile(s);
        cp_async_commit();
    }
    if (f.on) pdl_wait();
    pdl_trigger();  // the product that follows may start fetching its weights
    {
        constexpr int CH = HD / 8;
        const bf16* qsrc = (const bf16*)p.q + (int64_t)q_row * p.q_row_stride + (int64_t)h0 * HD;
        for (int idx = tid; idx < 16 * CH; idx += 128) {
            int row = idx / CH, c = idx - row * CH;
            bool ok = row < nh;
            cp_async16(Qs + row * SD + c * 8, ok ? qsrc + (int64_t)row * HD + c * 8 : qsrc, ok ? 16 : 0);
        }
        cp_async_commit();
    }

    // The CTA whose keys end with the token's own page has that key and value from the q/k/v product's
    // row, not from the cache: the last tile is patched in shared memory, and one CTA per kv head also
    // stores them in the cache for the steps to come.
    const bool owns_last = f.on && f.write_kv && n > 0 && my_hi == t_hi;  // a run that only reads another's cache finds the key there
    if (f.on && n > 0) {
        const int half = f.rot / 2;
        // rows whose position lies beyond the table are refused on the host
        const int tpos = (half == 0 || gb_check(pos, f.table_positions, GB_CHECK_ROPE_POSITION)) ? pos : 0;
        const float* cs = f.cos_t + (int64_t)tpos * half;
        const float* sn = f.sin_t + (int64_t)tpos * half;
        const bf16* row = (const bf16*)p.q + (int64_t)q_row * p.q_row_stride;
        if (owns_last) {
            const bf16* ksrc = row + (int64_t)(p.heads + kvh) * HD;
            const bf16* vsrc = row + (int64_t)(p.heads + p.kv_heads + kvh) * HD;
            for (int i = tid; i < 2 * HD; i += 128) fresh[i] = i < HD ? ksrc[i] : vsrc[i - HD];
        }
        cp_async_wait<0>();  // the queries have landed (the first tiles were requested before them)
        __syncthreads();
        for (int task = warp; task < nh + (owns_last ? 1 : 0); task += 4) {
            if (task < nh)
                norm_rope_row<HD>(Qs + task * SD, Ys + warp * HD, f.q_w, f.eps, cs, sn, f.rot, lane, f.consecutive != 0);
            else
                norm_rope_row<HD>(fresh, Ys + warp * HD, f.k_w, f.eps, cs, sn, f.rot, lane, f.consecutive != 0);
        }
        __syncthreads();
        if (owns_last && chunk == 0) {
            const int64_t page = page_of(bt, pos, p.bt_stride, p.pages);
            const int64_t at = ((page * p.kv_heads + kvh) * 64 + (pos & 63)) * (int64_t)HD;
            bf16* kdst = (bf16*)p.k_plane + at;
            bf16* vdst = (bf16*)p.v_plane + at;
            for (int i = tid; i < 2 * HD; i += 128) {
                if (i < HD)
                    kdst[i] = fresh[i];
                else
                    vdst[i - HD] = fresh[i];
            }
        }
    }

    const float sc = p.scale * LOG2E;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    float o[NF][4];
#pragma unroll
    for (int j = 0; j < NF; j++)
#pragma unroll
        for (int e = 0; e < 4; e++) o[j][e] = 0.f;
    uint32_t qf[QREG ? KS : 1][4];

    for (int i = 0; i < n; i++) {
        // tile i has landed; the queries, requested last, only once every group has (first iteration)
        if (i == 0)
            cp_async_wait<0>();
        else
            cp_async_wait<DSTAGES - 2>();
        __syncthreads();
        if (i + DSTAGES - 1 < n) load_tile(i + DSTAGES - 1);
        cp_async_commit();
        if (QREG && i == 0) {
#pragma unroll
            for (int ks = 0; ks < KS; ks++)
                ldmatrix_x4(qf[QREG ? ks : 0], Qs + ((lane & 7) + ((lane >> 3) & 1) * 8) * SD + ks * 16 + (lane >> 4) * 8);
        }
        if (owns_last && i == n - 1) {
            // the token's own key and value over whatever the cache held at its place
            bf16* krow = KV + (i % DSTAGES) * STAGE + (pos & 63) * SD;
            for (int idx = tid; idx < 2 * HD; idx += 128) {
                if (idx < HD)
                    krow[idx] = fresh[idx];
                else
                    krow[64 * SD + idx - HD] = fresh[idx];
            }
            __syncthreads();
        }
        const bf16* kt = KV + (i % DSTAGES) * STAGE;
        const bf16* vt = kt + 64 * SD;
        const int t = my_lo + i;
        float s[2][4];
#pragma unroll
        for (int j = 0; j < 2; j++)
#pragma unroll
            for (int e = 0; e < 4; e++) s[j][e] = 0.f;
#pragma unroll
        for (int ks = 0; ks < KS; ks++) {
            uint32_t a[4], b[4];
            if (QREG) {
#pragma unroll
                for (int e = 0; e < 4; e++) a[e] = qf[QREG ? ks : 0][e];
            } else {
                ldmatrix_x4(a, Qs + ((lane & 7) + ((lane >> 3) & 1) * 8) * SD + ks * 16 + (lane >> 4) * 8);
            }
            ldmatrix_x4(b, kt + (warp * 16 + (lane & 7) + (lane >> 4) * 8) * SD + ks * 16 + ((lane >> 3) & 1) * 8);
            mma_bf16_16816(s[0], a[0], a[1], a[2], a[3], b[0], b[1]);
            mma_bf16_16816(s[1], a[0], a[1], a[2], a[3], b[2], b[3]);
        }
        float mx0 = m0, mx1 = m1;
#pragma unroll
        for (int j = 0; j < 2; j++) {
#pragma unroll
            for (int e = 0; e < 4; e++) {
                int key = t * 64 + warp * 16 + j * 8 + t4 * 2 + (e & 1);
                bool ok = key <= pos && key >= lo_pos;
                float v = ok ? s[j][e] * sc : -INFINITY;
                s[j][e] = v;
                if (e & 2) mx1 = fmaxf(mx1, v); else mx0 = fmaxf(mx0, v);
            }
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float base0 = mx0 == -INFINITY ? 0.f : mx0, base1 = mx1 == -INFINITY ? 0.f : mx1;
        const float c0 = exp2f(m0 - base0), c1 = exp2f(m1 - base1);
        m0 = mx0;
        m1 = mx1;
        l0 *= c0;
        l1 *= c1;
#pragma unroll
        for (int j = 0; j < NF; j++) {
            o[j][0] *= c0;
            o[j][1] *= c0;
            o[j][2] *= c1;
            o[j][3] *= c1;
        }
        uint32_t pa[4];
        {
            float p00 = exp2f(s[0][0] - base0), p01 = exp2f(s[0][1] - base0), p02 = exp2f(s[0][2] - base1), p03 = exp2f(s[0][3] - base1);
            float p10 = exp2f(s[1][0] - base0), p11 = exp2f(s[1][1] - base0), p12 = exp2f(s[1][2] - base1), p13 = exp2f(s[1][3] - base1);
            l0 += p00 + p01 + p10 + p11;
            l1 += p02 + p03 + p12 + p13;
            pa[0] = pack_bf16(p00, p01);
            pa[1] = pack_bf16(p02, p03);
            pa[2] = pack_bf16(p10, p11);
            pa[3] = pack_bf16(p12, p13);
        }
#pragma unroll
        for (int c = 0; c < KS; c++) {
            uint32_t b[4];
            ldmatrix_x4_trans(b, vt + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * SD + c * 16 + (lane >> 4) * 8);
            mma_bf16_16816(o[c * 2], pa[0], pa[1], pa[2], pa[3], b[0], b[1]);
            mma_bf16_16816(o[c * 2 + 1], pa[0], pa[1], pa[2], pa[3], b[2], b[3]);
        }
    }
    cp_async_wait<0>();
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    __syncthreads();  // every warp is done with the tiles: reuse their memory for the merge

    // merge the four warps: Ms/Ls [4][16], Os [4][16][HD]
    float* Ms = reinterpret_cast<float*>(KV);
    float* Ls = Ms + 64;
    float* Os = Ls + 64;
    if (t4 == 0) {
        Ms[warp * 16 + g] = m0;
        Ms[warp * 16 + g + 8] = m1;
        Ls[warp * 16 + g] = l0;
        Ls[warp * 16 + g + 8] = l1;
    }
#pragma unroll
    for (int j = 0; j < NF; j++) {
        float* o0 = Os + ((size_t)warp * 16 + g) * HD + j * 8 + t4 * 2;
        float* o1 = Os + ((size_t)warp * 16 + g + 8) * HD + j * 8 + t4 * 2;
        o0[0] = o[j][0];
        o0[1] = o[j][1];
        o1[0] = o[j][2];
        o1[1] = o[j][3];
    }
    __syncthreads();
    for (int idx = tid; idx < nh * HD; idx += 128) {
        int r = idx / HD, c = idx - r * HD;
        float M = fmaxf(fmaxf(Ms[r], Ms[16 + r]), fmaxf(Ms[32 + r], Ms[48 + r]));
        float L = 0.f, acc = 0.f;
        if (M != -INFINITY) {
#pragma unroll
            for (int w = 0; w < 4; w++) {
                float f = exp2f(Ms[w * 16 + r] - M);
                L += f * Ls[w * 16 + r];
                acc += f * Os[((size_t)w * 16 + r) * HD + c];
            }
        }
        int head = h0 + r;
        if (p.num_splits == 1) {
            ((bf16*)p.out)[(int64_t)q_row * p.out_row_stride + (int64_t)head * HD + c] = __float2bfloat16_rn(acc / L);
        } else {
            float* sp = p.scratch + (((int64_t)seq * p.heads + head) * p.num_splits + split) * (HD + 2);
            if (c == 0) {
                sp[0] = M == -INFINITY ? -INFINITY : M * LN2;  // natural-log units, as the merge kernel expects
                sp[1] = L;
            }
            sp[2 + c] = acc;
        }
    }
}

template <int HD>
int launch_prefill(const AttnParams& p, cudaStream_t stream) {
    constexpr bool QREG = HD <= 128;
    constexpr int SD = HD + 8;
    const int smem = 5 * 64 * SD * 2;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_prefill_mma_kernel<HD, QREG>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) GB_REFUSE("attention_prefill_mma: cannot reserve %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
        configured = true;
    }
    dim3 grid(ceil_div(p.max_q_len, 64), p.heads, p.nseq);
    if (grid.y > 65535 || grid.z > 65535) GB_REFUSE("attention_prefill_mma: grid (%u, %u, %u) exceeds one launch", grid.x, grid.y, grid.z);
    attn_prefill_mma_kernel<HD, QREG><<<grid, 128, smem, stream>>>(p);
    GB_CHECK_LAUNCH("attention_prefill_mma");
    return 0;
}

template <int HD>
int launch_decode(const AttnParams& p, const RopeFuse& f, cudaStream_t stream) {
    constexpr bool QREG = HD <= 128;
    constexpr int SD = HD + 8;
    int smem = (16 * SD + DSTAGES * 2 * 64 * SD) * 2 + 4 * HD * 4 + 2 * HD * 2;
    const int merge = (128 + 64 * HD) * 4 + 16 * SD * 2;
    if (merge > smem) smem = merge;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_decode_mma_kernel<HD, QREG>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) GB_REFUSE("attention_decode_mma: cannot reserve %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
        configured = true;
    }
    const int G = p.heads / p.kv_heads;
    const int GC = G < 16 ? G : 16;
    const int hchunks = (G + GC - 1) / GC;
    dim3 grid(p.num_splits, p.kv_heads * hchunks, p.nseq);
    if (grid.y > 65535 || grid.z > 65535) GB_REFUSE("attention_decode_mma: grid (%u, %u, %u) exceeds one launch", grid.x, grid.y, grid.z);
    // Measured at 1 to 64 sequences of 4096 keys: launched early, this kernel gains a little when it
    // is alone (one split, many CTAs) and loses when its CTAs and those of the merge behind it sit
    // waiting beside the kernels ahead (also when it fetches its first pages while it waits), so only
    // the single-split form is a dependent launch.
    if (p.num_splits == 1)
        launch_pdl(attn_decode_mma_kernel<HD, QREG>, grid, dim3(128), (size_t)smem, stream, p, f);
    else
        attn_decode_mma_kernel<HD, QREG><<<grid, 128, smem, stream>>>(p, f);
    GB_CHECK_LAUNCH("attention_decode_mma");
    if (p.num_splits > 1)
        return gb_attention_merge_launch(p.scratch, p.out, GB_BF16, p.out_row_stride, p.seq_q_start, p.nseq, p.heads, p.d,
                                         p.num_splits, stream);
    return 0;
}

int check(const AttnParams& p, const char* who) {
    if (p.heads <= 0 || p.kv_heads <= 0 || p.heads % p.kv_heads) GB_REFUSE("%s: %d heads over %d kv heads", who, p.heads, p.kv_heads);
    if (p.d % 16 || p.d < 16 || (p.d > 128 && p.d != 256))
        GB_REFUSE("%s: head_dim %d is not one of 16, 32, ..., 128, 256 (other sizes up to 256 run on the CUDA-core kernel)", who, p.d);
    if (p.window < 0) GB_REFUSE("%s: window %d", who, p.window);
    if (((uintptr_t)p.q & 15) || (p.q_row_stride & 7)) GB_REFUSE("%s: query rows must be 16-byte aligned", who);
    if ((p.out_row_stride & 1) || ((uintptr_t)p.out & 3)) GB_REFUSE("%s: output rows must be 4-byte aligned", who);
    return 0;
}

}  // namespace

#define GB_DISPATCH_HD(fn, ...)                            \
    switch (p.d) {                                         \
        case 16: return fn<16>(p, ##__VA_ARGS__, stream);  \
        case 32: return fn<32>(p, ##__VA_ARGS__, stream);  \
        case 48: return fn<48>(p, ##__VA_ARGS__, stream);  \
        case 64: return fn<64>(p, ##__VA_ARGS__, stream);  \
        case 80: return fn<80>(p, ##__VA_ARGS__, stream);  \
        case 96: return fn<96>(p, ##__VA_ARGS__, stream);  \
        case 112: return fn<112>(p, ##__VA_ARGS__, stream); \
        case 128: return fn<128>(p, ##__VA_ARGS__, stream); \
        case 256: return fn<256>(p, ##__VA_ARGS__, stream); \
    }

GB_API int gb_attention_prefill_mma(const AttnParams* pp, cudaStream_t stream) {
    AttnParams p = *pp;
    if (p.nseq <= 0 || p.max_q_len <= 0) return 0;
    if (int rc = check(p, "attention_prefill_mma")) return rc;
    if (p.num_splits != 1) GB_REFUSE("attention_prefill_mma: key splits are for single-token rows");
    GB_DISPATCH_HD(launch_prefill)
    GB_REFUSE("attention_prefill_mma: head_dim %d", p.d);
}

GB_API int gb_attention_decode_mma(const AttnParams* pp, cudaStream_t stream) {
    AttnParams p = *pp;
    if (p.nseq <= 0) return 0;
    if (int rc = check(p, "attention_decode_mma")) return rc;
    if (p.max_q_len != 1) GB_REFUSE("attention_decode_mma: rows of up to %d tokens; this kernel takes single tokens", p.max_q_len);
    if (p.num_splits < 1) GB_REFUSE("attention_decode_mma: %d key splits", p.num_splits);
    if (p.num_splits > 1 && !p.scratch) GB_REFUSE("attention_decode_mma: %d key splits without scratch memory", p.num_splits);
    const RopeFuse off = {};
    GB_DISPATCH_HD(launch_decode, off)
    GB_REFUSE("attention_decode_mma: head_dim %d", p.d);
}

// Whether the single-token kernel can do the q/k norm, the rotation and the cache write of these rows
// itself (bfloat16, a head size it takes, one row a sequence).
GB_API int gb_attention_decode_rope_accepts(int dtype, int d, int rot, int max_q_len) {
    return dtype == GB_BF16 && max_q_len == 1 && !(d & 15) && (d <= 128 || d == 256) && rot >= 0 && rot <= d && !(rot & 1);
}

// Single-token attention on rows as the q/k/v product left them: `a` describes the attention call
// (a->q the rows of the fused q|k|v buffer), `r` what gb_qk_norm_rope_kv_write would have been given
// for the same rows.  Each CTA norms and rotates the queries of its heads; the CTA that reads a
// sequence's last page takes the token's own key and value from the row, and one CTA per kv head
// stores them in the cache.  The same bits as the two kernels one after the other.
GB_API int gb_attention_decode_mma_rope(const AttnParams* pp, const QkRopeParams* rp, cudaStream_t stream) {
    AttnParams p = *pp;
    const QkRopeParams& r = *rp;
    if (p.nseq <= 0) return 0;
    const char* who = "attention_decode_mma_rope";
    if (int rc = check(p, who)) return rc;
    if (p.max_q_len != 1) GB_REFUSE("%s: rows of up to %d tokens; this kernel takes single tokens", who, p.max_q_len);
    if (p.num_splits < 1) GB_REFUSE("%s: %d key splits", who, p.num_splits);
    if (p.num_splits > 1 && !p.scratch) GB_REFUSE("%s: %d key splits without scratch memory", who, p.num_splits);
    if (r.qkv != p.q || r.row_stride != p.q_row_stride || r.heads != p.heads || r.kv_heads != p.kv_heads || r.d != p.d ||
        r.rows != p.nseq || r.block_table != p.block_table || r.bt_stride != p.bt_stride)
        GB_REFUSE("%s: the two descriptions are not of the same rows", who);
    if (r.write_kv && (r.k_plane != p.k_plane || r.v_plane != p.v_plane)) GB_REFUSE("%s: keys would be written to another plane than is read", who);
    if (!gb_attention_decode_rope_accepts(GB_BF16, p.d, r.rot, p.max_q_len)) GB_REFUSE("%s: head_dim %d, rotary width %d", who, p.d, r.rot);
    if (r.rot > 0 && (!r.cos_t || !r.sin_t)) GB_REFUSE("%s: rotary width %d without an angle table", who, r.rot);
    RopeFuse f = {};
    f.on = 1;
    f.q_w = r.q_w;
    f.k_w = r.k_w;
    f.eps = r.eps;
    f.cos_t = r.cos_t;
    f.sin_t = r.sin_t;
    f.rot = r.rot;
    f.table_positions = r.table_positions;
    f.write_kv = r.write_kv;
    // the row-wise kernel's own condition for its fast path (elementwise.cu)
    f.consecutive = p.d == 128 && r.rot == 128 && !(r.row_stride & 3) && !((uintptr_t)r.qkv & 7) &&
                    !(((uintptr_t)r.q_w | (uintptr_t)r.k_w | (uintptr_t)r.cos_t | (uintptr_t)r.sin_t) & 15) && (r.q_w != nullptr) == (r.k_w != nullptr);
    GB_DISPATCH_HD(launch_decode, f)
    GB_REFUSE("%s: head_dim %d", who, p.d);
}

// the checked build's record of the first index this file's kernels found out of bounds
GB_CHECK_READER(gb_checked_status_attention_mma)
