// Row-wise kernels: embedding gather, residual add + RMSNorm, SwiGLU, and the fused
// per-head norm + rotary embedding + cache write.  All arithmetic is fp32; only storage varies.
#include "common.cuh"
#include "api.h"

#include <stdarg.h>
#include <stdio.h>

// ------------------------------------------------------------------------------------------
// error text
static thread_local char g_error[512];

void gb_set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

GB_API const char* gb_last_error() { return g_error; }

GB_API int gb_abi_version() { return 2; }

// 1 if the library was built with bounds-checked indices (see common.cuh)
GB_API int gb_is_checked() {
#ifdef GB_CHECKED
    return 1;
#else
    return 0;
#endif
}

// ------------------------------------------------------------------------------------------
// embedding: h[r, :] = float(table[ids[r], :])      (internal/qwen3lm/evaluator.go:594-599)
// With `stats`, the sum of squares of each row is left in stats[row * stats_stride] (one partial sum
// a row, taken in a fixed order), and with `next_w` also xn_out[row] = bf16(row * next_w): the first
// norm's output but for the row factor, for a product that applies that factor itself.
template <typename T>
__global__ void embed_gather_kernel(const T* __restrict__ table, const int* __restrict__ ids, int hidden,
                                    int vocab, float* __restrict__ out, float* __restrict__ stats, int64_t stats_stride,
                                    const float* __restrict__ next_w, __nv_bfloat16* __restrict__ xn_out, int64_t ldxn) {
    __shared__ float warp_part[8];
    int r = blockIdx.x;
    int id = ids[r];
    // ids are validated on the host; an id outside the table reads row 0 rather than faulting.
    if (!gb_check(id, vocab, GB_CHECK_TOKEN_ID) || id < 0 || id >= vocab) id = 0;
    const T* src = table + (int64_t)id * hidden;
    float* dst = out + (int64_t)r * hidden;
    float ss = 0.f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float v = to_f32<T>(src[i]);
        dst[i] = v;
        ss += v * v;
        if (next_w != nullptr) xn_out[(int64_t)r * ldxn + i] = __float2bfloat16_rn(v * next_w[i]);
    }
    if (stats == nullptr) return;
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) warp_part[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.f;
#pragma unroll
        for (int i = 0; i < 8; i++) t += warp_part[i];
        stats[(int64_t)r * stats_stride] = t;
    }
}

GB_API int gb_embed_gather(const void* table, int table_dtype, const int* ids, int rows, int hidden, int vocab,
                           float* out, float* stats, int64_t stats_stride, const float* next_w, void* xn_out, int64_t ldxn,
                           cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (hidden <= 0 || vocab <= 0) GB_REFUSE("embed_gather: hidden %d, vocab %d", hidden, vocab);
    if (next_w && (!xn_out || ldxn < hidden)) GB_REFUSE("embed_gather: a norm weight is given without room for its %d-wide rows", hidden);
    if (table_dtype == GB_F32)
        embed_gather_kernel<float><<<rows, 256, 0, stream>>>((const float*)table, ids, hidden, vocab, out, stats, stats_stride, next_w,
                                                             (__nv_bfloat16*)xn_out, ldxn);
    else if (table_dtype == GB_BF16)
        embed_gather_kernel<__nv_bfloat16><<<rows, 256, 0, stream>>>((const __nv_bfloat16*)table, ids, hidden, vocab, out, stats, stats_stride,
                                                                     next_w, (__nv_bfloat16*)xn_out, ldxn);
    else
        GB_REFUSE("embed_gather: unknown table dtype %d", table_dtype);
    GB_CHECK_LAUNCH("embed_gather");
    return 0;
}

// ids[i] = source[ids[i]]: a step whose tokens are the ones the sampler just left on the device takes
// them by position, so the host need not have read them.  A position outside the source gives 0.
__global__ void gather_tokens_kernel(int* __restrict__ ids, const int* __restrict__ source, int n, int source_n) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    int p = ids[i];
    gb_check(p, source_n, GB_CHECK_TOKEN_SOURCE);
    ids[i] = (p >= 0 && p < source_n) ? source[p] : 0;
}

GB_API int gb_gather_tokens(int* ids, const int* source, int n, int source_n, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (source_n <= 0) GB_REFUSE("gather_tokens: empty source");
    gather_tokens_kernel<<<ceil_div(n, 128), 128, 0, stream>>>(ids, source, n, source_n);
    GB_CHECK_LAUNCH("gather_tokens");
    return 0;
}

// ------------------------------------------------------------------------------------------
// residual add + RMSNorm                     (internal/qwen3lm/ops.go:94-108, 251-254)
//   v = h[row] (+ delta[row]);  if the rows are not gathered, h[row] = v
//   out[i] = v * (1 / sqrt(mean(v^2) + eps)) * w
// One CTA of 256 threads per row; the sum of squares is taken in a fixed order (strided partial
// sums, shuffle tree, then the 8 warp sums in order), so a row's result does not depend on what
// else is in the batch.
template <typename TO>
__global__ void add_rmsnorm_kernel(float* __restrict__ h, const float* __restrict__ delta,
                                   const float* __restrict__ w, float eps, int n, TO* __restrict__ out,
                                   const int* __restrict__ row_index) {
    __shared__ float warp_part[8];
    __shared__ float inv_s;
    int orow = blockIdx.x;
    int row = row_index ? row_index[orow] : orow;
    float* hr = h + (int64_t)row * n;
    const float* dr = delta ? delta + (int64_t)row * n : nullptr;
    bool write_back = (row_index == nullptr) && (delta != nullptr);
    float ss = 0.f;
    for (int i = threadIdx.x; i < n; i += 256) {
        float v = hr[i];
        if (dr) v += dr[i];
        if (write_back) hr[i] = v;
        ss += v * v;
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) warp_part[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.f;
#pragma unroll
        for (int i = 0; i < 8; i++) t += warp_part[i];
        inv_s = 1.0f / sqrtf(t / (float)n + eps);
    }
    __syncthreads();
    float inv = inv_s;
    TO* orow_p = out + (int64_t)orow * n;
    for (int i = threadIdx.x; i < n; i += 256) {
        float v = hr[i];
        if (dr && !write_back) v += dr[i];
        orow_p[i] = from_f32<TO>(v * inv * w[i]);
    }
}

// The same operation for rows whose width is a multiple of 4 and at most THREADS * 16: every
// thread keeps its (up to four) float4 pieces of the row in registers, so the row is read once.
template <typename TO, int THREADS>
__global__ void __launch_bounds__(THREADS) add_rmsnorm_vec_kernel(float* __restrict__ h, const float* __restrict__ delta,
                                                                  const float* __restrict__ w, float eps, int n, TO* __restrict__ out,
                                                                  const int* __restrict__ row_index) {
    __shared__ float warp_part[THREADS / 32];
    __shared__ float inv_s;
    pdl_wait();
    pdl_trigger();  // the product that follows may start fetching its weights
    const int orow = blockIdx.x;
    const int row = row_index ? row_index[orow] : orow;
    float4* hr = reinterpret_cast<float4*>(h + (int64_t)row * n);
    const float4* dr = delta ? reinterpret_cast<const float4*>(delta + (int64_t)row * n) : nullptr;
    const bool write_back = (row_index == nullptr) && (delta != nullptr);
    const int n4 = n >> 2;
    float4 v[4];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        int c = threadIdx.x + i * THREADS;
        if (c < n4) {
            v[i] = hr[c];
            if (dr) {
                float4 d = dr[c];
                v[i].x += d.x;
                v[i].y += d.y;
                v[i].z += d.z;
                v[i].w += d.w;
            }
            ss += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
        }
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) warp_part[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.f;
#pragma unroll
        for (int i = 0; i < THREADS / 32; i++) t += warp_part[i];
        inv_s = 1.0f / sqrtf(t / (float)n + eps);
    }
    __syncthreads();
    const float inv = inv_s;
    const float4* w4 = reinterpret_cast<const float4*>(w);
    TO* orow_p = out + (int64_t)orow * n;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        int c = threadIdx.x + i * THREADS;
        if (c < n4) {
            if (write_back) hr[c] = v[i];
            float4 ww = w4[c];
            float a = v[i].x * inv * ww.x, b = v[i].y * inv * ww.y, cc = v[i].z * inv * ww.z, d = v[i].w * inv * ww.w;
            if (sizeof(TO) == 4) {
                reinterpret_cast<float4*>(orow_p)[c] = make_float4(a, b, cc, d);
            } else {
                __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(cc, d);
                uint2 pk;
                pk.x = *reinterpret_cast<uint32_t*>(&lo);
                pk.y = *reinterpret_cast<uint32_t*>(&hi);
                reinterpret_cast<uint2*>(orow_p)[c] = pk;
            }
        }
    }
}

GB_API int gb_add_rmsnorm(float* h, const float* delta, const float* w, float eps, int n, void* out, int out_dtype,
                          const int* row_index, int out_rows, cudaStream_t stream) {
    if (out_rows <= 0) return 0;
    if (n <= 0) GB_REFUSE("add_rmsnorm: width %d", n);
    if (out_dtype != GB_F32 && out_dtype != GB_BF16) GB_REFUSE("add_rmsnorm: unknown output dtype %d", out_dtype);
    const bool aligned = !(((uintptr_t)h | (uintptr_t)delta | (uintptr_t)w | (uintptr_t)out) & 15);
    if ((n & 3) == 0 && n <= 1024 * 16 && aligned) {
        if (n <= 256 * 16) {
            if (out_dtype == GB_F32)
                launch_pdl(add_rmsnorm_vec_kernel<float, 256>, dim3(out_rows), dim3(256), 0, stream, h, delta, w, eps, n, (float*)out, row_index);
            else
                launch_pdl(add_rmsnorm_vec_kernel<__nv_bfloat16, 256>, dim3(out_rows), dim3(256), 0, stream, h, delta, w, eps, n, (__nv_bfloat16*)out, row_index);
        } else {
            if (out_dtype == GB_F32)
                launch_pdl(add_rmsnorm_vec_kernel<float, 1024>, dim3(out_rows), dim3(1024), 0, stream, h, delta, w, eps, n, (float*)out, row_index);
            else
                launch_pdl(add_rmsnorm_vec_kernel<__nv_bfloat16, 1024>, dim3(out_rows), dim3(1024), 0, stream, h, delta, w, eps, n, (__nv_bfloat16*)out, row_index);
        }
        GB_CHECK_LAUNCH("add_rmsnorm");
        return 0;
    }
    if (out_dtype == GB_F32)
        add_rmsnorm_kernel<float><<<out_rows, 256, 0, stream>>>(h, delta, w, eps, n, (float*)out, row_index);
    else if (out_dtype == GB_BF16)
        add_rmsnorm_kernel<__nv_bfloat16><<<out_rows, 256, 0, stream>>>(h, delta, w, eps, n, (__nv_bfloat16*)out, row_index);
    else
        GB_REFUSE("add_rmsnorm: unknown output dtype %d", out_dtype);
    GB_CHECK_LAUNCH("add_rmsnorm");
    return 0;
}

// h[row] += delta[row] for all rows (the residual add after the last layer when nothing is normed).
__global__ void add_rows_kernel(float* __restrict__ h, const float* __restrict__ delta, int64_t total) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < total) h[i] += delta[i];
}

GB_API int gb_add_rows(float* h, const float* delta, int rows, int n, cudaStream_t stream) {
    int64_t total = (int64_t)rows * n;
    if (total <= 0) return 0;
    int64_t blocks = (total + 255) / 256;
    if (blocks > 0x7fffffff) GB_REFUSE("add_rows: %lld elements are too many for one launch", (long long)total);
    add_rows_kernel<<<(unsigned)blocks, 256, 0, stream>>>(h, delta, total);
    GB_CHECK_LAUNCH("add_rows");
    return 0;
}

// ------------------------------------------------------------------------------------------
// SwiGLU: out[r, i] = silu(gu[r, i]) * gu[r, inter + i]      (internal/qwen3lm/ops.go:442-461)
// silu is evaluated with the exponential of a non-positive argument on both branches.
__device__ __forceinline__ float silu_f32(float x) {
    if (x >= 0.f) return x / (1.f + expf(-x));
    float e = expf(x);
    return x * e / (1.f + e);
}

// interleave8 = 0: gate in columns [0, I), up in [I, 2I).  interleave8 = 1: blocks of sixteen
// columns, eight gate columns followed by the eight up columns of the same outputs.
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, int inter, int64_t gu_stride, int interleave8) {
    int r = blockIdx.y;
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= inter) return;
    const T* g = gu + (int64_t)r * gu_stride;
    int gi = interleave8 ? ((i >> 3) << 4) + (i & 7) : i;
    int ui = interleave8 ? gi + 8 : inter + i;
    float a = to_f32<T>(g[gi]);
    float b = to_f32<T>(g[ui]);
    out[(int64_t)r * inter + i] = from_f32<T>(silu_f32(a) * b);
}

// bfloat16, width a multiple of 8: eight outputs a thread, 16-byte loads and stores
__global__ void swiglu_bf16x8_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out, int inter,
                                     int interleave8) {
    const int r = blockIdx.y;
    const int i = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (i >= inter) return;
    const __nv_bfloat16* g = gu + (int64_t)r * 2 * inter;
    const int gi = interleave8 ? i * 2 : i, ui = interleave8 ? i * 2 + 8 : inter + i;
    const uint4 a = *reinterpret_cast<const uint4*>(g + gi), b = *reinterpret_cast<const uint4*>(g + ui);
    const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&a);
    const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&b);
    uint4 o;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int j = 0; j < 4; j++)
        o2[j] = __floats2bfloat162_rn(silu_f32(__low2float(a2[j])) * __low2float(b2[j]), silu_f32(__high2float(a2[j])) * __high2float(b2[j]));
    *reinterpret_cast<uint4*>(out + (int64_t)r * inter + i) = o;
}

GB_API int gb_swiglu(const void* gu, void* out, int dtype, int rows, int inter, int interleave8, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (inter <= 0) GB_REFUSE("swiglu: width %d", inter);
    if (interleave8 && (inter & 7)) GB_REFUSE("swiglu: interleaved columns need a width that is a multiple of 8, got %d", inter);
    if (rows > 65535) GB_REFUSE("swiglu: %d rows exceed one launch (65535); the step splits larger batches", rows);
    if (dtype == GB_BF16 && (inter & 7) == 0 && !(((uintptr_t)gu | (uintptr_t)out) & 15)) {
        swiglu_bf16x8_kernel<<<dim3(ceil_div(inter / 8, 128), rows), 128, 0, stream>>>((const __nv_bfloat16*)gu, (__nv_bfloat16*)out, inter,
                                                                                     interleave8);
        GB_CHECK_LAUNCH("swiglu");
        return 0;
    }
    dim3 grid(ceil_div(inter, 256), rows);
    if (dtype == GB_F32)
        swiglu_kernel<float><<<grid, 256, 0, stream>>>((const float*)gu, (float*)out, inter, 2 * (int64_t)inter, interleave8);
    else if (dtype == GB_BF16)
        swiglu_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)gu, (__nv_bfloat16*)out, inter,
                                                               2 * (int64_t)inter, interleave8);
    else
        GB_REFUSE("swiglu: unknown dtype %d", dtype);
    GB_CHECK_LAUNCH("swiglu");
    return 0;
}

// ------------------------------------------------------------------------------------------
// per-head RMSNorm + rotate-half RoPE + cache write
//                                  (internal/qwen3lm/ops.go:231-248, kernels_scalar.go:73-80)
// qkv is [rows, (heads + 2 kv_heads) * d]: q heads, then k heads, then v heads.
//   q heads: normed (if q_w) and rotated in place;
//   k heads: normed (if k_w), rotated, stored at the row's position in the key plane;
//   v heads: stored as they are in the value plane.
// One warp per (row, head).  The angle table holds cos/sin of pos * theta^(-2i/rot) computed in
// float64 on the host and rounded to fp32 (internal/qwen3lm/evaluator.go:847-858).

template <typename T>
__global__ void qk_rope_kernel(QkRopeParams p) {
    extern __shared__ float sh[];  // [4 warps][d]
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int r = blockIdx.x;
    int head = blockIdx.y * 4 + warp;
    int total_heads = p.heads + 2 * p.kv_heads;
    if (head >= total_heads) return;
    int d = p.d;
    T* src = (T*)p.qkv + (int64_t)r * p.row_stride + (int64_t)head * d;
    int pos = p.row_pos[r];
    bool is_q = head < p.heads;
    bool is_k = !is_q && head < p.heads + p.kv_heads;
    int kvh = is_q ? 0 : (is_k ? head - p.heads : head - p.heads - p.kv_heads);

    T* dst = nullptr;
    if (is_q) {
        dst = src;
    } else {
        if (!p.write_kv) return;
        int slot = p.seq_slot[p.row_seq[r]];
        int64_t page = page_of(block_table_row(p.block_table, p.bt_stride, slot, p.max_slots), pos, p.bt_stride, p.pages);
        T* plane = (T*)(is_k ? p.k_plane : p.v_plane);
        dst = plane + ((page * p.kv_heads + kvh) * GB_PAGE + (pos % GB_PAGE)) * (int64_t)d;
    }
    if (!is_q && !is_k) {  // value head: copy
        for (int i = lane; i < d; i += 32) dst[i] = src[i];
        return;
    }
    const float* w = is_q ? p.q_w : p.k_w;
    float* y = sh + warp * d;
    float ss = 0.f;
    for (int i = lane; i < d; i += 32) {
        float v = to_f32<T>(src[i]);
        y[i] = v;
        ss += v * v;
    }
    float inv = 1.f;
    if (w) {
        ss = warp_sum(ss);
        inv = 1.0f / sqrtf(ss / (float)d + p.eps);
    }
    __syncwarp();
    if (w)
        for (int i = lane; i < d; i += 32) y[i] = y[i] * inv * w[i];
    __syncwarp();
    int half = p.rot / 2;
    // rows whose position lies beyond the table are refused on the host
    const int tpos = (half == 0 || gb_check(pos, p.table_positions, GB_CHECK_ROPE_POSITION)) ? pos : 0;
    const float* c = p.cos_t + (int64_t)tpos * half;
    const float* s = p.sin_t + (int64_t)tpos * half;
    for (int i = lane; i < d; i += 32) {
        float v;
        if (i < half)
            v = y[i] * c[i] - y[i + half] * s[i];
        else if (i < p.rot)
            v = y[i] * c[i - half] + y[i - half] * s[i - half];
        else
            v = y[i];
        dst[i] = from_f32<T>(v);
    }
}

// The common geometry (bfloat16, head_dim 128 rotated in full): a warp per head and ROPE_ROWS
// consecutive rows, every lane holds four consecutive elements of each row, so element i and its
// partner i + 64 sit in lanes l and l ^ 16.  All loads of the warp's rows (positions, elements,
// angles, page numbers) are issued before anything is computed: a row is only 256 bytes per head,
// and it takes several in flight per thread to keep the memory system busy.
constexpr int ROPE_ROWS = 4;

__global__ void __launch_bounds__(256) qk_rope_bf16_d128_kernel(QkRopeParams p) {
    pdl_wait();
    pdl_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r0 = blockIdx.x * ROPE_ROWS;
    const int head = blockIdx.y * 8 + warp;
    const int total_heads = p.heads + 2 * p.kv_heads;
    if (head >= total_heads) return;
    typedef __nv_bfloat16 bf;
    const bool is_q = head < p.heads;
    const bool is_k = !is_q && head < p.heads + p.kv_heads;
    if (!is_q && !p.write_kv) return;
    const int kvh = is_q ? 0 : (is_k ? head - p.heads : head - p.heads - p.kv_heads);
    const float* w = is_q ? p.q_w : p.k_w;
    const int ci = (lane & 15) * 4;  // index into the 64 angles of a position

    int pos[ROPE_ROWS];
    uint2 raw[ROPE_ROWS];
    bf* dst[ROPE_ROWS];
    float4 c[ROPE_ROWS], sn[ROPE_ROWS];
#pragma unroll
    for (int j = 0; j < ROPE_ROWS; j++) {
        const int r = r0 + j < p.rows ? r0 + j : p.rows - 1;  // rows past the end repeat the last one and are not stored
        pos[j] = p.row_pos[r];
        bf* src = (bf*)p.qkv + (int64_t)r * p.row_stride + (int64_t)head * 128 + lane * 4;
        raw[j] = *reinterpret_cast<const uint2*>(src);
        dst[j] = src;
    }
    if (!is_q) {
        int slot[ROPE_ROWS];
#pragma unroll
        for (int j = 0; j < ROPE_ROWS; j++) {
            const int r = r0 + j < p.rows ? r0 + j : p.rows - 1;
            slot[j] = p.seq_slot[p.row_seq[r]];
        }
#pragma unroll
        for (int j = 0; j < ROPE_ROWS; j++) {
            const int64_t page = page_of(block_table_row(p.block_table, p.bt_stride, slot[j], p.max_slots), pos[j], p.bt_stride, p.pages);
            bf* plane = (bf*)(is_k ? p.k_plane : p.v_plane);
            dst[j] = plane + ((page * p.kv_heads + kvh) * GB_PAGE + (pos[j] % GB_PAGE)) * (int64_t)128 + lane * 4;
        }
    }
    if (!is_q && !is_k) {
#pragma unroll
        for (int j = 0; j < ROPE_ROWS; j++)
            if (r0 + j < p.rows) *reinterpret_cast<uint2*>(dst[j]) = raw[j];
        return;
    }
#pragma unroll
    for (int j = 0; j < ROPE_ROWS; j++) {
        const int tpos = gb_check(pos[j], p.table_positions, GB_CHECK_ROPE_POSITION) ? pos[j] : 0;
        c[j] = *reinterpret_cast<const float4*>(p.cos_t + (int64_t)tpos * 64 + ci);
        sn[j] = *reinterpret_cast<const float4*>(p.sin_t + (int64_t)tpos * 64 + ci);
    }
    float4 ww = make_float4(1.f, 1.f, 1.f, 1.f);
    if (w) ww = *reinterpret_cast<const float4*>(w + lane * 4);
#pragma unroll
    for (int j = 0; j < ROPE_ROWS; j++) {
        const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&raw[j].x), hi = *reinterpret_cast<const __nv_bfloat162*>(&raw[j].y);
        float y[4] = {__low2float(lo), __high2float(lo), __low2float(hi), __high2float(hi)};
        if (w) {
            float ss = warp_sum(y[0] * y[0] + y[1] * y[1] + y[2] * y[2] + y[3] * y[3]);
            const float inv = 1.0f / sqrtf(ss / 128.f + p.eps);
            y[0] = y[0] * inv * ww.x;
            y[1] = y[1] * inv * ww.y;
            y[2] = y[2] * inv * ww.z;
            y[3] = y[3] * inv * ww.w;
        }
        const float cs[4] = {c[j].x, c[j].y, c[j].z, c[j].w}, sv[4] = {sn[j].x, sn[j].y, sn[j].z, sn[j].w};
        float o[4];
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const float partner = __shfl_xor_sync(0xffffffffu, y[e], 16);
            o[e] = lane < 16 ? y[e] * cs[e] - partner * sv[e] : y[e] * cs[e] + partner * sv[e];
        }
        const __nv_bfloat162 o0 = __floats2bfloat162_rn(o[0], o[1]), o1 = __floats2bfloat162_rn(o[2], o[3]);
        uint2 out;
        out.x = *reinterpret_cast<const uint32_t*>(&o0);
        out.y = *reinterpret_cast<const uint32_t*>(&o1);
        if (r0 + j < p.rows) *reinterpret_cast<uint2*>(dst[j]) = out;
    }
}

// The same geometry for prompts (many rows): half a warp per head and row, a lane holds eight
// consecutive elements (16-byte loads and stores), element i and its partner i + 64 sit in lanes l
// and l ^ 8 of the half.  Fewer instructions per element than the kernel above, which is bound by its
// instruction stream once there are rows enough to fill the GPU (2048 rows of 48 heads: 18.4 -> 15.0
// us; with several heads of a row per half warp, to load the row's angles once, 16.2).  A warp takes
// two heads of WIDE_ROWS consecutive rows.
constexpr int WIDE_ROWS = 4;

__global__ void __launch_bounds__(256) qk_rope_bf16_d128_wide_kernel(QkRopeParams p) {
    pdl_wait();
    pdl_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, l16 = lane & 15;
    const int r0 = blockIdx.x * WIDE_ROWS;
    const int total_heads = p.heads + 2 * p.kv_heads;
    int head = (blockIdx.y * 8 + warp) * 2 + (lane >> 4);
    const bool live = head < total_heads;  // a dead half takes part in the shuffles and stores nothing
    if (!live) head = total_heads - 1;
    typedef __nv_bfloat16 bf;
    const bool is_q = head < p.heads;
    const bool is_k = !is_q && head < p.heads + p.kv_heads;
    const bool stores = live && (is_q || p.write_kv);
    const int kvh = is_q ? 0 : (is_k ? head - p.heads : head - p.heads - p.kv_heads);
    const float* w = is_q ? p.q_w : p.k_w;
    const int ci = (l16 & 7) * 8;  // index into the 64 angles of a position

    int pos[WIDE_ROWS];
    uint4 raw[WIDE_ROWS];
    bf* dst[WIDE_ROWS];
#pragma unroll
    for (int j = 0; j < WIDE_ROWS; j++) {
        const int r = r0 + j < p.rows ? r0 + j : p.rows - 1;  // rows past the end repeat the last one and are not stored
        pos[j] = p.row_pos[r];
        bf* src = (bf*)p.qkv + (int64_t)r * p.row_stride + (int64_t)head * 128 + l16 * 8;
        raw[j] = *reinterpret_cast<const uint4*>(src);
        dst[j] = src;
    }
    if (!is_q) {
#pragma unroll
        for (int j = 0; j < WIDE_ROWS; j++) {
            const int r = r0 + j < p.rows ? r0 + j : p.rows - 1;
            const int slot = p.seq_slot[p.row_seq[r]];
            const int64_t page = page_of(block_table_row(p.block_table, p.bt_stride, slot, p.max_slots), pos[j], p.bt_stride, p.pages);
            bf* plane = (bf*)(is_k ? p.k_plane : p.v_plane);
            dst[j] = plane + ((page * p.kv_heads + kvh) * GB_PAGE + (pos[j] % GB_PAGE)) * (int64_t)128 + l16 * 8;
        }
    }
    const bool value = !is_q && !is_k;
    const bool normed = w != nullptr && !value;
    float ww[8];
#pragma unroll
    for (int e = 0; e < 8; e++) ww[e] = 1.f;
    if (normed) {
        const float4 a = *reinterpret_cast<const float4*>(w + l16 * 8), b = *reinterpret_cast<const float4*>(w + l16 * 8 + 4);
        ww[0] = a.x; ww[1] = a.y; ww[2] = a.z; ww[3] = a.w; ww[4] = b.x; ww[5] = b.y; ww[6] = b.z; ww[7] = b.w;
    }
#pragma unroll
    for (int j = 0; j < WIDE_ROWS; j++) {
        const uint32_t in[4] = {raw[j].x, raw[j].y, raw[j].z, raw[j].w};
        float y[8];
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const __nv_bfloat162 h2 = *reinterpret_cast<const __nv_bfloat162*>(&in[e]);
            y[2 * e] = __low2float(h2);
            y[2 * e + 1] = __high2float(h2);
        }
        // the halves of a warp may hold heads of different kinds: both run the same instructions and choose at the end
        float ss = 0.f;
#pragma unroll
        for (int e = 0; e < 8; e++) ss += y[e] * y[e];
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        const float inv = normed ? 1.0f / sqrtf(ss / 128.f + p.eps) : 1.f;
        const int tpos = gb_check(pos[j], p.table_positions, GB_CHECK_ROPE_POSITION) ? pos[j] : 0;
        const float4 c0 = *reinterpret_cast<const float4*>(p.cos_t + (int64_t)tpos * 64 + ci), c1 = *reinterpret_cast<const float4*>(p.cos_t + (int64_t)tpos * 64 + ci + 4);
        const float4 s0 = *reinterpret_cast<const float4*>(p.sin_t + (int64_t)tpos * 64 + ci), s1 = *reinterpret_cast<const float4*>(p.sin_t + (int64_t)tpos * 64 + ci + 4);
        const float cs[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w}, sv[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
        uint32_t out[4];
#pragma unroll
        for (int e = 0; e < 4; e++) {
            float o2[2];
#pragma unroll
            for (int u = 0; u < 2; u++) {
                const int i = 2 * e + u;
                const float v = normed ? y[i] * inv * ww[i] : y[i];
                const float partner = __shfl_xor_sync(0xffffffffu, v, 8);
                o2[u] = l16 < 8 ? v * cs[i] - partner * sv[i] : v * cs[i] + partner * sv[i];
            }
            const __nv_bfloat162 h2 = __floats2bfloat162_rn(o2[0], o2[1]);
            out[e] = value ? in[e] : *reinterpret_cast<const uint32_t*>(&h2);
        }
        if (stores && r0 + j < p.rows) *reinterpret_cast<uint4*>(dst[j]) = make_uint4(out[0], out[1], out[2], out[3]);
    }
}

GB_API int gb_qk_norm_rope_kv_write(const QkRopeParams* pp, int dtype, cudaStream_t stream) {
    QkRopeParams p = *pp;
    if (p.rows <= 0) return 0;
    if (p.d <= 0 || p.d > 1024) GB_REFUSE("qk_norm_rope: head_dim %d is outside [1, 1024]", p.d);
    if (p.rot < 0 || p.rot > p.d || (p.rot & 1)) GB_REFUSE("qk_norm_rope: rotary width %d must be even and <= head_dim %d", p.rot, p.d);
    if (p.rot > 0 && (!p.cos_t || !p.sin_t)) GB_REFUSE("qk_norm_rope: rotary width %d without an angle table", p.rot);
    if (p.heads <= 0 || p.kv_heads < 0) GB_REFUSE("qk_norm_rope: heads %d, kv heads %d", p.heads, p.kv_heads);
    if (p.rows > 0x7fffffff / 2) GB_REFUSE("qk_norm_rope: %d rows are too many", p.rows);
    int total_heads = p.heads + 2 * p.kv_heads;
    if (dtype == GB_BF16 && p.d == 128 && p.rot == 128 && !(p.row_stride & 3) && !((uintptr_t)p.qkv & 7) &&
        !(((uintptr_t)p.q_w | (uintptr_t)p.k_w | (uintptr_t)p.cos_t | (uintptr_t)p.sin_t) & 15) && (p.q_w != nullptr) == (p.k_w != nullptr) &&
        ceil_div(total_heads, 8) <= 65535) {
        // prompts: the kernel of 16-byte accesses (it adds a row's squares up in another order, so a key
        // may differ in its last bit from the one the kernel for few rows would write)
        if (p.rows >= 256 && !(p.row_stride & 7) && !((uintptr_t)p.qkv & 15)) {
            launch_pdl(qk_rope_bf16_d128_wide_kernel, dim3(ceil_div(p.rows, WIDE_ROWS), ceil_div(total_heads, 16)), dim3(256), 0, stream, p);
            GB_CHECK_LAUNCH("qk_norm_rope_kv_write");
            return 0;
        }
        launch_pdl(qk_rope_bf16_d128_kernel, dim3(ceil_div(p.rows, ROPE_ROWS), ceil_div(total_heads, 8)), dim3(256), 0, stream, p);
        GB_CHECK_LAUNCH("qk_norm_rope_kv_write");
        return 0;
    }
    dim3 grid(p.rows, ceil_div(total_heads, 4));
    if (grid.y > 65535) GB_REFUSE("qk_norm_rope: %d heads exceed one launch", total_heads);
    size_t smem = (size_t)4 * p.d * sizeof(float);
    if (dtype == GB_F32)
        qk_rope_kernel<float><<<grid, 128, smem, stream>>>(p);
    else if (dtype == GB_BF16)
        qk_rope_kernel<__nv_bfloat16><<<grid, 128, smem, stream>>>(p);
    else
        GB_REFUSE("qk_norm_rope: unknown dtype %d", dtype);
    GB_CHECK_LAUNCH("qk_norm_rope_kv_write");
    return 0;
}

// ------------------------------------------------------------------------------------------
// dtype conversion helpers used when rows are handed between precisions
__global__ void f32_to_bf16_kernel(const float* __restrict__ a, __nv_bfloat16* __restrict__ b, int64_t n) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) b[i] = __float2bfloat16_rn(a[i]);
}

GB_API int gb_f32_to_bf16(const float* a, void* b, int64_t n, cudaStream_t stream) {
    if (n <= 0) return 0;
    int64_t blocks = (n + 255) / 256;
    if (blocks > 0x7fffffff) GB_REFUSE("f32_to_bf16: %lld elements are too many", (long long)n);
    f32_to_bf16_kernel<<<(unsigned)blocks, 256, 0, stream>>>(a, (__nv_bfloat16*)b, n);
    GB_CHECK_LAUNCH("f32_to_bf16");
    return 0;
}

// the checked build's record of the first index this file's kernels found out of bounds
GB_CHECK_READER(gb_checked_status_rows)
