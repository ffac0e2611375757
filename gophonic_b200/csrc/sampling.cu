// Token selection on the device: greedy argmax, and temperature / top-k / top-p sampling with a
// counter-based draw.
//
// The sampler follows qwen3/chat.go:808-847: the k likeliest logits (k = top_k, or 1024 when
// top_k is 0 or larger than 1024) in descending order, weights exp((x - top) / T) in fp32 summed
// in that order, the nucleus cut at the first prefix whose sum reaches top_p * total, then a
// draw r = u * sum walked down the list.  Ties between equal logits go to the lower index, and
// the uniform u is splitmix64(seed + (draw + 1) * gamma) >> 40 scaled by 2^-24, as the
// reference's device sampler draws it (internal/qwen3lm/gpu.metal:575-582), so a token is a pure
// function of (logits, options, seed, draw) and does not depend on what else is in the batch.
// Greedy selection takes the first index of the maximum; a NaN never wins
// (qwen3/chat.go:905-914, internal/qwen3lm/gpu.metal:195-237).
#include "common.cuh"

#include <math.h>

namespace {

constexpr int ST = 1024;       // threads of the sampling CTA
constexpr int MAXK = 1024;     // candidate bound (qwen3/chat.go:796-799)

__device__ __forceinline__ uint32_t order_key(float f) {
    if (f != f) return 0u;  // NaN sorts below everything
    uint32_t u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ __forceinline__ float draw01(uint64_t seed, uint64_t draw) {
    uint64_t x = seed + (draw + 1ull) * 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    x ^= x >> 31;
    return (float)(x >> 40) * (1.0f / 16777216.0f);
}

// first index of the maximum of row[0..n); every thread of the CTA gets the result
__device__ int block_argmax(const float* __restrict__ row, int n, float* s_val, int* s_idx) {
    float best = -INFINITY;
    int at = 0x7fffffff;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        float v = row[i];
        if (v > best) {
            best = v;
            at = i;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, best, o);
        int oi = __shfl_xor_sync(0xffffffffu, at, o);
        if (ov > best || (ov == best && oi < at)) {
            best = ov;
            at = oi;
        }
    }
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) {
        s_val[warp] = best;
        s_idx[warp] = at;
    }
    __syncthreads();
    if (warp == 0) {
        int nw = blockDim.x >> 5;
        best = lane < nw ? s_val[lane] : -INFINITY;
        at = lane < nw ? s_idx[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            float ov = __shfl_xor_sync(0xffffffffu, best, o);
            int oi = __shfl_xor_sync(0xffffffffu, at, o);
            if (ov > best || (ov == best && oi < at)) {
                best = ov;
                at = oi;
            }
        }
        if (lane == 0) s_idx[0] = (at == 0x7fffffff) ? 0 : at;
    }
    __syncthreads();
    int r = s_idx[0];
    __syncthreads();
    return r;
}

__global__ void __launch_bounds__(ST) argmax_kernel(const float* __restrict__ logits, int vocab, int64_t stride,
                                                    int* __restrict__ out) {
    __shared__ float s_val[32];
    __shared__ int s_idx[32];
    int r = blockIdx.x;
    int t = block_argmax(logits + (int64_t)r * stride, vocab, s_val, s_idx);
    if (threadIdx.x == 0) out[r] = t;
}

// Two-stage argmax for wide rows: a CTA per (row, chunk of 8192 logits) leaves its best (value,
// index) in scratch, then one CTA per row takes the first maximum of the chunk results.
constexpr int ARG_CHUNK = 8192;

__global__ void __launch_bounds__(256) argmax_part_kernel(const float* __restrict__ logits, int vocab, int64_t stride,
                                                          float* __restrict__ part_val, int* __restrict__ part_idx, int chunks) {
    __shared__ float s_val[32];
    __shared__ int s_idx[32];
    const int r = blockIdx.y, c = blockIdx.x;
    const float* row = logits + (int64_t)r * stride;
    const int lo = c * ARG_CHUNK, hi = lo + ARG_CHUNK < vocab ? lo + ARG_CHUNK : vocab;
    float best = -INFINITY;
    int at = 0x7fffffff;
    for (int i = lo + threadIdx.x; i < hi; i += 256) {
        float v = row[i];
        if (v > best) {
            best = v;
            at = i;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, best, o);
        int oi = __shfl_xor_sync(0xffffffffu, at, o);
        if (ov > best || (ov == best && oi < at)) {
            best = ov;
            at = oi;
        }
    }
    if ((threadIdx.x & 31) == 0) {
        s_val[threadIdx.x >> 5] = best;
        s_idx[threadIdx.x >> 5] = at;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; w++)
            if (s_val[w] > best || (s_val[w] == best && s_idx[w] < at)) {
                best = s_val[w];
                at = s_idx[w];
            }
        part_val[(int64_t)r * chunks + c] = best;
        part_idx[(int64_t)r * chunks + c] = at;
    }
}

__global__ void argmax_final_kernel(const float* __restrict__ part_val, const int* __restrict__ part_idx, int chunks,
                                    int* __restrict__ out) {
    const int r = blockIdx.x;
    float best = -INFINITY;
    int at = 0x7fffffff;
    for (int c = threadIdx.x; c < chunks; c += 32) {
        float v = part_val[(int64_t)r * chunks + c];
        int i = part_idx[(int64_t)r * chunks + c];
        if (v > best || (v == best && i < at)) {
            best = v;
            at = i;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, best, o);
        int oi = __shfl_xor_sync(0xffffffffu, at, o);
        if (ov > best || (ov == best && oi < at)) {
            best = ov;
            at = oi;
        }
    }
    if (threadIdx.x == 0) out[r] = at == 0x7fffffff ? 0 : at;
}

// exclusive prefix sum of one unsigned per thread over the CTA, in thread order
__device__ __forceinline__ uint32_t block_scan_u32(uint32_t v, uint32_t* part, uint32_t* total) {
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint32_t inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        uint32_t n = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += n;
    }
    if (lane == 31) part[warp] = inc;
    __syncthreads();
    uint32_t before = 0, tot = 0;
    for (int i = 0; i < ST / 32; i++) {
        uint32_t pv = part[i];
        if (i < warp) before += pv;
        tot += pv;
    }
    __syncthreads();
    *total = tot;
    return before + inc - v;
}

struct SampleParams {
    const float* logits;
    int64_t stride;
    int rows, vocab;
    const float* temperature;  // per row
    const int* top_k;
    const float* top_p;
    const uint64_t* seed;
    uint64_t* draw;
    int* out;
    const int* opt_row;  // option index of logits row i (null: i itself)
    int advance;         // add one to draw[] of every sampled row
};

// The walk over the k likeliest candidates, most likely first (cand[i] = key << 32 | ~index, sorted
// descending): weights, nucleus cut, draw.  Thread 0 does the sums one after another in fp32, the
// order the reference adds them in.
__device__ void pick_from_sorted(const SampleParams& p, int r, int o, const float* __restrict__ row, int k, float temp,
                                 const unsigned long long* cand, float* prob) {
    const int tid = threadIdx.x;
    const float inv = 1.f / temp;
    const int top_i = (int)(0xFFFFFFFFu - (uint32_t)(cand[0] & 0xFFFFFFFFull));
    const float top = row[top_i];
    for (int i = tid; i < k; i += ST) {
        int idx = (int)(0xFFFFFFFFu - (uint32_t)(cand[i] & 0xFFFFFFFFull));
        prob[i] = expf((row[idx] - top) * inv);
    }
    __syncthreads();
    if (tid == 0) {
        float sum = 0.f;
        for (int i = 0; i < k; i++) sum += prob[i];
        int n = k;
        float tp = p.top_p[o];
        if (tp > 0.f && tp < 1.f) {
            float acc = 0.f;
            for (int i = 0; i < k; i++) {
                acc += prob[i];
                if (acc >= tp * sum) {
                    n = i + 1;
                    sum = acc;
                    break;
                }
            }
        }
        float rr = draw01(p.seed[o], p.draw[o]) * sum;
        int pick = n - 1;
        for (int i = 0; i < n; i++) {
            rr -= prob[i];
            if (rr <= 0.f) {
                pick = i;
                break;
            }
        }
        p.out[r] = (int)(0xFFFFFFFFu - (uint32_t)(cand[pick] & 0xFFFFFFFFull));
        if (p.advance) p.draw[o] += 1ull;
    }
}

// One CTA selects for one row by itself: radix select of the k-th largest logit over the whole row,
// gather, sort.  `cand` holds at least MAXK entries, `prob` MAXK.
__device__ void sample_row_full(const SampleParams& p, int r, int o, unsigned long long* cand, float* prob) {
    __shared__ float s_val[32];
    __shared__ int s_idx[32];
    __shared__ uint32_t bins[256];
    __shared__ uint32_t part[ST / 32];
    __shared__ uint32_t chosen[2];
    __shared__ uint32_t n_gt;

    const int tid = threadIdx.x;
    const float* row = p.logits + (int64_t)r * p.stride;
    const int V = p.vocab;
    const float temp = p.temperature[o];
    if (!(temp > 0.f)) {
        int t = block_argmax(row, V, s_val, s_idx);
        if (tid == 0) p.out[r] = t;
        return;
    }
    int k = p.top_k[o];
    if (k <= 0 || k > MAXK) k = MAXK;
    if (k > V) k = V;

    // radix select: the k-th largest key and how many keys equal to it are taken
    uint32_t prefix = 0, need = (uint32_t)k;
    for (int dgt = 3; dgt >= 0; dgt--) {
        uint32_t shift = (uint32_t)dgt * 8u;
        uint32_t high = dgt == 3 ? 0u : (0xFFFFFFFFu << (shift + 8u));
        if (tid < 256) bins[tid] = 0;
        __syncthreads();
        for (int i = tid; i < V; i += ST) {
            uint32_t key = order_key(row[i]);
            if ((key & high) == prefix) atomicAdd(&bins[(key >> shift) & 255u], 1u);
        }
        __syncthreads();
        if (tid == 0) {
            uint32_t b = 255;
            for (;; b--) {
                uint32_t n = bins[b];
                if (n >= need || b == 0) break;
                need -= n;
            }
            chosen[0] = prefix | (b << shift);
            chosen[1] = need;
        }
        __syncthreads();
        prefix = chosen[0];
        need = chosen[1];
        __syncthreads();
    }
    // gather: keys above the threshold, and of those equal to it the `need` of lowest index
    if (tid == 0) n_gt = 0;
    for (int i = tid; i < MAXK; i += ST) cand[i] = 0ull;
    __syncthreads();
    uint32_t eq_taken = 0;  // equals taken so far (same in every thread)
    const uint32_t n_above = (uint32_t)k - need;
    for (int base = 0; base < V; base += ST) {
        int i = base + tid;
        uint32_t key = i < V ? order_key(row[i]) : 0u;
        bool gt = i < V && key > prefix;
        bool eq = i < V && key == prefix;
        if (gt) {
            uint32_t slot = atomicAdd(&n_gt, 1u);
            if (slot < (uint32_t)MAXK) cand[slot] = ((unsigned long long)key << 32) | (uint32_t)(0xFFFFFFFFu - (uint32_t)i);
        }
        uint32_t total;
        uint32_t rank = block_scan_u32(eq ? 1u : 0u, part, &total);
        if (eq && eq_taken + rank < need) {
            uint32_t slot = n_above + eq_taken + rank;
            if (slot < (uint32_t)MAXK) cand[slot] = ((unsigned long long)key << 32) | (uint32_t)(0xFFFFFFFFu - (uint32_t)i);
        }
        eq_taken += total;
    }
    __syncthreads();
    // bitonic sort of the 1024 composite keys, descending (empty slots are 0 and sink)
    for (int size = 2; size <= MAXK; size <<= 1) {
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            int i = tid;
            int j = i ^ stride;
            if (j > i) {
                unsigned long long a = cand[i], b = cand[j];
                bool desc = (i & size) == 0;
                if (desc ? (a < b) : (a > b)) {
                    cand[i] = b;
                    cand[j] = a;
                }
            }
            __syncthreads();
        }
    }
    pick_from_sorted(p, r, o, row, k, temp, cand, prob);
}

__global__ void __launch_bounds__(ST) sample_kernel(SampleParams p) {
    __shared__ unsigned long long cand[MAXK];
    __shared__ float prob[MAXK];
    const int r = blockIdx.x;
    sample_row_full(p, r, p.opt_row ? p.opt_row[r] : r, cand, prob);
}

// ---- wide rows: three kernels ------------------------------------------------------------
// A row of a large vocabulary is too long for one CTA to scan five times.  (1) CTAs over chunks of
// the row count the logits by the top 12 bits of their order key into a histogram of the row.
// (2) Every CTA finds, from the histogram, the lowest bin that the k likeliest logits reach, and
// appends the logits of its chunk in that bin or above to the row's candidate list.  (3) One CTA
// per row sorts the candidates (k and the rest of the last bin: a few hundred to a few thousand)
// by (logit descending, index ascending) and walks them as above.  If the last bin is so crowded
// that the list overflows (many equal logits), that CTA selects over the whole row by itself.
// Greedy rows take the same path with k = 1.
constexpr int HB = 4096;        // histogram bins
constexpr int WCHUNK = 8192;    // logits per CTA in (1) and (2)
constexpr int MAXC = 4096;      // candidates kept per row
constexpr int HROW = HB + 2;    // per row: bins, then the candidate count

__device__ __forceinline__ int row_k(const SampleParams& p, int o) {
    if (!(p.temperature[o] > 0.f)) return 1;
    int k = p.top_k[o];
    if (k <= 0 || k > MAXK) k = MAXK;
    if (k > p.vocab) k = p.vocab;
    return k;
}

__global__ void __launch_bounds__(256) sample_hist_kernel(SampleParams p, uint32_t* __restrict__ hist) {
    __shared__ uint32_t sh[HB];
    const int r = blockIdx.y, tid = threadIdx.x;
    for (int i = tid; i < HB; i += 256) sh[i] = 0;
    __syncthreads();
    const float* row = p.logits + (int64_t)r * p.stride;
    const int lo = blockIdx.x * WCHUNK, hi = lo + WCHUNK < p.vocab ? lo + WCHUNK : p.vocab;
    for (int i = lo + tid; i < hi; i += 256) atomicAdd(&sh[order_key(row[i]) >> 20], 1u);
    __syncthreads();
    uint32_t* h = hist + (int64_t)r * HROW;
    for (int i = tid; i < HB; i += 256)
        if (sh[i]) atomicAdd(&h[i], sh[i]);
}

__global__ void __launch_bounds__(256) sample_gather_kernel(SampleParams p, uint32_t* __restrict__ hist,
                                                            unsigned long long* __restrict__ cands) {
    __shared__ uint32_t sh[HB];
    __shared__ uint32_t seg[256];
    __shared__ int s_bin;
    const int r = blockIdx.y, tid = threadIdx.x;
    const int o = p.opt_row ? p.opt_row[r] : r;
    uint32_t* h = hist + (int64_t)r * HROW;
    uint32_t local = 0;
    for (int i = 0; i < HB / 256; i++) {
        uint32_t v = h[tid * (HB / 256) + i];
        sh[tid * (HB / 256) + i] = v;
        local += v;
    }
    seg[tid] = local;
    __syncthreads();
    if (tid == 0) {
        const uint32_t k = (uint32_t)row_k(p, o);
        uint32_t cum = 0;
        int bin = 0;
        for (int t = 255; t >= 0; t--) {
            if (cum + seg[t] >= k) {
                for (int b = t * (HB / 256) + HB / 256 - 1; b >= t * (HB / 256); b--) {
                    cum += sh[b];
                    if (cum >= k) {
                        bin = b;
                        break;
                    }
                }
                break;
            }
            cum += seg[t];
        }
        s_bin = bin;
    }
    __syncthreads();
    const uint32_t bin = (uint32_t)s_bin;
    const float* row = p.logits + (int64_t)r * p.stride;
    unsigned long long* c = cands + (int64_t)r * MAXC;
    const int lo = blockIdx.x * WCHUNK, hi = lo + WCHUNK < p.vocab ? lo + WCHUNK : p.vocab;
    for (int i = lo + tid; i < hi; i += 256) {
        const uint32_t key = order_key(row[i]);
        if ((key >> 20) >= bin) {
            const uint32_t slot = atomicAdd(&h[HB], 1u);
            if (slot < (uint32_t)MAXC) c[slot] = ((unsigned long long)key << 32) | (uint32_t)(0xFFFFFFFFu - (uint32_t)i);
        }
    }
}

__global__ void __launch_bounds__(ST) sample_final_kernel(SampleParams p, const uint32_t* __restrict__ hist,
                                                          const unsigned long long* __restrict__ cands) {
    __shared__ unsigned long long cand[MAXC];
    __shared__ float prob[MAXK];
    const int r = blockIdx.x, tid = threadIdx.x;
    const int o = p.opt_row ? p.opt_row[r] : r;
    const uint32_t count = hist[(int64_t)r * HROW + HB];
    if (count > (uint32_t)MAXC) {
        sample_row_full(p, r, o, cand, prob);
        return;
    }
    const int n = (int)count;
    int P = 1024;
    while (P < n) P <<= 1;
    const unsigned long long* c = cands + (int64_t)r * MAXC;
    for (int i = tid; i < P; i += ST) cand[i] = i < n ? c[i] : 0ull;
    __syncthreads();
    // bitonic sort, descending (empty slots are 0 and sink)
    for (int size = 2; size <= P; size <<= 1) {
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            for (int t = tid; t < P / 2; t += ST) {
                const int i = ((t & ~(stride - 1)) << 1) | (t & (stride - 1));
                const int j = i | stride;
                unsigned long long a = cand[i], b = cand[j];
                const bool desc = (i & size) == 0;
                if (desc ? (a < b) : (a > b)) {
                    cand[i] = b;
                    cand[j] = a;
                }
            }
            __syncthreads();
        }
    }
    const float* row = p.logits + (int64_t)r * p.stride;
    const float temp = p.temperature[o];
    if (!(temp > 0.f)) {
        if (tid == 0) p.out[r] = n > 0 ? (int)(0xFFFFFFFFu - (uint32_t)(cand[0] & 0xFFFFFFFFull)) : 0;
        return;
    }
    int k = row_k(p, o);
    if (k > n) k = n;
    pick_from_sorted(p, r, o, row, k, temp, cand, prob);
}

// logits[r, v] -= presence[r] for every token v the reply of row r already holds
// (qwen3/chat.go:430-437); `seen` is one bit per (row slot, token).
__global__ void presence_kernel(float* __restrict__ logits, int64_t stride, int vocab, const uint32_t* __restrict__ seen,
                                int64_t seen_stride, const int* __restrict__ seen_row, const float* __restrict__ presence,
                                int indexed) {
    int r = blockIdx.y;
    float pen = presence[indexed ? seen_row[r] : r];
    if (pen == 0.f) return;
    int w = blockIdx.x * blockDim.x + threadIdx.x;
    int words = (vocab + 31) / 32;
    if (w >= words) return;
    uint32_t bits = seen[(int64_t)seen_row[r] * seen_stride + w];
    while (bits) {
        int b = __ffs(bits) - 1;
        bits &= bits - 1;
        int v = w * 32 + b;
        if (v < vocab) logits[(int64_t)r * stride + v] -= pen;
    }
}

__global__ void mark_seen_kernel(const int* __restrict__ tokens, int rows, int vocab, uint32_t* __restrict__ seen,
                                 int64_t seen_stride, const int* __restrict__ seen_row) {
    int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= rows) return;
    int t = tokens[r];
    if (t < 0 || t >= vocab) return;
    atomicOr(&seen[(int64_t)seen_row[r] * seen_stride + (t >> 5)], 1u << (t & 31));
}

}  // namespace

GB_API int gb_argmax(const float* logits, int rows, int vocab, int64_t stride, int* out, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0 || stride < vocab) GB_REFUSE("argmax: vocab %d, stride %lld", vocab, (long long)stride);
    argmax_kernel<<<rows, ST, 0, stream>>>(logits, vocab, stride, out);
    GB_CHECK_LAUNCH("argmax");
    return 0;
}

// scratch: rows * ceil(vocab / 8192) floats followed by as many ints
GB_API int gb_argmax_wide(const float* logits, int rows, int vocab, int64_t stride, int* out, void* scratch, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0 || stride < vocab) GB_REFUSE("argmax: vocab %d, stride %lld", vocab, (long long)stride);
    if (rows > 65535) GB_REFUSE("argmax: %d rows exceed one launch", rows);
    if (!scratch) GB_REFUSE("argmax: the two-stage kernel needs scratch");
    const int chunks = ceil_div(vocab, ARG_CHUNK);
    float* pv = (float*)scratch;
    int* pi = (int*)(pv + (int64_t)rows * chunks);
    argmax_part_kernel<<<dim3(chunks, rows), 256, 0, stream>>>(logits, vocab, stride, pv, pi, chunks);
    GB_CHECK_LAUNCH("argmax_part");
    argmax_final_kernel<<<rows, 32, 0, stream>>>(pv, pi, chunks, out);
    GB_CHECK_LAUNCH("argmax_final");
    return 0;
}

// Bytes of scratch gb_sample wants for `rows` rows of `vocab` logits (0: none).
GB_API int64_t gb_sample_scratch_bytes(int rows, int vocab) {
    if (vocab < 2 * WCHUNK || rows <= 0) return 0;
    return (int64_t)rows * (HROW * (int64_t)sizeof(uint32_t) + MAXC * (int64_t)sizeof(unsigned long long));
}

// One token per row.  opt_row (may be null): which entry of the option arrays row i uses.
// advance != 0: draw[] of every sampled row is increased by one after the draw.
GB_API int gb_sample(const float* logits, int rows, int vocab, int64_t stride, const int* opt_row, const float* temperature,
                     const int* top_k, const float* top_p, const uint64_t* seed, uint64_t* draw, int* out, int advance, void* scratch,
                     int64_t scratch_bytes, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0 || stride < vocab) GB_REFUSE("sample: vocab %d, stride %lld", vocab, (long long)stride);
    SampleParams p{logits, stride, rows, vocab, temperature, top_k, top_p, seed, draw, out, opt_row, advance};
    const int64_t want = gb_sample_scratch_bytes(rows, vocab);
    if (want == 0 || !scratch || scratch_bytes < want || rows > 65535) {
        sample_kernel<<<rows, ST, 0, stream>>>(p);
        GB_CHECK_LAUNCH("sample");
        return 0;
    }
    if ((uintptr_t)scratch & 7) GB_REFUSE("sample: scratch must be 8-byte aligned");
    unsigned long long* cands = (unsigned long long*)scratch;
    uint32_t* hist = (uint32_t*)(cands + (int64_t)rows * MAXC);
    if (cudaMemsetAsync(hist, 0, (size_t)rows * HROW * sizeof(uint32_t), stream) != cudaSuccess) GB_REFUSE("sample: cannot clear the histograms");
    const dim3 grid(ceil_div(vocab, WCHUNK), rows);
    sample_hist_kernel<<<grid, 256, 0, stream>>>(p, hist);
    GB_CHECK_LAUNCH("sample_hist");
    sample_gather_kernel<<<grid, 256, 0, stream>>>(p, hist, cands);
    GB_CHECK_LAUNCH("sample_gather");
    sample_final_kernel<<<rows, ST, 0, stream>>>(p, hist, cands);
    GB_CHECK_LAUNCH("sample_final");
    return 0;
}

// presence[r] belongs to logits row r, or, with indexed != 0, to the bitmap row seen_row[r]
GB_API int gb_presence_penalty(float* logits, int rows, int vocab, int64_t stride, const uint32_t* seen, int64_t seen_stride,
                               const int* seen_row, const float* presence, int indexed, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (rows > 65535) GB_REFUSE("presence_penalty: %d rows exceed one launch", rows);
    int words = (vocab + 31) / 32;
    presence_kernel<<<dim3(ceil_div(words, 256), rows), 256, 0, stream>>>(logits, stride, vocab, seen, seen_stride, seen_row, presence, indexed);
    GB_CHECK_LAUNCH("presence_penalty");
    return 0;
}

GB_API int gb_mark_seen(const int* tokens, int rows, int vocab, uint32_t* seen, int64_t seen_stride, const int* seen_row,
                        cudaStream_t stream) {
    if (rows <= 0) return 0;
    mark_seen_kernel<<<ceil_div(rows, 128), 128, 0, stream>>>(tokens, rows, vocab, seen, seen_stride, seen_row);
    GB_CHECK_LAUNCH("mark_seen");
    return 0;
}
