// Host-side dispatch: which kernel takes a product or an attention call of given types and sizes,
// and the issue of a whole pre-norm layer (norm, q/k/v product, q/k norm + rotation + cache write,
// attention, output projection, norm, gate/up product with SwiGLU, down projection) from one call.
//
// A prompt step of a few hundred rows is some 330 kernel launches; issued one by one from Python
// (argument checks, ctypes marshalling and an allocation per call, about 15 us each) the host needs
// longer than the GPU up to about 256 rows.  The layer call does the same launches, in the same
// order and with the same kernel choices, from C++ out of one workspace the caller provides.  The
// reference keeps a whole run in one submission for the same reason
// (internal/qwen3lm/gpu_darwin.go:1596-1622).
#include "api.h"
#include "common.cuh"

// ------------------------------------------------------------------------------------------
// products
enum GbGemmAlgo : int { GB_ALGO_SIMT = 0, GB_ALGO_SKINNY = 1, GB_ALGO_TC5 = 2, GB_ALGO_TC5_PAIR = 3, GB_ALGO_TC5_DECODE = 4 };

// rows up to which the fragment-streaming kernel is used for decode; above it the tcgen05 decode kernel
// (with 16 it took 9, 12 and 16 sequences 7 % longer a step: 5.07 / 5.30 / 5.70 against 4.72 / 4.95 / 5.36 ms)
constexpr int SKINNY_MAX_ROWS = 8;
// rows up to which the tcgen05 decode kernel takes a product (its batch side is one instruction wide)
constexpr int TC5_DECODE_MAX_ROWS = 256;
// rows from which the tcgen05 kernel that pairs two SMs on tiles of 256 x 256 is used
constexpr int TC5_PAIR_MIN_ROWS = 192;
// outputs this wide (the head) have enough tiles to fill the GPU without cutting K; the tcgen05 decode
// kernel then streams them a little faster than the fragment kernel at every row count
constexpr int WIDE_OUTPUT = 32768;
// prompts whose longest sequence brings at least this many rows use the tcgen05 attention kernel
constexpr int TC5_ATTENTION_MIN_ROWS = 65;
// few-row products of at least this many weights, and at least this long on both sides, run on the tcgen05
// decode kernel (inside a decode step of 8B sizes the 24576 x 4096 product, a little faster there by
// itself, cost the step a quarter: the width that counts is the one of the products around it as well)
constexpr int64_t BIG_PRODUCT = 40 << 20;
constexpr int BIG_PRODUCT_MIN_SIDE = 5120;

GB_API int gb_dispatch_constant(int which) {
    switch (which) {
        case 0: return SKINNY_MAX_ROWS;
        case 1: return TC5_DECODE_MAX_ROWS;
        case 2: return TC5_PAIR_MIN_ROWS;
        case 3: return WIDE_OUTPUT;
        case 4: return TC5_ATTENTION_MIN_ROWS;
        case 5: return GB_FOLD_MAX_ROWS;
    }
    return -1;
}

// The tensor-core kernel for aligned bfloat16 operands of these sizes (measured on the four products
// of a layer at 1.7B, 8B and 32B sizes, 1 to 2048 rows).
GB_API int gb_gemm_algo(int M, int N, int K, int sms) {
    // Few rows: the weights streamed straight into mma.sync fragments, except for the largest products, which
    // the tcgen05 decode kernel streams faster (one row, us: 10240 x 5120 18.4 against 21.1, 5120 x 8192 16.2
    // against 17.8, 5120 x 25600 41.0 against 49.4; but 4096 x 12288 18.7 against 17.5 and 6144 x 4096 10.6
    // against 9.8)
    const bool large = (int64_t)N * K >= BIG_PRODUCT && N >= BIG_PRODUCT_MIN_SIDE && K >= BIG_PRODUCT_MIN_SIDE;
    if (M <= SKINNY_MAX_ROWS && N < WIDE_OUTPUT && !large) return GB_ALGO_SKINNY;
    // tcgen05, weights on the M side, K slices across a cluster; a head-sized output has tiles enough for the
    // tiled kernel, which reads the activations once per 256 columns (151936 x 4096 at 64 rows: 222 against 241 us)
    if (M <= 64) return N >= WIDE_OUTPUT && M > 16 ? GB_ALGO_TC5 : GB_ALGO_TC5_DECODE;
    // Up to 256 rows a narrow output is still bound by reading its weights, and the decode kernel gives
    // every SM a share of them by cutting K; its CTAs all read the activations, though, so a wide output
    // is better off on the tiled kernels.  Tiles of 128 output columns against the SM count: at 65 to
    // 128 rows the decode kernel won at 80 tiles (10240 x 5120: 36 against 45 us) and lost at 96
    // (12288 x 2048: 28 against 18 us); at 129 to 256 rows it won at 40 (5120 x 8192: 44 against 48 us;
    // 4096 x 4096: 19 against 26 us), tied at 48 and lost at 80 (75 against 38 us).
    const int tiles = (N + 127) / 128;
    if (M <= TC5_DECODE_MAX_ROWS / 2) return 5 * tiles <= 3 * sms ? GB_ALGO_TC5_DECODE : GB_ALGO_TC5;
    if (M <= TC5_DECODE_MAX_ROWS && 10 * tiles <= 3 * sms) return GB_ALGO_TC5_DECODE;
    if (M >= TC5_PAIR_MIN_ROWS) return GB_ALGO_TC5_PAIR;                  // tcgen05 on pairs of SMs, 256 x 256 tiles
    return GB_ALGO_TC5;                                                   // tcgen05, 128 x 256 tiles
}

// The kernel for a few-row product that applies row factors from statistics (the first product of a part
// in a folded decode step).  As gb_gemm_algo, and the tcgen05 decode kernel also for a product as large as
// the gate/up of an 8B layer (24576 x 4096: 34.0 against 37.7 us at eight rows), provided the few-row kernel
// behind it is then launched as an ordinary kernel (see gb_gemm_skinny_residual): as a dependent launch it
// would come in beside the decode kernel's CTAs one to an SM and run its other CTAs as a second wave.
GB_API int gb_gemm_scaled_algo(int M, int N, int K, int sms) {
    const int algo = gb_gemm_algo(M, N, K, sms);
    // (whole 8B decode steps: 0.4 to 0.9 % slower at one to three sequences, 0.8 to 2.4 % faster at four to eight)
    if (algo == GB_ALGO_SKINNY && M >= 4 && (int64_t)N * K >= BIG_PRODUCT && N >= BIG_PRODUCT_MIN_SIDE && K >= 4096) return GB_ALGO_TC5_DECODE;
    return algo;
}

static bool tensor_core_operands(const void* A, int a_dtype, const void* W, int w_dtype, int K, int64_t lda) {
    return a_dtype == GB_BF16 && w_dtype == GB_BF16 && (K & 7) == 0 && (lda & 7) == 0 && !((uintptr_t)A & 15) && !((uintptr_t)W & 15);
}

// C = A W^T with the kernel chosen by operand types and sizes (W contiguous: row stride K).  What the
// tensor-core kernels cannot take (float32 operands, rows that are not 16-byte aligned) runs on the
// fp32 CUDA-core kernel.  *algo receives the choice.
GB_API int gb_gemm_auto(const void* A, int a_dtype, const void* W, int w_dtype, void* C, int c_dtype, int M, int N, int K, int64_t lda,
                        int64_t ldc, int sms, int* algo, cudaStream_t stream) {
    int a = GB_ALGO_SIMT;
    if (tensor_core_operands(A, a_dtype, W, w_dtype, K, lda)) a = gb_gemm_algo(M, N, K, sms);
    if (algo) *algo = a;
    switch (a) {
        case GB_ALGO_SKINNY: return gb_gemm_skinny(A, W, C, c_dtype, M, N, K, lda, ldc, stream);
        case GB_ALGO_TC5: return gb_gemm_tc5(A, W, C, c_dtype, M, N, K, lda, ldc, stream);
        case GB_ALGO_TC5_PAIR: return gb_gemm_tc5_pair(A, W, C, c_dtype, M, N, K, lda, ldc, stream);
        case GB_ALGO_TC5_DECODE:
            return gb_gemm_tc5_decode(A, W, C, c_dtype, M, N, K, lda, ldc, 0, gb_gemm_tc5_decode_splits(M, N, K, sms), stream);
        default: return gb_gemm_simt(A, a_dtype, W, w_dtype, C, c_dtype, M, N, K, lda, K, ldc, stream);
    }
}

static bool swiglu_operands(const void* A, int a_dtype, const void* W, int w_dtype, int N, int K, int64_t lda) {
    return tensor_core_operands(A, a_dtype, W, w_dtype, K, lda) && (N & 15) == 0;
}

// C[M, N / 2] = silu(A Wg^T) * (A Wu^T), gate and up rows of W interleaved in blocks of eight, in the
// kernel gb_gemm_auto would pick.  Returns 1 (nothing launched) if the operands do not allow the
// fused epilogue.
GB_API int gb_gemm_swiglu_auto(const void* A, int a_dtype, const void* W, int w_dtype, void* C, int c_dtype, int M, int N, int K,
                               int64_t lda, int64_t ldc, int sms, int* algo, cudaStream_t stream) {
    if (!swiglu_operands(A, a_dtype, W, w_dtype, N, K, lda)) return 1;
    const int a = gb_gemm_algo(M, N, K, sms);
    if (algo) *algo = a;
    switch (a) {
        case GB_ALGO_SKINNY: return gb_gemm_skinny_swiglu(A, W, C, c_dtype, M, N, K, lda, ldc, stream);
        case GB_ALGO_TC5: return gb_gemm_tc5_swiglu(A, W, C, c_dtype, M, N, K, lda, ldc, stream);
        case GB_ALGO_TC5_PAIR: return gb_gemm_tc5_pair_swiglu(A, W, C, c_dtype, M, N, K, lda, ldc, stream);
        default: return gb_gemm_tc5_decode(A, W, C, c_dtype, M, N, K, lda, ldc, 1, gb_gemm_tc5_decode_splits(M, N, K, sms), stream);
    }
}

// Whether C += A W^T can run in the epilogue of the paired-SM kernel (a prompt-sized bfloat16
// product into the float32 residual).
GB_API int gb_gemm_add_accepts(const void* A, int a_dtype, const void* W, int w_dtype, const void* C, int M, int N, int K, int64_t lda,
                               int64_t ldc, int sms) {
    return tensor_core_operands(A, a_dtype, W, w_dtype, K, lda) && M >= TC5_PAIR_MIN_ROWS && (ldc & 3) == 0 && !((uintptr_t)C & 15) &&
           gb_gemm_algo(M, N, K, sms) == GB_ALGO_TC5_PAIR;
}

// ------------------------------------------------------------------------------------------
// attention
enum GbAttnAlgo : int { GB_ATTN_SIMT = 0, GB_ATTN_DECODE_MMA = 1, GB_ATTN_PREFILL_MMA = 2, GB_ATTN_PREFILL_TC5 = 3 };

GB_API int gb_attention_algo(const AttnParams* p, int dtype) {
    if (dtype != GB_BF16 || (p->d & 15) || !(p->d <= 128 || p->d == 256)) return GB_ATTN_SIMT;
    if (p->max_q_len == 1) return GB_ATTN_DECODE_MMA;
    if (p->max_q_len >= TC5_ATTENTION_MIN_ROWS && p->d == 128 && !((uintptr_t)p->q & 15) && !(p->q_row_stride & 7) && !(p->out_row_stride & 7))
        return GB_ATTN_PREFILL_TC5;
    return GB_ATTN_PREFILL_MMA;
}

// rows: packed query rows in the q buffer; pages: pages in each cache plane.  *kernels receives the
// number of kernels launched (a split-key call merges with a second one).
GB_API int gb_attention_auto(const AttnParams* p, int dtype, int rows, int pages, int* algo, int* kernels, cudaStream_t stream) {
    const int a = gb_attention_algo(p, dtype);
    if (algo) *algo = a;
    if (kernels) *kernels = (a == GB_ATTN_SIMT || a == GB_ATTN_DECODE_MMA) && p->num_splits > 1 ? 2 : 1;
    switch (a) {
        case GB_ATTN_DECODE_MMA: return gb_attention_decode_mma(p, stream);
        case GB_ATTN_PREFILL_MMA: return gb_attention_prefill_mma(p, stream);
        case GB_ATTN_PREFILL_TC5: return gb_attention_prefill_tc5(p, rows, pages, stream);
        default: return gb_attention_simt(p, dtype, stream);
    }
}

// ------------------------------------------------------------------------------------------
// a whole pre-norm layer
struct GbPrenormLayer {
    // sizes and constants, from the parts' specs
    int hidden, heads, kv_heads, head_dim, intermediate;
    float mixer_norm_eps, ffn_norm_eps, qk_norm_eps, scale;
    int window, rotary_dim, table_positions;
    int act_dtype;        // GB_F32 or GB_BF16: activations and cache
    int gate_up_interleaved;
    // tensors
    const float* mixer_norm_w;
    const float* ffn_norm_w;
    const void* w_qkv;
    int w_qkv_dtype;
    const void* w_o;
    int w_o_dtype;
    const void* w_gate_up;
    int w_gate_up_dtype;
    const void* w_down;
    int w_down_dtype;
    const float* q_norm_w;  // null: no per-head norm
    const float* k_norm_w;
    const float* cos_t;
    const float* sin_t;
};

struct GbStepRows {
    int rows, nseq, max_q_len;
    const int* row_pos;
    const int* row_seq;
    const int* seq_slot;
    const int* seq_q_start;
    const int* seq_q_len;
    const int* seq_kv_len;
    int num_splits;
    float* split_scratch;
    // this run's cache plane
    const int* block_table;
    int bt_stride;
    void* k_plane;
    void* v_plane;
    int pages;
    int write_kv;
    int max_slots;  // rows of the block table
};

static int64_t align256(int64_t n) { return (n + 255) & ~(int64_t)255; }

struct LayerWorkspace {
    unsigned char *x, *qkv, *ctx, *act, *gate_up;
    float *mixed, *out;
    int64_t bytes;
};

static LayerWorkspace carve(const GbPrenormLayer& L, int rows, unsigned char* base) {
    const int64_t es = L.act_dtype == GB_BF16 ? 2 : 4;
    const int64_t q_dim = (int64_t)L.heads * L.head_dim, kv_dim = (int64_t)L.kv_heads * L.head_dim;
    LayerWorkspace w;
    int64_t at = 0;
    auto take = [&](int64_t n) {
        unsigned char* p = base ? base + at : nullptr;
        at += align256(n);
        return p;
    };
    w.x = take(rows * L.hidden * es);
    w.qkv = take(rows * (q_dim + 2 * kv_dim) * es);
    w.ctx = take(rows * q_dim * es);
    w.mixed = (float*)take((int64_t)rows * L.hidden * 4);
    w.act = take((int64_t)rows * L.intermediate * es);
    w.out = (float*)take((int64_t)rows * L.hidden * 4);
    w.gate_up = take((int64_t)rows * 2 * L.intermediate * es);  // only used when the fused SwiGLU epilogue cannot be
    w.bytes = at;
    return w;
}

GB_API int64_t gb_prenorm_layer_workspace(const GbPrenormLayer* L, int rows) { return carve(*L, rows, nullptr).bytes; }

#define GB_TRY(call)               \
    do {                           \
        int rc__ = (call);         \
        if (rc__ < 0) return rc__; \
    } while (0)

// Runs the layer on the fp32 residual h[rows, hidden] (updated in place).  `delta` (or null) is an
// addend the residual is still owed; it is added by the first norm.  On return *delta_out is the
// addend the layer itself leaves owed (a pointer into the workspace: the down projection's output),
// or null if the layer added everything itself (prompt-sized steps do, in the epilogues of the
// output and down projections).  *launches receives the number of kernels launched.
GB_API int gb_prenorm_layer_forward(const GbPrenormLayer* Lp, const GbStepRows* Sp, float* h, const float* delta, void* workspace,
                                    int64_t workspace_bytes, int sms, float** delta_out, int* launches, cudaStream_t stream) {
    const GbPrenormLayer& L = *Lp;
    const GbStepRows& S = *Sp;
    const int rows = S.rows;
    if (delta_out) *delta_out = nullptr;
    if (launches) *launches = 0;
    if (rows <= 0) return 0;
    if (((uintptr_t)workspace & 255)) GB_REFUSE("prenorm_layer: the workspace must be 256-byte aligned");
    LayerWorkspace ws = carve(L, rows, (unsigned char*)workspace);
    if (ws.bytes > workspace_bytes) GB_REFUSE("prenorm_layer: the workspace holds %lld bytes, %lld are needed", (long long)workspace_bytes, (long long)ws.bytes);
    const int act = L.act_dtype;
    const int q_dim = L.heads * L.head_dim, kv_dim = L.kv_heads * L.head_dim, qkv_dim = q_dim + 2 * kv_dim;
    int n = 0, algo = 0, kernels = 0;

    // h += delta; x = norm(h)
    GB_TRY(gb_add_rmsnorm(h, delta, L.mixer_norm_w, L.mixer_norm_eps, L.hidden, ws.x, act, nullptr, rows, stream));
    n++;
    GB_TRY(gb_gemm_auto(ws.x, act, L.w_qkv, L.w_qkv_dtype, ws.qkv, act, rows, qkv_dim, L.hidden, L.hidden, qkv_dim, sms, &algo, stream));
    n++;
    QkRopeParams r = {ws.qkv, qkv_dim, L.q_norm_w, L.k_norm_w, L.qk_norm_eps, L.cos_t, L.sin_t, L.rotary_dim, L.table_positions,
                      S.row_pos, S.row_seq, S.seq_slot, S.block_table, S.bt_stride, S.k_plane, S.v_plane, S.write_kv,
                      rows, L.heads, L.kv_heads, L.head_dim, S.pages, S.max_slots};
    AttnParams a = {ws.qkv, qkv_dim, ws.ctx, q_dim, S.k_plane, S.v_plane, S.block_table, S.bt_stride, S.seq_slot, S.seq_q_start,
                    S.seq_q_len, S.seq_kv_len, S.nseq, L.heads, L.kv_heads, L.head_dim, S.max_q_len, L.scale, L.window,
                    S.num_splits > 1 ? S.num_splits : 1, S.num_splits > 1 ? S.split_scratch : nullptr, S.pages, S.max_slots};
    if (gb_attention_decode_rope_accepts(act, L.head_dim, L.rotary_dim, S.max_q_len) && rows == S.nseq) {
        // single tokens: the attention kernel norms and rotates its queries and places the token's key and value itself
        GB_TRY(gb_attention_decode_mma_rope(&a, &r, stream));
        n += a.num_splits > 1 ? 2 : 1;
    } else {
        GB_TRY(gb_qk_norm_rope_kv_write(&r, act, stream));
        n++;
        GB_TRY(gb_attention_auto(&a, act, rows, S.pages, &algo, &kernels, stream));
        n += kernels;
    }
    // output projection: into the residual itself where the paired-SM kernel takes it, else an addend for the next norm
    const float* mixed = nullptr;
    if (gb_gemm_add_accepts(ws.ctx, act, L.w_o, L.w_o_dtype, h, rows, L.hidden, q_dim, q_dim, L.hidden, sms) && (L.hidden & 3) == 0) {
        GB_TRY(gb_gemm_tc5_pair_add(ws.ctx, L.w_o, h, rows, L.hidden, q_dim, q_dim, L.hidden, stream));
    } else {
        GB_TRY(gb_gemm_auto(ws.ctx, act, L.w_o, L.w_o_dtype, ws.mixed, GB_F32, rows, L.hidden, q_dim, q_dim, L.hidden, sms, &algo, stream));
        mixed = ws.mixed;
    }
    n++;
    GB_TRY(gb_add_rmsnorm(h, mixed, L.ffn_norm_w, L.ffn_norm_eps, L.hidden, ws.x, act, nullptr, rows, stream));
    n++;
    // gate/up with SwiGLU in the product's epilogue where the operands allow it
    int fused = 1;
    if (L.gate_up_interleaved) {
        fused = gb_gemm_swiglu_auto(ws.x, act, L.w_gate_up, L.w_gate_up_dtype, ws.act, act, rows, 2 * L.intermediate, L.hidden, L.hidden,
                                    L.intermediate, sms, &algo, stream);
        if (fused < 0) return fused;
    }
    if (fused == 0) {
        n++;
    } else {
        GB_TRY(gb_gemm_auto(ws.x, act, L.w_gate_up, L.w_gate_up_dtype, ws.gate_up, act, rows, 2 * L.intermediate, L.hidden, L.hidden,
                            2 * L.intermediate, sms, &algo, stream));
        GB_TRY(gb_swiglu(ws.gate_up, ws.act, act, rows, L.intermediate, L.gate_up_interleaved, stream));
        n += 2;
    }
    if (gb_gemm_add_accepts(ws.act, act, L.w_down, L.w_down_dtype, h, rows, L.hidden, L.intermediate, L.intermediate, L.hidden, sms) &&
        (L.hidden & 3) == 0) {
        GB_TRY(gb_gemm_tc5_pair_add(ws.act, L.w_down, h, rows, L.hidden, L.intermediate, L.intermediate, L.hidden, stream));
    } else {
        GB_TRY(gb_gemm_auto(ws.act, act, L.w_down, L.w_down_dtype, ws.out, GB_F32, rows, L.hidden, L.intermediate, L.intermediate, L.hidden,
                            sms, &algo, stream));
        if (delta_out) *delta_out = ws.out;
    }
    n++;
    if (launches) *launches = n;
    return 0;
}
