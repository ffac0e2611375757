// The C interface of the kernel library: parameter blocks and entry points.
//
// Every entry point has C linkage, takes raw device pointers and a cudaStream_t, launches on that
// stream and returns 0, or a negative status with the reason in gb_last_error().  Sizes a kernel
// cannot take are refused before anything is launched.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#ifndef GB_API
#define GB_API extern "C" __attribute__((visibility("default")))
#endif

// Attention over the paged cache: rows of a step, packed sequence by sequence.
struct AttnParams {
    const void* q;
    int64_t q_row_stride;
    void* out;
    int64_t out_row_stride;
    const void* k_plane;
    const void* v_plane;
    const int* block_table;
    int bt_stride;
    const int* seq_slot;
    const int* seq_q_start;
    const int* seq_q_len;
    const int* seq_kv_len;
    int nseq, heads, kv_heads, d;
    int max_q_len;
    float scale;
    int window;
    int num_splits;
    float* scratch;  // [nseq][heads][num_splits][d + 2] when num_splits > 1
    int pages;       // pages of each cache plane, and slots (rows) of the block table: the bounds the
    int max_slots;   // checked build holds every page and slot index against
};

// Per-head q/k RMSNorm, rotary embedding and cache write on the rows of a fused q|k|v buffer.
struct QkRopeParams {
    void* qkv;
    int64_t row_stride;
    const float* q_w;
    const float* k_w;
    float eps;
    const float* cos_t;  // [capacity, rot/2] or null when rot == 0
    const float* sin_t;
    int rot;             // rotary width (even, <= d); 0: no rotation
    int table_positions;
    const int* row_pos;
    const int* row_seq;
    const int* seq_slot;
    const int* block_table;
    int bt_stride;
    void* k_plane;
    void* v_plane;
    int write_kv;
    int rows, heads, kv_heads, d;
    int pages;      // pages of each cache plane, and slots (rows) of the block table: the bounds the
    int max_slots;  // checked build holds every page and slot index against
};

GB_API const char* gb_last_error();

// row-wise kernels
GB_API int gb_add_rmsnorm(float* h, const float* delta, const float* w, float eps, int n, void* out, int out_dtype, const int* row_index,
                          int out_rows, cudaStream_t stream);
GB_API int gb_swiglu(const void* gu, void* out, int dtype, int rows, int inter, int interleave8, cudaStream_t stream);
GB_API int gb_qk_norm_rope_kv_write(const QkRopeParams* p, int dtype, cudaStream_t stream);

// matrix products: C[M, N] = A[M, K] W[N, K]^T
GB_API int gb_gemm_simt(const void* A, int a_dtype, const void* W, int w_dtype, void* C, int c_dtype, int M, int N, int K, int64_t lda,
                        int64_t ldw, int64_t ldc, cudaStream_t stream);
GB_API int gb_gemm_skinny(const void* X, const void* W, void* Y, int c_dtype, int M, int N, int K, int64_t ldx, int64_t ldy, cudaStream_t stream);
GB_API int gb_gemm_skinny_swiglu(const void* X, const void* W, void* Y, int c_dtype, int M, int N, int K, int64_t ldx, int64_t ldy,
                                 cudaStream_t stream);
GB_API int gb_gemm_tc5(const void* A, const void* W, void* C, int c_dtype, int M, int N, int K, int64_t lda, int64_t ldc, cudaStream_t stream);
GB_API int gb_gemm_tc5_swiglu(const void* A, const void* W, void* C, int c_dtype, int M, int N, int K, int64_t lda, int64_t ldc,
                              cudaStream_t stream);
GB_API int gb_gemm_tc5_pair(const void* A, const void* W, void* C, int c_dtype, int M, int N, int K, int64_t lda, int64_t ldc,
                            cudaStream_t stream);
GB_API int gb_gemm_tc5_pair_swiglu(const void* A, const void* W, void* C, int c_dtype, int M, int N, int K, int64_t lda, int64_t ldc,
                                   cudaStream_t stream);
GB_API int gb_gemm_tc5_pair_add(const void* A, const void* W, void* C, int M, int N, int K, int64_t lda, int64_t ldc, cudaStream_t stream);
// most rows the products with the residual's row-wise work folded in take
constexpr int GB_FOLD_MAX_ROWS = 64;
GB_API int gb_gemm_tc5_decode_splits(int M, int N, int K, int sms);
GB_API int gb_gemm_tc5_decode(const void* X, const void* W, void* Y, int c_dtype, int M, int N, int K, int64_t ldx, int64_t ldy, int epi,
                              int splits, cudaStream_t stream);

// attention
GB_API int gb_attention_simt(const AttnParams* p, int dtype, cudaStream_t stream);
GB_API int gb_attention_decode_mma(const AttnParams* p, cudaStream_t stream);
GB_API int gb_attention_prefill_mma(const AttnParams* p, cudaStream_t stream);
GB_API int gb_attention_decode_rope_accepts(int dtype, int d, int rot, int max_q_len);
GB_API int gb_attention_decode_mma_rope(const AttnParams* p, const QkRopeParams* r, cudaStream_t stream);
GB_API int gb_attention_prefill_tc5(const AttnParams* p, int rows, int pages, cudaStream_t stream);
