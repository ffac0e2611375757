// Warp-level tensor-core and asynchronous-copy primitives shared by the bfloat16 kernels that
// run on mma.sync (the tile-streaming kernels whose operands arrive from the paged cache or in
// fragment order straight from global memory).
#pragma once

#include "common.cuh"

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// 16-byte asynchronous copy global -> shared; src_bytes = 0 writes zeros and reads nothing.
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_u32(smem_dst)), "l"(gmem_src), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem_row) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(smem_u32(smem_row)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem_row) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(smem_u32(smem_row)));
}
__device__ __forceinline__ void ldmatrix_x2(uint32_t (&r)[2], const void* smem_row) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0, %1}, [%2];\n"
                 : "=r"(r[0]), "=r"(r[1])
                 : "r"(smem_u32(smem_row)));
}
__device__ __forceinline__ void ldmatrix_x2_trans(uint32_t (&r)[2], const void* smem_row) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0, %1}, [%2];\n"
                 : "=r"(r[0]), "=r"(r[1])
                 : "r"(smem_u32(smem_row)));
}

// D[16x8] += A[16x16] * B[16x8], bf16 operands, fp32 accumulate.
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                               uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// 16-byte streaming load that does not allocate in L1 (weights are read once).
__device__ __forceinline__ uint4 ld_stream16(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// Warps a CTA of the fragment-streaming products gets at most (they split K), for `tiles` CTAs of 16
// weight rows: few tiles (narrow outputs) leave SMs short of loads in flight, so their CTAs get 16
// warps, wide outputs 8.  Timed alone in chains of the same product, a rule that keeps every CTA
// resident at once (16 warps up to two tiles an SM, 8 up to four, 4 up to eight) looked better at
// the 32B sizes (320 tiles x K 25600: 57.7 -> 49.3 us; 640 x 5120: 23.1 -> 21.0), but inside the
// decode step, between its other kernels, the same rule cost 40 us a layer; the step decides.
static inline int skinny_warps(int tiles) { return tiles <= 320 ? 16 : 8; }

// SMs of the current device (asked once per device).
static inline int gb_sm_count() {
    static int cached[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

// Whether a fragment-streaming product of `tiles` CTAs of `kw` warps is launched as a programmatic
// dependent launch (its CTAs become resident and request their first weights while the kernel ahead
// still runs).  Not when its last wave is thin: two CTAs of 16 warps or four of 8 fit an SM, and a
// grid that fills these places once and leaves a few CTAs over (the 32B sizes: 320 tiles of 16
// warps on 296 places, 640 of 8 on 592) ran a decode step of sixteen 32B layers in 4.50 ms as
// dependent launches and in 3.61 ms as ordinary ones, at one sequence (4.87 and 4.26 ms at eight).
// Grids of one wave, or with a well-filled last wave (the 8B and 1.7B sizes), gain 1-2 % as dependents.
static inline bool skinny_dependent(int tiles, int kw) {
    const int places = (kw >= 16 ? 2 : 4) * gb_sm_count();
    const int last = tiles % places;
    return tiles <= places || last == 0 || 4 * last >= places;
}
