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

// How a fragment-streaming product of `tiles` CTAs of 16 weight rows is launched: the most warps a
// CTA gets (they split K), and whether it is a programmatic dependent launch (its CTAs become
// resident and request their first weights while the kernel ahead still runs).  At 64 registers a
// thread an SM holds two CTAs of 16 warps, four of 8 or eight of 4.  Few tiles (narrow outputs)
// leave SMs short of loads in flight, so their CTAs get more warps; a product whose CTAs are not all
// resident at once ends in a thin wave that costs as much as a full one.  Measured inside decode
// steps of the 1.7B, 8B and 32B sizes (alone, in chains of the same product, the picture differs:
// the step decides):
//   up to two tiles an SM (8B output and down projections, 256 tiles): 16 warps, dependent;
//   up to 320 tiles (32B output and down projections): 8 warps, ordinary launch; with 16 warps
//     they leave 24 CTAs for a second wave, and as dependents of 8 warps they cost a third more;
//   up to four tiles an SM (8B q/k/v, 384 tiles): 8 warps, dependent;
//   up to eight (32B q/k/v, 640; 1.7B gate/up, 768): 4 warps, ordinary launch;
//   wider (8B gate/up, 1536): 8 warps, dependent.
// Against 16 warps up to 320 tiles, 8 beyond, all dependents: sixteen 32B layers at one sequence
// 4.50 -> 3.26 ms (eight: 4.87 -> 3.62), 1.7B 1.30 -> 1.26 ms, 8B unchanged.
static inline int skinny_warps(int tiles) {
    const int sms = gb_sm_count();
    if (tiles <= 2 * sms) return 16;
    if (tiles <= 4 * sms) return 8;
    if (tiles <= 8 * sms) return 4;
    return 8;
}

static inline bool skinny_dependent(int tiles) {
    const int sms = gb_sm_count();
    if (tiles <= 2 * sms) return true;
    if (tiles <= 320) return false;
    if (tiles <= 4 * sms) return true;
    if (tiles <= 8 * sms) return false;
    return true;
}
