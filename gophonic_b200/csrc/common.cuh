// Shared helpers of the sm_100a kernel library.
//
// Every exported function has C linkage, takes raw device pointers plus a cudaStream_t, launches
// on that stream and returns 0 or a negative status; the text of the last refusal is kept per
// thread and read with gb_last_error().  Sizes a kernel cannot take are refused on the host
// before anything is launched, never computed wrongly.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define GB_API extern "C" __attribute__((visibility("default")))

enum GbDtype : int { GB_F32 = 0, GB_BF16 = 1 };

// Tokens per cache page.  Keys and values of one (page, kv head) are contiguous: [64][head_dim].
#define GB_PAGE 64

void gb_set_error(const char* fmt, ...);

#define GB_REFUSE(...)            \
    do {                          \
        gb_set_error(__VA_ARGS__); \
        return -1;                \
    } while (0)

#define GB_CHECK_LAUNCH(what)                                                       \
    do {                                                                            \
        cudaError_t e__ = cudaGetLastError();                                       \
        if (e__ != cudaSuccess) {                                                   \
            gb_set_error("%s: launch failed: %s", what, cudaGetErrorString(e__));   \
            return -2;                                                              \
        }                                                                           \
    } while (0)

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// The checked build (compiled with -DGB_CHECKED; the stand-in for a memory checker where none can be
// run): every index that reaches the block table, a cache plane, the embedding table or a token
// source is compared with its bound first.  An index out of bounds is recorded (the first one with
// its value and bound, and a count of all) in a status word of the translation unit, and the
// access is skipped or redirected to element 0, so the kernel neither faults nor reads what it should
// not.  The host reads the words of all translation units with gb_checked_status().  In the
// ordinary build the checks compile to nothing.
enum GbCheckCode : int {
    GB_CHECK_TOKEN_ID = 1,       // a token id outside the vocabulary
    GB_CHECK_TOKEN_SOURCE = 2,   // a position outside the token source
    GB_CHECK_SLOT = 3,           // a cache slot outside the block table
    GB_CHECK_LOGICAL_PAGE = 4,   // a position beyond the pages a block-table row has
    GB_CHECK_PHYSICAL_PAGE = 5,  // a block-table entry outside the cache plane
    GB_CHECK_ROPE_POSITION = 6,  // a position beyond the rotation tables
    GB_CHECK_KV_LENGTH = 7,      // a sequence longer than its block-table row can hold, or shorter than its new rows
    GB_CHECK_TRIPLE = 8,         // a (slot, logical, physical) triple outside the table or the plane
};
#ifdef GB_CHECKED
static __device__ int gb_check_word[4];  // first code, its value, its bound, count of all
__device__ __forceinline__ bool gb_check(long long v, long long bound, int code) {
    if (v >= 0 && v < bound) return true;
    if (atomicCAS(&gb_check_word[0], 0, code) == 0) {
        gb_check_word[1] = (int)v;
        gb_check_word[2] = (int)bound;
    }
    atomicAdd(&gb_check_word[3], 1);
    return false;
}
#define GB_CHECK_READER(name)                                                                           \
    GB_API int name(int* out4) {                                                                        \
        int zero[4] = {0, 0, 0, 0};                                                                     \
        if (cudaMemcpyFromSymbol(out4, gb_check_word, sizeof(zero)) != cudaSuccess) return -1;          \
        if (out4[0] != 0 || out4[3] != 0) cudaMemcpyToSymbol(gb_check_word, zero, sizeof(zero));        \
        return out4[0];                                                                                 \
    }
#else
__device__ __forceinline__ bool gb_check(long long, long long, int) { return true; }
#define GB_CHECK_READER(name)                      \
    GB_API int name(int* out4) {                   \
        out4[0] = out4[1] = out4[2] = out4[3] = 0; \
        return 0;                                  \
    }
#endif

// Physical page of token `pos` of the sequence whose block-table row is `bt` (bt_stride entries), in
// a plane of `pages` pages.
__device__ __forceinline__ int64_t page_of(const int* __restrict__ bt, int pos, int bt_stride, int pages) {
    const int lp = pos / GB_PAGE;
    if (!gb_check(lp, bt_stride, GB_CHECK_LOGICAL_PAGE)) return 0;
    const int page = bt[lp];
    if (!gb_check(page, pages, GB_CHECK_PHYSICAL_PAGE)) return 0;
    return (int64_t)page;
}

// Block-table row of the cache slot a sequence lives in.
__device__ __forceinline__ const int* block_table_row(const int* __restrict__ table, int bt_stride, int slot, int max_slots) {
    if (!gb_check(slot, max_slots, GB_CHECK_SLOT)) slot = 0;
    return table + (int64_t)slot * bt_stride;
}

static inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

// Programmatic dependent launch.  A kernel launched with the programmatic-serialization attribute
// may begin while the kernel before it on the stream is still running; it must call pdl_wait()
// before it touches anything that an earlier kernel or copy of the stream writes (or writes
// anything one of them reads): before the wait it may use only its parameters and memory that
// never changes (weights).  Every CTA calls pdl_wait(), also one that has nothing to do, so that
// a kernel never completes before the kernel ahead of it.  A kernel calls pdl_trigger() once the
// kernel after it may begin its own prologue; the kernels here do so after their own wait, so at
// most two kernels overlap.  Both calls are no-ops for ordinary launches.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
// The same wait taken by one thread for its CTA: the others park at the CTA barrier instead of
// each waiting on the grid dependency, which leaves the issue slots of the SM to the kernel that is
// still running beside them.  Every thread of the CTA must call it.
__device__ __forceinline__ void pdl_wait_cta() {
    if (threadIdx.x == 0) pdl_wait();
    __syncthreads();
}
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }

// Launch `kernel` so that it may overlap the tail of its predecessor (see pdl_wait); with
// `dependent` false, as an ordinary launch (the kernel's own wait and trigger are then no-ops).
template <typename... KArgs, typename... Args>
static inline cudaError_t launch_maybe_pdl(bool dependent, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                           cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = dependent ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

template <typename... KArgs, typename... Args>
static inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// The same for a kernel whose CTAs form thread-block clusters of cluster_x x cluster_y.
template <typename... KArgs, typename... Args>
static inline cudaError_t launch_pdl_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                             unsigned cluster_x, unsigned cluster_y, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = cluster_x;
    attr[1].val.clusterDim.y = cluster_y;
    attr[1].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
