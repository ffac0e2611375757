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

// Physical page of token `pos` of the sequence whose block-table row is `bt`.
__device__ __forceinline__ int64_t page_of(const int* __restrict__ bt, int pos) { return (int64_t)bt[pos / GB_PAGE]; }

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
