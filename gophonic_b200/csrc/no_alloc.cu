// See no_alloc.h: single-token split-key attention whose scratch is a static device array.
#include "no_alloc.h"
#include "api.h"

#include "common.cuh"

// the layout of attention_simt.cu's parameters

extern "C" int gb_attention_simt(const AttnParams* pp, int dtype, cudaStream_t stream);

// Partial results of the key splits: [nseq][heads][num_splits][head_dim + 2] floats.  In host code
// this name is only a handle for cudaGetSymbolAddress, never a pointer a kernel may be given.
static __device__ __align__(256) float g_static_scratch[GB_STATIC_SCRATCH_FLOATS];

// Device code may name the array directly; this kernel is never launched and only keeps the
// array referenced from device code, so that it stays in the image.
__global__ void static_scratch_reference_kernel(float* out) {
    if (out) out[0] = g_static_scratch[0];
}

namespace {
constexpr int MAX_DEVICES = 64;
float* g_scratch_address[MAX_DEVICES];  // per device, filled by that device's first call
}  // namespace

GB_API unsigned int gb_static_scratch_floats(void) { return GB_STATIC_SCRATCH_FLOATS; }

GB_API int gb_attention_decode_static(const AttnParams* params, int dtype, cudaStream_t stream) {
    if (!params) GB_REFUSE("attention_decode_static: no parameters");
    AttnParams p = *params;
    if (p.nseq <= 0) return 0;
    if (p.max_q_len != 1) GB_REFUSE("attention_decode_static: rows of up to %d tokens; this entry point takes single tokens", p.max_q_len);
    if (p.num_splits < 2) GB_REFUSE("attention_decode_static: %d key splits; at least 2 are needed for the scratch to be used", p.num_splits);
    if (p.heads <= 0 || p.d <= 0) GB_REFUSE("attention_decode_static: %d heads of width %d", p.heads, p.d);
    unsigned long long need = (unsigned long long)p.nseq * (unsigned long long)p.heads * (unsigned long long)p.num_splits *
                              (unsigned long long)(p.d + 2);
    if (need > GB_STATIC_SCRATCH_FLOATS)
        GB_REFUSE("attention_decode_static: %d sequences x %d heads x %d splits x (%d + 2) = %llu floats exceed the static "
                  "scratch of %u floats; use fewer splits or the entry point that takes caller scratch",
                  p.nseq, p.heads, p.num_splits, p.d, need, GB_STATIC_SCRATCH_FLOATS);
    int device = -1;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) GB_REFUSE("attention_decode_static: cudaGetDevice: %s", cudaGetErrorString(e));
    if (device < 0 || device >= MAX_DEVICES) GB_REFUSE("attention_decode_static: device %d is beyond the %d this entry point tracks", device, MAX_DEVICES);
    if (g_scratch_address[device] == nullptr) {
        // set-up, once per device, with that device current
        float* ptr = nullptr;
        e = cudaGetSymbolAddress((void**)&ptr, g_static_scratch);
        if (e != cudaSuccess || ptr == nullptr)
            GB_REFUSE("attention_decode_static: cannot find the static scratch on device %d: %s", device, cudaGetErrorString(e));
        g_scratch_address[device] = ptr;
    }
    p.scratch = g_scratch_address[device];
    return gb_attention_simt(&p, dtype, stream);
}
