// Single-token attention for callers that must not allocate device memory.
//
// This entry point has no counterpart in GetStream/gophonic; it exists for hosts of this library
// that cannot call cudaMalloc on the path that runs a decode step.  Two kinds of caller are
// meant.  The first is a plain C or C++ serving loop on a latency-critical thread (a voice
// agent's reply loop, for instance): the CUDA allocator takes a process-wide lock and may wait
// for the whole device, so one call can stall every stream for an unbounded time.  The second is
// a process whose device memory has already been handed out in full, for example to another
// component's pool, so that an allocation here would simply fail.
//
// gb_attention_decode_static does what gb_attention_simt does for single-token rows whose keys
// are cut into splits, except that the partial results of the splits do not go through a
// caller-supplied scratch buffer: they go through one array that is part of the library image,
//
//     static __device__ __align__(256) float  of  GB_STATIC_SCRATCH_FLOATS  elements (8 MiB),
//
// which every GPU that loads the library holds until the process exits.  The caller still passes
// every input and the output; the `scratch` field of the parameters is ignored.
//
// Limit.  nseq * heads * num_splits * (head_dim + 2) must not exceed GB_STATIC_SCRATCH_FLOATS;
// a larger request is refused with an error text (gb_last_error) and nothing is launched.
// num_splits must be at least 2 (with one split there is no scratch to speak of: use
// gb_attention_simt) and rows must be single tokens.
//
// Set-up.  The first call on each device looks up the array's device address
// (cudaGetSymbolAddress, with that device current) and keeps it; make that first call before any
// stream capture begins.  No call allocates or frees: not through the CUDA runtime and not
// through any library.  The address is kept in a plain per-device table without a lock: two host
// threads that make the first call on one device at the same time both look the address up and
// both store the same value, which is harmless.
//
// Sharing.  All calls on a device use the same array, and it keeps what the last call left in
// it.  Nothing in it has to start at zero: every slot that the merge reads is written first by
// the same call, including the slots of splits that had no keys.  Two calls that overlap in time
// on one GPU (different streams, or different host threads) race on the array and may both return
// wrong results; run them one after the other.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#define GB_STATIC_SCRATCH_FLOATS (2u * 1024u * 1024u)

struct AttnParams;

extern "C" __attribute__((visibility("default"))) int gb_attention_decode_static(const struct AttnParams* params, int dtype,
                                                                                 cudaStream_t stream);

// the largest nseq * heads * num_splits * (head_dim + 2) the entry point takes
extern "C" __attribute__((visibility("default"))) unsigned int gb_static_scratch_floats(void);
