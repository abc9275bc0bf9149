// Decode attention for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference implementation; it exists for embedders of this
// library that cannot call cudaMalloc themselves and cannot let a library do it for them: code running
// inside a memory pool that owns the whole device, plugins of a host process whose allocator must see
// every byte, and real-time loops in which an allocation (an implicit device synchronisation) is not
// acceptable.  b2_attn_decode needs two scratch buffers for the split-K partial results; here those buffers
// are fixed-size arrays inside the library's own device image, so a call allocates nothing: no cudaMalloc,
// no cudaFree, no allocating library routine.
//
// Cost: every GPU on which the library is loaded holds B2_NA_MAX_ACC_FLOATS * 4 + B2_NA_MAX_ML_ENTRIES * 8
// bytes (about 8.5 MB) until the process exits.
//
// Limits: nb * n_heads * n_splits <= B2_NA_MAX_ML_ENTRIES and nb * n_heads * n_splits * hd <=
// B2_NA_MAX_ACC_FLOATS (for example 8 sequences x 32 heads x 16 splits x head size 128).  Larger problems are
// rejected with B2_NA_ERR_TOO_LARGE before anything is launched.
//
// First call: the first call on each device looks up the device address of the arrays (with that device
// current) and caches it.  Make that first call outside of any stream capture.
//
// Sharing: all calls on a device use the same arrays and each call overwrites what the previous one left
// there.  Nothing needs to start at zero (every slot that is read was written earlier in the same call).
// Two calls whose kernels overlap on the GPU -- different streams without an ordering between them --
// race on the arrays; order them on one stream or with events.
//
// Arguments are those of b2_attn_decode (see attn_decode.cu); the part_acc / part_ml fields of both
// structs are ignored, and so are n_heads / n_splits / hd of the combine struct (taken from the decode
// arguments).  Returns 0, a cudaError_t value, or B2_NA_ERR_TOO_LARGE.
#pragma once
#include <cuda_runtime.h>

#define B2_NA_MAX_ACC_FLOATS (2 * 1024 * 1024)
#define B2_NA_MAX_ML_ENTRIES (16 * 1024)
#define B2_NA_ERR_TOO_LARGE (-2)

struct AttnDecodeArgs;
struct AttnCombineArgs;

extern "C" __attribute__((visibility("default"))) int b2_attn_decode_noalloc(const AttnDecodeArgs* a, const AttnCombineArgs* c, int nb,
                                                                           int hd, cudaStream_t st);
