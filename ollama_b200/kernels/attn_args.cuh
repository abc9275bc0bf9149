// Argument block shared by the decode-attention kernels (scalar split-K kernel and tensor-core split-K kernel).
#pragma once
#include "common.cuh"

struct AttnDecodeArgs {
    const float* q;          // [nb][H][HD]
    const __half* k_cache;   // [slots][Hkv][n_ctx][HD]
    const __half* v_cache;
    const int* positions;    // [nb] position of the query token (its K/V is already in the cache)
    const int* slots;        // [nb]
    int n_heads, n_kv_heads, n_ctx, n_splits;
    float scale, softcap;
    int window;              // 0 = full
    float* part_acc;         // scratch [nb][H][splits][HD]
    float2* part_ml;         // scratch [nb][H][splits] (max, sum)
    const __half* k_scale;   // q8_0 cache (k_cache / v_cache hold int8): [slots][Hkv][n_ctx][HD/32] scales, or null for f16
    const __half* v_scale;
};

// Optional second argument of the tensor-core kernel: with `qkv` set the kernel takes the query rows straight from the
// projection output and rotates them itself, and the CTA whose split holds the query's own position rotates the new key,
// appends key and value to the cache (f16 caches only) and uses them from shared memory, so that no rotary-embedding launch
// precedes the attention.
struct AttnRopeArgs {
    const float* qkv;        // [nb][(H + 2 Hkv) * HD] raw projections (q | k | v), or null: q comes rotated from a.q
    const float* inv_freq;   // [n_rot / 2]
    float mscale;
    int n_rot, neox;
};

// Tensor-core variant (attn_decode_mma.cu): same partial outputs, so the same combine kernel follows.
// Returns cudaErrorNotSupported for shapes it does not take (head size other than 64 / 128, more than 16 query heads per KV head).
int attn_decode_mma_launch(const AttnDecodeArgs& a, int nb, int hd, int pdl, cudaStream_t st);
// The same with the rotary embedding and the cache append inside; cudaErrorNotSupported also for quantised caches and more
// than 256 rotated dimensions.
int attn_decode_mma_rope_launch(const AttnDecodeArgs& a, const AttnRopeArgs& r, int nb, int hd, int pdl, cudaStream_t st);
