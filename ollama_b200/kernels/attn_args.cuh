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

// Tensor-core variant (attn_decode_mma.cu): same partial outputs, so the same combine kernel follows.
// Returns cudaErrorNotSupported for shapes it does not take (head size other than 64 / 128, more than 16 query heads per KV head).
int attn_decode_mma_launch(const AttnDecodeArgs& a, int nb, int hd, int pdl, cudaStream_t st);
