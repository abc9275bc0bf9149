// Split-K decode attention over the slot-partitioned f16 KV cache, sm_100a.
//
// One query token per sequence.  grid = (splits, kv_head * head_groups, sequences).  Every CTA owns
// a contiguous range of cached positions of one (sequence, kv head) and G query heads that share
// that kv head (grouped-query attention: K/V are read once for G heads).  Inside a warp, LP = HD/16
// lanes cooperate on one cached position (each lane holds 16 dims = one 32-byte load of K and one of
// V), so a warp walks 32/LP positions per step with fully coalesced loads and keeps the running
// soft-max statistics and the output accumulator in registers.  Lane groups, warps and finally the
// splits are merged with the usual (max, sum, acc) rescaling; the merge of the splits, the attention
// sinks, the normalisation and the int8 re-quantisation for the output projection happen in the
// combine kernel.  Masks: causal by construction (only positions <= the query position are stored),
// optional sliding window, optional logit soft-cap.
#include <stdlib.h>

#include "attn_args.cuh"

template <int HD, int G>
__device__ __forceinline__ void attn_decode_body(const AttnDecodeArgs& a) {
    constexpr int LP = HD / 16;          // lanes per position
    constexpr int PPW = 32 / LP;         // positions per warp step
    const int split = blockIdx.x, b = blockIdx.z;
    const int group = a.n_heads / a.n_kv_heads;
    const int hg_per_kv = group / G;
    const int kvh = blockIdx.y / hg_per_kv, hg = blockIdx.y % hg_per_kv;
    const int head0 = kvh * group + hg * G;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int sub = lane % LP, pg = lane / LP;

    pdl_launch();
    pdl_wait();
    const int qpos = a.positions[b], slot = a.slots[b];
    const int kv_len = qpos + 1;
    const int start = (a.window > 0 && kv_len > a.window) ? kv_len - a.window : 0;
    const int span = kv_len - start;
    int chunk = (span + a.n_splits - 1) / a.n_splits;
    chunk = ((chunk + PPW * 4 - 1) / (PPW * 4)) * (PPW * 4);
    const int p0 = start + split * chunk, p1 = min(p0 + chunk, kv_len);

    float q[G][16], acc[G][16], m[G], l[G];
#pragma unroll
    for (int g = 0; g < G; g++) {
        const float* qp = a.q + ((size_t)b * a.n_heads + head0 + g) * HD + sub * 16;
#pragma unroll
        for (int i = 0; i < 16; i += 4) {
            const float4 t = *(const float4*)(qp + i);
            q[g][i] = t.x * a.scale; q[g][i + 1] = t.y * a.scale; q[g][i + 2] = t.z * a.scale; q[g][i + 3] = t.w * a.scale;
        }
#pragma unroll
        for (int i = 0; i < 16; i++) acc[g][i] = 0.f;
        m[g] = -1e30f;
        l[g] = 0.f;
    }
    const size_t base = ((size_t)slot * a.n_kv_heads + kvh) * a.n_ctx;
    // uniform trip count for the whole warp (the shuffles below need every lane); lanes whose position
    // falls beyond the range load a clamped address and skip the soft-max update
    for (int pb = p0 + warp * PPW; pb < p1; pb += 4 * PPW) {
        const int p = pb + pg;
        const bool valid = p < p1;
        const int pc = valid ? p : p1 - 1;
        float kf[16], vf[16];
        if (a.k_scale) {      // q8_0 cache: 16 int8 per lane and the scale of their block of 32
            const uint4 kq = *(const uint4*)(reinterpret_cast<const int8_t*>(a.k_cache) + (base + pc) * HD + sub * 16);
            const uint4 vq = *(const uint4*)(reinterpret_cast<const int8_t*>(a.v_cache) + (base + pc) * HD + sub * 16);
            const float dk = __half2float(a.k_scale[(base + pc) * (HD / 32) + (sub >> 1)]);
            const float dv = __half2float(a.v_scale[(base + pc) * (HD / 32) + (sub >> 1)]);
            const uint32_t kw[4] = {kq.x, kq.y, kq.z, kq.w}, vw[4] = {vq.x, vq.y, vq.z, vq.w};
#pragma unroll
            for (int i = 0; i < 16; i++) {
                kf[i] = dk * (float)(int8_t)((kw[i >> 2] >> (8 * (i & 3))) & 0xff);
                vf[i] = dv * (float)(int8_t)((vw[i >> 2] >> (8 * (i & 3))) & 0xff);
            }
        } else {
            const __half* kp = a.k_cache + (base + pc) * HD + sub * 16;
            const __half* vp = a.v_cache + (base + pc) * HD + sub * 16;
            const uint4 k0 = *(const uint4*)kp, k1 = *(const uint4*)(kp + 8);
            const uint4 v0 = *(const uint4*)vp, v1 = *(const uint4*)(vp + 8);
            const __half2* h = reinterpret_cast<const __half2*>(&k0);
            const __half2* h2 = reinterpret_cast<const __half2*>(&k1);
            const __half2* w = reinterpret_cast<const __half2*>(&v0);
            const __half2* w2 = reinterpret_cast<const __half2*>(&v1);
#pragma unroll
            for (int i = 0; i < 4; i++) {
                float2 t = __half22float2(h[i]); kf[2 * i] = t.x; kf[2 * i + 1] = t.y;
                t = __half22float2(h2[i]); kf[8 + 2 * i] = t.x; kf[8 + 2 * i + 1] = t.y;
                t = __half22float2(w[i]); vf[2 * i] = t.x; vf[2 * i + 1] = t.y;
                t = __half22float2(w2[i]); vf[8 + 2 * i] = t.x; vf[8 + 2 * i + 1] = t.y;
            }
        }
#pragma unroll
        for (int g = 0; g < G; g++) {
            float s = 0.f;
#pragma unroll
            for (int i = 0; i < 16; i++) s += q[g][i] * kf[i];
#pragma unroll
            for (int o = 1; o < LP; o <<= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
            if (a.softcap > 0.f) s = a.softcap * tanhf(s / a.softcap);
            // no divergent control flow here: the next head's shuffles need the whole warp converged
            const float mn = valid ? fmaxf(m[g], s) : m[g];
            const float corr = __expf(m[g] - mn), pr = valid ? __expf(s - mn) : 0.f;
            l[g] = l[g] * corr + pr;
#pragma unroll
            for (int i = 0; i < 16; i++) acc[g][i] = acc[g][i] * corr + pr * vf[i];
            m[g] = mn;
        }
    }
    __syncwarp();
    // merge the PPW lane groups of the warp
#pragma unroll
    for (int o = LP; o < 32; o <<= 1) {
#pragma unroll
        for (int g = 0; g < G; g++) {
            const float mo = __shfl_xor_sync(0xffffffffu, m[g], o), lo = __shfl_xor_sync(0xffffffffu, l[g], o);
            const float mn = fmaxf(m[g], mo);
            const float c0 = __expf(m[g] - mn), c1 = __expf(mo - mn);
            l[g] = l[g] * c0 + lo * c1;
#pragma unroll
            for (int i = 0; i < 16; i++) {
                const float ao = __shfl_xor_sync(0xffffffffu, acc[g][i], o);
                acc[g][i] = acc[g][i] * c0 + ao * c1;
            }
            m[g] = mn;
        }
    }
    // merge the four warps through shared memory
    __shared__ float s_acc[4][G][HD];
    __shared__ float s_m[4][G], s_l[4][G];
    if (pg == 0) {
#pragma unroll
        for (int g = 0; g < G; g++) {
#pragma unroll
            for (int i = 0; i < 16; i++) s_acc[warp][g][sub * 16 + i] = acc[g][i];
            if (sub == 0) { s_m[warp][g] = m[g]; s_l[warp][g] = l[g]; }
        }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < G * HD; idx += 128) {
        const int g = idx / HD, d = idx % HD;
        float mn = fmaxf(fmaxf(s_m[0][g], s_m[1][g]), fmaxf(s_m[2][g], s_m[3][g]));
        float o = 0.f, lt = 0.f;
#pragma unroll
        for (int w = 0; w < 4; w++) {
            const float c = __expf(s_m[w][g] - mn);
            o += s_acc[w][g][d] * c;
            lt += s_l[w][g] * c;
        }
        const size_t pi = ((size_t)b * a.n_heads + head0 + g) * a.n_splits + split;
        a.part_acc[pi * HD + d] = o;
        if (d == 0) a.part_ml[pi] = make_float2(mn, lt);
    }
}

template <int HD, int G>
__global__ void __launch_bounds__(128) attn_decode_kernel(const __grid_constant__ AttnDecodeArgs a) {
    attn_decode_body<HD, G>(a);
}

struct AttnCombineArgs {
    const float* part_acc;
    const float2* part_ml;
    const float* sinks;      // [H] or null
    int n_heads, n_splits, hd;
    float* out;              // [nb][H*hd] or null
    int8_t* out_q;           // [nb][H*hd] or null
    float2* out_ds;          // [nb][H*hd/32]
};

// grid = (H, nb), block = hd threads (multiple of 32)
__global__ void attn_combine_kernel(const __grid_constant__ AttnCombineArgs a) {
    const int h = blockIdx.x, b = blockIdx.y, d = threadIdx.x;
    pdl_launch();
    pdl_wait();
    const size_t p0 = ((size_t)b * a.n_heads + h) * a.n_splits;
    float mn = -1e30f;
    for (int s = 0; s < a.n_splits; s++) mn = fmaxf(mn, a.part_ml[p0 + s].x);
    if (a.sinks) mn = fmaxf(mn, a.sinks[h]);
    float o = 0.f, l = 0.f;
    for (int s = 0; s < a.n_splits; s++) {
        const float2 ml = a.part_ml[p0 + s];
        const float c = __expf(ml.x - mn);
        o += a.part_acc[(p0 + s) * a.hd + d] * c;
        l += ml.y * c;
    }
    if (a.sinks) l += __expf(a.sinks[h] - mn);
    const float v = l > 0.f ? o / l : 0.f;
    const size_t oi = ((size_t)b * a.n_heads + h) * a.hd + d;
    if (a.out) a.out[oi] = v;
    if (a.out_q) {
        const float amax = warp_max(fabsf(v));
        const float dq = amax / 127.f;
        const int q = dq > 0.f ? __float2int_rn(v / dq) : 0;
        const float s = dq * warp_sum((float)q);
        a.out_q[oi] = (int8_t)q;
        if ((d & 31) == 0) a.out_ds[oi >> 5] = make_float2(dq, s);
    }
}

// Split-K attention with the combine folded in: the CTA that finishes last for a (sequence, head group) merges the
// splits of its heads, applies the sink, normalises and re-quantises, so the step needs one launch instead of two.
struct AttnFusedArgs {
    AttnDecodeArgs d;
    AttnCombineArgs c;
    unsigned* tickets;       // [nb][gridDim.y], zero before the first launch (the last CTA of a group resets its counter)
};

template <int HD, int G>
__global__ void __launch_bounds__(128) attn_decode_fused_kernel(const __grid_constant__ AttnFusedArgs f) {
    attn_decode_body<HD, G>(f.d);
    __shared__ int s_last;
    __threadfence();                     // this CTA's partials are visible before its ticket is
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned* t = f.tickets + (size_t)blockIdx.z * gridDim.y + blockIdx.y;
        const unsigned prev = atomicAdd(t, 1u);
        s_last = prev == gridDim.x - 1;
        if (s_last) *t = 0u;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    const AttnCombineArgs& c = f.c;
    const int b = blockIdx.z;
    const int group = f.d.n_heads / f.d.n_kv_heads, hg_per_kv = group / G;
    const int head0 = (blockIdx.y / hg_per_kv) * group + (blockIdx.y % hg_per_kv) * G;
    for (int idx = threadIdx.x; idx < G * HD; idx += 128) {
        const int h = head0 + idx / HD, d = idx % HD;
        const size_t p0 = ((size_t)b * c.n_heads + h) * c.n_splits;
        float mn = -1e30f;
        for (int s = 0; s < c.n_splits; s++) mn = fmaxf(mn, __ldcg(&c.part_ml[p0 + s]).x);
        if (c.sinks) mn = fmaxf(mn, c.sinks[h]);
        float o = 0.f, l = 0.f;
        for (int s = 0; s < c.n_splits; s++) {
            const float2 ml = __ldcg(&c.part_ml[p0 + s]);
            const float w = __expf(ml.x - mn);
            o += __ldcg(&c.part_acc[(p0 + s) * HD + d]) * w;
            l += ml.y * w;
        }
        if (c.sinks) l += __expf(c.sinks[h] - mn);
        const float v = l > 0.f ? o / l : 0.f;
        const size_t oi = ((size_t)b * c.n_heads + h) * HD + d;
        if (c.out) c.out[oi] = v;
        if (c.out_q) {
            const float amax = warp_max(fabsf(v));
            const float dq = amax / 127.f;
            const int q = dq > 0.f ? __float2int_rn(v / dq) : 0;
            const float sq = dq * warp_sum((float)q);
            c.out_q[oi] = (int8_t)q;
            if ((d & 31) == 0) c.out_ds[oi >> 5] = make_float2(dq, sq);
        }
    }
}

template <int HD>
static const void* pick_decode_fused(int g) {
    if (g >= 4) return (const void*)attn_decode_fused_kernel<HD, 4>;
    if (g >= 2) return (const void*)attn_decode_fused_kernel<HD, 2>;
    return (const void*)attn_decode_fused_kernel<HD, 1>;
}

template <int HD>
static const void* pick_decode(int g) {
    if (g >= 4) return (const void*)attn_decode_kernel<HD, 4>;
    if (g >= 2) return (const void*)attn_decode_kernel<HD, 2>;
    return (const void*)attn_decode_kernel<HD, 1>;
}

static cudaError_t launch1(const void* fn, dim3 grid, dim3 block, void** args, cudaStream_t st, int pdl) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = pdl ? 1 : 0;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    return cudaLaunchKernelExC(&cfg, fn, args);
}

// Tensor-core kernel or scalar kernel: B200_ATTN_MMA = 1 / 0 forces the choice; otherwise grouped-query models
// (two or more query heads per KV head, head size 64 or 128) take the tensor-core kernel.  Measured on Llama-8B
// (4 heads per KV head): 443 against 428 tok/s at 0.6 k tokens of context, 383 against 329 at 6.2 k.
static int g_mma_mode = -2, g_mma_min_ctx = 0;      // -2: not read from the environment yet, -1: automatic

static bool use_mma(const AttnDecodeArgs& a, int hd) {
    if (g_mma_mode == -2) {
        const char* e = getenv("B200_ATTN_MMA");
        g_mma_mode = e ? atoi(e) : -1;
        const char* c = getenv("B200_ATTN_MMA_CTX");
        if (c) g_mma_min_ctx = atoi(c);
    }
    if (hd != 64 && hd != 128) return false;
    if (g_mma_mode >= 0) return g_mma_mode != 0;
    return a.n_heads / a.n_kv_heads >= 2 && a.n_ctx >= g_mma_min_ctx;
}

// Overrides the choice for this process: 1 tensor-core kernel, 0 scalar kernel, -1 automatic.
B2_API void b2_attn_decode_mode(int mode) { g_mma_mode = mode < -1 ? -1 : mode; }

// Scratch needed by b2_attn_decode: part_acc = nb*H*splits*hd floats, part_ml = nb*H*splits float2.
B2_API int b2_attn_decode(const AttnDecodeArgs* a, const AttnCombineArgs* c, int nb, int hd, int pdl, cudaStream_t st) {
    const int group = a->n_heads / a->n_kv_heads;
    int G = group >= 4 && group % 4 == 0 ? 4 : (group % 2 == 0 ? 2 : 1);
    const void* fn = nullptr;
    if (hd == 64) fn = pick_decode<64>(G);
    else if (hd == 128) fn = pick_decode<128>(G);
    else if (hd == 256) fn = pick_decode<256>(G);
    else if (hd == 32) fn = pick_decode<32>(G);
    else return (int)cudaErrorInvalidValue;
    dim3 grid(a->n_splits, a->n_kv_heads * (group / G), nb);
    AttnDecodeArgs ca = *a;
    void* args[] = {&ca};
    cudaError_t e = cudaErrorNotSupported;
    if (use_mma(*a, hd)) e = (cudaError_t)attn_decode_mma_launch(*a, nb, hd, pdl, st);
    if (e == cudaErrorNotSupported) e = launch1(fn, grid, dim3(128), args, st, pdl);
    if (e != cudaSuccess) return (int)e;
    AttnCombineArgs cc = *c;
    void* args2[] = {&cc};
    return (int)launch1((const void*)attn_combine_kernel, dim3(a->n_heads, nb), dim3(hd), args2, st, pdl);
}

// Split-K attention on raw projections: rotary embedding of the queries, rotation + cache append of the new key / value and the
// attention itself in one launch (tensor-core kernel only), then the merge of the splits.  Returns cudaErrorNotSupported
// (nothing launched) for shapes, cache encodings or rotary settings that kernel does not take: the caller then runs
// b2_rope_kv + b2_attn_decode.
B2_API int b2_attn_decode_rope(const AttnDecodeArgs* a, const AttnRopeArgs* r, const AttnCombineArgs* c, int nb, int hd, int pdl, cudaStream_t st) {
    if (!r || !r->qkv) return (int)cudaErrorInvalidValue;
    const cudaError_t e = (cudaError_t)attn_decode_mma_rope_launch(*a, *r, nb, hd, pdl, st);
    if (e != cudaSuccess) return (int)e;
    AttnCombineArgs cc = *c;
    void* args2[] = {&cc};
    return (int)launch1((const void*)attn_combine_kernel, dim3(a->n_heads, nb), dim3(hd), args2, st, pdl);
}

// One launch: split-K attention with the merge of the splits done by the last CTA of every head group.
// `tickets`: nb * n_kv_heads * (group / G) zero-initialised counters (at most nb * n_heads).
B2_API int b2_attn_decode_fused(const AttnDecodeArgs* a, const AttnCombineArgs* c, unsigned* tickets, int nb, int hd, int pdl, cudaStream_t st) {
    const int group = a->n_heads / a->n_kv_heads;
    int G = group >= 4 && group % 4 == 0 ? 4 : (group % 2 == 0 ? 2 : 1);
    const void* fn = nullptr;
    if (hd == 64) fn = pick_decode_fused<64>(G);
    else if (hd == 128) fn = pick_decode_fused<128>(G);
    else if (hd == 256) fn = pick_decode_fused<256>(G);
    else if (hd == 32) fn = pick_decode_fused<32>(G);
    else return (int)cudaErrorInvalidValue;
    dim3 grid(a->n_splits, a->n_kv_heads * (group / G), nb);
    AttnFusedArgs f{*a, *c, tickets};
    void* args[] = {&f};
    return (int)launch1(fn, grid, dim3(128), args, st, pdl);
}

// ---------------------------------------------------------------------------------------------
// Allocation-free entry point (declared in no_alloc.h)
// ---------------------------------------------------------------------------------------------
#include "no_alloc.h"

#include <mutex>

// The split-K partials live in these two arrays instead of caller-provided scratch.  They belong to the
// library image: every GPU that loads the library carries them (about 8.5 MB) until the process exits.
static __device__ __align__(256) float g_na_part_acc[B2_NA_MAX_ACC_FLOATS];
static __device__ __align__(256) float2 g_na_part_ml[B2_NA_MAX_ML_ENTRIES];

// In host code the two names above are only handles for the runtime; the device addresses that a kernel
// can dereference are looked up once per device and kept here.
static constexpr int kNaMaxDevices = 64;
static float* s_na_acc[kNaMaxDevices];
static float2* s_na_ml[kNaMaxDevices];
static std::mutex s_na_mutex;

B2_API int b2_attn_decode_noalloc(const AttnDecodeArgs* a, const AttnCombineArgs* c, int nb, int hd, cudaStream_t st) {
    if (!a || !c || nb < 1 || a->n_heads < 1 || a->n_kv_heads < 1 || a->n_splits < 1 || hd < 1) return (int)cudaErrorInvalidValue;
    const long long entries = (long long)nb * a->n_heads * a->n_splits;
    if (entries > B2_NA_MAX_ML_ENTRIES || entries * hd > B2_NA_MAX_ACC_FLOATS) return B2_NA_ERR_TOO_LARGE;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= kNaMaxDevices) return (int)cudaErrorInvalidDevice;
    float* acc;
    float2* ml;
    {
        std::lock_guard<std::mutex> lock(s_na_mutex);
        if (!s_na_acc[dev]) {      // first call on this device (the device is current): resolve the symbols
            void* p0 = nullptr;
            void* p1 = nullptr;
            e = cudaGetSymbolAddress(&p0, g_na_part_acc);
            if (e != cudaSuccess) return (int)e;
            e = cudaGetSymbolAddress(&p1, g_na_part_ml);
            if (e != cudaSuccess) return (int)e;
            s_na_acc[dev] = (float*)p0;
            s_na_ml[dev] = (float2*)p1;
        }
        acc = s_na_acc[dev];
        ml = s_na_ml[dev];
    }
    AttnDecodeArgs da = *a;
    AttnCombineArgs ca = *c;
    da.part_acc = acc;
    da.part_ml = ml;
    ca.part_acc = acc;
    ca.part_ml = ml;
    ca.n_heads = a->n_heads;
    ca.n_splits = a->n_splits;
    ca.hd = hd;
    // Every (sequence, head, split) slot that the combine step reads is written by the attention kernel of
    // the same call -- empty splits store a neutral partial -- so nothing has to be cleared between calls.
    return b2_attn_decode(&da, &ca, nb, hd, 0, st);
}
