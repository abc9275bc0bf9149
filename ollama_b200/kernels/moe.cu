// Mixture-of-experts glue for sm_100a: router gating (softmax / top-k in either order) and the weighted
// combination of the selected experts' outputs.  The expert matrix products themselves are the indirect
// forms of the GEMV / GLU kernels (kernels/gemv.cu, `ids`): one grid row per (token, expert-slot) pair.
//
// In the reference stack these are ggml-cuda's topk-moe / argsort / softmax kernels and the ids paths of
// mul_mat_id and add_id.
#include "comm.cuh"

struct MoeRouteArgs {
    const float* logits;   // [tokens][ld]
    int ld;
    int n_experts;         // <= 512
    int k;                 // experts per token, <= 16
    int mode;              // 0: softmax over all experts, then top-k (optionally renormalised); 1: top-k, then softmax over the selected
    int norm_topk;
    int e_lo, e_cnt;       // experts resident on this GPU: [e_lo, e_lo + e_cnt)
    int* ids;              // [tokens][k] global expert ids
    int* lids;             // [tokens][k] id relative to e_lo, or -1 when the expert lives elsewhere
    float* wts;            // [tokens][k]
};

// one warp per token
__global__ void __launch_bounds__(128) moe_route_kernel(const __grid_constant__ MoeRouteArgs a, int tokens) {
    constexpr int MAXJ = 16;
    pdl_launch();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int t = blockIdx.x * 4 + (threadIdx.x >> 5);
    if (t >= tokens) return;
    const float* lg = a.logits + (size_t)t * a.ld;
    float v[MAXJ];
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < MAXJ; j++) {
        const int e = lane + 32 * j;
        v[j] = e < a.n_experts ? lg[e] : -INFINITY;
        mx = fmaxf(mx, v[j]);
    }
    mx = warp_max(mx);
    float denom = 0.f;
    if (a.mode == 0) {
#pragma unroll
        for (int j = 0; j < MAXJ; j++) denom += (lane + 32 * j < a.n_experts) ? __expf(v[j] - mx) : 0.f;
        denom = warp_sum(denom);
    }
    float sel_v = 0.f;     // lane s keeps the value of the s-th selected expert
    int sel_e = 0;
    for (int s = 0; s < a.k; s++) {
        float bv = -INFINITY;
        int be = 0x7fffffff;
#pragma unroll
        for (int j = 0; j < MAXJ; j++) {
            const int e = lane + 32 * j;
            if (v[j] > bv) { bv = v[j]; be = e; }      // ascending e within a lane: the lowest index wins ties
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oe = __shfl_xor_sync(0xffffffffu, be, o);
            if (ov > bv || (ov == bv && oe < be)) { bv = ov; be = oe; }
        }
        if (lane == s) { sel_v = bv; sel_e = be; }
#pragma unroll
        for (int j = 0; j < MAXJ; j++)
            if (lane + 32 * j == be) v[j] = -INFINITY;
    }
    const bool mine = lane < a.k;
    float w;
    if (a.mode == 0) {
        w = mine ? __expf(sel_v - mx) / denom : 0.f;
        if (a.norm_topk) w /= warp_sum(w);
    } else {
        const float top = __shfl_sync(0xffffffffu, sel_v, 0);          // the first selected is the largest
        const float ex = mine ? __expf(sel_v - top) : 0.f;
        w = ex / warp_sum(ex);
    }
    if (mine) {
        const size_t o = (size_t)t * a.k + lane;
        a.ids[o] = sel_e;
        const int l = sel_e - a.e_lo;
        a.lids[o] = (l >= 0 && l < a.e_cnt) ? l : -1;
        a.wts[o] = w;
    }
}

B2_API int b2_moe_route(const MoeRouteArgs* a, int tokens, int pdl, cudaStream_t st) {
    if (tokens < 1 || a->n_experts < 1 || a->n_experts > 512 || a->k < 1 || a->k > 16 || a->k > a->n_experts) return (int)cudaErrorInvalidValue;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((tokens + 3) / 4);
    cfg.blockDim = dim3(128);
    cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = pdl ? 1 : 0;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    MoeRouteArgs copy = *a;
    void* args[] = {&copy, &tokens};
    return (int)cudaLaunchKernelExC(&cfg, (const void*)moe_route_kernel, args);
}

// ---------------------------------------------------------------------------------------------
// x[t] += sum_s wts[t][s] * y[t * k + s]      (y rows of experts that live elsewhere are zero)
// With a CommSend (low-latency protocol) the weighted sum is not added locally: it is this GPU's partial
// result of an expert-parallel layer and goes, tagged with the epoch, into every rank's receive buffer; the
// following add + RMSNorm kernel sums the ranks' partial rows into the residual stream.
// ---------------------------------------------------------------------------------------------
struct MoeCombineArgs {
    const float* y;        // [tokens * k][d]
    const float* wts;      // [tokens][k]
    int k;
    int d;                 // multiple of 4
    float* x;              // [tokens][d]
    CommSend cm;
};

__global__ void __launch_bounds__(256) moe_combine_kernel(const __grid_constant__ MoeCombineArgs a) {
    pdl_launch();
    pdl_wait();
    const int t = blockIdx.x;
    const unsigned ep = a.cm.n_dst > 0 ? comm_next_epoch(a.cm) : 0u;
    const long long poff = a.cm.n_dst > 0 ? comm_parity_off(a.cm, ep) : 0ll;
    for (int c = threadIdx.x; c < (a.d >> 2); c += 256) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int s = 0; s < a.k; s++) {
            const float w = a.wts[(size_t)t * a.k + s];
            const float4 v = *(const float4*)(a.y + ((size_t)t * a.k + s) * a.d + 4 * c);
            acc.x += w * v.x; acc.y += w * v.y; acc.z += w * v.z; acc.w += w * v.w;
        }
        if (a.cm.n_dst > 0) {
            const long long o = poff + (long long)t * a.d + 4 * c;
            const uint4 lo = make_uint4(__float_as_uint(acc.x), ep, __float_as_uint(acc.y), ep);
            const uint4 hi = make_uint4(__float_as_uint(acc.z), ep, __float_as_uint(acc.w), ep);
            for (int r = 0; r < a.cm.n_dst; r++) {
                uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<uint2*>(a.cm.dst[r]) + o);
                dst[0] = lo;
                dst[1] = hi;
            }
        } else {
            float4* xp = (float4*)(a.x + (size_t)t * a.d + 4 * c);
            float4 xv = *xp;
            xv.x += acc.x; xv.y += acc.y; xv.z += acc.z; xv.w += acc.w;
            *xp = xv;
        }
    }
}

B2_API int b2_moe_combine(const MoeCombineArgs* a, int tokens, int pdl, cudaStream_t st) {
    if (tokens < 1 || (a->d & 3) || a->k < 1 || (a->cm.n_dst > 0 && !a->cm.ll)) return (int)cudaErrorInvalidValue;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(tokens);
    cfg.blockDim = dim3(256);
    cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = pdl ? 1 : 0;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    MoeCombineArgs copy = *a;
    void* args[] = {&copy};
    return (int)cudaLaunchKernelExC(&cfg, (const void*)moe_combine_kernel, args);
}

// ---------------------------------------------------------------------------------------------
// Grouped prefill.  The (token, expert-slot) pairs of a chunk are laid out in a buffer sorted by expert in which every
// expert's rows start at a multiple of 128, so that one tensor-core GEMM launch with a tile -> expert table covers all
// experts (kernels/gemm_tc.cu, b2_gemm_bf16_grouped).  Everything happens on the device: no count ever visits the host.
// ---------------------------------------------------------------------------------------------
struct MoePlanArgs {
    const int* lids;       // [pairs] expert index on this GPU, or -1
    int pairs;
    int n_experts;         // experts on this GPU, <= 512
    int* row_of_pair;      // [pairs] row of the pair in the sorted buffer, or -1
    int* tile_expert;      // [max_tiles] expert of every 128-row tile, -1 for tiles without rows
    int max_tiles;
};

// one CTA: count, scan the padded counts, hand out rows.  The order of the pairs inside an expert depends on the atomics, the
// value computed for a pair does not.
__global__ void __launch_bounds__(1024) moe_plan_kernel(const __grid_constant__ MoePlanArgs a) {
    __shared__ int cnt[512], off[513], cur[512];
    const int tid = threadIdx.x;
    for (int e = tid; e < a.n_experts; e += 1024) cnt[e] = cur[e] = 0;
    __syncthreads();
    for (int p = tid; p < a.pairs; p += 1024) {
        const int l = a.lids[p];
        if (l >= 0 && l < a.n_experts) atomicAdd(&cnt[l], 1);
    }
    __syncthreads();
    if (tid == 0) {
        int o = 0;
        for (int e = 0; e < a.n_experts; e++) {
            off[e] = o;
            o += (cnt[e] + 127) & ~127;
        }
        off[a.n_experts] = o;
    }
    __syncthreads();
    for (int t = tid; t < a.max_tiles; t += 1024) {
        // the expert whose padded range holds row 128 t (ranges are ascending: a short linear search per tile)
        int e = -1;
        const int row = t * 128;
        if (row < off[a.n_experts]) {
            int lo = 0, hi = a.n_experts - 1;
            while (lo < hi) {
                const int mid = (lo + hi + 1) >> 1;
                if (off[mid] <= row) lo = mid; else hi = mid - 1;
            }
            e = lo;
            // experts without rows share their offset with the next one: step to the one that owns the row
            while (e < a.n_experts - 1 && off[e + 1] <= row) e++;
            if (row >= off[e] + ((cnt[e] + 127) & ~127)) e = -1;
        }
        a.tile_expert[t] = e;
    }
    for (int p = tid; p < a.pairs; p += 1024) {
        const int l = a.lids[p];
        int r = -1;
        if (l >= 0 && l < a.n_experts) r = off[l] + atomicAdd(&cur[l], 1);
        a.row_of_pair[p] = r < a.max_tiles * 128 ? r : -1;
    }
}

B2_API int b2_moe_plan(const MoePlanArgs* a, cudaStream_t st) {
    if (a->pairs < 1 || a->n_experts < 1 || a->n_experts > 512 || a->max_tiles < 1) return (int)cudaErrorInvalidValue;
    moe_plan_kernel<<<1, 1024, 0, st>>>(*a);
    return (int)cudaGetLastError();
}

// xs[row_of_pair[p]] = h[p / k]   (bf16 rows of d elements, d % 8 == 0)
__global__ void __launch_bounds__(128) moe_gather_kernel(const uint4* h, const int* row_of_pair, int k, int d8, uint4* xs) {
    const int p = blockIdx.x, r = row_of_pair[p];
    if (r < 0) return;
    const uint4* src = h + (size_t)(p / k) * d8;
    uint4* dst = xs + (size_t)r * d8;
    for (int c = threadIdx.x; c < d8; c += 128) dst[c] = src[c];
}

B2_API int b2_moe_gather(const void* h, const int* row_of_pair, int pairs, int k, int d, void* xs, cudaStream_t st) {
    if (pairs < 1 || k < 1 || (d & 7) || ((uintptr_t)h & 15) || ((uintptr_t)xs & 15)) return (int)cudaErrorInvalidValue;
    moe_gather_kernel<<<pairs, 128, 0, st>>>((const uint4*)h, row_of_pair, k, d >> 3, (uint4*)xs);
    return (int)cudaGetLastError();
}

// out[t] (+)= sum_s wts[t][s] * ys[row_of_pair[t k + s]]   (pairs whose expert lives elsewhere contribute nothing)
__global__ void __launch_bounds__(256) moe_scatter_combine_kernel(const float* ys, const int* row_of_pair, const float* wts, int k, int d,
                                                                  float* out, int accumulate) {
    const int t = blockIdx.x;
    for (int c = threadIdx.x; c < (d >> 2); c += 256) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int s = 0; s < k; s++) {
            const int r = row_of_pair[(size_t)t * k + s];
            if (r < 0) continue;
            const float w = wts[(size_t)t * k + s];
            const float4 v = *(const float4*)(ys + (size_t)r * d + 4 * c);
            acc.x += w * v.x; acc.y += w * v.y; acc.z += w * v.z; acc.w += w * v.w;
        }
        float4* o = (float4*)(out + (size_t)t * d + 4 * c);
        if (accumulate) {
            const float4 x = *o;
            acc.x += x.x; acc.y += x.y; acc.z += x.z; acc.w += x.w;
        }
        *o = acc;
    }
}

B2_API int b2_moe_scatter_combine(const float* ys, const int* row_of_pair, const float* wts, int tokens, int k, int d, float* out,
                                  int accumulate, cudaStream_t st) {
    if (tokens < 1 || k < 1 || (d & 3)) return (int)cudaErrorInvalidValue;
    moe_scatter_combine_kernel<<<tokens, 256, 0, st>>>(ys, row_of_pair, wts, k, d, out, accumulate);
    return (int)cudaGetLastError();
}
