// Normalisation, activation quantisation, rotary embedding + KV-cache append, embedding gather,
// arg-max.  These are the memory-bound glue ops of a decode step; each one is fused with its
// neighbours where the data flow allows (RMSNorm + int8 block quantisation of the GEMV input;
// per-head QK-norm + RoPE + f16 conversion + scatter into the slot-partitioned cache).
#include "common.cuh"
#include "comm.cuh"

// ---------------------------------------------------------------------------------------------
// y = rmsnorm(x) * w  ->  fp32 copy (optional) + int8 blocks of 32 with (d, d*sum q)
// one CTA per token
// ---------------------------------------------------------------------------------------------
struct NormQuantArgs {
    const float* x;      // [nb][k]
    const float* w;      // [k] or null (no scaling)
    float eps;
    int k;
    int do_norm;         // 0: quantise x as is
    int8_t* xq;          // [nb][k] or null
    float2* xds;         // [nb][k/32]
    float* xf;           // [nb][k] or null
    float* residual;     // if set: residual[b][i] += y   (post-norm residual add of sandwich-norm models)
    // tensor parallel: x[b] += sum over ranks of the partial rows received from the group, before anything else
    const uint2* parts;      // [2 halves][n_part][rows][k] (value, epoch) pairs in this rank's peer-mapped region (null: none)
    int n_part;
    long long part_stride;   // pairs between the slabs of two ranks
    long long parity_stride; // pairs between the two halves
    CommChan* chan;
};

// Each thread owns float4 chunks c = tid + 256 j; a quantisation block of 32 is 8 consecutive chunks =
// 8 consecutive lanes, so block maxima and sums are 3-step shuffles.  All loads of a row are issued
// before the first use (rows up to 8192 elements stay in registers).
__global__ void __launch_bounds__(256) rmsnorm_quant_kernel(const __grid_constant__ NormQuantArgs a) {
    constexpr int MAXJ = 8;
    __shared__ float red[8];
    const int b = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nchunk = a.k >> 2;
    float4 wv[MAXJ];
    if (a.w) {   // the norm weights do not depend on the producer kernel
#pragma unroll
        for (int j = 0; j < MAXJ; j++) {
            const int c = tid + 256 * j;
            wv[j] = c < nchunk ? *(const float4*)(a.w + 4 * c) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    pdl_launch();
    pdl_wait();
    const float* x = a.x + (size_t)b * a.k;
    const uint2* part = nullptr;
    unsigned ep = 0;
    if (a.n_part) {      // low-latency exchange: the words of this epoch arrive from every rank while we poll them
        ep = ld_volatile_u32(&a.chan->epoch) + 1u;
        part = a.parts + ((ep & 1u) ? a.parity_stride : 0ll) + (size_t)b * a.k;
    }
    for (int c0 = 0; c0 < nchunk; c0 += 256 * MAXJ) {     // one trip for k <= 8192
        float4 v[MAXJ];
#pragma unroll
        for (int j = 0; j < MAXJ; j++) {
            const int c = c0 + tid + 256 * j;
            v[j] = c < nchunk ? *(const float4*)(x + 4 * c) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        if (part) {      // k <= 8192 here (checked by the launcher): the reduced row is complete in registers
            for (int r = 0; r < a.n_part; r++) ll_add_row<MAXJ>(part + r * a.part_stride, tid, nchunk, ep, a.chan, v);
#pragma unroll
            for (int j = 0; j < MAXJ; j++) {
                const int c = tid + 256 * j;
                if (c < nchunk) *(float4*)(const_cast<float*>(x) + 4 * c) = v[j];
            }
        }
        float inv = 1.f;
        if (a.do_norm) {
            float ss = 0.f;
            if (nchunk <= 256 * MAXJ) {
#pragma unroll
                for (int j = 0; j < MAXJ; j++) ss += v[j].x * v[j].x + v[j].y * v[j].y + v[j].z * v[j].z + v[j].w * v[j].w;
            } else {
                for (int c = tid; c < nchunk; c += 256) {
                    const float4 t = *(const float4*)(x + 4 * c);
                    ss += t.x * t.x + t.y * t.y + t.z * t.z + t.w * t.w;
                }
            }
            ss = warp_sum(ss);
            __syncthreads();
            if (lane == 0) red[warp] = ss;
            __syncthreads();
            float t = lane < 8 ? red[lane] : 0.f;
            t = warp_sum(t);
            inv = rsqrtf(t / (float)a.k + a.eps);
        }
#pragma unroll
        for (int j = 0; j < MAXJ; j++) {
            const int c = c0 + tid + 256 * j;
            const bool ok = c < nchunk;
            float4 y = v[j];
            y.x *= inv; y.y *= inv; y.z *= inv; y.w *= inv;
            if (a.w) {
                float4 ww = wv[j];
                if (c0) ww = ok ? *(const float4*)(a.w + 4 * c) : ww;
                y.x *= ww.x; y.y *= ww.y; y.z *= ww.z; y.w *= ww.w;
            }
            const size_t o = (size_t)b * a.k + 4 * (size_t)c;
            if (ok && a.xf) *(float4*)(a.xf + o) = y;
            if (ok && a.residual) {
                float4 r = *(float4*)(a.residual + o);
                r.x += y.x; r.y += y.y; r.z += y.z; r.w += y.w;
                *(float4*)(a.residual + o) = r;
            }
            if (a.xq) {
                float amax = fmaxf(fmaxf(fabsf(y.x), fabsf(y.y)), fmaxf(fabsf(y.z), fabsf(y.w)));
                amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
                amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
                amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
                const float d = amax / 127.f, id = d > 0.f ? 1.f / d : 0.f;
                const int q0 = __float2int_rn(y.x * id), q1 = __float2int_rn(y.y * id), q2 = __float2int_rn(y.z * id), q3 = __float2int_rn(y.w * id);
                float qs = (float)(q0 + q1 + q2 + q3);
                qs += __shfl_xor_sync(0xffffffffu, qs, 1);
                qs += __shfl_xor_sync(0xffffffffu, qs, 2);
                qs += __shfl_xor_sync(0xffffffffu, qs, 4);
                if (ok) {
                    *(uint32_t*)(a.xq + o) = (uint32_t)(q0 & 0xff) | ((uint32_t)(q1 & 0xff) << 8) | ((uint32_t)(q2 & 0xff) << 16) | ((uint32_t)(q3 & 0xff) << 24);
                    if ((lane & 7) == 0) a.xds[(size_t)b * (a.k >> 5) + (c >> 3)] = make_float2(d, d * qs);
                }
            }
        }
    }
    if (a.n_part) ll_consumed(a.chan, gridDim.x, ep);
}

B2_API int b2_rmsnorm_quant(const NormQuantArgs* a, int nb, int pdl, cudaStream_t st) {
    if (a->k & 31) return (int)cudaErrorInvalidValue;
    if (a->n_part && (a->k > 8192 || a->n_part > COMM_MAX_RANKS || !a->parts || !a->chan)) return (int)cudaErrorInvalidValue;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(nb);
    cfg.blockDim = dim3(256);
    cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = pdl ? 1 : 0;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    NormQuantArgs copy = *a;
    void* args[] = {&copy};
    return (int)cudaLaunchKernelExC(&cfg, (const void*)rmsnorm_quant_kernel, args);
}

// ---------------------------------------------------------------------------------------------
// QKV post-processing: optional per-head RMSNorm of q and k, RoPE, write q (fp32) and append K/V
// (f16) to the cache at [slot][kv_head][position][dim].  grid = (tokens, n_heads + 2 n_kv_heads)
// ---------------------------------------------------------------------------------------------
struct RopeKvArgs {
    const float* qkv;        // [nt][(H + 2 Hkv) * hd]  (q | k | v)
    const int* positions;    // [nt]
    const int* slots;        // [nt]
    const float* inv_freq;   // [n_rot/2]
    const float* q_norm;     // [hd] or null
    const float* k_norm;     // [hd] or null
    float eps, mscale;
    int n_heads, n_kv_heads, hd, n_rot, neox, n_ctx;
    float* q_out;            // [nt][H][hd]
    __half* k_cache;         // [slots][Hkv][n_ctx][hd]  (int8 when the scale arrays are given)
    __half* v_cache;
    __half* k_scale;         // q8_0 cache: [slots][Hkv][n_ctx][hd/32] one f16 scale per 32 dims, or null for an f16 cache
    __half* v_scale;
};

__global__ void __launch_bounds__(128) rope_kv_kernel(const __grid_constant__ RopeKvArgs a) {
    const int t = blockIdx.x, head = blockIdx.y, tid = threadIdx.x;
    const int H = a.n_heads, Hkv = a.n_kv_heads, hd = a.hd;
    pdl_launch();
    pdl_wait();
    const int pos = a.positions[t], slot = a.slots[t];
    const float* src = a.qkv + (size_t)t * (H + 2 * Hkv) * hd + (size_t)head * hd;
    const bool is_q = head < H, is_k = !is_q && head < H + Hkv;
    __shared__ float sh[512];
    __shared__ float red[4];
    for (int i = tid; i < hd; i += 128) sh[i] = src[i];
    __syncthreads();
    const float* nw = is_q ? a.q_norm : (is_k ? a.k_norm : nullptr);
    if (nw) {
        float ss = 0.f;
        for (int i = tid; i < hd; i += 128) ss += sh[i] * sh[i];
        ss = warp_sum(ss);
        if ((tid & 31) == 0) red[tid >> 5] = ss;
        __syncthreads();
        const float tot = red[0] + red[1] + red[2] + red[3];
        const float inv = rsqrtf(tot / (float)hd + a.eps);
        for (int i = tid; i < hd; i += 128) sh[i] = sh[i] * inv * nw[i];
        __syncthreads();
    }
    if (is_q || is_k) {
        const int half_rot = a.n_rot >> 1;
        for (int p = tid; p < half_rot; p += 128) {
            const int i0 = a.neox ? p : 2 * p, i1 = a.neox ? p + half_rot : 2 * p + 1;
            float sn, cs;
            sincosf((float)pos * a.inv_freq[p], &sn, &cs);
            sn *= a.mscale; cs *= a.mscale;
            const float x0 = sh[i0], x1 = sh[i1];
            sh[i0] = x0 * cs - x1 * sn;
            sh[i1] = x0 * sn + x1 * cs;
        }
        __syncthreads();
    }
    if (is_q) {
        float* dst = a.q_out + ((size_t)t * H + head) * hd;
        for (int i = tid; i < hd; i += 128) dst[i] = sh[i];
    } else {
        const int kvh = is_k ? head - H : head - H - Hkv;
        const size_t rowi = ((size_t)slot * Hkv + kvh) * a.n_ctx + pos;
        __half* sc = is_k ? a.k_scale : a.v_scale;
        if (sc) {      // q8_0: a warp covers one block of 32 dims per trip (hd is a multiple of 32)
            int8_t* dst = reinterpret_cast<int8_t*>(is_k ? a.k_cache : a.v_cache) + rowi * hd;
            for (int i0 = 0; i0 < hd; i0 += 128) {
                const int i = i0 + tid;
                const float v = i < hd ? sh[i] : 0.f;
                const __half dh = __float2half_rn(warp_max(fabsf(v)) / 127.f);
                const float d = __half2float(dh);
                if (i < hd) {
                    dst[i] = (int8_t)(d > 0.f ? max(-127, min(127, __float2int_rn(v / d))) : 0);
                    if ((tid & 31) == 0) sc[rowi * (hd >> 5) + (i >> 5)] = dh;
                }
            }
        } else {
            __half* dst = (is_k ? a.k_cache : a.v_cache) + rowi * hd;
            for (int i = tid; i < hd; i += 128) dst[i] = __float2half_rn(sh[i]);
        }
    }
}

// Prefill form of the kernel above: one CTA per token, a warp per head (eight heads in flight, the rest in turns).  The
// sines and cosines of the token's position are computed once per token, not once per head (a chunk of 2048 tokens of a
// 48-head model otherwise evaluates 6 M full-range sincosf), and nothing but the warp has to synchronise.
__global__ void __launch_bounds__(256) rope_kv_rows_kernel(const __grid_constant__ RopeKvArgs a) {
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int H = a.n_heads, Hkv = a.n_kv_heads, hd = a.hd;
    const int half_rot = a.n_rot >> 1;
    __shared__ float s_cs[256], s_sn[256];
    __shared__ float sh_all[8][512];
    const int pos = a.positions[t], slot = a.slots[t];
    for (int p = threadIdx.x; p < half_rot; p += 256) {
        float sn, cs;
        sincosf((float)pos * a.inv_freq[p], &sn, &cs);
        s_cs[p] = cs * a.mscale;
        s_sn[p] = sn * a.mscale;
    }
    __syncthreads();
    float* sh = sh_all[warp];
    for (int head = warp; head < H + 2 * Hkv; head += 8) {
        const float* src = a.qkv + (size_t)t * (H + 2 * Hkv) * hd + (size_t)head * hd;
        const bool is_q = head < H, is_k = !is_q && head < H + Hkv;
        for (int i = lane; i < hd; i += 32) sh[i] = src[i];
        __syncwarp();
        const float* nw = is_q ? a.q_norm : (is_k ? a.k_norm : nullptr);
        if (nw) {
            float ss = 0.f;
            for (int i = lane; i < hd; i += 32) ss += sh[i] * sh[i];
            ss = warp_sum(ss);
            const float inv = rsqrtf(ss / (float)hd + a.eps);
            for (int i = lane; i < hd; i += 32) sh[i] = sh[i] * inv * nw[i];
            __syncwarp();
        }
        if (is_q || is_k) {
            for (int p = lane; p < half_rot; p += 32) {
                const int i0 = a.neox ? p : 2 * p, i1 = a.neox ? p + half_rot : 2 * p + 1;
                const float cs = s_cs[p], sn = s_sn[p];
                const float x0 = sh[i0], x1 = sh[i1];
                sh[i0] = x0 * cs - x1 * sn;
                sh[i1] = x0 * sn + x1 * cs;
            }
            __syncwarp();
        }
        if (is_q) {
            float* dst = a.q_out + ((size_t)t * H + head) * hd;
            for (int i = lane; i < hd; i += 32) dst[i] = sh[i];
        } else {
            const int kvh = is_k ? head - H : head - H - Hkv;
            const size_t rowi = ((size_t)slot * Hkv + kvh) * a.n_ctx + pos;
            __half* sc = is_k ? a.k_scale : a.v_scale;
            if (sc) {      // q8_0: the warp covers one block of 32 dims per trip (hd is a multiple of 32)
                int8_t* dst = reinterpret_cast<int8_t*>(is_k ? a.k_cache : a.v_cache) + rowi * hd;
                for (int i0 = 0; i0 < hd; i0 += 32) {
                    const float v = sh[i0 + lane];
                    const __half dh = __float2half_rn(warp_max(fabsf(v)) / 127.f);
                    const float d = __half2float(dh);
                    dst[i0 + lane] = (int8_t)(d > 0.f ? max(-127, min(127, __float2int_rn(v / d))) : 0);
                    if (lane == 0) sc[rowi * (hd >> 5) + (i0 >> 5)] = dh;
                }
            } else {
                __half* dst = (is_k ? a.k_cache : a.v_cache) + rowi * hd;
                for (int i = lane; i < hd; i += 32) dst[i] = __float2half_rn(sh[i]);
            }
        }
        __syncwarp();
    }
}

B2_API int b2_rope_kv(const RopeKvArgs* a, int nt, int pdl, cudaStream_t st) {
    if (a->hd > 512 || ((a->k_scale || a->v_scale) && ((a->hd & 31) || !a->k_scale || !a->v_scale))) return (int)cudaErrorInvalidValue;
    if (nt >= 64 && a->n_rot <= 512) {          // prefill chunks: a CTA per token
        RopeKvArgs copy = *a;
        rope_kv_rows_kernel<<<nt, 256, 0, st>>>(copy);
        return (int)cudaGetLastError();
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(nt, a->n_heads + 2 * a->n_kv_heads);
    cfg.blockDim = dim3(128);
    cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = pdl ? 1 : 0;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    RopeKvArgs copy = *a;
    void* args[] = {&copy};
    return (int)cudaLaunchKernelExC(&cfg, (const void*)rope_kv_kernel, args);
}

// ---------------------------------------------------------------------------------------------
// Embedding gather from a (possibly quantised) table: out[t][:] = scale * dequant(table[ids[t]][:])
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float deq_elem(const WDesc& w, int row, int i) {
    const int K = w.k;
    switch (w.type) {
        case WT_F32: return ((const float*)w.p0)[(size_t)row * K + i];
        case WT_F16: return __half2float(((const __half*)w.p0)[(size_t)row * K + i]);
        case WT_BF16: return __bfloat162float(((const __nv_bfloat16*)w.p0)[(size_t)row * K + i]);
        case WT_Q8_0: {
            const int8_t q = ((const int8_t*)w.p0)[(size_t)row * K + i];
            return (float)q * __half2float(((const __half*)w.p1)[(size_t)row * (K >> 5) + (i >> 5)]);
        }
        case WT_Q4_0: {
            const int blk = i >> 5, l = i & 31;
            const uint8_t q = ((const uint8_t*)w.p0)[(size_t)row * (K >> 1) + blk * 16 + (l & 15)];
            const int v = (l < 16 ? (q & 15) : (q >> 4)) - 8;
            return (float)v * __half2float(((const __half*)w.p1)[(size_t)row * (K >> 5) + blk]);
        }
        case WT_MXFP4: {
            const int blk = i >> 5, l = i & 31;
            const uint8_t q = ((const uint8_t*)w.p0)[(size_t)row * (K >> 1) + blk * 16 + (l & 15)];
            const int code = l < 16 ? (q & 15) : (q >> 4);
            const float mags[8] = {0.f, 0.5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};
            const float v = (code & 8) ? -mags[code & 7] : mags[code & 7];
            return v * e8m0_to_float(((const uint8_t*)w.p1)[(size_t)row * (K >> 5) + blk]);
        }
        case WT_Q4_K:
        case WT_Q5_K: {
            const int sb = i >> 8, r = i & 255, j = r >> 6, hi = (r >> 5) & 1, l = r & 31;
            const uint8_t* sm = (const uint8_t*)w.p1 + ((size_t)row * (K >> 8) + sb) * 16 + 4 * j;
            const __half2 dm = ((const __half2*)w.p2)[(size_t)row * (K >> 8) + sb];
            const int s = sm[hi], m = sm[2 + hi];
            const uint8_t qb = ((const uint8_t*)w.p0)[(size_t)row * (K >> 1) + sb * 128 + j * 32 + l];
            int q = hi ? (qb >> 4) : (qb & 15);
            if (w.type == WT_Q5_K) {
                const uint8_t h = ((const uint8_t*)w.p3)[(size_t)row * (K >> 3) + sb * 32 + l];
                q |= ((h >> (2 * j + hi)) & 1) << 4;
            }
            return __low2float(dm) * (float)s * (float)q - __high2float(dm) * (float)m;
        }
        case WT_Q6_K: {
            const int sb = i >> 8, r = i & 255, n = r >> 7, qd = (r >> 5) & 3, l = r & 31;
            const uint8_t qlb = ((const uint8_t*)w.p0)[(size_t)row * (K >> 1) + sb * 128 + n * 64 + (qd & 1) * 32 + l];
            const uint8_t qhb = ((const uint8_t*)w.p1)[(size_t)row * (K >> 2) + sb * 64 + n * 32 + l];
            const int q = ((qd < 2 ? (qlb & 15) : (qlb >> 4)) | (((qhb >> (2 * qd)) & 3) << 4)) - 32;
            const int8_t s = ((const int8_t*)w.p2)[(size_t)row * (K >> 4) + sb * 16 + n * 8 + (l >> 4) + 2 * qd];
            return __half2float(((const __half*)w.p3)[(size_t)row * (K >> 8) + sb]) * (float)s * (float)q;
        }
    }
    return 0.f;
}

struct EmbedArgs {
    WDesc table;
    const int* ids;      // [nt]
    float scale;
    float* out;          // [nt][k]
};

// grid (tokens, slices): a slice is EMBED_SLICE consecutive elements of the row, so that one token's row is decoded by
// several CTAs at once (a single CTA took 10-12 us for a 4096-wide Q4_K row)
constexpr int EMBED_SLICE = 512;

__global__ void __launch_bounds__(256) embed_kernel(const __grid_constant__ EmbedArgs a) {
    pdl_launch();
    pdl_wait();
    const int t = blockIdx.x;
    int row = a.ids[t];
    row = min(max(row, 0), a.table.n - 1);
    const int lo = blockIdx.y * EMBED_SLICE, hi = min(a.table.k, lo + EMBED_SLICE);
    for (int i = lo + threadIdx.x; i < hi; i += 256) a.out[(size_t)t * a.table.k + i] = a.scale * deq_elem(a.table, row, i);
}

B2_API int b2_embed(const EmbedArgs* a, int nt, cudaStream_t st) {
    EmbedArgs copy = *a;
    embed_kernel<<<dim3((unsigned)nt, (unsigned)((a->table.k + EMBED_SLICE - 1) / EMBED_SLICE)), 256, 0, st>>>(copy);
    return (int)cudaGetLastError();
}

// Dequantise rows [row0, row0+nrows) of a weight into bf16 (used to stage operands for the
// tensor-core GEMM and by the tests that check the plane layouts).
struct DequantArgs {
    WDesc w;
    int row0, nrows;
    __nv_bfloat16* out;   // [nrows][k]
};

__global__ void __launch_bounds__(256) dequant_rows_kernel(const __grid_constant__ DequantArgs a) {
    const int r = blockIdx.x;
    if (r >= a.nrows) return;
    for (int i = threadIdx.x; i < a.w.k; i += 256)
        a.out[(size_t)r * a.w.k + i] = __float2bfloat16(deq_elem(a.w, a.row0 + r, i));
}

B2_API int b2_dequant_rows(const DequantArgs* a, cudaStream_t st) {
    DequantArgs copy = *a;
    dequant_rows_kernel<<<a->nrows, 256, 0, st>>>(copy);
    return (int)cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------
// arg-max over the vocabulary, one CTA per row; optional soft-cap is monotonic so it is skipped
// ---------------------------------------------------------------------------------------------
// One CTA per row.  The row is read as float4 with eight loads in flight per thread; ties go to the lowest index.  With
// `tokens` the winner is also fed back as the next step's input token and the row's position advances (the decode loop's
// bookkeeping, otherwise a launch of its own).
__global__ void __launch_bounds__(1024) argmax_kernel(const float* logits, int n, int ld, int* out, int* tokens, int* positions) {
    pdl_launch();
    pdl_wait();
    const float* x = logits + (size_t)blockIdx.x * ld;
    float best = -INFINITY;
    int bi = 0x7fffffff;
    const int n4 = (((uintptr_t)x & 15) == 0) ? n >> 2 : 0;
    const float4* x4 = reinterpret_cast<const float4*>(x);
#pragma unroll 8
    for (int i = threadIdx.x; i < n4; i += 1024) {
        const float4 v = __ldcs(x4 + i);
        const int e = 4 * i;
        if (v.x > best) { best = v.x; bi = e; }
        if (v.y > best) { best = v.y; bi = e + 1; }
        if (v.z > best) { best = v.z; bi = e + 2; }
        if (v.w > best) { best = v.w; bi = e + 3; }
    }
    for (int i = 4 * n4 + threadIdx.x; i < n; i += 1024) {
        const float v = x[i];
        if (v > best) { best = v; bi = i; }
    }
    __shared__ float sv[32];
    __shared__ int si[32];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = best; si[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x < 32) {
        best = sv[threadIdx.x]; bi = si[threadIdx.x];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
        }
        if (threadIdx.x == 0) {
            out[blockIdx.x] = bi;
            if (tokens) {
                tokens[blockIdx.x] = bi;
                positions[blockIdx.x] += 1;
            }
        }
    }
}

B2_API int b2_argmax(const float* logits, int rows, int n, int ld, int* out, cudaStream_t st) {
    argmax_kernel<<<rows, 1024, 0, st>>>(logits, n, ld, out, nullptr, nullptr);
    return (int)cudaGetLastError();
}

// arg-max of every row, and the row's token / position advanced for the next decode step, in one launch
B2_API int b2_argmax_advance(const float* logits, int rows, int n, int ld, int* out, int* tokens, int* positions, cudaStream_t st) {
    if (!tokens || !positions) return (int)cudaErrorInvalidValue;
    argmax_kernel<<<rows, 1024, 0, st>>>(logits, n, ld, out, tokens, positions);
    return (int)cudaGetLastError();
}

// Decode-step bookkeeping kept on the device so that a captured step can be replayed:
// tokens[b] = sampled[b]; positions[b] += 1
__global__ void advance_kernel(int* tokens, int* positions, const int* sampled, int nb) {
    const int b = threadIdx.x;
    if (b < nb) { tokens[b] = sampled[b]; positions[b] += 1; }
}

B2_API int b2_advance(int* tokens, int* positions, const int* sampled, int nb, cudaStream_t st) {
    advance_kernel<<<1, 32, 0, st>>>(tokens, positions, sampled, nb);
    return (int)cudaGetLastError();
}

// fp32 -> bf16 with optional row-wise RMSNorm (prefill activations feeding the tensor-core GEMM)
struct NormCastArgs {
    const float* x;
    const float* w;
    float eps;
    int k, do_norm;
    __nv_bfloat16* out;
};

__global__ void __launch_bounds__(256) rmsnorm_bf16_kernel(const __grid_constant__ NormCastArgs a) {
    __shared__ float red[8];
    const int b = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* x = a.x + (size_t)b * a.k;
    float inv = 1.f;
    if (a.do_norm) {
        float ss = 0.f;
        for (int i = tid; i < a.k; i += 256) ss += x[i] * x[i];
        ss = warp_sum(ss);
        if (lane == 0) red[warp] = ss;
        __syncthreads();
        float t = lane < 8 ? red[lane] : 0.f;
        t = warp_sum(t);
        inv = rsqrtf(t / (float)a.k + a.eps);
    }
    for (int i = tid; i < a.k; i += 256) {
        float v = x[i] * inv;
        if (a.w) v *= a.w[i];
        a.out[(size_t)b * a.k + i] = __float2bfloat16(v);
    }
}

B2_API int b2_rmsnorm_bf16(const NormCastArgs* a, int rows, cudaStream_t st) {
    NormCastArgs copy = *a;
    rmsnorm_bf16_kernel<<<rows, 256, 0, st>>>(copy);
    return (int)cudaGetLastError();
}
