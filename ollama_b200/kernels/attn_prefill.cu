// Flash attention for prefill chunks over the slot-partitioned f16 KV cache, sm_100a.
//
//   out[t][h] = softmax_k( scale * q[t][h] . K[k] (soft-capped, causal / sliding-window masked) ) V        k < kv_len
//
// One CTA = 64 consecutive query tokens of one head (4 warps x 16 rows); keys are visited in tiles of 64
// that land in shared memory through cp.async (two stages, the next tile loads while the current one is
// multiplied).  QK^T and PV run on the tensor cores as m16n8k16 f16 MMAs with fp32 accumulation, the
// softmax is the usual online form (running row maximum and sum, exp2 with the scale folded in), and the
// probabilities go from the accumulator layout of the first product straight into the A-operand layout of
// the second without touching shared memory.  Attention sinks (one extra logit per head in the
// denominator) and logit soft-capping are part of the kernel.  The result is written as bf16 rows
// [token][head * D], which is the operand layout of the following output-projection GEMM.
//
// The query rows of a chunk start at position pos0; rows of the cache are [slot][kv_head][position][D].
// In the reference stack this is ggml-cuda's fattn family (mma / tile / vec variants).
#include <mma.h>

#include "common.cuh"

struct AttnPrefillArgs {
    const float* q;          // [T][H][D] fp32, rotary embedding already applied
    const __half* k_cache;   // [slots][Hkv][n_ctx][D]
    const __half* v_cache;
    __nv_bfloat16* out;      // [T][H * D]
    const float* sinks;      // [H] or null
    int T, H, Hkv, n_ctx;
    int slot, pos0;
    int kv_len;              // keys visible to the chunk: positions [0, kv_len)
    int causal;
    int window;              // 0 = none; key k is visible to query p when p - k < window
    float scale, softcap;
    const __half* k_scale;   // q8_0 cache (k_cache / v_cache hold int8): [slots][Hkv][n_ctx][D/32] scales, or null for f16
    const __half* v_scale;
};

namespace {

constexpr int BM = 64, BN = 64, PAD = 8;

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_f16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ uint32_t pack_half2(float a, float b) {
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&h);
}

template <int D>
__global__ void __launch_bounds__(128) attn_prefill_kernel(const __grid_constant__ AttnPrefillArgs a) {
    constexpr int LD = D + PAD;                 // padded row length (halfs): rows start 16 bytes apart modulo 128
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __half* sQ = reinterpret_cast<__half*>(smem_raw);            // [BM][LD]
    __half* sK = sQ + BM * LD;                                   // [2][BN][LD]
    __half* sV = sK + 2 * BN * LD;                               // [2][BN][LD]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, tq = lane & 3;
    const int m0 = blockIdx.x * BM, h = blockIdx.y, hkv = h / (a.H / a.Hkv);
    const __half* kbase = a.k_cache + ((size_t)a.slot * a.Hkv + hkv) * a.n_ctx * D;
    const __half* vbase = a.v_cache + ((size_t)a.slot * a.Hkv + hkv) * a.n_ctx * D;

    // key range of this tile of queries
    const int q_lo = a.pos0 + m0, q_hi = a.pos0 + min(m0 + BM, a.T) - 1;
    int k_end = a.causal ? min(a.kv_len, q_hi + 1) : a.kv_len;
    int k_begin = a.window > 0 ? max(0, q_lo - a.window + 1) : 0;
    k_begin &= ~(BN - 1);
    const int n_tiles = k_end > k_begin ? (k_end - k_begin + BN - 1) / BN : 0;

    auto load_kv = [&](int tile, int stage) {
        const int n0 = k_begin + tile * BN;
        __half* dk = sK + stage * BN * LD;
        __half* dv = sV + stage * BN * LD;
        if (a.k_scale) {      // q8_0 cache: plain loads, expanded to f16 on the way into shared memory (16 dims per thread and trip)
            const int8_t* kq = reinterpret_cast<const int8_t*>(a.k_cache) + ((size_t)a.slot * a.Hkv + hkv) * a.n_ctx * D;
            const int8_t* vq = reinterpret_cast<const int8_t*>(a.v_cache) + ((size_t)a.slot * a.Hkv + hkv) * a.n_ctx * D;
            const __half* ks = a.k_scale + ((size_t)a.slot * a.Hkv + hkv) * a.n_ctx * (D / 32);
            const __half* vs = a.v_scale + ((size_t)a.slot * a.Hkv + hkv) * a.n_ctx * (D / 32);
            for (int c = tid; c < BN * (D / 16); c += 128) {
                const int r = c / (D / 16), col = (c % (D / 16)) * 16;
                const int pos = min(n0 + r, a.n_ctx - 1);
                const uint4 k4 = *(const uint4*)(kq + (size_t)pos * D + col), v4 = *(const uint4*)(vq + (size_t)pos * D + col);
                const float dkf = __half2float(ks[(size_t)pos * (D / 32) + (col >> 5)]), dvf = __half2float(vs[(size_t)pos * (D / 32) + (col >> 5)]);
                const uint32_t kw[4] = {k4.x, k4.y, k4.z, k4.w}, vw[4] = {v4.x, v4.y, v4.z, v4.w};
                uint32_t ko[8], vo[8];
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const uint32_t kb = kw[i >> 1] >> (16 * (i & 1)), vb = vw[i >> 1] >> (16 * (i & 1));
                    ko[i] = pack_half2(dkf * (float)(int8_t)(kb & 0xff), dkf * (float)(int8_t)((kb >> 8) & 0xff));
                    vo[i] = pack_half2(dvf * (float)(int8_t)(vb & 0xff), dvf * (float)(int8_t)((vb >> 8) & 0xff));
                }
                *(uint4*)(dk + r * LD + col) = make_uint4(ko[0], ko[1], ko[2], ko[3]);
                *(uint4*)(dk + r * LD + col + 8) = make_uint4(ko[4], ko[5], ko[6], ko[7]);
                *(uint4*)(dv + r * LD + col) = make_uint4(vo[0], vo[1], vo[2], vo[3]);
                *(uint4*)(dv + r * LD + col + 8) = make_uint4(vo[4], vo[5], vo[6], vo[7]);
            }
            asm volatile("cp.async.commit_group;" ::: "memory");      // keeps the group counting of the f16 path
            return;
        }
        for (int c = tid; c < BN * (D / 8); c += 128) {
            const int r = c / (D / 8), col = (c % (D / 8)) * 8;
            const int pos = min(n0 + r, a.n_ctx - 1);           // rows past the cache repeat its last row (masked below)
            cp_async16(dk + r * LD + col, kbase + (size_t)pos * D + col);
            cp_async16(dv + r * LD + col, vbase + (size_t)pos * D + col);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    if (n_tiles > 0) load_kv(0, 0);
    // Q tile: fp32 -> f16
    for (int c = tid; c < BM * (D / 4); c += 128) {
        const int r = c / (D / 4), col = (c % (D / 4)) * 4;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (m0 + r < a.T) v = *(const float4*)(a.q + ((size_t)(m0 + r) * a.H + h) * D + col);
        *reinterpret_cast<uint2*>(sQ + r * LD + col) = make_uint2(pack_half2(v.x, v.y), pack_half2(v.z, v.w));
    }
    __syncthreads();
    uint32_t qf[D / 16][4];
#pragma unroll
    for (int kk = 0; kk < D / 16; kk++)
        ldmatrix_x4(qf[kk], smem_addr(sQ + (warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * LD + kk * 16 + 8 * (lane >> 4)));

    float o[D / 8][4];
#pragma unroll
    for (int j = 0; j < D / 8; j++) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const float LOG2E = 1.4426950408889634f;
    const float sl2 = a.scale * LOG2E;
    const int qp0 = a.pos0 + m0 + warp * 16 + g, qp1 = qp0 + 8;

    for (int tile = 0; tile < n_tiles; tile++) {
        const int stage = tile & 1;
        if (tile + 1 < n_tiles) {
            load_kv(tile + 1, stage ^ 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        const __half* tk = sK + stage * BN * LD;
        const __half* tv = sV + stage * BN * LD;
        const int n0 = k_begin + tile * BN;

        float s[BN / 8][4];
#pragma unroll
        for (int j = 0; j < BN / 8; j++) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
        for (int kk = 0; kk < D / 16; kk++) {
#pragma unroll
            for (int j = 0; j < BN / 8; j += 2) {
                uint32_t b[4];
                ldmatrix_x4(b, smem_addr(tk + (8 * j + (lane & 7) + 8 * (lane >> 4)) * LD + kk * 16 + 8 * ((lane >> 3) & 1)));
                mma_f16(s[j], qf[kk], b[0], b[1]);
                mma_f16(s[j + 1], qf[kk], b[2], b[3]);
            }
        }
        // scale, soft-cap, mask; scores end up in the log2 domain
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int j = 0; j < BN / 8; j++) {
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int kp = n0 + 8 * j + 2 * tq + (e & 1);
                const int qp = (e & 2) ? qp1 : qp0;
                float v = s[j][e];
                v = a.softcap > 0.f ? a.softcap * tanhf(v * a.scale / a.softcap) * LOG2E : v * sl2;
                const bool ok = kp < a.kv_len && (!a.causal || kp <= qp) && (a.window <= 0 || qp - kp < a.window);
                v = ok ? v : -INFINITY;
                s[j][e] = v;
                mx[e >> 1] = fmaxf(mx[e >> 1], v);
            }
        }
        float corr[2];
#pragma unroll
        for (int r = 0; r < 2; r++) {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
            const float m_new = fmaxf(m_run[r], mx[r]);
            corr[r] = m_new == -INFINITY ? 1.f : exp2f(m_run[r] - m_new);
            m_run[r] = m_new;
            l_run[r] *= corr[r];
        }
        float ls[2] = {0.f, 0.f};
#pragma unroll
        for (int j = 0; j < BN / 8; j++) {
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const float mr = m_run[e >> 1];
                const float p = mr == -INFINITY ? 0.f : exp2f(s[j][e] - mr);
                s[j][e] = p;
                ls[e >> 1] += p;
            }
        }
        l_run[0] += ls[0];
        l_run[1] += ls[1];
#pragma unroll
        for (int j = 0; j < D / 8; j++) {
            o[j][0] *= corr[0]; o[j][1] *= corr[0];
            o[j][2] *= corr[1]; o[j][3] *= corr[1];
        }
        // O += P V: the accumulator fragments of S are the A fragments of P
#pragma unroll
        for (int kk = 0; kk < BN / 16; kk++) {
            uint32_t pa[4];
            pa[0] = pack_half2(s[2 * kk][0], s[2 * kk][1]);
            pa[1] = pack_half2(s[2 * kk][2], s[2 * kk][3]);
            pa[2] = pack_half2(s[2 * kk + 1][0], s[2 * kk + 1][1]);
            pa[3] = pack_half2(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
            for (int j = 0; j < D / 8; j += 2) {
                uint32_t b[4];
                ldmatrix_x4_trans(b, smem_addr(tv + (16 * kk + (lane & 7) + 8 * ((lane >> 3) & 1)) * LD + 8 * j + 8 * (lane >> 4)));
                mma_f16(o[j], pa, b[0], b[1]);
                mma_f16(o[j + 1], pa, b[2], b[3]);
            }
        }
        __syncthreads();        // everyone is done with this stage before it is overwritten two iterations later
    }

    // finish: row sums across the quad, attention sink, normalise, store bf16
#pragma unroll
    for (int r = 0; r < 2; r++) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
        if (a.sinks) {
            const float sk = a.sinks[h] * LOG2E;
            const float m_new = fmaxf(m_run[r], sk);
            const float c = m_run[r] == -INFINITY ? 0.f : exp2f(m_run[r] - m_new);
            l_run[r] = l_run[r] * c + exp2f(sk - m_new);
#pragma unroll
            for (int j = 0; j < D / 8; j++) { o[j][2 * r] *= c; o[j][2 * r + 1] *= c; }
        }
    }
#pragma unroll
    for (int r = 0; r < 2; r++) {
        const int row = m0 + warp * 16 + g + 8 * r;
        if (row >= a.T) continue;
        const float inv = l_run[r] > 0.f ? 1.f / l_run[r] : 0.f;
        __nv_bfloat16* op = a.out + (size_t)row * a.H * D + (size_t)h * D;
#pragma unroll
        for (int j = 0; j < D / 8; j++) {
            const __nv_bfloat162 v = __floats2bfloat162_rn(o[j][2 * r] * inv, o[j][2 * r + 1] * inv);
            *reinterpret_cast<__nv_bfloat162*>(op + 8 * j + 2 * tq) = v;
        }
    }
}

template <int D>
int launch(const AttnPrefillArgs& a, cudaStream_t st) {
    constexpr int SMEM = (BM + 4 * BN) * (D + PAD) * 2;
    static PerDeviceOnce once;
    if (once.first()) cudaFuncSetAttribute(attn_prefill_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    dim3 grid((a.T + BM - 1) / BM, a.H);
    attn_prefill_kernel<D><<<grid, 128, SMEM, st>>>(a);
    return (int)cudaGetLastError();
}

}  // namespace

// head_dim 32, 64, 128 or 256 (others: cudaErrorNotSupported).  Returns a cudaError_t value.
B2_API int b2_attn_prefill(const AttnPrefillArgs* a, int head_dim, cudaStream_t st) {
    if (a->T < 1 || a->H < 1 || a->Hkv < 1 || a->H % a->Hkv || a->kv_len < 1 || a->kv_len > a->n_ctx) return (int)cudaErrorInvalidValue;
    if (head_dim == 128) return launch<128>(*a, st);
    if (head_dim == 64) return launch<64>(*a, st);
    if (head_dim == 256) return launch<256>(*a, st);      // gemma family; 255 registers with a 96-byte spill
    if (head_dim == 32) return launch<32>(*a, st);
    return (int)cudaErrorNotSupported;
}
