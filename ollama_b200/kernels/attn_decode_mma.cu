// Split-K decode attention on the tensor cores, sm_100a.
//
// Same contract as the scalar kernel of attn_decode.cu (one query token per sequence, partial results
// (max, sum, unnormalised output) per split, merged by the combine kernel), different inner loop: the
// query heads that share a KV head are the rows of an m16n8k16 MMA tile (grouped-query attention gives
// 4..16 such heads; missing rows are zero), so one tile of 64 cached positions costs each warp 32 MMAs
// instead of some 1800 scalar instructions per 16 positions.  grid = (splits, kv heads, sequences), 4 warps.
// Cache rows arrive in shared memory through cp.async (two stages, or three / four when the launch has so few CTAs that each SM
// holds two / one: the bytes in flight per SM, not the math, bound this kernel at long contexts); warp w owns positions 16w..16w+15 of
// every tile and keeps its own running soft-max statistics and output accumulator, the four warps are merged
// through shared memory at the end.  The scalar kernel stays the choice for short contexts and for head
// sizes without an instantiation here.
#include "attn_args.cuh"

namespace {

constexpr int BN = 64, PAD = 8, ROWS = 16;

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

template <int D, int NS>
__global__ void __launch_bounds__(128) attn_decode_mma_kernel(const __grid_constant__ AttnDecodeArgs a, const __grid_constant__ AttnRopeArgs r) {
    constexpr int LD = D + PAD;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __half* sQ = reinterpret_cast<__half*>(smem_raw);            // [ROWS][LD]
    __half* sK = sQ + ROWS * LD;                                 // [NS][BN][LD]
    __half* sV = sK + NS * BN * LD;                              // [NS][BN][LD]
    __shared__ float s_m[4][ROWS], s_l[4][ROWS];
    __shared__ float s_cs[128], s_sn[128];                        // cos / sin of the query position per rotated pair (fused form)
    __shared__ __half s_newk[D], s_newv[D];                       // the query token's own key and value rows (fused form, owning split)
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, tq = lane & 3;
    const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    const int group = a.n_heads / a.n_kv_heads;                  // query heads per KV head (<= ROWS, checked by the launcher)
    const int head0 = kvh * group;

    pdl_launch();
    pdl_wait();
    const int qpos = a.positions[b], slot = a.slots[b];
    const int kv_len = qpos + 1;
    const int start = (a.window > 0 && kv_len > a.window) ? kv_len - a.window : 0;
    const int span = kv_len - start;
    int chunk = (span + a.n_splits - 1) / a.n_splits;
    chunk = ((chunk + BN - 1) / BN) * BN;
    const int p0 = start + split * chunk, p1 = min(p0 + chunk, kv_len);
    const int n_tiles = p1 > p0 ? (p1 - p0 + BN - 1) / BN : 0;
    const size_t row0 = ((size_t)slot * a.n_kv_heads + kvh) * a.n_ctx;      // first cache row of this (slot, kv head)

    auto load_kv = [&](int tile, int stage) {
        const int n0 = p0 + tile * BN;
        __half* dk = sK + stage * BN * LD;
        __half* dv = sV + stage * BN * LD;
        if (a.k_scale) {      // q8_0 cache: plain loads, expanded to f16 on the way into shared memory
            const int8_t* kq = reinterpret_cast<const int8_t*>(a.k_cache) + row0 * D;
            const int8_t* vq = reinterpret_cast<const int8_t*>(a.v_cache) + row0 * D;
            const __half* ks = a.k_scale + row0 * (D / 32);
            const __half* vs = a.v_scale + row0 * (D / 32);
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
        const __half* kbase = a.k_cache + row0 * D;
        const __half* vbase = a.v_cache + row0 * D;
        for (int c = tid; c < BN * (D / 8); c += 128) {
            const int r = c / (D / 8), col = (c % (D / 8)) * 8;
            const int pos = min(n0 + r, a.n_ctx - 1);           // rows past the range repeat a valid row (masked below)
            cp_async16(dk + r * LD + col, kbase + (size_t)pos * D + col);
            cp_async16(dv + r * LD + col, vbase + (size_t)pos * D + col);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    // the first NS - 1 tiles are requested at once (one commit group each, empty past the end, so that the counting stays uniform)
#pragma unroll
    for (int t = 0; t < NS - 1; t++) {
        if (t < n_tiles) load_kv(t, t);
        else asm volatile("cp.async.commit_group;" ::: "memory");
    }
    const bool fresh = r.qkv != nullptr;
    const bool owner = fresh && n_tiles > 0 && qpos >= p0 && qpos < p1;      // this split holds the query token's own position
    // element i of a raw head row after the rotary embedding (pairs (2p, 2p+1), or (p, p + n_rot/2) in the neox order)
    auto rotated = [&](const float* row, int i) -> float {
        const float x = row[i];
        if (i >= r.n_rot) return x;
        const int half_rot = r.n_rot >> 1;
        const bool first = r.neox ? i < half_rot : !(i & 1);
        const int p = r.neox ? (first ? i : i - half_rot) : i >> 1;
        const float y = row[r.neox ? (first ? i + half_rot : i - half_rot) : (i ^ 1)];
        return first ? x * s_cs[p] - y * s_sn[p] : y * s_sn[p] + x * s_cs[p];
    };
    if (fresh) {
        // the raw rows (query heads of this group, the key and the value) are staged in the last K stage, which stays unused
        // until the tile loop requests tile NS - 1; cos / sin of the position are computed once per CTA meanwhile
        float* raw = reinterpret_cast<float*>(sK + (NS - 1) * BN * LD);       // [group + 2][D]
        const float* tok = r.qkv + (size_t)b * (a.n_heads + 2 * a.n_kv_heads) * D;
        const int nrows = group + (owner ? 2 : 0);
        for (int c = tid; c < nrows * (D / 4); c += 128) {
            const int rr = c / (D / 4), col = (c % (D / 4)) * 4;
            const float* src = rr < group ? tok + (size_t)(head0 + rr) * D
                                          : tok + (size_t)(a.n_heads + (rr == group ? 0 : a.n_kv_heads) + kvh) * D;
            *reinterpret_cast<float4*>(raw + rr * D + col) = __ldcg(reinterpret_cast<const float4*>(src + col));
        }
        for (int p = tid; p < (r.n_rot >> 1); p += 128) {
            float sn, cs;
            sincosf((float)qpos * r.inv_freq[p], &sn, &cs);
            s_sn[p] = sn * r.mscale;
            s_cs[p] = cs * r.mscale;
        }
        __syncthreads();
        if (owner) {      // append the new key / value rows to the cache and keep them for the last tile
            const float* krow = raw + group * D;
            const float* vrow = raw + (group + 1) * D;
            __half* kc = const_cast<__half*>(a.k_cache) + (row0 + qpos) * D;
            __half* vc = const_cast<__half*>(a.v_cache) + (row0 + qpos) * D;
            for (int i = tid; i < D; i += 128) {
                const __half kh = __float2half_rn(rotated(krow, i)), vh = __float2half_rn(vrow[i]);
                s_newk[i] = kh;
                s_newv[i] = vh;
                kc[i] = kh;
                vc[i] = vh;
            }
        }
        for (int c = tid; c < ROWS * (D / 4); c += 128) {
            const int rr = c / (D / 4), col = (c % (D / 4)) * 4;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (rr < group) {
                const float* qrow = raw + rr * D;
                v = make_float4(rotated(qrow, col), rotated(qrow, col + 1), rotated(qrow, col + 2), rotated(qrow, col + 3));
            }
            *reinterpret_cast<uint2*>(sQ + rr * LD + col) = make_uint2(pack_half2(v.x, v.y), pack_half2(v.z, v.w));
        }
    } else {
        // Q rows: the heads of this KV head, fp32 -> f16, rows beyond the group are zero
        for (int c = tid; c < ROWS * (D / 4); c += 128) {
            const int rr = c / (D / 4), col = (c % (D / 4)) * 4;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (rr < group) v = *(const float4*)(a.q + ((size_t)b * a.n_heads + head0 + rr) * D + col);
            *reinterpret_cast<uint2*>(sQ + rr * LD + col) = make_uint2(pack_half2(v.x, v.y), pack_half2(v.z, v.w));
        }
    }
    __syncthreads();
    uint32_t qf[D / 16][4];
#pragma unroll
    for (int kk = 0; kk < D / 16; kk++)
        ldmatrix_x4(qf[kk], smem_addr(sQ + ((lane & 7) + 8 * ((lane >> 3) & 1)) * LD + kk * 16 + 8 * (lane >> 4)));

    float o[D / 8][4];
#pragma unroll
    for (int j = 0; j < D / 8; j++) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
    float m_run[2] = {-1e30f, -1e30f}, l_run[2] = {0.f, 0.f};

    for (int tile = 0; tile < n_tiles; tile++) {
        const int stage = tile % NS;
        if (tile + NS - 1 < n_tiles) load_kv(tile + NS - 1, (tile + NS - 1) % NS);      // into the stage that tile - 1 has just left
        else asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group %0;" ::"n"(NS - 1) : "memory");               // tile's own group is complete
        __syncthreads();
        if (owner && tile == n_tiles - 1) {      // the query's own row did not come from the cache: put it into the tile
            const int rr = qpos - (p0 + tile * BN);
            for (int i = tid; i < D; i += 128) {
                sK[stage * BN * LD + rr * LD + i] = s_newk[i];
                sV[stage * BN * LD + rr * LD + i] = s_newv[i];
            }
            __syncthreads();
        }
        const __half* tk = sK + stage * BN * LD + 16 * warp * LD;       // this warp's 16 positions of the tile
        const __half* tv = sV + stage * BN * LD + 16 * warp * LD;
        const int n0 = p0 + tile * BN + 16 * warp;

        float s[2][4];
        s[0][0] = s[0][1] = s[0][2] = s[0][3] = s[1][0] = s[1][1] = s[1][2] = s[1][3] = 0.f;
#pragma unroll
        for (int kk = 0; kk < D / 16; kk++) {
            uint32_t kb[4];
            ldmatrix_x4(kb, smem_addr(tk + ((lane & 7) + 8 * (lane >> 4)) * LD + kk * 16 + 8 * ((lane >> 3) & 1)));
            mma_f16(s[0], qf[kk], kb[0], kb[1]);
            mma_f16(s[1], qf[kk], kb[2], kb[3]);
        }
        // element e of block j: row g + 8 (e >> 1) (a query head), position n0 + 8 j + 2 tq + (e & 1)
        float mx[2] = {-1e30f, -1e30f};
        bool ok[2][2];
#pragma unroll
        for (int j = 0; j < 2; j++) {
#pragma unroll
            for (int e = 0; e < 2; e++) ok[j][e] = n0 + 8 * j + 2 * tq + e < p1;
#pragma unroll
            for (int e = 0; e < 4; e++) {
                float v = s[j][e] * a.scale;
                if (a.softcap > 0.f) v = a.softcap * tanhf(v / a.softcap);
                s[j][e] = v;
                if (ok[j][e & 1]) mx[e >> 1] = fmaxf(mx[e >> 1], v);
            }
        }
        float corr[2];
#pragma unroll
        for (int r = 0; r < 2; r++) {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
            const float m_new = fmaxf(m_run[r], mx[r]);
            corr[r] = __expf(m_run[r] - m_new);
            m_run[r] = m_new;
            l_run[r] *= corr[r];
        }
#pragma unroll
        for (int j = 0; j < 2; j++) {
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const float p = ok[j][e & 1] ? __expf(s[j][e] - m_run[e >> 1]) : 0.f;
                s[j][e] = p;
                l_run[e >> 1] += p;
            }
        }
#pragma unroll
        for (int j = 0; j < D / 8; j++) {
            o[j][0] *= corr[0]; o[j][1] *= corr[0];
            o[j][2] *= corr[1]; o[j][3] *= corr[1];
        }
        // O += P V: the accumulator fragments of S are the A fragments of P (16 positions = one k step)
        uint32_t pa[4];
        pa[0] = pack_half2(s[0][0], s[0][1]);
        pa[1] = pack_half2(s[0][2], s[0][3]);
        pa[2] = pack_half2(s[1][0], s[1][1]);
        pa[3] = pack_half2(s[1][2], s[1][3]);
#pragma unroll
        for (int j = 0; j < D / 8; j += 2) {
            uint32_t vb[4];
            ldmatrix_x4_trans(vb, smem_addr(tv + ((lane & 7) + 8 * ((lane >> 3) & 1)) * LD + 8 * j + 8 * (lane >> 4)));
            mma_f16(o[j], pa, vb[0], vb[1]);
            mma_f16(o[j + 1], pa, vb[2], vb[3]);
        }
        __syncthreads();        // everyone is done with this stage before the next iteration's request overwrites it
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");

    // merge the four warps: (max, sum, acc) of every query head through shared memory (the staging area is free now)
#pragma unroll
    for (int r = 0; r < 2; r++) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }
    float* s_acc = reinterpret_cast<float*>(sK);                 // [4][ROWS][D]
#pragma unroll
    for (int r = 0; r < 2; r++) {
        const int row = g + 8 * r;
        if (row < group) {
            float* dst = s_acc + ((size_t)warp * ROWS + row) * D;
#pragma unroll
            for (int j = 0; j < D / 8; j++) *reinterpret_cast<float2*>(dst + 8 * j + 2 * tq) = make_float2(o[j][2 * r], o[j][2 * r + 1]);
            if (tq == 0) {
                s_m[warp][row] = m_run[r];
                s_l[warp][row] = l_run[r];
            }
        }
    }
    __syncthreads();
    for (int idx = tid; idx < group * D; idx += 128) {
        const int row = idx / D, d = idx % D;
        const float mn = fmaxf(fmaxf(s_m[0][row], s_m[1][row]), fmaxf(s_m[2][row], s_m[3][row]));
        float acc = 0.f, lt = 0.f;
#pragma unroll
        for (int w = 0; w < 4; w++) {
            const float c = __expf(s_m[w][row] - mn);
            acc += s_acc[((size_t)w * ROWS + row) * D + d] * c;
            lt += s_l[w][row] * c;
        }
        const size_t pi = ((size_t)b * a.n_heads + head0 + row) * a.n_splits + split;
        a.part_acc[pi * D + d] = acc;
        if (d == 0) a.part_ml[pi] = make_float2(mn, lt);
    }
}

template <int D, int NS>
int launch(const AttnDecodeArgs& a, const AttnRopeArgs& r, int nb, int pdl, cudaStream_t st) {
    constexpr int SMEM = (ROWS + 2 * NS * BN) * (D + PAD) * 2;
    static PerDeviceOnce once;
    if (once.first()) cudaFuncSetAttribute(attn_decode_mma_kernel<D, NS>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(a.n_splits, a.n_kv_heads, nb);
    cfg.blockDim = dim3(128);
    cfg.dynamicSmemBytes = SMEM;
    cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = pdl ? 1 : 0;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    AttnDecodeArgs copy = a;
    AttnRopeArgs rcopy = r;
    void* args[] = {&copy, &rcopy};
    return (int)cudaLaunchKernelExC(&cfg, (const void*)attn_decode_mma_kernel<D, NS>, args);
}

int g_stages = 0;      // 0: by the size of the launch; 2, 3 or 4: forced (tests)

// Four stages take 140 KB of shared memory (one CTA per SM), three 109 KB (two per SM), two 74 KB (three per SM).  A launch that
// gives every SM at most one CTA runs four stages, one that gives it at most two runs three, larger ones keep two: the bytes in
// flight per SM stay about the same and no launch needs a second round because of its shared memory.
int stages_for(const AttnDecodeArgs& a, int nb) {
    if (g_stages) return g_stages;
    static int sms = 0;
    if (!sms) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (sms <= 0) sms = 148;
    }
    const long ctas = (long)a.n_splits * a.n_kv_heads * nb;
    if (a.n_ctx / a.n_splits < 2 * BN) return 2;
    return ctas <= sms ? 4 : (ctas <= 2L * sms ? 3 : 2);
}

template <int D>
int launch_d(const AttnDecodeArgs& a, const AttnRopeArgs& r, int nb, int pdl, cudaStream_t st) {
    switch (stages_for(a, nb)) {
        case 4: return launch<D, 4>(a, r, nb, pdl, st);
        case 3: return launch<D, 3>(a, r, nb, pdl, st);
        default: return launch<D, 2>(a, r, nb, pdl, st);
    }
}

}  // namespace

int attn_decode_mma_rope_launch(const AttnDecodeArgs& a, const AttnRopeArgs& r, int nb, int hd, int pdl, cudaStream_t st) {
    if (a.n_kv_heads < 1 || a.n_heads % a.n_kv_heads || a.n_heads / a.n_kv_heads > ROWS) return (int)cudaErrorNotSupported;
    if (r.qkv && (a.k_scale || a.v_scale || r.n_rot > 256 || r.n_rot > hd || (r.n_rot & 1) || !r.inv_freq)) return (int)cudaErrorNotSupported;
    if (hd == 128) return launch_d<128>(a, r, nb, pdl, st);
    if (hd == 64) return launch_d<64>(a, r, nb, pdl, st);
    return (int)cudaErrorNotSupported;
}

// Pipeline depth of the tensor-core decode kernel: 0 = chosen per launch (default), 2, 3 or 4 = forced.  Returns the previous setting.
B2_API int b2_attn_decode_stages(int n) {
    const int old = g_stages;
    if (n == 0 || (n >= 2 && n <= 4)) g_stages = n;
    return old;
}

int attn_decode_mma_launch(const AttnDecodeArgs& a, int nb, int hd, int pdl, cudaStream_t st) {
    const AttnRopeArgs none = {};
    return attn_decode_mma_rope_launch(a, none, nb, hd, pdl, st);
}
