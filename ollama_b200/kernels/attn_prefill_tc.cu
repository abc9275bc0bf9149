// Flash attention for prefill chunks on the fifth-generation tensor cores (tcgen05 + TMEM + TMA), sm_100a.
//
//   out[t][h] = softmax_k( scale * q[t][h] . K[k] (soft-capped, causal / sliding-window masked) ) V        k < kv_len
//
// One CTA = 128 consecutive query tokens of one head.  Keys and values are visited in tiles of 128 cache rows that TMA
// drops into two shared-memory stages in the 128-byte-swizzled layout (the f16 cache rows [position][D] are K-major for
// Q K^T and MN-major for P V, so neither product needs a transposed copy).  One elected thread issues the MMAs:
// S = Q K^T (M = 128 queries, N = 128 keys) into TMEM columns 0..127, and O_tile = P V (N = D) into columns 128..128+D.
// Eight softmax warps read S from TMEM (a warp reaches the 32 TMEM lanes of its quarter, so two warps share a quarter
// and split the columns), keep the running row maximum and sum, write the probabilities as f16 into the swizzled A-operand
// tile of the second product, and add each O_tile to their register accumulators after rescaling those.  S of the next
// tile is issued right after P V of the current one, so the tensor pipe works on it while the softmax warps accumulate.
// Roles: warps 0-7 softmax, warp 8 TMA producer, warp 9 MMA issue and TMEM allocation.  Every mbarrier wait is bounded; a
// wait that runs out sets KS_TIMEOUT in the status word, and all roles leave their loops (TMEM is freed on the way out).
//
// The kernel that runs by default is the pipelined form further down (two score buffers, probabilities kept in TMEM, the
// accumulation of a tile deferred behind the next tile's softmax); the single-buffered forms above it stay selectable.
//
// Attention sinks, logit soft-capping and sliding windows follow attn_prefill.cu, which stays the kernel for int8 caches
// and head sizes other than 64 / 128.  In the reference stack this is ggml-cuda's fattn family (mma / tile / vec).
#include "tc_common.cuh"

struct AttnPrefillArgs {      // the same block as in attn_prefill.cu
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
    const __half* k_scale;   // int8 cache: not taken by this kernel
    const __half* v_scale;
};

__device__ int g_attn_tc_status = 0;

namespace {

using namespace tc;
constexpr int BQ = 128, BKV = 128;
constexpr int ATOM_BYTES = 128 * 128;          // 128 rows x 64 f16: one swizzle atom column of a tile
constexpr int SOFTMAX_WARPS = 8;
constexpr int THREADS = (SOFTMAX_WARPS + 2) * 32;
constexpr int TMEM_COLS = 256;
constexpr int O_COL = 128;                     // first TMEM column of the P V tile

template <int D>
struct Lay {
    static constexpr int ATOMS = D / 64;
    static constexpr int Q_BYTES = ATOMS * ATOM_BYTES;
    static constexpr int KV_BYTES = ATOMS * ATOM_BYTES;      // one of K / V, one stage
    static constexpr int P_BYTES = 2 * ATOM_BYTES;
    static constexpr int OFF_K = Q_BYTES, OFF_V = OFF_K + 2 * KV_BYTES, OFF_P = OFF_V + 2 * KV_BYTES, OFF_BAR = OFF_P + P_BYTES;
    static constexpr int TOTAL = OFF_BAR + 256 + 2 * 2 * 128 * 4 + 1024;
};

// f16 x f16 -> fp32; B operand K-major (keys x D for Q K^T) or MN-major (keys x D for P V)
__host__ __device__ constexpr uint32_t idesc_f16(int m, int n, int b_mn_major) {
    return (1u << 4) | ((uint32_t)b_mn_major << 16) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// MN-major operand, 128-byte swizzle: 64 contiguous elements per row of 128 bytes, 8-row groups 1024 bytes apart along K,
// 64-element column blocks `lbo_bytes` apart.
__device__ __forceinline__ uint64_t umma_desc_mn(const void* smem_tile, uint32_t lbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_u32(smem_tile) & 0x3FFFF) >> 4);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}

// A operand from TMEM (lane = row, one 32-bit column = two consecutive K elements), B from shared memory
__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}

// 32 consecutive 32-bit columns of this thread's TMEM lane
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]),
          "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]),
          "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]),
          "r"(v[30]), "r"(v[31])
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&h);
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// 2-D f16 tensor [rows][d] (d contiguous), box = 64 x 128 rows, 128-byte swizzle, out-of-range rows read as zero.
bool make_kv_map(CUtensorMap* map, const void* base, size_t rows, int d) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {(cuuint64_t)d, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)d * 2};
    cuuint32_t box[2] = {64u, (cuuint32_t)BKV};
    cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// PT: the probabilities stay in TMEM (written over the first 64 columns of S, two f16 per column) and are the A operand of
// P V from there; otherwise they go through the swizzled shared-memory tile.
template <int D, bool PT>
__global__ void __launch_bounds__(THREADS, 1) attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                                                                     const __grid_constant__ AttnPrefillArgs a) {
    using L = Lay<D>;
    constexpr int ATOMS = L::ATOMS;
    constexpr int OH = D / 2;                  // output columns per softmax thread
    extern __shared__ uint8_t smem_raw[];
    uint8_t* sm = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* sQ = sm;
    uint8_t* sP = sm + L::OFF_P;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sm + L::OFF_BAR);
    uint64_t* kv_full = bars;            // [2]
    uint64_t* kv_empty = bars + 2;       // [2]
    uint64_t* s_full = bars + 4;
    uint64_t* p_ready = bars + 5;
    uint64_t* o_full = bars + 6;
    uint64_t* pair = bars + 7;           // [4]: the two warps of a TMEM lane quarter
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 11);
    float* x_max = reinterpret_cast<float*>(sm + L::OFF_BAR + 256);      // [2][128] row maxima of the two column halves
    float* x_sum = x_max + 256;                                           // [2][128] row sums at the end
    __shared__ int s_failed;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int mt = gridDim.x - 1 - blockIdx.x;       // late query tiles see the most keys: they start first
    const int m0 = mt * BQ, h = blockIdx.y, hkv = h / (a.H / a.Hkv);
    const int q_lo = a.pos0 + m0, q_hi = a.pos0 + min(m0 + BQ, a.T) - 1;
    const int k_end = a.causal ? min(a.kv_len, q_hi + 1) : a.kv_len;
    const int k_begin = (a.window > 0 ? max(0, q_lo - a.window + 1) : 0) & ~(BKV - 1);
    const int n_tiles = k_end > k_begin ? (k_end - k_begin + BKV - 1) / BKV : 0;

    if (threadIdx.x == 0) {
        s_failed = 0;
        for (int s = 0; s < 2; s++) {
            mbar_init(&kv_full[s], 1);
            mbar_init(&kv_empty[s], 1);
        }
        mbar_init(s_full, 1);
        mbar_init(p_ready, SOFTMAX_WARPS);
        mbar_init(o_full, 1);
        for (int q = 0; q < 4; q++) mbar_init(&pair[q], 2);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 9) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (warp < SOFTMAX_WARPS) {
        // Q tile: fp32 -> f16 in the swizzled K-major layout; thread = (row, column half)
        const int r = 32 * (warp & 3) + lane, c = warp >> 2;
        const bool live = m0 + r < a.T;
        const float* qp = a.q + ((size_t)(m0 + r) * a.H + h) * D + OH * c;
#pragma unroll
        for (int j = 0; j < OH / 8; j++) {           // 16-byte chunks of 8 values
            float4 v0 = make_float4(0.f, 0.f, 0.f, 0.f), v1 = v0;
            if (live) {
                v0 = *(const float4*)(qp + 8 * j);
                v1 = *(const float4*)(qp + 8 * j + 4);
            }
            const int col = OH * c + 8 * j;           // first column of the chunk
            const int atom = col >> 6, chunk = (col & 63) >> 3;
            *(uint4*)(sQ + atom * ATOM_BYTES + r * 128 + ((chunk ^ (r & 7)) << 4)) =
                make_uint4(pack_h2(v0.x, v0.y), pack_h2(v0.z, v0.w), pack_h2(v1.x, v1.y), pack_h2(v1.z, v1.w));
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp == 8) {
        if (lane == 0) {
            const int row0 = (a.slot * a.Hkv + hkv) * a.n_ctx + k_begin;
            for (int t = 0; t < n_tiles; t++) {
                const int s = t & 1;
                if (t >= 2 && !mbar_wait(&kv_empty[s], ((t >> 1) - 1) & 1)) { atomicExch(&s_failed, 1); break; }
                mbar_expect_tx(&kv_full[s], 2 * L::KV_BYTES);
#pragma unroll
                for (int at = 0; at < ATOMS; at++) {
                    tma_load_2d(sm + L::OFF_K + s * L::KV_BYTES + at * ATOM_BYTES, &map_k, 64 * at, row0 + t * BKV, &kv_full[s]);
                    tma_load_2d(sm + L::OFF_V + s * L::KV_BYTES + at * ATOM_BYTES, &map_v, 64 * at, row0 + t * BKV, &kv_full[s]);
                }
            }
        }
    } else if (warp == 9) {
        if (lane == 0 && n_tiles > 0) {
            constexpr uint32_t id_s = idesc_f16(BQ, BKV, 0), id_o = idesc_f16(BQ, D, 1);
            bool ok = true;
            auto issue_s = [&](int s) {          // S = Q K^T over the D / 16 K-steps
                const uint8_t* kt = sm + L::OFF_K + s * L::KV_BYTES;
#pragma unroll
                for (int at = 0; at < ATOMS; at++) {
                    const uint64_t qd = umma_desc(sQ + at * ATOM_BYTES), kd = umma_desc(kt + at * ATOM_BYTES);
#pragma unroll
                    for (int k = 0; k < 4; k++) umma_f16(tmem, qd + 2 * k, kd + 2 * k, id_s, (at | k) != 0);
                }
                umma_commit(s_full);
            };
            if (!mbar_wait(&kv_full[0], 0)) ok = false;
            if (ok) {
                tc_fence_after();
                issue_s(0);
            }
            for (int t = 0; t < n_tiles && ok; t++) {
                const int s = t & 1;
                if (!mbar_wait(p_ready, t & 1)) { ok = false; break; }
                tc_fence_after();
                const uint8_t* vt = sm + L::OFF_V + s * L::KV_BYTES;
#pragma unroll
                for (int kk = 0; kk < BKV / 16; kk++) {      // O_tile = P V, 16 keys per step
                    const uint64_t vd = umma_desc_mn(vt + kk * 16 * 128, ATOM_BYTES);
                    if (PT) {
                        umma_f16_ts(tmem + O_COL, tmem + 8 * kk, vd, id_o, kk != 0);
                    } else {
                        const uint64_t pd = umma_desc(sP + (kk >> 2) * ATOM_BYTES) + 2 * (kk & 3);
                        umma_f16(tmem + O_COL, pd, vd, id_o, kk != 0);
                    }
                }
                umma_commit(o_full);
                umma_commit(&kv_empty[s]);
                if (t + 1 < n_tiles) {
                    if (!mbar_wait(&kv_full[s ^ 1], ((t + 1) >> 1) & 1)) { ok = false; break; }
                    tc_fence_after();
                    issue_s(s ^ 1);
                }
            }
            if (!ok) atomicExch(&s_failed, 1);
        }
    } else {
        const int q = warp & 3, c = warp >> 2;
        const int r = 32 * q + lane;
        const int qp = a.pos0 + m0 + r;
        const float LOG2E = 1.4426950408889634f;
        const float sl2 = a.scale * LOG2E;
        const uint32_t lane_base = (uint32_t)(32 * q) << 16;
        float o[OH];
#pragma unroll
        for (int j = 0; j < OH; j++) o[j] = 0.f;
        float m_run = -INFINITY, l_run = 0.f;
        bool ok = true;
        for (int t = 0; t < n_tiles && ok; t++) {
            const int n0 = k_begin + t * BKV;
            if (!mbar_wait(s_full, t & 1)) { ok = false; break; }
            tc_fence_after();
            uint32_t v[2][32];
            tmem_ld32(tmem + lane_base + (uint32_t)(64 * c), v[0]);
            tmem_ld32(tmem + lane_base + (uint32_t)(64 * c + 32), v[1]);
            const bool masked = (a.causal && n0 + BKV - 1 > q_lo) || n0 + BKV > a.kv_len || a.window > 0;
            float mx = -INFINITY;
            if (a.softcap > 0.f) {                // scores end up in the log2 domain either way
                const float cap2 = a.softcap * LOG2E, inv_cap = a.scale / a.softcap;
#pragma unroll
                for (int i = 0; i < 2; i++)
#pragma unroll
                    for (int j = 0; j < 32; j++) v[i][j] = __float_as_uint(cap2 * tanhf(__uint_as_float(v[i][j]) * inv_cap));
            } else {
#pragma unroll
                for (int i = 0; i < 2; i++)
#pragma unroll
                    for (int j = 0; j < 32; j++) v[i][j] = __float_as_uint(__uint_as_float(v[i][j]) * sl2);
            }
            if (masked) {                         // warp-uniform: only tiles on the diagonal, at the window edge or at the end of the keys
                const int kp0 = n0 + 64 * c;
                const int hi = min(a.causal ? qp : a.kv_len - 1, a.kv_len - 1), lo = a.window > 0 ? qp - a.window + 1 : 0;
#pragma unroll
                for (int i = 0; i < 2; i++)
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        const int kp = kp0 + 32 * i + j;
                        if (kp > hi || kp < lo) v[i][j] = 0xff800000u;      // -inf
                    }
            }
#pragma unroll
            for (int i = 0; i < 2; i++)
#pragma unroll
                for (int j = 0; j < 32; j++) mx = fmaxf(mx, __uint_as_float(v[i][j]));
            // the other half of the row sits with the partner warp of this lane quarter
            x_max[c * 128 + r] = mx;
            __syncwarp();
            if (lane == 0) mbar_arrive(&pair[q]);
            if (!mbar_wait(&pair[q], t & 1)) { ok = false; break; }
            mx = fmaxf(mx, x_max[(c ^ 1) * 128 + r]);
            const float m_new = fmaxf(m_run, mx);
            const float corr = m_new == -INFINITY ? 1.f : ex2(m_run - m_new);
            const float mref = m_new == -INFINITY ? 0.f : m_new;
            m_run = m_new;
            float ls = 0.f;
            if (PT) {
                uint32_t pw[32];
#pragma unroll
                for (int i = 0; i < 2; i++)
#pragma unroll
                    for (int j = 0; j < 32; j += 2) {
                        const float p0 = ex2(__uint_as_float(v[i][j]) - mref), p1 = ex2(__uint_as_float(v[i][j + 1]) - mref);
                        ls += p0 + p1;
                        pw[16 * i + (j >> 1)] = pack_h2(p0, p1);
                    }
                // keys 64 c .. 64 c + 63 of this row = columns 32 c .. 32 c + 31; both warps of the quarter have read all of S by now
                tmem_st32(tmem + lane_base + (uint32_t)(32 * c), pw);
            } else {
                uint8_t* prow = sP + c * ATOM_BYTES + r * 128;
#pragma unroll
                for (int i = 0; i < 2; i++) {
#pragma unroll
                    for (int j = 0; j < 32; j += 8) {
                        float p[8];
#pragma unroll
                        for (int e = 0; e < 8; e++) {
                            p[e] = ex2(__uint_as_float(v[i][j + e]) - mref);
                            ls += p[e];
                        }
                        const int chunk = 4 * i + (j >> 3);
                        *(uint4*)(prow + ((chunk ^ (r & 7)) << 4)) = make_uint4(pack_h2(p[0], p[1]), pack_h2(p[2], p[3]), pack_h2(p[4], p[5]), pack_h2(p[6], p[7]));
                    }
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            }
            l_run = l_run * corr + ls;
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_ready);
            if (!mbar_wait(o_full, t & 1)) { ok = false; break; }
            tc_fence_after();
#pragma unroll
            for (int j0 = 0; j0 < OH; j0 += 32) {
                uint32_t ov[32];
                tmem_ld32(tmem + lane_base + (uint32_t)(O_COL + OH * c + j0), ov);
#pragma unroll
                for (int j = 0; j < 32; j++) o[j0 + j] = o[j0 + j] * corr + __uint_as_float(ov[j]);
            }
            tc_fence_before();
        }
        if (!ok) atomicExch(&s_failed, 1);
        // row sum of both halves, attention sink, normalise, store bf16
        x_sum[c * 128 + r] = l_run;
        __syncwarp();
        if (lane == 0) mbar_arrive(&pair[q]);
        if (ok && !mbar_wait(&pair[q], n_tiles & 1)) {
            ok = false;
            atomicExch(&s_failed, 1);
        }
        if (ok) {
            float l = l_run + x_sum[(c ^ 1) * 128 + r];
            float oc = 1.f;
            if (a.sinks) {
                const float sk = a.sinks[h] * LOG2E;
                const float m_new = fmaxf(m_run, sk);
                oc = m_run == -INFINITY ? 0.f : ex2(m_run - m_new);
                l = l * oc + ex2(sk - m_new);
            }
            const float inv = l > 0.f ? oc / l : 0.f;
            if (m0 + r < a.T) {
                __nv_bfloat16* op = a.out + (size_t)(m0 + r) * a.H * D + (size_t)h * D + OH * c;
#pragma unroll
                for (int j = 0; j < OH; j += 8) {
                    uint32_t w[4];
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        const __nv_bfloat162 b = __floats2bfloat162_rn(o[j + 2 * e] * inv, o[j + 2 * e + 1] * inv);
                        w[e] = *reinterpret_cast<const uint32_t*>(&b);
                    }
                    *(uint4*)(op + j) = make_uint4(w[0], w[1], w[2], w[3]);
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 9) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
    if (threadIdx.x == 0 && s_failed) atomicExch(&g_attn_tc_status, KS_TIMEOUT);
}

// The tensor map of a cache tensor depends on its address and extent only, and a model asks for the same few dozen tensors
// on every chunk: encoded maps are kept (per thread, so no lock) and found again by (address, rows, head size).
struct MapKey {
    const void* base;
    size_t rows;
    int d;
};
struct MapEntry {
    MapKey key;
    CUtensorMap map;
};
bool cached_kv_map(CUtensorMap* out, const void* base, size_t rows, int d) {
    constexpr int CAP = 512;                      // K and V of up to 256 layers; beyond that the oldest entries are replaced
    static thread_local MapEntry* table = nullptr;
    static thread_local int used = 0, next = 0;
    if (!table) table = new MapEntry[CAP];
    for (int i = 0; i < used; i++)
        if (table[i].key.base == base && table[i].key.rows == rows && table[i].key.d == d) {
            *out = table[i].map;
            return true;
        }
    if (!make_kv_map(out, base, rows, d)) return false;
    const int at = used < CAP ? used++ : (next++ % CAP);
    table[at] = MapEntry{{base, rows, d}, *out};
    return true;
}

// ---------------------------------------------------------------------------------------------------------------------
// Pipelined form.  Two score buffers and two P V tiles in TMEM (all 512 columns), the probabilities in TMEM over the scores
// they came from.  S of tile t + 2 is issued as soon as the softmax warps are done with S of tile t, so the scores of the next
// tile are always waiting when a softmax pass ends; and the softmax warps add P V of tile t - 1 to their accumulators after
// they have handed the probabilities of tile t to the tensor pipe, so that product runs under the accumulation instead of in
// front of it.  Roles: warps 0-7 softmax, warp 8 K loads, warp 9 MMA issue and TMEM allocation, warp 10 V loads.
// ---------------------------------------------------------------------------------------------------------------------
constexpr int THREADS2 = (SOFTMAX_WARPS + 3) * 32;
constexpr int TMEM_COLS2 = 512;

template <int D>
struct Lay2 {
    static constexpr int ATOMS = D / 64;
    static constexpr int Q_BYTES = ATOMS * ATOM_BYTES;
    static constexpr int KV_BYTES = ATOMS * ATOM_BYTES;
    static constexpr int OFF_K = Q_BYTES, OFF_V = OFF_K + 2 * KV_BYTES, OFF_BAR = OFF_V + 2 * KV_BYTES;
    static constexpr int TOTAL = OFF_BAR + 256 + 2 * 2 * 128 * 4 + 1024;
};

template <int D>
__global__ void __launch_bounds__(THREADS2, 1) attn_prefill_tc2_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                                                                       const __grid_constant__ AttnPrefillArgs a) {
    using L = Lay2<D>;
    constexpr int ATOMS = L::ATOMS;
    constexpr int OH = D / 2;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* sm = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* sQ = sm;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sm + L::OFF_BAR);
    uint64_t* k_full = bars;             // every barrier below: one per buffer
    uint64_t* k_empty = bars + 2;
    uint64_t* v_full = bars + 4;
    uint64_t* v_empty = bars + 6;
    uint64_t* s_full = bars + 8;
    uint64_t* p_ready = bars + 10;
    uint64_t* o_full = bars + 12;
    uint64_t* pair = bars + 14;          // [4]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 18);
    int* failed = reinterpret_cast<int*>(bars + 19);
    float* x_max = reinterpret_cast<float*>(sm + L::OFF_BAR + 256);
    float* x_sum = x_max + 256;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int mt = gridDim.x - 1 - blockIdx.x;
    const int m0 = mt * BQ, h = blockIdx.y, hkv = h / (a.H / a.Hkv);
    const int q_lo = a.pos0 + m0, q_hi = a.pos0 + min(m0 + BQ, a.T) - 1;
    const int k_end = a.causal ? min(a.kv_len, q_hi + 1) : a.kv_len;
    const int k_begin = (a.window > 0 ? max(0, q_lo - a.window + 1) : 0) & ~(BKV - 1);
    const int n_tiles = k_end > k_begin ? (k_end - k_begin + BKV - 1) / BKV : 0;

    if (threadIdx.x == 0) {
        *failed = 0;
        for (int b = 0; b < 2; b++) {
            mbar_init(&k_full[b], 1);
            mbar_init(&k_empty[b], 1);
            mbar_init(&v_full[b], 1);
            mbar_init(&v_empty[b], 1);
            mbar_init(&s_full[b], 1);
            mbar_init(&p_ready[b], SOFTMAX_WARPS);
            mbar_init(&o_full[b], 1);
        }
        for (int q = 0; q < 4; q++) mbar_init(&pair[q], 2);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 9) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS2) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (warp < SOFTMAX_WARPS) {
        const int r = 32 * (warp & 3) + lane, c = warp >> 2;
        const bool live = m0 + r < a.T;
        const float* qp = a.q + ((size_t)(m0 + r) * a.H + h) * D + OH * c;
#pragma unroll
        for (int j = 0; j < OH / 8; j++) {
            float4 v0 = make_float4(0.f, 0.f, 0.f, 0.f), v1 = v0;
            if (live) {
                v0 = *(const float4*)(qp + 8 * j);
                v1 = *(const float4*)(qp + 8 * j + 4);
            }
            const int col = OH * c + 8 * j;
            const int atom = col >> 6, chunk = (col & 63) >> 3;
            *(uint4*)(sQ + atom * ATOM_BYTES + r * 128 + ((chunk ^ (r & 7)) << 4)) =
                make_uint4(pack_h2(v0.x, v0.y), pack_h2(v0.z, v0.w), pack_h2(v1.x, v1.y), pack_h2(v1.z, v1.w));
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const int row0 = (a.slot * a.Hkv + hkv) * a.n_ctx + k_begin;

    if (warp == 8 || warp == 10) {
        if (lane == 0) {                 // one thread streams the K tiles, another the V tiles: each waits only for its own buffers
            const bool is_k = warp == 8;
            const CUtensorMap* map = is_k ? &map_k : &map_v;
            uint64_t* full = is_k ? k_full : v_full;
            uint64_t* empty = is_k ? k_empty : v_empty;
            uint8_t* base = sm + (is_k ? L::OFF_K : L::OFF_V);
            for (int t = 0; t < n_tiles; t++) {
                const int b = t & 1;
                if (t >= 2 && !mbar_wait(&empty[b], ((t >> 1) - 1) & 1)) { atomicExch(failed, 1); break; }
                mbar_expect_tx(&full[b], L::KV_BYTES);
#pragma unroll
                for (int at = 0; at < ATOMS; at++) tma_load_2d(base + b * L::KV_BYTES + at * ATOM_BYTES, map, 64 * at, row0 + t * BKV, &full[b]);
            }
        }
    } else if (warp == 9) {
        if (lane == 0 && n_tiles > 0) {
            constexpr uint32_t id_s = idesc_f16(BQ, BKV, 0), id_o = idesc_f16(BQ, D, 1);
            bool ok = true;
            auto issue_s = [&](int t) {          // S(t) = Q K(t)^T into score buffer t & 1
                const int b = t & 1;
                if (!mbar_wait(&k_full[b], (t >> 1) & 1)) { ok = false; return; }
                tc_fence_after();
                const uint8_t* kt = sm + L::OFF_K + b * L::KV_BYTES;
#pragma unroll
                for (int at = 0; at < ATOMS; at++) {
                    const uint64_t qd = umma_desc(sQ + at * ATOM_BYTES), kd = umma_desc(kt + at * ATOM_BYTES);
#pragma unroll
                    for (int k = 0; k < 4; k++) umma_f16(tmem + 128 * b, qd + 2 * k, kd + 2 * k, id_s, (at | k) != 0);
                }
                umma_commit(&s_full[b]);
                umma_commit(&k_empty[b]);
            };
            issue_s(0);
            if (ok && n_tiles > 1) issue_s(1);
            for (int t = 0; t < n_tiles && ok; t++) {
                const int b = t & 1, ph = (t >> 1) & 1;
                if (!mbar_wait(&p_ready[b], ph) || !mbar_wait(&v_full[b], ph)) { ok = false; break; }
                tc_fence_after();
                const uint8_t* vt = sm + L::OFF_V + b * L::KV_BYTES;
#pragma unroll
                for (int kk = 0; kk < BKV / 16; kk++)      // O_tile(t) = P(t) V(t); P sits in the first 64 columns of its score buffer
                    umma_f16_ts(tmem + 256 + 128 * b, tmem + 128 * b + 8 * kk, umma_desc_mn(vt + kk * 16 * 128, ATOM_BYTES), id_o, kk != 0);
                umma_commit(&o_full[b]);
                umma_commit(&v_empty[b]);
                if (t + 2 < n_tiles) issue_s(t + 2);       // runs behind P V(t), which still reads the buffer it overwrites
            }
            if (!ok) atomicExch(failed, 1);
        }
    } else {
        const int q = warp & 3, c = warp >> 2;
        const int r = 32 * q + lane;
        const int qp = a.pos0 + m0 + r;
        const float LOG2E = 1.4426950408889634f;
        const float sl2 = a.scale * LOG2E;
        const uint32_t lane_base = (uint32_t)(32 * q) << 16;
        float o[OH];
#pragma unroll
        for (int j = 0; j < OH; j++) o[j] = 0.f;
        float m_run = -INFINITY, l_run = 0.f, corr_prev = 1.f;
        bool ok = true;
        auto accumulate = [&](int t, float corr) {      // o = o * corr + O_tile(t)
            const int b = t & 1;
            if (!mbar_wait(&o_full[b], (t >> 1) & 1)) { ok = false; return; }
            tc_fence_after();
#pragma unroll
            for (int j0 = 0; j0 < OH; j0 += 32) {
                uint32_t ov[32];
                tmem_ld32(tmem + lane_base + (uint32_t)(256 + 128 * b + OH * c + j0), ov);
#pragma unroll
                for (int j = 0; j < 32; j++) o[j0 + j] = o[j0 + j] * corr + __uint_as_float(ov[j]);
            }
            tc_fence_before();
        };
        for (int t = 0; t < n_tiles && ok; t++) {
            const int b = t & 1;
            const int n0 = k_begin + t * BKV;
            if (!mbar_wait(&s_full[b], (t >> 1) & 1)) { ok = false; break; }
            tc_fence_after();
            uint32_t v[2][32];
            tmem_ld32(tmem + lane_base + (uint32_t)(128 * b + 64 * c), v[0]);
            tmem_ld32(tmem + lane_base + (uint32_t)(128 * b + 64 * c + 32), v[1]);
            const bool masked = (a.causal && n0 + BKV - 1 > q_lo) || n0 + BKV > a.kv_len || a.window > 0;
            float mx = -INFINITY;
            if (a.softcap > 0.f) {
                const float cap2 = a.softcap * LOG2E, inv_cap = a.scale / a.softcap;
#pragma unroll
                for (int i = 0; i < 2; i++)
#pragma unroll
                    for (int j = 0; j < 32; j++) v[i][j] = __float_as_uint(cap2 * tanhf(__uint_as_float(v[i][j]) * inv_cap));
            } else {
#pragma unroll
                for (int i = 0; i < 2; i++)
#pragma unroll
                    for (int j = 0; j < 32; j++) v[i][j] = __float_as_uint(__uint_as_float(v[i][j]) * sl2);
            }
            if (masked) {
                const int kp0 = n0 + 64 * c;
                const int hi = min(a.causal ? qp : a.kv_len - 1, a.kv_len - 1), lo = a.window > 0 ? qp - a.window + 1 : 0;
#pragma unroll
                for (int i = 0; i < 2; i++)
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        const int kp = kp0 + 32 * i + j;
                        if (kp > hi || kp < lo) v[i][j] = 0xff800000u;
                    }
            }
#pragma unroll
            for (int i = 0; i < 2; i++)
#pragma unroll
                for (int j = 0; j < 32; j++) mx = fmaxf(mx, __uint_as_float(v[i][j]));
            x_max[c * 128 + r] = mx;
            __syncwarp();
            if (lane == 0) mbar_arrive(&pair[q]);
            if (!mbar_wait(&pair[q], t & 1)) { ok = false; break; }
            mx = fmaxf(mx, x_max[(c ^ 1) * 128 + r]);
            const float m_new = fmaxf(m_run, mx);
            const float corr = m_new == -INFINITY ? 1.f : ex2(m_run - m_new);
            const float mref = m_new == -INFINITY ? 0.f : m_new;
            m_run = m_new;
            float ls = 0.f;
            uint32_t pw[32];
#pragma unroll
            for (int i = 0; i < 2; i++)
#pragma unroll
                for (int j = 0; j < 32; j += 2) {
                    const float p0 = ex2(__uint_as_float(v[i][j]) - mref), p1 = ex2(__uint_as_float(v[i][j + 1]) - mref);
                    ls += p0 + p1;
                    pw[16 * i + (j >> 1)] = pack_h2(p0, p1);
                }
            tmem_st32(tmem + lane_base + (uint32_t)(128 * b + 32 * c), pw);      // both warps of the quarter have read all of S(t) by now
            l_run = l_run * corr + ls;
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_ready[b]);
            if (t >= 1) accumulate(t - 1, corr_prev);      // P V(t - 1) finished long ago; P V(t) runs under this
            corr_prev = corr;
        }
        if (ok && n_tiles > 0) accumulate(n_tiles - 1, corr_prev);
        if (!ok) atomicExch(failed, 1);
        x_sum[c * 128 + r] = l_run;
        __syncwarp();
        if (lane == 0) mbar_arrive(&pair[q]);
        if (ok && !mbar_wait(&pair[q], n_tiles & 1)) {
            ok = false;
            atomicExch(failed, 1);
        }
        if (ok) {
            float l = l_run + x_sum[(c ^ 1) * 128 + r];
            float oc = 1.f;
            if (a.sinks) {
                const float sk = a.sinks[h] * LOG2E;
                const float m_new = fmaxf(m_run, sk);
                oc = m_run == -INFINITY ? 0.f : ex2(m_run - m_new);
                l = l * oc + ex2(sk - m_new);
            }
            const float inv = l > 0.f ? oc / l : 0.f;
            if (m0 + r < a.T) {
                __nv_bfloat16* op = a.out + (size_t)(m0 + r) * a.H * D + (size_t)h * D + OH * c;
#pragma unroll
                for (int j = 0; j < OH; j += 8) {
                    uint32_t w[4];
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        const __nv_bfloat162 bb = __floats2bfloat162_rn(o[j + 2 * e] * inv, o[j + 2 * e + 1] * inv);
                        w[e] = *reinterpret_cast<const uint32_t*>(&bb);
                    }
                    *(uint4*)(op + j) = make_uint4(w[0], w[1], w[2], w[3]);
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 9) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS2) : "memory");
    }
    if (threadIdx.x == 0 && *failed) atomicExch(&g_attn_tc_status, KS_TIMEOUT);
}


int g_variant = 2;      // 0: probabilities through shared memory, 1: probabilities in TMEM, 2: the pipelined kernel (default)

template <int D, bool PT>
int launch(const AttnPrefillArgs& a, int n_slots, cudaStream_t st) {
    CUtensorMap mk, mv;
    const size_t rows = (size_t)n_slots * a.Hkv * a.n_ctx;
    if (!cached_kv_map(&mk, a.k_cache, rows, D) || !cached_kv_map(&mv, a.v_cache, rows, D)) return (int)cudaErrorNotSupported;
    static PerDeviceOnce once;
    if (once.first()) cudaFuncSetAttribute(attn_prefill_tc_kernel<D, PT>, cudaFuncAttributeMaxDynamicSharedMemorySize, Lay<D>::TOTAL);
    dim3 grid((a.T + BQ - 1) / BQ, a.H);
    attn_prefill_tc_kernel<D, PT><<<grid, THREADS, Lay<D>::TOTAL, st>>>(mk, mv, a);
    return (int)cudaGetLastError();
}

template <int D>
int launch2(const AttnPrefillArgs& a, int n_slots, cudaStream_t st) {
    CUtensorMap mk, mv;
    const size_t rows = (size_t)n_slots * a.Hkv * a.n_ctx;
    if (!cached_kv_map(&mk, a.k_cache, rows, D) || !cached_kv_map(&mv, a.v_cache, rows, D)) return (int)cudaErrorNotSupported;
    static PerDeviceOnce once;
    if (once.first()) cudaFuncSetAttribute(attn_prefill_tc2_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, Lay2<D>::TOTAL);
    dim3 grid((a.T + BQ - 1) / BQ, a.H);
    attn_prefill_tc2_kernel<D><<<grid, THREADS2, Lay2<D>::TOTAL, st>>>(mk, mv, a);
    return (int)cudaGetLastError();
}

}  // namespace

// Prefill attention on tcgen05: f16 caches, head size 64 or 128 (anything else: cudaErrorNotSupported, nothing launched; the
// caller then runs b2_attn_prefill).  `n_slots`: slots of the cache tensors (the extent of the TMA maps).  Returns a cudaError_t value.
B2_API int b2_attn_prefill_tc(const AttnPrefillArgs* a, int head_dim, int n_slots, cudaStream_t st) {
    if (!a || a->T < 1 || a->H < 1 || a->Hkv < 1 || a->H % a->Hkv || a->kv_len < 1 || a->kv_len > a->n_ctx || n_slots < 1 || a->slot < 0 ||
        a->slot >= n_slots)
        return (int)cudaErrorInvalidValue;
    if (a->k_scale || a->v_scale) return (int)cudaErrorNotSupported;
    if (((uintptr_t)a->k_cache & 15) || ((uintptr_t)a->v_cache & 15) || ((uintptr_t)a->q & 15) || ((uintptr_t)a->out & 15)) return (int)cudaErrorNotSupported;
    if ((size_t)n_slots * a->Hkv * a->n_ctx >= ((size_t)1 << 31)) return (int)cudaErrorNotSupported;
    if (g_variant == 2 && head_dim == 128) return launch2<128>(*a, n_slots, st);
    if (g_variant == 2 && head_dim == 64) return launch2<64>(*a, n_slots, st);
    if (head_dim == 128) return g_variant ? launch<128, true>(*a, n_slots, st) : launch<128, false>(*a, n_slots, st);
    if (head_dim == 64) return g_variant ? launch<64, true>(*a, n_slots, st) : launch<64, false>(*a, n_slots, st);
    return (int)cudaErrorNotSupported;
}

// 0: the probabilities go through shared memory; 1: they stay in TMEM; 2: the pipelined kernel (default).  Returns the previous setting.
B2_API int b2_attn_prefill_tc_variant(int v) {
    const int old = g_variant;
    if (v >= 0 && v <= 2) g_variant = v;
    return old;
}

B2_API int b2_attn_prefill_tc_status() {
    int v = 0;
    cudaMemcpyFromSymbol(&v, g_attn_tc_status, sizeof(int));
    return v;
}

B2_API void b2_attn_prefill_tc_clear_status() {
    const int v = 0;
    cudaMemcpyToSymbol(g_attn_tc_status, &v, sizeof(int));
}
