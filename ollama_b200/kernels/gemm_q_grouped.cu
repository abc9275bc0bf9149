// Grouped expert GEMM that streams the experts in their 4-bit encoding (MXFP4), sm_100a:
//   out[rows of tile t][:] = X[rows of tile t][K] (bf16) . W[expert(t)][N][K]^T + bias[expert(t)]      (+ gated activation)
//
// Mixture-of-experts prefill: the (token, expert) rows are sorted by expert into 128-row tiles (kernels/moe.cu builds the
// tile -> expert table on the device).  A 16-bit copy of the experts would have to be streamed from HBM for every chunk
// (3.8 x the bytes of the MXFP4 blocks, and it does not fit beside them for the large models), so this kernel reads the
// blocks themselves.  One CTA = one 128-row tile x 128 weight rows of that tile's expert:
//   * warp 0 brings the activation tile of every K block (64 columns) by TMA into a 2-stage ring (two CTAs share an SM);
//   * warps 2-9 stream the weight bytes: each thread owns 32 columns of one weight row per K block (16 bytes of nibbles and
//     one E8M0 scale), keeps six K blocks in flight with cp.async into a private shared-memory ring (enough bytes per SM to
//     cover HBM latency), turns the codes into bf16 with one integer multiply, one mask and one packed multiply per pair (the 3 magnitude bits dropped into
//     the exponent / mantissa of a bf16 are 2^-126 times the value, subnormals included) and writes them into the stage buffer
//     in the 128-byte-swizzled K-major layout the tensor core reads;
//   * warp 1 issues tcgen05.mma (M 128 x N 128 x K 16, bf16) into a TMEM accumulator;
//   * warps 2-9 drain the accumulator: bias, then either fp32 rows or the gated activation of interleaved gate / up columns as bf16.
// Tiles of the table's padding (expert -1) return at once.  Every mbarrier wait is bounded (KS_TIMEOUT in the status word).
//
// In the reference stack the same product is ggml-cuda's mul_mat_id over MXFP4 experts (mmq / mmvq kernels with in-kernel
// dequantisation feeding mma.sync); this is its tcgen05 / TMEM / TMA form.
#include "tc_common.cuh"

__device__ int g_gemm_qg_status = 0;

namespace {

using namespace tc;
constexpr int BN = 128;
constexpr int STAGES = 2;
constexpr int DEPTH = 6;                       // K blocks of weight bytes in flight per thread
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2;
constexpr int DEQ_WARPS = 8;
constexpr int THREADS = (2 + DEQ_WARPS) * 32;
constexpr int RING_BYTES = DEPTH * DEQ_WARPS * 32 * 16;

struct QGroupedParams {
    WDesc w;                 // MXFP4 planes of all experts stacked: row e * n + r
    int m;                   // rows of x: a multiple of 128
    const int* tile_expert;  // [m / 128]: expert of the tile, -1 = padding
    void* out;               // fp32 [m][ldo], or bf16 [m][ldo] holding n / 2 columns with glu
    int ldo;
    const float* bias;       // [experts][n] or null
    int glu;                 // 0: off, 1 + activation otherwise (columns 2i / 2i + 1 = gate / up of output i)
    float alpha, limit;
    int scale_pitch;         // bytes per row of the shared-memory copy of the E8M0 scales
};

__device__ __forceinline__ uint32_t mul_bf16x2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

// Four E2M1 codes, one per byte of `codes` (sign in bit 3) -> two bf16x2 words of value * 2^(e-127).
// A code c spread over a 16-bit lane and multiplied by 0x1040 is (c << 6) + (c << 12): the magnitude bits EEM land in bits 8..6
// and the sign in bit 15 (mask 0x81C0 drops the rest).  Read as bf16 that is 2^(E-127) (1 + M/2), or M 2^-127 for E = 0: the E2M1
// value times 2^-126 in every case, subnormal or not.  One packed multiply by `mult2` = bf16x2 2^(e-1) restores the value and
// applies the block scale (exact: a power of two); blocks with e > 128 (scales above 2, which 2^(e-1) cannot hold next to the
// 2^126) take two multiplies, by 2^126 and by 2^(e-127).
__device__ __forceinline__ void expand_fp4x4(uint32_t codes, uint32_t mult2, uint32_t& w01, uint32_t& w23) {
    const uint32_t b01 = (__byte_perm(codes, 0u, 0x4140) * 0x1040u) & 0x81C081C0u;      // {c0, 0, c1, 0}
    const uint32_t b23 = (__byte_perm(codes, 0u, 0x4342) * 0x1040u) & 0x81C081C0u;
    w01 = mul_bf16x2(b01, mult2);
    w23 = mul_bf16x2(b23, mult2);
}

__global__ void __launch_bounds__(THREADS, 2) gemm_q_grouped_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ QGroupedParams p) {
    const int mt = blockIdx.y;
    const int e = p.tile_expert[mt];
    if (e < 0) return;                                   // padding of the tile table: the whole CTA leaves before it owns anything

    extern __shared__ uint8_t smem_raw[];
    uint8_t* tiles = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* ring = tiles + STAGES * (A_BYTES + B_BYTES);
    uint64_t* full = reinterpret_cast<uint64_t*>(ring + RING_BYTES);
    uint64_t* empty = full + STAGES;
    uint64_t* acc_ready = empty + STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_ready + 1);
    int* failed = reinterpret_cast<int*>(tmem_slot + 1);
    uint8_t* scales = ring + RING_BYTES + 128;            // [128][scale_pitch]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * BN, m0 = mt * BM;
    const int K = p.w.k, k_blocks = K / BK, n = p.w.n;

    if (threadIdx.x == 0) {
        *failed = 0;
        for (int s = 0; s < STAGES; s++) {
            mbar_init(&full[s], 1 + DEQ_WARPS);          // the TMA producer (with its byte count) + one arrival per expanding warp
            mbar_init(&empty[s], 1);
        }
        mbar_init(acc_ready, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(BN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // weight streaming starts before anything else is ready: the first DEPTH - 1 K blocks of this thread's row
    const int dt = threadIdx.x - 64;
    const int r = dt & 127, h = dt >> 7;
    const size_t wrow = (size_t)e * n + min(n0 + r, n - 1);
    const uint8_t* qrow = (const uint8_t*)p.w.p0 + wrow * (size_t)(K >> 1) + 16 * h;
    uint4* my_ring = reinterpret_cast<uint4*>(ring) + dt;
    if (warp >= 2) {
        for (int kb = 0; kb < DEPTH - 1; kb++) {
            if (kb < k_blocks) cp_async16(my_ring + (kb % DEPTH) * (DEQ_WARPS * 32), qrow + kb * 32);
            asm volatile("cp.async.commit_group;" ::: "memory");
        }
        // the E8M0 scales of the tile's 128 weight rows, all K blocks: K / 32 bytes per row
        const int spr = K >> 5;
        for (int i = dt; i < 128 * spr; i += DEQ_WARPS * 32) {
            const int rr = i / spr, c = i - rr * spr;
            scales[rr * p.scale_pitch + c] = __ldg((const uint8_t*)p.w.p1 + ((size_t)e * n + min(n0 + rr, n - 1)) * spr + c);
        }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_acc = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            for (int kb = 0; kb < k_blocks; kb++) {
                const int s = kb % STAGES;
                if (kb >= STAGES && !mbar_wait(&empty[s], ((kb / STAGES) - 1) & 1)) { atomicExch(failed, 1); break; }
                mbar_expect_tx(&full[s], A_BYTES);
                tma_load_2d(tiles + s * (A_BYTES + B_BYTES), &map_a, kb * BK, m0, &full[s]);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc(BM, BN);
            bool ok = true;
            for (int kb = 0; kb < k_blocks; kb++) {
                const int s = kb % STAGES;
                if (!mbar_wait(&full[s], (kb / STAGES) & 1)) { ok = false; atomicExch(failed, 1); break; }
                tc_fence_after();
                const uint8_t* a_src = tiles + s * (A_BYTES + B_BYTES);
                const uint64_t adesc = umma_desc(a_src), bdesc = umma_desc(a_src + A_BYTES);
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; k++) umma_bf16(tmem_acc, adesc + 2 * k, bdesc + 2 * k, idesc, (kb | k) != 0);
                umma_commit(&empty[s]);
            }
            if (ok) umma_commit(acc_ready);
        }
    } else {
        bool ok = true;
        for (int kb = 0; kb < k_blocks && ok; kb++) {
            const int s = kb % STAGES;
            const int nxt = kb + DEPTH - 1;
            if (nxt < k_blocks) cp_async16(my_ring + (nxt % DEPTH) * (DEQ_WARPS * 32), qrow + nxt * 32);
            asm volatile("cp.async.commit_group;" ::: "memory");
            asm volatile("cp.async.wait_group %0;" ::"n"(DEPTH - 1) : "memory");
            const uint4 q = my_ring[(kb % DEPTH) * (DEQ_WARPS * 32)];
            const uint32_t eb = scales[r * p.scale_pitch + 2 * kb + h];                     // E8M0: the block scale is 2^(eb - 127)
            const bool wide = eb > 128u;
            const uint32_t m1 = wide ? 0x7E80u : (eb == 0u ? 0u : (eb + 126u) << 7);           // bf16 2^126, or 2^(eb - 1) (eb = 0 reads as zero)
            const uint32_t mult2 = m1 | (m1 << 16);
            // byte j of the 16: low nibble = column j, high nibble = column 16 + j of this thread's 32
            const uint32_t qw[4] = {q.x, q.y, q.z, q.w};
            uint32_t vals[16];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                expand_fp4x4(qw[i] & 0x0f0f0f0fu, mult2, vals[2 * i], vals[2 * i + 1]);
                expand_fp4x4((qw[i] >> 4) & 0x0f0f0f0fu, mult2, vals[8 + 2 * i], vals[8 + 2 * i + 1]);
            }
            if (wide) {                                   // rare: scales above 2
                const uint32_t s1 = eb << 7, s2 = s1 | (s1 << 16);
#pragma unroll
                for (int i = 0; i < 16; i++) vals[i] = mul_bf16x2(vals[i], s2);
            }
            if (kb >= STAGES) ok = mbar_wait(&empty[s], ((kb / STAGES) - 1) & 1);
            if (ok) {
                uint8_t* row = tiles + s * (A_BYTES + B_BYTES) + A_BYTES + r * 128;
#pragma unroll
                for (int c = 0; c < 4; c++)
                    *reinterpret_cast<uint4*>(row + (((4 * h + c) ^ (r & 7)) << 4)) = make_uint4(vals[4 * c], vals[4 * c + 1], vals[4 * c + 2], vals[4 * c + 3]);
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            }
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&full[s])) : "memory");
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        if (!ok) atomicExch(failed, 1);
        const int q4 = warp & 3;                              // TMEM lane quarter this warp may read
        const int chalf = (warp - 2) >> 2;                    // which 64 accumulator columns this warp drains
        const bool ready = ok && mbar_wait(acc_ready, 0);
        if (!ready) atomicExch(failed, 1);
        tc_fence_after();
        const int row = m0 + q4 * 32 + lane;
        if (ready && row < p.m) {
#pragma unroll 1
            for (int c0 = 64 * chalf; c0 < 64 * chalf + 64; c0 += 32) {
                uint32_t v[32];
                tmem_ld32(tmem_acc + ((uint32_t)(q4 * 32) << 16) + (uint32_t)c0, v);
                const int col0 = n0 + c0;
                if (col0 >= n) continue;
                const float* bias = p.bias ? p.bias + (size_t)e * n + col0 : nullptr;
                if (p.glu) {
                    __nv_bfloat16* o = (__nv_bfloat16*)p.out + (size_t)row * p.ldo + (col0 >> 1);
#pragma unroll
                    for (int j = 0; j < 32; j += 8) {
                        if (col0 + j >= n) break;
                        uint32_t w[2];
#pragma unroll
                        for (int t = 0; t < 2; t++) {
                            float g0 = __uint_as_float(v[j + 4 * t]), u0 = __uint_as_float(v[j + 4 * t + 1]);
                            float g1 = __uint_as_float(v[j + 4 * t + 2]), u1 = __uint_as_float(v[j + 4 * t + 3]);
                            if (bias) {
                                g0 += bias[j + 4 * t]; u0 += bias[j + 4 * t + 1];
                                g1 += bias[j + 4 * t + 2]; u1 += bias[j + 4 * t + 3];
                            }
                            w[t] = pack2(glu_act(g0, u0, p.glu - 1, p.alpha, p.limit), glu_act(g1, u1, p.glu - 1, p.alpha, p.limit));
                        }
                        *reinterpret_cast<uint2*>(o + (j >> 1)) = make_uint2(w[0], w[1]);
                    }
                } else {
                    float* o = (float*)p.out + (size_t)row * p.ldo + col0;
#pragma unroll
                    for (int j = 0; j < 32; j += 4) {
                        if (col0 + j >= n) break;
                        float4 t = make_float4(__uint_as_float(v[j]), __uint_as_float(v[j + 1]), __uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
                        if (bias) {
                            t.x += bias[j]; t.y += bias[j + 1]; t.z += bias[j + 2]; t.w += bias[j + 3];
                        }
                        *reinterpret_cast<float4*>(o + j) = t;
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "r"(BN) : "memory");
    }
    if (threadIdx.x == 0 && *failed) atomicExch(&g_gemm_qg_status, KS_TIMEOUT);
}

}  // namespace

// Grouped product over MXFP4 experts.  x: bf16 [m][k], m a multiple of 128, rows sorted by expert in 128-row tiles;
// w: the stacked experts (w->n rows each, `experts` of them; w->type must be WT_MXFP4, k a multiple of 64, n of 8);
// out: fp32 [m][ldo] (glu_act_id < 0), or bf16 [m][ldo] with n / 2 activated columns; bias: [experts][n] or null.
// Other encodings or shapes: cudaErrorNotSupported (nothing launched).  Returns a cudaError_t value.
B2_API int b2_gemm_q_grouped(const void* x, int m, const WDesc* w, int experts, const int* tile_expert, void* out, int ldo, const float* bias,
                             int glu_act_id, float alpha, float limit, cudaStream_t st) {
    if (!x || !w || !tile_expert || !out || m < 128 || (m & 127) || experts < 1 || glu_act_id > 2 || ((uintptr_t)x & 15) || ((uintptr_t)out & 15))
        return (int)cudaErrorInvalidValue;
    if (w->type != WT_MXFP4 || (w->k & 63) || w->k < 64 || (w->n & 7) || ((uintptr_t)w->p0 & 15)) return (int)cudaErrorNotSupported;
    if (glu_act_id >= 0 ? (ldo & 3) : (ldo & 3)) return (int)cudaErrorInvalidValue;
    CUtensorMap ma;
    if (!tc::make_map(&ma, x, m, w->k, BM)) return (int)cudaErrorNotSupported;
    const int scale_pitch = ((w->k >> 5) + 3) & ~3;
    const int smem = STAGES * (A_BYTES + B_BYTES) + RING_BYTES + 128 + 128 * scale_pitch + 1024;
    if (smem > 227 * 1024) return (int)cudaErrorNotSupported;
    static PerDeviceOnce once;
    if (once.first()) cudaFuncSetAttribute(gemm_q_grouped_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    QGroupedParams p{*w, m, tile_expert, out, ldo, bias, glu_act_id >= 0 ? 1 + glu_act_id : 0, alpha, limit, scale_pitch};
    dim3 grid((w->n + BN - 1) / BN, m / BM);
    gemm_q_grouped_kernel<<<grid, THREADS, smem, st>>>(ma, p);
    return (int)cudaGetLastError();
}

B2_API int b2_gemm_q_grouped_status() {
    int v = 0;
    cudaMemcpyFromSymbol(&v, g_gemm_qg_status, sizeof(int));
    return v;
}
