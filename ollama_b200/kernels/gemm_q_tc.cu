// Dequantisation-fused tensor-core GEMM for prefill on sm_100a:
//   out[M, N] (+)= X[M, K] (bf16) . W[N, K]^T (GGUF-quantised, plane layout) + bias
//
// The activation tile (A operand) arrives by TMA as in gemm_tc.cu.  The weight tile (B operand) never
// exists in global memory in 16-bit form: eight producer warps read the quantised planes of 128 weight
// rows x 64 columns (one thread = 32 columns of one row), expand them to bf16 in registers and write
// them into the stage buffer in exactly the 128-byte-swizzled K-major layout that the tcgen05
// shared-memory descriptor expects (16-byte chunk c of row r lives at chunk c ^ (r & 7)); a proxy
// fence publishes those generic-proxy writes to the tensor core.  The raw bytes of the next K block
// are requested before the current one is expanded, so global latency stays off the critical path.
// 4- and 6-bit codes become bf16 with one byte-permute, one packed subtraction and one packed FMA per
// pair: the code q is dropped into the mantissa of 128.0 (bf16 0x43qq = 128 + q, exact for q < 128),
// 128 + zero-point is subtracted (exact) and w = (q - zero) * scale + offset is a fma.rn.bf16x2.
// One elected thread issues tcgen05.mma (M = 128 tokens, N = 128 weight rows) into a TMEM accumulator;
// four of the producer warps drain it once their last stage is written.  All mbarrier waits are
// bounded (KS_TIMEOUT in the status word on expiry).
//
// This is the counterpart of ggml-cuda's mmq kernels (in-kernel dequantisation feeding mma.sync) and of
// its dequantise-then-cuBLAS path, redone for tcgen05 / TMEM.
#include "tc_common.cuh"
#include "comm.cuh"

__device__ int g_gemm_q_status = 0;

namespace {

using namespace tc;
constexpr int BN = 128;          // weight rows per CTA (MMA N)
constexpr int STAGES = 3;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int SMEM_TOTAL = STAGES * STAGE_BYTES + 1024 + 256;
constexpr int DEQ_WARPS = 8;
constexpr int THREADS = (2 + DEQ_WARPS) * 32;

struct QGemmParams {
    WDesc w;                // quantised weight [n][k]
    int m;
    float* out;
    int ldo;
    int accumulate;
    // tensor parallel (cm.n_dst > 0): row m of the result belongs to rank m / rows_per_rank; the tile is stored into that
    // rank's buffer cm.dst[owner] (pitch ldo, row index relative to the owner's first row) and the exchange is announced.
    CommSend cm;
    int rows_per_rank;
};

// Raw bytes of 32 columns of one weight row (what a producer thread fetches per K block).
struct Raw {
    uint4 a, b, c, d;
    uint32_t s0, s1;
};

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}
__device__ __forceinline__ uint32_t bf16x2_fma(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ uint32_t bf16x2_splat(float v) { return pack_bf16(v, v); }

__device__ __forceinline__ uint32_t bf16x2_sub(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}

// Four byte-sized codes (one per byte of `codes`) -> two bf16x2 words of scale * (code - zero) + offset.
// `magic_zero2` is bf16x2 (128 + zero); the subtraction is exact, so the only roundings are those of scale, offset and the result.
__device__ __forceinline__ void expand4(uint32_t codes, uint32_t magic_zero2, uint32_t scale2, uint32_t off2, uint32_t& w01, uint32_t& w23) {
    const uint32_t m01 = __byte_perm(codes, 0x43434343u, 0x4140);      // {code0, 0x43, code1, 0x43} = bf16 (128 + code0), (128 + code1)
    const uint32_t m23 = __byte_perm(codes, 0x43434343u, 0x4342);
    w01 = bf16x2_fma(bf16x2_sub(m01, magic_zero2), scale2, off2);
    w23 = bf16x2_fma(bf16x2_sub(m23, magic_zero2), scale2, off2);
}

// half h (0/1) of K block kb of row `row`: columns 64 kb + 32 h .. + 31
__device__ __forceinline__ void load_raw(const WDesc& w, int row, int kb, int h, Raw& r) {
    const int K = w.k;
    switch (w.type) {
        case WT_Q4_K: {
            const uint8_t* qp = (const uint8_t*)w.p0 + (size_t)row * (K >> 1) + kb * 32;
            r.a = ldg16(qp);
            r.b = ldg16(qp + 16);
            r.s0 = __ldg((const uint32_t*)((const uint8_t*)w.p1 + (size_t)row * (K >> 4) + kb * 4));
            r.s1 = __ldg((const uint32_t*)w.p2 + (size_t)row * (K >> 8) + (kb >> 2));
            break;
        }
        case WT_Q6_K: {
            const int sb = kb >> 2, n = (kb >> 1) & 1, hi = kb & 1;
            const uint8_t* lp = (const uint8_t*)w.p0 + (size_t)row * (K >> 1) + sb * 128 + 64 * n + 32 * h;
            const uint8_t* hp = (const uint8_t*)w.p1 + (size_t)row * (K >> 2) + sb * 64 + 32 * n;
            r.a = ldg16(lp);
            r.b = ldg16(lp + 16);
            r.c = ldg16(hp);
            r.d = ldg16(hp + 16);
            r.s0 = __ldg((const uint32_t*)((const int8_t*)w.p2 + (size_t)row * (K >> 4) + sb * 16 + 8 * n + 4 * hi));
            r.s1 = __ldg((const unsigned short*)w.p3 + (size_t)row * (K >> 8) + sb);
            break;
        }
        case WT_Q8_0: {
            const int8_t* qp = (const int8_t*)w.p0 + (size_t)row * K + kb * 64 + 32 * h;
            r.a = ldg16(qp);
            r.b = ldg16(qp + 16);
            r.s1 = __ldg((const unsigned short*)w.p1 + (size_t)row * (K >> 5) + kb * 2 + h);
            break;
        }
        default: {   // BF16 / F16: 32 values = 64 bytes
            const uint8_t* p = (const uint8_t*)w.p0 + ((size_t)row * K + kb * 64 + 32 * h) * 2;
            r.a = ldg16(p);
            r.b = ldg16(p + 16);
            r.c = ldg16(p + 32);
            r.d = ldg16(p + 48);
            break;
        }
    }
}

__device__ __forceinline__ float half_bits_to_float(uint32_t bits) {
    return __half2float(__ushort_as_half((unsigned short)bits));
}

// Raw -> 16 bf16x2 words (32 consecutive columns)
__device__ __forceinline__ void expand_raw(int type, const Raw& r, int kb, int h, uint32_t (&o)[16]) {
    switch (type) {
        case WT_Q4_K: {
            const float2 df = __half22float2(*reinterpret_cast<const __half2*>(&r.s1));
            const float sc = df.x * (float)((r.s0 >> (8 * h)) & 0xff), mn = df.y * (float)((r.s0 >> (16 + 8 * h)) & 0xff);
            const uint32_t s2 = bf16x2_splat(sc), o2 = bf16x2_splat(-mn);
            const uint32_t q[8] = {r.a.x, r.a.y, r.a.z, r.a.w, r.b.x, r.b.y, r.b.z, r.b.w};
#pragma unroll
            for (int i = 0; i < 8; i++) {      // byte j of word i = column 4i + j (low nibble: half 0, high nibble: half 1)
                const uint32_t codes = (h ? (q[i] >> 4) : q[i]) & 0x0f0f0f0fu;
                expand4(codes, 0x43004300u, s2, o2, o[2 * i], o[2 * i + 1]);
            }
            return;
        }
        case WT_Q6_K: {
            // quarter 2 hi + h of the half: low (hi = 0) or high (hi = 1) nibbles of ql, two bits of qh at 2 (2 hi + h)
            const int hi = kb & 1, hs = 2 * (2 * hi + h);
            const float d = half_bits_to_float(r.s1);
            const uint32_t L[8] = {r.a.x, r.a.y, r.a.z, r.a.w, r.b.x, r.b.y, r.b.z, r.b.w};
            const uint32_t H[8] = {r.c.x, r.c.y, r.c.z, r.c.w, r.d.x, r.d.y, r.d.z, r.d.w};
#pragma unroll
            for (int c = 0; c < 2; c++) {      // 16 columns share one scale
                const float sc = d * (float)(int8_t)((r.s0 >> (8 * (2 * h + c))) & 0xff);
                const uint32_t s2 = bf16x2_splat(sc);
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const uint32_t lo = (hi ? (L[4 * c + i] >> 4) : L[4 * c + i]) & 0x0f0f0f0fu;
                    const uint32_t codes = lo | (((H[4 * c + i] >> hs) & 0x03030303u) << 4);
                    expand4(codes, 0x43204320u, s2, 0u, o[8 * c + 2 * i], o[8 * c + 2 * i + 1]);      // bf16 0x4320 = 160 = 128 + 32
                }
            }
            return;
        }
        case WT_Q8_0: {
            const float d = half_bits_to_float(r.s1);
            const uint32_t Q[8] = {r.a.x, r.a.y, r.a.z, r.a.w, r.b.x, r.b.y, r.b.z, r.b.w};
#pragma unroll
            for (int i = 0; i < 8; i++) {
                o[2 * i] = pack_bf16(d * (float)(int8_t)(Q[i] & 0xff), d * (float)(int8_t)((Q[i] >> 8) & 0xff));
                o[2 * i + 1] = pack_bf16(d * (float)(int8_t)((Q[i] >> 16) & 0xff), d * (float)(int8_t)(Q[i] >> 24));
            }
            return;
        }
        case WT_BF16: {
            const uint32_t V[16] = {r.a.x, r.a.y, r.a.z, r.a.w, r.b.x, r.b.y, r.b.z, r.b.w, r.c.x, r.c.y, r.c.z, r.c.w, r.d.x, r.d.y, r.d.z, r.d.w};
#pragma unroll
            for (int i = 0; i < 16; i++) o[i] = V[i];
            return;
        }
        default: {   // F16
            const uint32_t V[16] = {r.a.x, r.a.y, r.a.z, r.a.w, r.b.x, r.b.y, r.b.z, r.b.w, r.c.x, r.c.y, r.c.z, r.c.w, r.d.x, r.d.y, r.d.z, r.d.w};
#pragma unroll
            for (int i = 0; i < 16; i++) {
                const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&V[i]));
                o[i] = pack_bf16(f.x, f.y);
            }
            return;
        }
    }
}

// Store 32 consecutive K values (16 words) of row r, half h, into the swizzled stage tile.
__device__ __forceinline__ void store_half_row(uint8_t* tile, int r, int h, const uint32_t (&w)[16]) {
    uint8_t* row = tile + r * 128;
#pragma unroll
    for (int c = 0; c < 4; c++) {
        const uint4 v = make_uint4(w[4 * c], w[4 * c + 1], w[4 * c + 2], w[4 * c + 3]);
        *reinterpret_cast<uint4*>(row + (((4 * h + c) ^ (r & 7)) << 4)) = v;
    }
}

// grid = (M tiles, N tiles): CTAs that share a weight tile are adjacent in launch order and run together,
// so the quantised planes are fetched from HBM once and re-read from L2.
__global__ void __launch_bounds__(THREADS, 2) gemm_q_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ QGemmParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* tiles = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* full = reinterpret_cast<uint64_t*>(tiles + STAGES * STAGE_BYTES);
    uint64_t* empty = full + STAGES;
    uint64_t* acc_ready = empty + STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_ready + 1);
    __shared__ int s_failed;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = blockIdx.x * BM, n0 = blockIdx.y * BN;
    const int k_blocks = p.w.k / BK;

    if (threadIdx.x == 0) {
        s_failed = 0;
        for (int s = 0; s < STAGES; s++) {
            mbar_init(&full[s], 1 + DEQ_WARPS);      // TMA producer (with its byte count) + one arrival per dequant warp
            mbar_init(&empty[s], 1);
        }
        mbar_init(acc_ready, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(BN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_acc = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            for (int kb = 0; kb < k_blocks; kb++) {
                const int s = kb % STAGES;
                if (kb >= STAGES && !mbar_wait(&empty[s], ((kb / STAGES) - 1) & 1)) { atomicExch(&s_failed, 1); break; }
                mbar_expect_tx(&full[s], A_BYTES);
                tma_load_2d(tiles + s * STAGE_BYTES, &map_a, kb * BK, m0, &full[s]);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc(BM, BN);
            bool ok = true;
            for (int kb = 0; kb < k_blocks; kb++) {
                const int s = kb % STAGES;
                if (!mbar_wait(&full[s], (kb / STAGES) & 1)) { ok = false; atomicExch(&s_failed, 1); break; }
                tc_fence_after();
                const uint8_t* a_src = tiles + s * STAGE_BYTES;
                const uint64_t adesc = umma_desc(a_src), bdesc = umma_desc(a_src + A_BYTES);
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; k++) umma_bf16(tmem_acc, adesc + 2 * k, bdesc + 2 * k, idesc, (kb | k) != 0);
                umma_commit(&empty[s]);
            }
            if (ok) umma_commit(acc_ready);
        }
    } else {
        // warps 2..9: expand the weight tile (thread = 32 columns of one row), then drain the accumulator
        const int dt = threadIdx.x - 64;
        const int r = dt & 127, h = dt >> 7;
        const int wrow = min(n0 + r, p.w.n - 1);
        const int type = p.w.type;
        bool ok = true;
        Raw cur, nxt;
        load_raw(p.w, wrow, 0, h, cur);
        for (int kb = 0; kb < k_blocks && ok; kb++) {
            const int s = kb % STAGES;
            if (kb + 1 < k_blocks) load_raw(p.w, wrow, kb + 1, h, nxt);      // next block's bytes are in flight while this one is expanded
            uint32_t vals[16];
            expand_raw(type, cur, kb, h, vals);
            if (kb >= STAGES) ok = mbar_wait(&empty[s], ((kb / STAGES) - 1) & 1);
            if (ok) {
                store_half_row(tiles + s * STAGE_BYTES + A_BYTES, r, h, vals);
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // make the stores visible to the tensor core
            }
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&full[s])) : "memory");
            cur = nxt;
        }
        if (!ok) atomicExch(&s_failed, 1);
        const int q = warp & 3;                               // TMEM lane quarter this warp may read
        const int chalf = (warp - 2) >> 2;                    // which 64 accumulator columns this warp drains
        const bool ready = ok && mbar_wait(acc_ready, 0);
        if (!ready) atomicExch(&s_failed, 1);
        tc_fence_after();
        const int row = m0 + q * 32 + lane;
        if (ready) {
#pragma unroll 1
            for (int c0 = 64 * chalf; c0 < 64 * chalf + 64; c0 += 32) {
                uint32_t v[32];
                tmem_ld32(tmem_acc + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, v);
                if (row < p.m) {
                    float* o;
                    if (p.cm.n_dst > 0) {
                        const int owner = row / p.rows_per_rank;
                        o = p.cm.dst[owner] + (size_t)(row - owner * p.rows_per_rank) * p.ldo + p.w.out_off + n0 + c0;
                    } else {
                        o = p.out + (size_t)row * p.ldo + p.w.out_off + n0 + c0;
                    }
#pragma unroll
                    for (int j = 0; j < 32; j += 4) {
                        if (n0 + c0 + j >= p.w.n) break;
                        float4 t = make_float4(__uint_as_float(v[j]), __uint_as_float(v[j + 1]), __uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
                        if (p.w.bias) {
                            const float4 b = *(const float4*)(p.w.bias + n0 + c0 + j);
                            t.x += b.x; t.y += b.y; t.z += b.z; t.w += b.w;
                        }
                        if (p.accumulate) {
                            const float4 old = *(const float4*)(o + j);
                            t.x += old.x; t.y += old.y; t.z += old.z; t.w += old.w;
                        }
                        *(float4*)(o + j) = t;
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
    if (threadIdx.x == 0 && s_failed) atomicExch(&g_gemm_q_status, KS_TIMEOUT);
    if (p.cm.n_dst > 0) comm_publish(p.cm, gridDim.x * gridDim.y, comm_next_epoch(p.cm));
}

bool q_supported(const WDesc& w) {
    switch (w.type) {
        case WT_Q4_K: case WT_Q6_K: return w.k % 256 == 0;
        case WT_Q8_0: case WT_BF16: case WT_F16: return w.k % 64 == 0;
        default: return false;
    }
}

}  // namespace

// out[m][out_off + n] (+)= x[m][k] (bf16) . W[n][k]^T + bias.  Weight encodings: Q4_K, Q6_K, Q8_0, BF16, F16 (others: cudaErrorNotSupported).
// Requirements: n % 4 == 0, ldo % 4 == 0, out_off % 4 == 0, x 16-byte aligned.  Returns a cudaError_t value.
B2_API int b2_gemm_q(const void* x, int m, const WDesc* w, float* out, int ldo, int accumulate, cudaStream_t st) {
    if (!w || m < 1 || w->n < 1 || (w->n & 3) || (ldo & 3) || (w->out_off & 3) || ((uintptr_t)x & 15) || ((uintptr_t)out & 15))
        return (int)cudaErrorInvalidValue;
    if (!q_supported(*w)) return (int)cudaErrorNotSupported;
    CUtensorMap ma;
    if (!tc::make_map(&ma, x, m, w->k, BM)) return (int)cudaErrorNotSupported;
    static PerDeviceOnce once;
    if (once.first()) cudaFuncSetAttribute(gemm_q_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_TOTAL);
    QGemmParams p{*w, m, out, ldo, accumulate, {}, 0};
    dim3 grid((m + BM - 1) / BM, (w->n + BN - 1) / BN);
    gemm_q_tc_kernel<<<grid, THREADS, SMEM_TOTAL, st>>>(ma, p);
    return (int)cudaGetLastError();
}

// Row-parallel GEMM of a tensor-parallel group: the partial result tile of rows owned by rank r is stored straight into
// cm->dst[r] (a peer address, pitch ldo) from the epilogue and the exchange is announced on cm's channel.
B2_API int b2_gemm_q_scatter(const void* x, int m, const WDesc* w, int ldo, const CommSend* cm, int rows_per_rank, cudaStream_t st) {
    if (!w || !cm || m < 1 || w->n < 1 || (w->n & 3) || (ldo & 3) || (w->out_off & 3) || ((uintptr_t)x & 15) || rows_per_rank < 1 ||
        cm->n_dst < 1 || cm->n_dst > COMM_MAX_RANKS || (m + rows_per_rank - 1) / rows_per_rank > cm->n_dst)
        return (int)cudaErrorInvalidValue;
    if (!q_supported(*w)) return (int)cudaErrorNotSupported;
    CUtensorMap ma;
    if (!tc::make_map(&ma, x, m, w->k, BM)) return (int)cudaErrorNotSupported;
    cudaFuncSetAttribute(gemm_q_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_TOTAL);
    QGemmParams p{*w, m, nullptr, ldo, 0, *cm, rows_per_rank};
    dim3 grid((m + BM - 1) / BM, (w->n + BN - 1) / BN);
    gemm_q_tc_kernel<<<grid, THREADS, SMEM_TOTAL, st>>>(ma, p);
    return (int)cudaGetLastError();
}

B2_API int b2_gemm_q_status() {
    int v = 0;
    cudaMemcpyFromSymbol(&v, g_gemm_q_status, sizeof(int));
    return v;
}
