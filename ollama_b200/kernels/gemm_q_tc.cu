// Dequantisation-fused tensor-core GEMM for prefill on sm_100a:
//   out[M, N] (+)= X[M, K] (bf16) . W[N, K]^T (GGUF-quantised, plane layout) + bias
//
// The activation tile (A operand) arrives by TMA as in gemm_tc.cu.  The weight tile (B operand) never
// exists in global memory in 16-bit form: four producer warps read the quantised planes of 128 weight
// rows x 64 columns, expand them to bf16 in registers and write them into the stage buffer in exactly
// the 128-byte-swizzled K-major layout that the tcgen05 shared-memory descriptor expects (16-byte chunk
// c of row r lives at chunk c ^ (r & 7)); a proxy fence publishes those generic-proxy writes to the
// tensor core.  One elected thread issues tcgen05.mma (M = 128 tokens, N = 128 weight rows) into a TMEM
// accumulator; the producer warps turn into epilogue warps once their last stage is written.  Two CTAs
// fit on an SM (96 KB of stages, 128 TMEM columns each), so one CTA's epilogue overlaps the other's
// main loop.  All mbarrier waits are bounded (KS_TIMEOUT in the status word on expiry).
//
// This is the counterpart of ggml-cuda's mmq kernels (in-kernel dequantisation feeding mma.sync) and of
// its dequantise-then-cuBLAS path, redone for tcgen05 / TMEM.
#include "tc_common.cuh"

__device__ int g_gemm_q_status = 0;

namespace {

using namespace tc;
constexpr int BN = 128;          // weight rows per CTA (MMA N)
constexpr int STAGES = 3;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int SMEM_TOTAL = STAGES * STAGE_BYTES + 1024 + 256;
constexpr int DEQ_WARPS = 4;

struct QGemmParams {
    WDesc w;                // quantised weight [n][k]
    int m;
    float* out;
    int ldo;
    int accumulate;
};

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

// Store 64 consecutive K values of one weight row (already bf16-packed, 32 words) into the swizzled stage tile.
__device__ __forceinline__ void store_row_swizzled(uint8_t* tile, int r, const uint32_t (&w)[32]) {
    uint8_t* row = tile + r * 128;
#pragma unroll
    for (int c = 0; c < 8; c++) {
        const uint4 v = make_uint4(w[4 * c], w[4 * c + 1], w[4 * c + 2], w[4 * c + 3]);
        *reinterpret_cast<uint4*>(row + ((c ^ (r & 7)) << 4)) = v;
    }
}

// Expand columns [64 kb, 64 kb + 64) of weight row `row` to bf16 words.
__device__ __forceinline__ void dequant64(const WDesc& w, int row, int kb, uint32_t (&o)[32]) {
    const int K = w.k;
    switch (w.type) {
        case WT_Q4_K: {
            const uint8_t* qp = (const uint8_t*)w.p0 + (size_t)row * (K >> 1) + kb * 32;
            const uint4 qa = ldg16(qp), qb = ldg16(qp + 16);
            const uint32_t sm = __ldg((const uint32_t*)((const uint8_t*)w.p1 + (size_t)row * (K >> 4) + kb * 4));
            const float2 df = __half22float2(__ldg((const __half2*)w.p2 + (size_t)row * (K >> 8) + (kb >> 2)));
            const float dl = df.x * (float)(sm & 0xff), dh = df.x * (float)((sm >> 8) & 0xff);
            const float ml = df.y * (float)((sm >> 16) & 0xff), mh = df.y * (float)(sm >> 24);
            const uint32_t q[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
#pragma unroll
            for (int i = 0; i < 8; i++) {      // word i: bytes 4i .. 4i+3 -> low nibbles = columns 4i.., high = 32 + 4i..
                const uint32_t v = q[i];
                o[2 * i] = pack_bf16(dl * (float)(v & 15) - ml, dl * (float)((v >> 8) & 15) - ml);
                o[2 * i + 1] = pack_bf16(dl * (float)((v >> 16) & 15) - ml, dl * (float)((v >> 24) & 15) - ml);
                o[16 + 2 * i] = pack_bf16(dh * (float)((v >> 4) & 15) - mh, dh * (float)((v >> 12) & 15) - mh);
                o[16 + 2 * i + 1] = pack_bf16(dh * (float)((v >> 20) & 15) - mh, dh * (float)(v >> 28) - mh);
            }
            return;
        }
        case WT_Q6_K: {
            // 64 columns = two quarters (32 each) of half n of super-block sb
            const int sb = kb >> 2, n = (kb >> 1) & 1, hi = kb & 1;      // hi: quarters 2,3 use the high nibbles
            const uint8_t* lp = (const uint8_t*)w.p0 + (size_t)row * (K >> 1) + sb * 128 + 64 * n;
            const uint8_t* hp = (const uint8_t*)w.p1 + (size_t)row * (K >> 2) + sb * 64 + 32 * n;
            const int8_t* sp = (const int8_t*)w.p2 + (size_t)row * (K >> 4) + sb * 16 + 8 * n + 4 * hi;
            const float d = __half2float(__ldg((const __half*)w.p3 + (size_t)row * (K >> 8) + sb));
            const uint32_t s4 = __ldg((const uint32_t*)sp);             // scales of (quarter 2hi, l<16), (2hi, l>=16), (2hi+1, ..)
            const float sc[4] = {d * (float)(int8_t)(s4 & 0xff), d * (float)(int8_t)((s4 >> 8) & 0xff),
                                 d * (float)(int8_t)((s4 >> 16) & 0xff), d * (float)(int8_t)(s4 >> 24)};
#pragma unroll
            for (int qd = 0; qd < 2; qd++) {           // quarter 2hi + qd reads ql[32 qd + l], qh bits 2(2hi+qd)
#pragma unroll
                for (int c = 0; c < 2; c++) {          // 16 values per 16-byte load
                    const uint4 lq = ldg16(lp + 32 * qd + 16 * c), hq = ldg16(hp + 16 * c);
                    const uint32_t L[4] = {lq.x, lq.y, lq.z, lq.w}, H[4] = {hq.x, hq.y, hq.z, hq.w};
                    const float s = sc[2 * qd + c];
                    const int hs = 2 * (2 * hi + qd);
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const uint32_t lo = hi ? (L[i] >> 4) & 0x0f0f0f0fu : L[i] & 0x0f0f0f0fu;
                        const uint32_t v = lo | (((H[i] >> hs) & 0x03030303u) << 4);
                        const int base = 16 * qd + 8 * c + 2 * i;
                        o[base] = pack_bf16(s * (float)((int)(v & 63) - 32), s * (float)((int)((v >> 8) & 63) - 32));
                        o[base + 1] = pack_bf16(s * (float)((int)((v >> 16) & 63) - 32), s * (float)((int)((v >> 24) & 63) - 32));
                    }
                }
            }
            return;
        }
        case WT_Q8_0: {
            const int8_t* qp = (const int8_t*)w.p0 + (size_t)row * K + kb * 64;
            const __half* dp = (const __half*)w.p1 + (size_t)row * (K >> 5) + kb * 2;
#pragma unroll
            for (int h = 0; h < 2; h++) {
                const float d = __half2float(__ldg(dp + h));
#pragma unroll
                for (int c = 0; c < 2; c++) {
                    const uint4 q = ldg16(qp + 32 * h + 16 * c);
                    const uint32_t Q[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const int base = 16 * h + 8 * c + 2 * i;
                        o[base] = pack_bf16(d * (float)(int8_t)(Q[i] & 0xff), d * (float)(int8_t)((Q[i] >> 8) & 0xff));
                        o[base + 1] = pack_bf16(d * (float)(int8_t)((Q[i] >> 16) & 0xff), d * (float)(int8_t)(Q[i] >> 24));
                    }
                }
            }
            return;
        }
        case WT_BF16: {
            const uint8_t* p = (const uint8_t*)w.p0 + ((size_t)row * K + kb * 64) * 2;
#pragma unroll
            for (int c = 0; c < 8; c++) {
                const uint4 v = ldg16(p + 16 * c);
                o[4 * c] = v.x; o[4 * c + 1] = v.y; o[4 * c + 2] = v.z; o[4 * c + 3] = v.w;
            }
            return;
        }
        case WT_F16: {
            const uint8_t* p = (const uint8_t*)w.p0 + ((size_t)row * K + kb * 64) * 2;
#pragma unroll
            for (int c = 0; c < 8; c++) {
                const uint4 v = ldg16(p + 16 * c);
                const uint32_t V[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&V[i]));
                    o[4 * c + i] = pack_bf16(f.x, f.y);
                }
            }
            return;
        }
    }
#pragma unroll
    for (int i = 0; i < 32; i++) o[i] = 0;
}

// grid = (M tiles, N tiles): CTAs that share a weight tile are adjacent in launch order and run together,
// so the quantised planes are fetched from HBM once and re-read from L2.
__global__ void __launch_bounds__(192, 2) gemm_q_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ QGemmParams p) {
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
        // warps 2..5: dequantise the weight tile, one row per thread, then drain the accumulator
        const int r = (warp - 2) * 32 + lane;                 // row inside the tile
        const int wrow = min(n0 + r, p.w.n - 1);
        bool ok = true;
        for (int kb = 0; kb < k_blocks && ok; kb++) {
            const int s = kb % STAGES;
            uint32_t vals[32];
            dequant64(p.w, wrow, kb, vals);                   // global loads first, they do not need the stage
            if (kb >= STAGES) ok = mbar_wait(&empty[s], ((kb / STAGES) - 1) & 1);
            if (ok) {
                store_row_swizzled(tiles + s * STAGE_BYTES + A_BYTES, r, vals);
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // make the stores visible to the tensor core
            }
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&full[s])) : "memory");
        }
        if (!ok) atomicExch(&s_failed, 1);
        const int q = warp & 3;                               // TMEM lane quarter this warp may read
        const bool ready = ok && mbar_wait(acc_ready, 0);
        if (!ready) atomicExch(&s_failed, 1);
        tc_fence_after();
        const int row = m0 + q * 32 + lane;
        if (ready) {
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                uint32_t v[32];
                tmem_ld32(tmem_acc + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, v);
                if (row < p.m) {
                    float* o = p.out + (size_t)row * p.ldo + p.w.out_off + n0 + c0;
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
    static bool attr = false;
    if (!attr) {
        cudaFuncSetAttribute(gemm_q_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_TOTAL);
        attr = true;
    }
    QGemmParams p{*w, m, out, ldo, accumulate};
    dim3 grid((m + BM - 1) / BM, (w->n + BN - 1) / BN);
    gemm_q_tc_kernel<<<grid, 192, SMEM_TOTAL, st>>>(ma, p);
    return (int)cudaGetLastError();
}


B2_API int b2_gemm_q_status() {
    int v = 0;
    cudaMemcpyFromSymbol(&v, g_gemm_q_status, sizeof(int));
    return v;
}
