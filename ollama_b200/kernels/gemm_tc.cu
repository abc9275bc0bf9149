// Tensor-core GEMM for prefill on sm_100a: D[M,N] (+)= A[M,K] . B[N,K]^T (+ bias), bf16 operands, fp32 result.
//
// Blackwell path: operand tiles are fetched by TMA (cp.async.bulk.tensor, 128-byte swizzle) into a
// multi-stage shared-memory ring, one elected thread issues tcgen05.mma (cta_group::1, M = 128, N up to
// 256, K = 16 per instruction) with the accumulator in tensor memory, and four epilogue warps read the
// accumulator back with tcgen05.ld, add the bias and store / accumulate into the fp32 output.  Roles
// are warp-specialised: warp 0 = TMA producer, warp 1 = MMA issuer (+ TMEM allocation), warps 2..5 =
// epilogue.  Every mbarrier wait is bounded; on expiry the kernel records KS_TIMEOUT in its status word,
// skips the remaining work, still releases its tensor memory and returns.
//
// In the reference stack this role is played by ggml-cuda's mmq kernels (int8 mma.sync tiles) and the
// dequantise + cuBLAS path.
#include "tc_common.cuh"

__device__ int g_gemm_status = 0;

namespace {

using namespace tc;
constexpr int STAGES = 4;

struct GemmParams {
    int m, n, k;
    float* out;
    int ldo;
    const float* bias;      // [n] or null
    int accumulate;         // out += result
};

template <int BN>
struct SmemLayout {
    static constexpr int A_BYTES = BM * BK * 2;
    static constexpr int B_BYTES = BN * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int TOTAL = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
};

template <int BN>
__global__ void __launch_bounds__(192, 1) gemm_bf16_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                                                              const GemmParams p) {
    extern __shared__ uint8_t smem_raw[];
    using L = SmemLayout<BN>;
    uint8_t* tiles = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);     // 128-byte swizzle wants 1024-byte alignment
    uint64_t* full = reinterpret_cast<uint64_t*>(tiles + STAGES * L::STAGE_BYTES);
    uint64_t* empty = full + STAGES;
    uint64_t* acc_ready = empty + STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_ready + 1);
    __shared__ int s_failed;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int k_blocks = (p.k + BK - 1) / BK;

    if (threadIdx.x == 0) {
        s_failed = 0;
        for (int s = 0; s < STAGES; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        mbar_init(acc_ready, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {     // one warp allocates the accumulator columns (power of two >= 32)
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
                uint8_t* a_dst = tiles + s * L::STAGE_BYTES;
                uint8_t* b_dst = a_dst + L::A_BYTES;
                mbar_expect_tx(&full[s], L::STAGE_BYTES);
                tma_load_2d(a_dst, &map_a, kb * BK, m0, &full[s]);
                tma_load_2d(b_dst, &map_b, kb * BK, n0, &full[s]);
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
                const uint8_t* a_src = tiles + s * L::STAGE_BYTES;
                const uint64_t adesc = umma_desc(a_src), bdesc = umma_desc(a_src + L::A_BYTES);
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; k++) {
                    // advancing 16 elements along K inside the swizzle span = 32 bytes = 2 descriptor units
                    umma_bf16(tmem_acc, adesc + 2 * k, bdesc + 2 * k, idesc, (kb | k) != 0);
                }
                umma_commit(&empty[s]);        // frees the stage once these MMAs have read it
            }
            if (ok) umma_commit(acc_ready);
        }
    } else {
        // epilogue warps 2..5: warp w may touch TMEM lanes 32*(w%4) .. +31
        const int q = warp & 3;
        const bool ready = mbar_wait(acc_ready, 0);
        if (!ready) atomicExch(&s_failed, 1);
        tc_fence_after();
        const int row = m0 + q * 32 + lane;
        if (ready) {
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                uint32_t v[32];
                const uint32_t taddr = tmem_acc + ((uint32_t)(q * 32) << 16) + (uint32_t)c0;
                tmem_ld32(taddr, v);
                if (row < p.m) {
                    float* o = p.out + (size_t)row * p.ldo + n0 + c0;
#pragma unroll
                    for (int j = 0; j < 32; j += 4) {
                        if (n0 + c0 + j >= p.n) break;
                        float4 r = make_float4(__uint_as_float(v[j]), __uint_as_float(v[j + 1]), __uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
                        if (p.bias) {
                            const float4 b = *(const float4*)(p.bias + n0 + c0 + j);
                            r.x += b.x; r.y += b.y; r.z += b.z; r.w += b.w;
                        }
                        if (p.accumulate) {
                            const float4 old = *(const float4*)(o + j);
                            r.x += old.x; r.y += old.y; r.z += old.z; r.w += old.w;
                        }
                        *(float4*)(o + j) = r;
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
    if (threadIdx.x == 0 && s_failed) atomicExch(&g_gemm_status, KS_TIMEOUT);
}

template <int BN>
int launch(const void* a, const void* b, const GemmParams& p, cudaStream_t st) {
    CUtensorMap ma, mb;
    if (!make_map(&ma, a, p.m, p.k, BM) || !make_map(&mb, b, p.n, p.k, BN)) return (int)cudaErrorNotSupported;
    static bool attr = false;
    if (!attr) {
        cudaFuncSetAttribute(gemm_bf16_tc_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, SmemLayout<BN>::TOTAL);
        attr = true;
    }
    dim3 grid((p.n + BN - 1) / BN, (p.m + BM - 1) / BM);
    gemm_bf16_tc_kernel<BN><<<grid, 192, SmemLayout<BN>::TOTAL, st>>>(ma, mb, p);
    return (int)cudaGetLastError();
}

}  // namespace

// out[m][n] (+)= a[m][k] . b[n][k]^T + bias[n];  a, b bf16 row-major with k % 8 == 0 and 16-byte aligned bases,
// out fp32 with ldo % 4 == 0, n % 4 == 0.  Returns a cudaError_t value.
B2_API int b2_gemm_bf16(const void* a, const void* b, int m, int n, int k, float* out, int ldo, const float* bias, int accumulate,
                        cudaStream_t st) {
    if (m < 1 || n < 1 || k < 8 || (k & 7) || (n & 3) || (ldo & 3) || ((uintptr_t)a & 15) || ((uintptr_t)b & 15) || ((uintptr_t)out & 15))
        return (int)cudaErrorInvalidValue;
    GemmParams p{m, n, k, out, ldo, bias, accumulate};
    if (n >= 256) return launch<256>(a, b, p, st);
    if (n >= 128) return launch<128>(a, b, p, st);
    return launch<64>(a, b, p, st);
}

B2_API int b2_gemm_status() {
    int v = 0;
    cudaMemcpyFromSymbol(&v, g_gemm_status, sizeof(int));
    return v;
}
