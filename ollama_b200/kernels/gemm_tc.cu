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
#include "common.cuh"

#include <cuda.h>

__device__ int g_gemm_status = 0;

namespace {

constexpr int BM = 128;          // rows of A per CTA (MMA M)
constexpr int BK = 64;           // K elements per stage = one 128-byte swizzle span of bf16
constexpr int UMMA_K = 16;       // K per tcgen05.mma for 16-bit operands
constexpr int STAGES = 4;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.b32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait (roughly a second at most); false = gave up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    for (int i = 0; i < (1 << 22); i++) {
        if (mbar_try_wait(bar, parity)) return true;
        if (i > 128) __nanosleep(100);
    }
    return false;
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}

// Shared-memory matrix descriptor: K-major tile, 128-byte swizzle, rows 128 bytes apart, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc(const void* smem_tile) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_u32(smem_tile) & 0x3FFFF) >> 4);        // start address
    d |= (uint64_t)1 << 16;                                        // leading byte offset (unused with swizzle)
    d |= (uint64_t)(1024 >> 4) << 32;                              // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                                        // descriptor version of sm_100
    d |= (uint64_t)2 << 61;                                        // SWIZZLE_128B
    return d;
}

// Instruction descriptor: bf16 x bf16 -> fp32, both operands K-major, dense.
__host__ __device__ constexpr uint32_t umma_idesc(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

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
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                    "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                    : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
                      "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]),
                      "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
                      "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                    : "r"(taddr));
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
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

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

// 2-D bf16 tensor [rows][k] (k contiguous), box = 64 x box_rows, 128-byte swizzle, out-of-range reads give zero.
bool make_map(CUtensorMap* map, const void* base, int rows, int k, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)k * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
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
