// Tensor-core GEMM for prefill on sm_100a: D[M,N] (+)= A[M,K] . B[N,K]^T (+ bias), bf16 operands, fp32 or bf16 result.
//
// Blackwell path: operand tiles are fetched by TMA (cp.async.bulk.tensor, 128-byte swizzle) into a
// multi-stage shared-memory ring, one elected thread issues tcgen05.mma (cta_group::1, M = 128, N up to
// 256, K = 16 per instruction) with the accumulator in tensor memory, and four epilogue warps read the
// accumulator back with tcgen05.ld, add the bias and store / accumulate into the output.  Roles are
// warp-specialised: warp 0 = TMA producer, warp 1 = MMA issuer (+ TMEM allocation), warps 2..5 = epilogue.
//
// The kernel is persistent: one CTA per SM walks a static list of output tiles.  The accumulator is double
// buffered in tensor memory (2 x BN columns), so the epilogue of tile i overlaps the MMAs of tile i+1, and
// the shared-memory ring keeps running across tile boundaries.  Tiles are ordered M-fastest inside groups
// of 16 M-tiles: the CTAs that run at the same time share a handful of weight tiles (read from HBM once,
// from L2 afterwards) and the activation panel stays in L2.
//
// Tensor-parallel variant: with a CommSend the epilogue stores each row of the partial result straight into
// the buffer of the rank that owns that row (peer addresses over NVLink) and announces the exchange, which
// makes the kernel a fused GEMM + reduce-scatter (the reduction itself happens in the consumer).
//
// Every mbarrier wait is bounded; on expiry the kernel records KS_TIMEOUT in its status word, skips the
// remaining work, still releases its tensor memory and returns.
//
// In the reference stack this role is played by ggml-cuda's mmq kernels (int8 mma.sync tiles) and the
// dequantise + cuBLAS path.
#include "tc_common.cuh"
#include "comm.cuh"

__device__ int g_gemm_status = 0;

namespace {

using namespace tc;
constexpr int GROUP_M = 16;      // M-tiles per rasterisation group

struct GemmParams {
    int m, n, k;
    void* out;              // fp32 or bf16 [m][ldo]
    int ldo;                // elements
    const float* bias;      // [n] or null
    int accumulate;         // out += result (fp32 output only)
    int out_bf16;
    CommSend cm;            // cm.n_dst > 0: row r goes to cm.dst[r / rows_per_rank] at row r % rows_per_rank (bf16)
    int rows_per_rank;
    // grouped (mixture of experts): b holds E stacked [n][k] matrices and bias E x n values; the rows of a are sorted by expert
    // and every 128-row tile belongs to one expert.  tile_expert[mt] = that expert, or -1: the tile holds no rows.
    const int* tile_expert;
    // gated activation in the epilogue: columns 2i / 2i + 1 are gate / up of output i; out is bf16 [m][ldo] with n / 2 columns
    int glu;                // 0: off, 1 + act otherwise (0 silu, 1 gelu_tanh, 2 clamped swiglu)
    float glu_alpha, glu_limit;
};

template <int BN>
struct Cfg {
    static constexpr int STAGES = BN == 256 ? 4 : (BN == 192 ? 5 : 6);
    static constexpr int A_BYTES = BM * BK * 2;
    static constexpr int B_BYTES = BN * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int EPI_LD = 36;                                   // padded row of the epilogue's 32 x 32 transpose tile (floats)
    static constexpr int EPI_BYTES = 4 * 32 * EPI_LD * 4;              // one tile per epilogue warp
    static constexpr int TOTAL = STAGES * STAGE_BYTES + EPI_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
    static constexpr int ACC_STRIDE = BN == 192 ? 256 : BN;            // column distance of the two accumulators
    static constexpr int TMEM_COLS = 2 * ACC_STRIDE < 32 ? 32 : 2 * ACC_STRIDE;      // a power of two
};

__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int& mt, int& nt) {
    const int per_group = GROUP_M * tiles_n;
    const int g = t / per_group, r = t - g * per_group;
    const int gm = min(GROUP_M, tiles_m - g * GROUP_M);
    mt = g * GROUP_M + r % gm;
    nt = r / gm;
}

__device__ __forceinline__ uint32_t pack2_bf16(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

template <int BN>
__global__ void __launch_bounds__(192, 1) gemm_bf16_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                                                              const __grid_constant__ GemmParams p) {
    extern __shared__ uint8_t smem_raw[];
    using L = Cfg<BN>;
    constexpr int STAGES = L::STAGES;
    uint8_t* tiles = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);     // 128-byte swizzle wants 1024-byte alignment
    float* epi = reinterpret_cast<float*>(tiles + STAGES * L::STAGE_BYTES);
    uint64_t* full = reinterpret_cast<uint64_t*>(tiles + STAGES * L::STAGE_BYTES + L::EPI_BYTES);
    uint64_t* empty = full + STAGES;
    uint64_t* acc_full = empty + STAGES;
    uint64_t* acc_empty = acc_full + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    __shared__ int s_failed;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_m = (p.m + BM - 1) / BM, tiles_n = (p.n + BN - 1) / BN, total = tiles_m * tiles_n;
    const int k_blocks = (p.k + BK - 1) / BK;

    if (threadIdx.x == 0) {
        s_failed = 0;
        for (int s = 0; s < STAGES; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], 4);       // one arrival per epilogue warp
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {     // one warp allocates the accumulator columns (power of two >= 32)
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(L::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            int it = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
                int mt, nt;
                tile_coords(t, tiles_m, tiles_n, mt, nt);
                const int e = p.tile_expert ? p.tile_expert[mt] : 0;
                if (e < 0) continue;               // every role skips the same tiles
                for (int kb = 0; kb < k_blocks; kb++, it++) {
                    const int s = it % STAGES;
                    if (it >= STAGES && !mbar_wait(&empty[s], ((it / STAGES) - 1) & 1)) { ok = false; break; }
                    uint8_t* a_dst = tiles + s * L::STAGE_BYTES;
                    mbar_expect_tx(&full[s], L::STAGE_BYTES);
                    tma_load_2d(a_dst, &map_a, kb * BK, mt * BM, &full[s]);
                    tma_load_2d(a_dst + L::A_BYTES, &map_b, kb * BK, e * p.n + nt * BN, &full[s]);
                }
            }
            if (!ok) atomicExch(&s_failed, 1);
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc(BM, BN);
            int it = 0, i = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
                if (p.tile_expert) {
                    int mt, nt;
                    tile_coords(t, tiles_m, tiles_n, mt, nt);
                    if (p.tile_expert[mt] < 0) continue;
                }
                const int buf = i & 1, use = i >> 1;
                i++;
                if (use >= 1 && !mbar_wait(&acc_empty[buf], (use - 1) & 1)) { ok = false; break; }
                tc_fence_after();
                const uint32_t acc = tmem_base + (uint32_t)(buf * L::ACC_STRIDE);
                for (int kb = 0; kb < k_blocks; kb++, it++) {
                    const int s = it % STAGES;
                    if (!mbar_wait(&full[s], (it / STAGES) & 1)) { ok = false; break; }
                    tc_fence_after();
                    const uint8_t* a_src = tiles + s * L::STAGE_BYTES;
                    const uint64_t adesc = umma_desc(a_src), bdesc = umma_desc(a_src + L::A_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; k++) {
                        // advancing 16 elements along K inside the swizzle span = 32 bytes = 2 descriptor units
                        umma_bf16(acc, adesc + 2 * k, bdesc + 2 * k, idesc, (kb | k) != 0);
                    }
                    umma_commit(&empty[s]);        // frees the stage once these MMAs have read it
                }
                if (ok) umma_commit(&acc_full[buf]);
            }
            if (!ok) atomicExch(&s_failed, 1);
        }
    } else {
        // epilogue warps 2..5: warp w may touch TMEM lanes 32*(w%4) .. +31
        const int q = warp & 3;
        int i = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
            int mt, nt;
            tile_coords(t, tiles_m, tiles_n, mt, nt);
            const int e = p.tile_expert ? p.tile_expert[mt] : 0;
            if (e < 0) continue;
            const int buf = i & 1, use = i >> 1;
            i++;
            if (!mbar_wait(&acc_full[buf], use & 1)) { ok = false; break; }
            tc_fence_after();
            // Each thread reads 32 columns of its own accumulator row; a 32 x 32 transpose through shared memory turns that into
            // stores of 4 rows x 128 contiguous bytes per warp instruction (full lines for HBM, full packets for NVLink peers).
            const int n0 = nt * BN;
            float* st = epi + (warp - 2) * 32 * L::EPI_LD;
            const int sub = lane >> 3, cq = (lane & 7) * 4;                 // store phase: row within a group of 4, first of 4 columns
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                uint32_t v[32];
                const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * L::ACC_STRIDE + c0);
                tmem_ld32(taddr, v);
                if (n0 + c0 >= p.n) continue;       // warp-uniform
#pragma unroll
                for (int j = 0; j < 32; j += 4)
                    *(uint4*)(st + lane * L::EPI_LD + j) = make_uint4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                __syncwarp();
                const int col = n0 + c0 + cq;
                float4 bias = make_float4(0.f, 0.f, 0.f, 0.f);
                if (p.bias && col < p.n) bias = *(const float4*)(p.bias + (size_t)e * p.n + col);
#pragma unroll
                for (int rr = 0; rr < 8; rr++) {
                    const int lr = rr * 4 + sub;
                    const int row = mt * BM + q * 32 + lr;
                    if (row >= p.m || col >= p.n) continue;
                    float4 r = *(const float4*)(st + lr * L::EPI_LD + cq);
                    r.x += bias.x; r.y += bias.y; r.z += bias.z; r.w += bias.w;
                    if (p.glu) {               // (gate, up, gate, up) -> two activated outputs
                        const float h0 = glu_act(r.x, r.y, p.glu - 1, p.glu_alpha, p.glu_limit), h1 = glu_act(r.z, r.w, p.glu - 1, p.glu_alpha, p.glu_limit);
                        *(uint32_t*)((__nv_bfloat16*)p.out + (size_t)row * p.ldo + (col >> 1)) = pack2_bf16(h0, h1);
                    } else if (p.cm.n_dst > 0) {      // partial rows travel as bf16: half the NVLink bytes of fp32
                        const int owner = row / p.rows_per_rank;
                        __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.cm.dst[owner]) + (size_t)(row - owner * p.rows_per_rank) * p.ldo + col;
                        *(uint2*)dst = make_uint2(pack2_bf16(r.x, r.y), pack2_bf16(r.z, r.w));
                    } else if (p.out_bf16) {
                        *(uint2*)((__nv_bfloat16*)p.out + (size_t)row * p.ldo + col) = make_uint2(pack2_bf16(r.x, r.y), pack2_bf16(r.z, r.w));
                    } else {
                        float* o = (float*)p.out + (size_t)row * p.ldo + col;
                        if (p.accumulate) {
                            const float4 old = *(const float4*)o;
                            r.x += old.x; r.y += old.y; r.z += old.z; r.w += old.w;
                        }
                        *(float4*)o = r;
                    }
                }
                __syncwarp();
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&acc_empty[buf])) : "memory");
        }
        if (!ok) atomicExch(&s_failed, 1);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(L::TMEM_COLS) : "memory");
    }
    if (threadIdx.x == 0 && s_failed) atomicExch(&g_gemm_status, KS_TIMEOUT);
    if (p.cm.n_dst > 0) comm_publish(p.cm, gridDim.x, comm_next_epoch(p.cm));
}

int sm_count() {
    static int n = 0;
    if (!n) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        if (n <= 0) n = 148;
    }
    return n;
}

template <int BN>
int launch(const void* a, const void* b, const GemmParams& p, cudaStream_t st, int b_rows = 0) {
    CUtensorMap ma, mb;
    if (!make_map(&ma, a, p.m, p.k, BM) || !make_map(&mb, b, b_rows ? b_rows : p.n, p.k, BN)) return (int)cudaErrorNotSupported;
    static PerDeviceOnce once;
    if (once.first()) cudaFuncSetAttribute(gemm_bf16_tc_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<BN>::TOTAL);
    const int total = ((p.m + BM - 1) / BM) * ((p.n + BN - 1) / BN);
    const int grid = total < sm_count() ? total : sm_count();
    gemm_bf16_tc_kernel<BN><<<grid, 192, Cfg<BN>::TOTAL, st>>>(ma, mb, p);
    return (int)cudaGetLastError();
}

int dispatch(const void* a, const void* b, const GemmParams& p, cudaStream_t st, int b_rows = 0) {
    // wide tiles once they fill the machine; narrower ones keep more SMs busy on small problems
    const long tiles_m = (p.m + BM - 1) / BM;
    // a handful of rows (a decode step of several sequences): the product streams b once, so the narrowest tile that spreads
    // b over the most SMs wins
    if (p.m <= 32 && !p.out_bf16 && !p.glu && p.cm.n_dst == 0 && !b_rows && p.n >= 64 && (p.n + 127) / 128 < sm_count())
        return launch<64>(a, b, p, st, b_rows);
    if (p.n >= 256 && tiles_m * ((p.n + 255) / 256) >= sm_count()) return launch<256>(a, b, p, st, b_rows);
    // one round either way: the widest tile that still gives every SM at most one tile
    if (p.n >= 192 && tiles_m * ((p.n + 191) / 192) <= sm_count() && tiles_m * ((p.n + 127) / 128) > sm_count()) return launch<192>(a, b, p, st, b_rows);
    if (p.n >= 128) return launch<128>(a, b, p, st, b_rows);
    return launch<64>(a, b, p, st, b_rows);
}

bool bad_operands(const void* a, const void* b, int m, int n, int k, int ldo) {
    return m < 1 || n < 1 || k < 8 || (k & 7) || (n & 3) || (ldo & 3) || ((uintptr_t)a & 15) || ((uintptr_t)b & 15);
}

}  // namespace

// out[m][n] (+)= a[m][k] . b[n][k]^T + bias[n];  a, b bf16 row-major with k % 8 == 0 and 16-byte aligned bases,
// out fp32 with ldo % 4 == 0, n % 4 == 0.  Returns a cudaError_t value.
B2_API int b2_gemm_bf16(const void* a, const void* b, int m, int n, int k, float* out, int ldo, const float* bias, int accumulate,
                        cudaStream_t st) {
    if (bad_operands(a, b, m, n, k, ldo) || ((uintptr_t)out & 15)) return (int)cudaErrorInvalidValue;
    GemmParams p{m, n, k, out, ldo, bias, accumulate, 0, {}, 0, nullptr, 0, 0.f, 0.f};
    return dispatch(a, b, p, st);
}

// Same product with a bf16 result (n % 8 == 0, ldo % 8 == 0); no accumulation.
B2_API int b2_gemm_bf16_out16(const void* a, const void* b, int m, int n, int k, void* out, int ldo, const float* bias, cudaStream_t st) {
    if (bad_operands(a, b, m, n, k, ldo) || (n & 7) || (ldo & 7) || ((uintptr_t)out & 15)) return (int)cudaErrorInvalidValue;
    GemmParams p{m, n, k, out, ldo, bias, 0, 1, {}, 0, nullptr, 0, 0.f, 0.f};
    return dispatch(a, b, p, st);
}

// Row-parallel GEMM of a tensor-parallel group: row r of the partial result is stored, as bf16, into cm->dst[r / rows_per_rank]
// (a peer address; row index relative to the owner's first row, pitch ldo elements) and the exchange is announced on cm's channel.
B2_API int b2_gemm_bf16_scatter(const void* a, const void* b, int m, int n, int k, int ldo, const float* bias, const CommSend* cm,
                                int rows_per_rank, cudaStream_t st) {
    if (bad_operands(a, b, m, n, k, ldo) || !cm || rows_per_rank < 1 || cm->n_dst < 1 || cm->n_dst > COMM_MAX_RANKS ||
        (m + rows_per_rank - 1) / rows_per_rank > cm->n_dst)
        return (int)cudaErrorInvalidValue;
    GemmParams p{m, n, k, nullptr, ldo, bias, 0, 0, *cm, rows_per_rank, nullptr, 0, 0.f, 0.f};
    return dispatch(a, b, p, st);
}

// Gate/up product with the gated activation in the epilogue: out[m][n / 2] (bf16) = act(gate, up) of the interleaved columns of
// a . b^T + bias.  act: 0 silu, 1 gelu_tanh, 2 clamped swiglu (alpha, limit).
B2_API int b2_gemm_bf16_glu(const void* a, const void* b, int m, int n, int k, void* out, int ldo, const float* bias, int act, float alpha,
                            float limit, cudaStream_t st) {
    if (bad_operands(a, b, m, n, k, ldo) || (n & 7) || (ldo & 1) || ((uintptr_t)out & 3) || act < 0 || act > 2) return (int)cudaErrorInvalidValue;
    GemmParams p{m, n, k, out, ldo, bias, 0, 1, {}, 0, nullptr, 1 + act, alpha, limit};
    return dispatch(a, b, p, st);
}

// Grouped product over the experts of a mixture-of-experts layer in one launch.  a: [m][k] rows sorted by expert, every 128-row
// tile owned by one expert (tile_expert[m / 128] on the device: expert index, or -1 for a tile without rows); b: `experts`
// stacked [n][k] matrices; bias: experts x n or null.  glu_act < 0: out fp32 [m][ldo] = a . b_e^T + bias_e; otherwise the gated
// activation of interleaved gate/up columns, out bf16 [m][ldo] with n / 2 columns.
B2_API int b2_gemm_bf16_grouped(const void* a, const void* b, int m, int n, int k, int experts, const int* tile_expert, void* out, int ldo,
                                const float* bias, int glu_act_id, float alpha, float limit, cudaStream_t st) {
    if (bad_operands(a, b, m, n, k, ldo) || !tile_expert || experts < 1 || glu_act_id > 2 || ((uintptr_t)out & 15)) return (int)cudaErrorInvalidValue;
    if (glu_act_id >= 0 && ((n & 7) || (ldo & 1))) return (int)cudaErrorInvalidValue;
    GemmParams p{m, n, k, out, ldo, bias, 0, glu_act_id >= 0 ? 1 : 0, {}, 0, tile_expert, glu_act_id >= 0 ? 1 + glu_act_id : 0, alpha, limit};
    return dispatch(a, b, p, st, experts * n);
}

B2_API int b2_gemm_status() {
    int v = 0;
    cudaMemcpyFromSymbol(&v, g_gemm_status, sizeof(int));
    return v;
}
