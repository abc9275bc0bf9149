// Quantised matrix-vector kernels for decode (1..8 tokens per step), sm_100a.
//
// The role of these kernels in the reference stack is played by ggml's mmvq family (int8 dot
// products of block-quantised weights against block-quantised activations).  Design here:
//   * weights are re-laid out at load time into dense, naturally aligned planes (see WType); the FFN
//     gate and up matrices are additionally interleaved row by row into one matrix so that one warp
//     streams both rows of an output together;
//   * a warp owns four consecutive rows; its lanes stride over 16/32/48-byte items of those rows and
//     the item loop is unrolled, so every lane keeps 8+ independent 16-byte loads in flight (the
//     kernels are bound by memory-level parallelism: the whole 9 MB attention-output matrix of an 8B
//     model is smaller than what the SMs can have in flight).  Small matrices additionally split the
//     row length over KS warps of the CTA (partials meet in shared memory) so that every byte of the
//     matrix is requested in the first few hundred nanoseconds;
//   * activations arrive as int8 blocks of 32 with an fp32 scale d and the pre-multiplied block sum
//     s = d * sum(q) (needed by formats with a per-block minimum or a fixed offset); integer dot
//     products use dp4a;
//   * the epilogue stores, accumulates into the fp32 residual stream, or applies the gated FFN
//     activation and re-quantises the result for the following down projection.
// Weight loads bypass L1 (streamed once); activation loads stay cached.
#include "gemv_dot.cuh"
#include "comm.cuh"

struct GemvArgs {
    WDesc seg[4];
    int nseg;
    int nb;               // tokens (<= template NB)
    const int8_t* xq;     // [nb][k]
    const float2* xds;    // [nb][k/32]  (d, d*sum q)
    const float* xf;      // [nb][k]     fp32 activations for the float weight types
    float* out;           // [nb][ldo]
    int ldo;
    int accumulate;       // 1: out += result (residual add)
    CommSend cm;          // cm.n_dst > 0: write the result to every rank's buffer instead of `out` (pitch ldo) and announce it
    // mixture of experts (ids != null, nb = 1, one segment holding E stacked [n][k] matrices): grid.y enumerates
    // (token, expert-slot) pairs; pair p multiplies expert ids[p] with activation row p / x_div and writes output row p.
    // ids[p] < 0 (expert not resident on this GPU) gives a zero row.
    const int* ids;
    int x_div;
    int n_pairs;
};

struct GluArgs {
    WDesc gu;             // interleaved rows: 2i = gate row i, 2i+1 = up row i; n = 2 * d_ff
    int nb;
    const int8_t* xq;
    const float2* xds;
    const float* xf;
    int act;              // 0 silu, 1 gelu_tanh, 2 clamped swiglu (alpha, limit)
    float alpha, limit;
    int8_t* hq;           // [nb][d_ff]
    float2* hds;          // [nb][d_ff/32]
    float* hf;            // [nb][d_ff] or null
    // mixture of experts (ids != null, nb = 1, gu holds E stacked matrices): see GemvArgs
    const int* ids;
    int x_div;
    int n_pairs;
};

__device__ __forceinline__ Planes planes_of(const WDesc& w) {
    Planes p;
    p.p[0] = (const uint8_t*)w.p0; p.p[1] = (const uint8_t*)w.p1; p.p[2] = (const uint8_t*)w.p2; p.p[3] = (const uint8_t*)w.p3;
    plane_pitches(w.type, w.k, p.rb);
    return p;
}

// Sum M per-lane values across the warp with a halving exchange (about M + 5 shuffles instead of
// 5 M).  On return lane L owns elements e = base(L) + i, i < max(M/32, 1), in v[i]; base(L) is
// returned.  For M < 32 several lanes own the same element (the one with the low bits clear stores).
template <int M>
__device__ __forceinline__ int warp_reduce_scatter(float (&v)[M], int lane) {
    int base = 0;
    int cnt = M;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        if (cnt > 1) {
            const int half = cnt >> 1;
            const bool up = (lane & o) != 0;
#pragma unroll
            for (int i = 0; i < M / 2; i++) {
                if (i < half) {
                    const float send = up ? v[i] : v[i + half];
                    const float keep = up ? v[i + half] : v[i];
                    v[i] = keep + __shfl_xor_sync(0xffffffffu, send, o);
                }
            }
            if (up) base += half;
            cnt = half;
        } else {
            v[0] += __shfl_xor_sync(0xffffffffu, v[0], o);
        }
    }
    return base;
}

constexpr int R = 4;      // rows per warp

// Ask L2 for the weight bytes of rows [row0, row0 + nrows) before the grid-dependency wait: weights do
// not depend on the producer kernel, so they stream in while it drains and the dot loop then hits L2.
__device__ __forceinline__ void prefetch_rows(const Planes& pl, int row0, int nrows, int n_total, int idx, int n_idx) {
    nrows = min(nrows, n_total - row0);
    if (nrows <= 0) return;
#pragma unroll
    for (int p = 0; p < 4; p++) {
        if (pl.rb[p] == 0) continue;
        const uint8_t* base = pl.p[p] + (size_t)row0 * pl.rb[p];
        const uint32_t bytes = pl.rb[p] * (uint32_t)nrows;
        for (uint32_t off = (uint32_t)idx * 128u; off < bytes; off += (uint32_t)n_idx * 128u)
            asm volatile("prefetch.global.L2 [%0];" ::"l"(base + off));
    }
}

// CTA = 8 warps = (8/KS) row groups x KS slices of the row length.
// COMM: the epilogue stores to every rank of the tensor-parallel group (peer addresses) and publishes the exchange.
template <int NB, int KS, bool COMM>
__global__ void __launch_bounds__(256, (NB <= 2 ? 2 : 1)) gemv_kernel(const __grid_constant__ GemvArgs a) {
    constexpr int RGS = 8 / KS;
    constexpr int M = R * NB;
    constexpr int OWN = (M >= 32) ? (M / 32) : 1;
    __shared__ float red[8][M];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int rg = warp / KS, ks = warp % KS;
    int g = blockIdx.x * RGS + rg;
    int s = 0;
    for (; s < a.nseg; s++) {
        const int groups = (a.seg[s].n + R - 1) / R;
        if (g < groups) break;
        g -= groups;
    }
    const bool active = s < a.nseg;
    const WDesc& w = a.seg[active ? s : 0];
    const int row0 = g * R;
    float acc[R][NB];
#pragma unroll
    for (int r = 0; r < R; r++)
#pragma unroll
        for (int b = 0; b < NB; b++) acc[r][b] = 0.f;
    pdl_launch();
    const Planes pl = planes_of(w);
    if (active && !a.ids) prefetch_rows(pl, row0, R, w.n, ks * 32 + lane, KS * 32);
    pdl_wait();
    const int pair = a.ids ? (int)blockIdx.y : 0;
    const int expert = a.ids ? a.ids[pair] : 0;
    const int erow = expert * w.n;                   // first row of the selected expert in the stacked planes
    if (active && expert >= 0) {
        const size_t xo = a.ids ? (size_t)(pair / a.x_div) : 0;
        XRef<NB> x{a.xq + xo * w.k, a.xds + xo * (w.k >> 5), a.xf ? a.xf + xo * w.k : nullptr, w.k, a.nb};
        dot_any<R, NB>(w.type, pl, erow + row0, erow + w.n - 1, x, acc, ks * 32 + lane, KS * 32);
    }
    float(&flat)[M] = reinterpret_cast<float(&)[M]>(acc);
    const int base = warp_reduce_scatter<M>(flat, lane);
    const bool owner = M >= 32 || (lane & (32 / (M < 32 ? M : 32) - 1)) == 0;
    if (KS > 1) {
        if (owner) {
#pragma unroll
            for (int e = 0; e < OWN; e++) red[warp][base + e] = flat[e];
        }
        __syncthreads();
        if (!COMM && (ks != 0 || !active)) return;
        if (owner && ks == 0 && active) {
#pragma unroll
            for (int e = 0; e < OWN; e++) {
                float v = 0.f;
#pragma unroll
                for (int k2 = 0; k2 < KS; k2++) v += red[rg * KS + k2][base + e];
                flat[e] = v;
            }
        }
    }
    if (!COMM) {
        if (!active || !owner) return;
#pragma unroll
        for (int e = 0; e < OWN; e++) {
            const int idx = base + e, r = idx / NB, b = idx % NB;
            const int row = row0 + r;
            if (row < w.n && b < a.nb) {
                float* o = a.out + (size_t)(pair + b) * a.ldo + w.out_off + row;
                const float v = expert >= 0 ? flat[e] + (w.bias ? w.bias[erow + row] : 0.f) : 0.f;
                *o = a.accumulate ? *o + v : v;
            }
        }
    } else {
        const unsigned ep = comm_next_epoch(a.cm);
        if (active && owner && ks == 0) {
            const long long poff = comm_parity_off(a.cm, ep);
#pragma unroll
            for (int e = 0; e < OWN; e++) {
                const int idx = base + e, r = idx / NB, b = idx % NB;
                const int row = row0 + r;
                if (row < w.n && b < a.nb) {
                    const float v = flat[e] + (w.bias ? w.bias[row] : 0.f);
                    const long long o = poff + (long long)b * a.ldo + w.out_off + row;
                    if (a.cm.ll) {
                        const uint2 pair = make_uint2(__float_as_uint(v), ep);       // the value travels with its epoch
                        for (int d = 0; d < a.cm.n_dst; d++) reinterpret_cast<uint2*>(a.cm.dst[d])[o] = pair;
                    } else {
                        for (int d = 0; d < a.cm.n_dst; d++) a.cm.dst[d][o] = v;
                    }
                }
            }
        }
        if (!a.cm.ll) comm_publish(a.cm, gridDim.x, ep);
    }
}

// Gated FFN front half on the interleaved gate/up matrix: 16 warps x 2 outputs = one quantisation
// block of 32 outputs per CTA.
// WARPS = 16: one pass (few tokens, registers capped at 128); WARPS = 8: two passes per warp.
template <int NB, int WARPS>
__global__ void __launch_bounds__(WARPS * 32) glu_kernel(const __grid_constant__ GluArgs a) {
    constexpr int PASSES = 16 / WARPS;
    __shared__ float sh[NB][32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int n_out = a.gu.n >> 1;
    pdl_launch();
    const Planes pl = planes_of(a.gu);
    if (!a.ids) prefetch_rows(pl, (blockIdx.x * 32 + warp * PASSES * 2) * 2, R * PASSES, a.gu.n, lane, 32);
    pdl_wait();
    const int pair = a.ids ? (int)blockIdx.y : 0;
    const int expert = a.ids ? a.ids[pair] : 0;
    const int erow = expert * a.gu.n;
    const size_t xo = a.ids ? (size_t)(pair / a.x_div) : 0;
    XRef<NB> x{a.xq + xo * a.gu.k, a.xds + xo * (a.gu.k >> 5), a.xf ? a.xf + xo * a.gu.k : nullptr, a.gu.k, a.nb};
#pragma unroll 1
    for (int pass = 0; pass < PASSES; pass++) {
        const int slot = (warp * PASSES + pass) * 2;         // position of this warp's two outputs in the block of 32
        const int out0 = blockIdx.x * 32 + slot;
        const int row0 = out0 * 2;
        float acc[R][NB];
#pragma unroll
        for (int r = 0; r < R; r++)
#pragma unroll
            for (int b = 0; b < NB; b++) acc[r][b] = 0.f;
        if (out0 < n_out && expert >= 0) dot_any<R, NB>(a.gu.type, pl, erow + row0, erow + a.gu.n - 1, x, acc, lane, 32);
        // biases join lane 0's partial sums: row r of the warp is gate (r even) or up (r odd)
        if (a.gu.bias && out0 < n_out && lane == 0 && expert >= 0) {
#pragma unroll
            for (int r = 0; r < R; r++)
#pragma unroll
                for (int b = 0; b < NB; b++) acc[r][b] += a.gu.bias[erow + min(row0 + r, a.gu.n - 1)];
        }
        // plain reductions here: gate and up of one output must end up in the same lane
#pragma unroll
        for (int r = 0; r < R; r++)
#pragma unroll
            for (int b = 0; b < NB; b++) acc[r][b] = warp_sum(acc[r][b]);
        if (lane == 0) {
#pragma unroll
            for (int o = 0; o < 2; o++)
#pragma unroll
                for (int b = 0; b < NB; b++)
                    sh[b][slot + o] = (out0 + o < n_out) ? glu_act(acc[2 * o][b], acc[2 * o + 1][b], a.act, a.alpha, a.limit) : 0.f;
        }
    }
    __syncthreads();
    for (int b = warp; b < a.nb; b += WARPS) {
        const float v = sh[b][lane];
        const float amax = warp_max(fabsf(v));
        const float d = amax / 127.f;
        const int q = d > 0.f ? __float2int_rn(v / d) : 0;
        const float s = d * warp_sum((float)q);
        const int col = blockIdx.x * 32 + lane;
        const size_t orow = (size_t)(pair + b);
        if (col < n_out) {
            a.hq[orow * n_out + col] = (int8_t)q;
            if (a.hf) a.hf[orow * n_out + col] = v;
        }
        if (lane == 0) a.hds[orow * (n_out >> 5) + blockIdx.x] = make_float2(d, s);
    }
}

// ---------------------------------------------------------------------------------------------
// host launchers
// ---------------------------------------------------------------------------------------------
static cudaError_t launch_pdl(const void* fn, dim3 grid, dim3 block, size_t smem, void** args, cudaStream_t st, int pdl) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = pdl ? 1 : 0;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    return cudaLaunchKernelExC(&cfg, fn, args);
}

template <int NB, bool COMM>
static const void* pick_ks(int ks) {
    switch (ks) {
        case 8: return (const void*)gemv_kernel<NB, 8, COMM>;
        case 4: return (const void*)gemv_kernel<NB, 4, COMM>;
        case 2: return (const void*)gemv_kernel<NB, 2, COMM>;
        default: return (const void*)gemv_kernel<NB, 1, COMM>;
    }
}

template <bool COMM>
static const void* pick_nb(int nb, int ks) {
    return nb <= 1 ? pick_ks<1, COMM>(ks) : nb <= 2 ? pick_ks<2, COMM>(ks) : nb <= 4 ? pick_ks<4, COMM>(ks) : pick_ks<8, COMM>(ks);
}

// Runs y = W x for 1..8 tokens.  Returns a cudaError_t value.
B2_API int b2_gemv(const GemvArgs* a, int pdl, cudaStream_t st) {
    if (a->nb < 1 || a->nb > 8 || a->nseg < 1 || a->nseg > 4) return (int)cudaErrorInvalidValue;
    long groups = 0;
    int min_items = 1 << 30;
    for (int s = 0; s < a->nseg; s++) {
        groups += (a->seg[s].n + R - 1) / R;
        min_items = min(min_items, items_per_row(a->seg[s].type, a->seg[s].k));
    }
    // split the row length over KS warps until ~4000 warps exist (148 SMs x ~28) or a lane has one item left
    const int pairs = a->ids ? a->n_pairs : 1;
    if (a->ids && (a->nb != 1 || a->nseg != 1 || a->cm.n_dst > 0 || a->x_div < 1 || pairs < 1 || pairs > 65535)) return (int)cudaErrorInvalidValue;
    int ks = 1;
    while (ks < 8 && groups * pairs * ks < 4000 && min_items / (32 * ks * 2) >= 1) ks <<= 1;
    const int rgs = 8 / ks;
    dim3 grid((unsigned)((groups + rgs - 1) / rgs), (unsigned)pairs), block(256);
    GemvArgs copy = *a;
    void* args[] = {&copy};
    if (a->cm.n_dst < 0 || a->cm.n_dst > COMM_MAX_RANKS || (a->cm.n_dst > 0 && a->accumulate)) return (int)cudaErrorInvalidValue;
    const void* fn = a->cm.n_dst > 0 ? pick_nb<true>(a->nb, ks) : pick_nb<false>(a->nb, ks);
    return (int)launch_pdl(fn, grid, block, 0, args, st, pdl);
}

B2_API int b2_gemv_glu_quant(const GluArgs* a, int pdl, cudaStream_t st) {
    if (a->nb < 1 || a->nb > 8 || (a->gu.n & 63)) return (int)cudaErrorInvalidValue;
    if (a->ids && (a->nb != 1 || a->x_div < 1 || a->n_pairs < 1 || a->n_pairs > 65535)) return (int)cudaErrorInvalidValue;
    dim3 grid(a->gu.n / 64, a->ids ? a->n_pairs : 1), block(a->nb <= 2 ? 512 : 256);
    GluArgs copy = *a;
    void* args[] = {&copy};
    const void* fn = a->nb <= 1 ? (const void*)glu_kernel<1, 16> : a->nb <= 2 ? (const void*)glu_kernel<2, 16>
                   : a->nb <= 4 ? (const void*)glu_kernel<4, 8> : (const void*)glu_kernel<8, 8>;
    return (int)launch_pdl(fn, grid, block, 0, args, st, pdl);
}
