// Quantised matrix-vector kernels for decode (1..8 tokens per step), sm_100a.
//
// The role of these kernels in the reference stack is played by ggml's mmvq family (int8 dot
// products of block-quantised weights against block-quantised activations).  Design here:
//   * weights are re-laid out at load time into dense, naturally aligned planes (see WType);
//   * activations arrive as int8 blocks of 32 with an fp32 scale d and the pre-multiplied block sum
//     s = d * sum(q) (needed by the formats that carry a per-block minimum or a fixed offset);
//   * one warp owns R output rows, its lanes stride over 16/32/48-byte "items" of the rows so that
//     every lane has R independent 16-byte loads in flight; integer dot products use dp4a;
//   * the epilogue either stores, accumulates into the fp32 residual stream, or applies the gated
//     activation of the FFN and re-quantises the result for the following down projection.
// Weight loads bypass L1 (streamed once); activation loads stay cached.
#include "common.cuh"

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
};

template <int NB>
struct XRef {
    const int8_t* q;
    const float2* ds;
    const float* f;
    int k;
    int nb;    // valid tokens; template slots beyond it re-read token 0 and are never stored
    __device__ __forceinline__ size_t tok(int b) const { return (size_t)(b < nb ? b : 0); }
};

__device__ __forceinline__ void k4_scales(uint32_t s0, uint32_t s1, uint32_t s2, int j, float& sc_lo, float& m_lo, float& sc_hi, float& m_hi) {
    // sub-blocks 2j and 2j+1 of the 12-byte packed table (6-bit scale, 6-bit min each)
    int i = 2 * j;
    uint32_t a, b, c, d;
    if (j < 2) {
        a = (s0 >> (8 * i)) & 63;
        b = (s1 >> (8 * i)) & 63;
        c = (s0 >> (8 * i + 8)) & 63;
        d = (s1 >> (8 * i + 8)) & 63;
    } else {
        int t = i - 4;
        a = ((s2 >> (8 * t)) & 0xF) | (((s0 >> (8 * t + 6)) & 3) << 4);
        b = ((s2 >> (8 * t + 4)) & 0xF) | (((s1 >> (8 * t + 6)) & 3) << 4);
        c = ((s2 >> (8 * t + 8)) & 0xF) | (((s0 >> (8 * t + 14)) & 3) << 4);
        d = ((s2 >> (8 * t + 12)) & 0xF) | (((s1 >> (8 * t + 14)) & 3) << 4);
    }
    sc_lo = (float)a; m_lo = (float)b; sc_hi = (float)c; m_hi = (float)d;
}

__device__ __forceinline__ int dot16(const uint4& w, const int4& x) {
    int s = __dp4a((int)w.x, x.x, 0);
    s = __dp4a((int)w.y, x.y, s);
    s = __dp4a((int)w.z, x.z, s);
    return __dp4a((int)w.w, x.w, s);
}

// ---------------------------------------------------------------------------------------------
// per-format partial dot products: lane-strided over the row, R rows x NB tokens
// ---------------------------------------------------------------------------------------------
template <int R, int NB>
__device__ __forceinline__ void dot_q4k(const WDesc& w, int row0, const XRef<NB>& x, float (&acc)[R][NB], int lane, bool has_qh) {
    const int K = w.k, nsb = K >> 8, items = nsb * 8;
    const uint8_t* qs = (const uint8_t*)w.p0;
    const uint4* hdr = (const uint4*)w.p1;
    const uint8_t* qhp = (const uint8_t*)w.p2;
    for (int it = lane; it < items; it += 32) {
        const int sb = it >> 3, c = it & 7, j = c >> 1, h = c & 1;
        uint4 q[R], hd[R], qh[R];
#pragma unroll
        for (int r = 0; r < R; r++) {
            const int row = min(row0 + r, w.n - 1);
            q[r] = ldg16(qs + (size_t)row * (K >> 1) + sb * 128 + c * 16);
            hd[r] = __ldg(hdr + (size_t)row * nsb + sb);
            if (has_qh) qh[r] = ldg16(qhp + (size_t)row * (K >> 3) + sb * 32 + h * 16);
        }
        const int xoff = sb * 256 + 64 * j + 16 * h;
        int4 xlo[NB], xhi[NB];
        float2 dlo[NB], dhi[NB];
#pragma unroll
        for (int b = 0; b < NB; b++) {
            xlo[b] = *(const int4*)(x.q + x.tok(b) * K + xoff);
            xhi[b] = *(const int4*)(x.q + x.tok(b) * K + xoff + 32);
            dlo[b] = x.ds[x.tok(b) * (K >> 5) + sb * 8 + 2 * j];
            dhi[b] = x.ds[x.tok(b) * (K >> 5) + sb * 8 + 2 * j + 1];
        }
#pragma unroll
        for (int r = 0; r < R; r++) {
            const __half2 dm = *reinterpret_cast<const __half2*>(&hd[r].x);
            const float d = __low2float(dm), dmin = __high2float(dm);
            float sc_lo, m_lo, sc_hi, m_hi;
            k4_scales(hd[r].y, hd[r].z, hd[r].w, j, sc_lo, m_lo, sc_hi, m_hi);
            uint4 lo, hi;
            lo.x = q[r].x & 0x0f0f0f0fu; lo.y = q[r].y & 0x0f0f0f0fu; lo.z = q[r].z & 0x0f0f0f0fu; lo.w = q[r].w & 0x0f0f0f0fu;
            hi.x = (q[r].x >> 4) & 0x0f0f0f0fu; hi.y = (q[r].y >> 4) & 0x0f0f0f0fu;
            hi.z = (q[r].z >> 4) & 0x0f0f0f0fu; hi.w = (q[r].w >> 4) & 0x0f0f0f0fu;
            if (has_qh) {   // Q5_K: fifth bit of sub-block i is bit i of qh[l]
                const int s = 2 * j;
                lo.x |= ((qh[r].x >> s) & 0x01010101u) << 4; lo.y |= ((qh[r].y >> s) & 0x01010101u) << 4;
                lo.z |= ((qh[r].z >> s) & 0x01010101u) << 4; lo.w |= ((qh[r].w >> s) & 0x01010101u) << 4;
                hi.x |= ((qh[r].x >> (s + 1)) & 0x01010101u) << 4; hi.y |= ((qh[r].y >> (s + 1)) & 0x01010101u) << 4;
                hi.z |= ((qh[r].z >> (s + 1)) & 0x01010101u) << 4; hi.w |= ((qh[r].w >> (s + 1)) & 0x01010101u) << 4;
            }
            const float dl = d * sc_lo, dh = d * sc_hi;
            const float ml = (h == 0) ? dmin * m_lo : 0.f, mh = (h == 0) ? dmin * m_hi : 0.f;
#pragma unroll
            for (int b = 0; b < NB; b++) {
                const int sl = dot16(lo, xlo[b]), sh = dot16(hi, xhi[b]);
                acc[r][b] += dl * dlo[b].x * (float)sl + dh * dhi[b].x * (float)sh - ml * dlo[b].y - mh * dhi[b].y;
            }
        }
    }
}

template <int R, int NB>
__device__ __forceinline__ void dot_q6k(const WDesc& w, int row0, const XRef<NB>& x, float (&acc)[R][NB], int lane) {
    const int K = w.k, nsb = K >> 8, items = nsb * 4;
    const uint8_t* ql = (const uint8_t*)w.p0;
    const uint8_t* qh = (const uint8_t*)w.p1;
    const int8_t* sc = (const int8_t*)w.p2;
    const __half* dp = (const __half*)w.p3;
    for (int it = lane; it < items; it += 32) {
        const int sb = it >> 2, n = (it >> 1) & 1, c = it & 1;
        uint4 a[R], bq[R], hq[R];
        uint2 s8[R];
        float d[R];
#pragma unroll
        for (int r = 0; r < R; r++) {
            const int row = min(row0 + r, w.n - 1);
            const uint8_t* base = ql + (size_t)row * (K >> 1) + sb * 128 + 64 * n + 16 * c;
            a[r] = ldg16(base);
            bq[r] = ldg16(base + 32);
            hq[r] = ldg16(qh + (size_t)row * (K >> 2) + sb * 64 + 32 * n + 16 * c);
            s8[r] = __ldg((const uint2*)(sc + (size_t)row * (K >> 4) + sb * 16 + 8 * n));
            d[r] = __half2float(__ldg(dp + (size_t)row * nsb + sb));
        }
        const int xoff = sb * 256 + 128 * n + 16 * c;
        int4 xv[NB][4];
        float dx[NB][4];
#pragma unroll
        for (int b = 0; b < NB; b++)
#pragma unroll
            for (int qd = 0; qd < 4; qd++) {
                xv[b][qd] = *(const int4*)(x.q + x.tok(b) * K + xoff + 32 * qd);
                dx[b][qd] = x.ds[x.tok(b) * (K >> 5) + sb * 8 + 4 * n + qd].x;
            }
#pragma unroll
        for (int r = 0; r < R; r++) {
            uint4 v[4];
            const uint32_t* A = &a[r].x; const uint32_t* B = &bq[r].x; const uint32_t* H = &hq[r].x;
            uint32_t* v0 = &v[0].x; uint32_t* v1 = &v[1].x; uint32_t* v2 = &v[2].x; uint32_t* v3 = &v[3].x;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                v0[i] = __vsub4((A[i] & 0x0f0f0f0fu) | ((H[i] << 4) & 0x30303030u), 0x20202020u);
                v1[i] = __vsub4((B[i] & 0x0f0f0f0fu) | ((H[i] << 2) & 0x30303030u), 0x20202020u);
                v2[i] = __vsub4(((A[i] >> 4) & 0x0f0f0f0fu) | (H[i] & 0x30303030u), 0x20202020u);
                v3[i] = __vsub4(((B[i] >> 4) & 0x0f0f0f0fu) | ((H[i] >> 2) & 0x30303030u), 0x20202020u);
            }
            // scales for the four quarters: bytes c, c+2, c+4, c+6 of the 8-byte group
            const uint64_t sraw = ((uint64_t)s8[r].y << 32) | s8[r].x;
            float scq[4];
#pragma unroll
            for (int qd = 0; qd < 4; qd++) scq[qd] = d[r] * (float)(int8_t)((sraw >> (8 * (c + 2 * qd))) & 0xff);
#pragma unroll
            for (int b = 0; b < NB; b++) {
                float t = 0.f;
#pragma unroll
                for (int qd = 0; qd < 4; qd++) t += scq[qd] * dx[b][qd] * (float)dot16(v[qd], xv[b][qd]);
                acc[r][b] += t;
            }
        }
    }
}

template <int R, int NB>
__device__ __forceinline__ void dot_q8_0(const WDesc& w, int row0, const XRef<NB>& x, float (&acc)[R][NB], int lane) {
    const int K = w.k, items = K >> 5;
    const int8_t* qs = (const int8_t*)w.p0;
    const __half* dp = (const __half*)w.p1;
    for (int it = lane; it < items; it += 32) {
        uint4 a[R], bq[R];
        float d[R];
#pragma unroll
        for (int r = 0; r < R; r++) {
            const int row = min(row0 + r, w.n - 1);
            a[r] = ldg16(qs + (size_t)row * K + it * 32);
            bq[r] = ldg16(qs + (size_t)row * K + it * 32 + 16);
            d[r] = __half2float(__ldg(dp + (size_t)row * items + it));
        }
#pragma unroll
        for (int b = 0; b < NB; b++) {
            const int4 x0 = *(const int4*)(x.q + x.tok(b) * K + it * 32);
            const int4 x1 = *(const int4*)(x.q + x.tok(b) * K + it * 32 + 16);
            const float dx = x.ds[x.tok(b) * items + it].x;
#pragma unroll
            for (int r = 0; r < R; r++) acc[r][b] += d[r] * dx * (float)(dot16(a[r], x0) + dot16(bq[r], x1));
        }
    }
}

template <int R, int NB>
__device__ __forceinline__ void dot_q4_0(const WDesc& w, int row0, const XRef<NB>& x, float (&acc)[R][NB], int lane) {
    const int K = w.k, items = K >> 5;
    const uint8_t* qs = (const uint8_t*)w.p0;
    const __half* dp = (const __half*)w.p1;
    for (int it = lane; it < items; it += 32) {
        uint4 q[R];
        float d[R];
#pragma unroll
        for (int r = 0; r < R; r++) {
            const int row = min(row0 + r, w.n - 1);
            q[r] = ldg16(qs + (size_t)row * (K >> 1) + it * 16);
            d[r] = __half2float(__ldg(dp + (size_t)row * items + it));
        }
#pragma unroll
        for (int b = 0; b < NB; b++) {
            const int4 x0 = *(const int4*)(x.q + x.tok(b) * K + it * 32);
            const int4 x1 = *(const int4*)(x.q + x.tok(b) * K + it * 32 + 16);
            const float2 ds = x.ds[x.tok(b) * items + it];
#pragma unroll
            for (int r = 0; r < R; r++) {
                uint4 lo, hi;
                lo.x = q[r].x & 0x0f0f0f0fu; lo.y = q[r].y & 0x0f0f0f0fu; lo.z = q[r].z & 0x0f0f0f0fu; lo.w = q[r].w & 0x0f0f0f0fu;
                hi.x = (q[r].x >> 4) & 0x0f0f0f0fu; hi.y = (q[r].y >> 4) & 0x0f0f0f0fu;
                hi.z = (q[r].z >> 4) & 0x0f0f0f0fu; hi.w = (q[r].w >> 4) & 0x0f0f0f0fu;
                acc[r][b] += d[r] * (ds.x * (float)(dot16(lo, x0) + dot16(hi, x1)) - 8.f * ds.y);
            }
        }
    }
}

// e2m1 code -> 2 * value as int8, four codes at a time
__device__ __forceinline__ uint32_t fp4x4_to_i8(uint32_t idx) {
    const uint32_t sel = (idx & 0x7u) | ((idx >> 4) & 0x70u) | ((idx >> 8) & 0x700u) | ((idx >> 12) & 0x7000u);
    const uint32_t mag = __byte_perm(0x03020100u, 0x0c080604u, sel);
    const uint32_t neg = ((idx >> 3) & 0x01010101u) * 0xffu;
    return __vsub4(mag ^ neg, neg);
}

template <int R, int NB>
__device__ __forceinline__ void dot_mxfp4(const WDesc& w, int row0, const XRef<NB>& x, float (&acc)[R][NB], int lane) {
    const int K = w.k, items = K >> 5;
    const uint8_t* qs = (const uint8_t*)w.p0;
    const uint8_t* ep = (const uint8_t*)w.p1;
    for (int it = lane; it < items; it += 32) {
        uint4 q[R];
        float d[R];
#pragma unroll
        for (int r = 0; r < R; r++) {
            const int row = min(row0 + r, w.n - 1);
            q[r] = ldg16(qs + (size_t)row * (K >> 1) + it * 16);
            d[r] = 0.5f * e8m0_to_float(__ldg(ep + (size_t)row * items + it));
        }
#pragma unroll
        for (int b = 0; b < NB; b++) {
            const int4 x0 = *(const int4*)(x.q + x.tok(b) * K + it * 32);
            const int4 x1 = *(const int4*)(x.q + x.tok(b) * K + it * 32 + 16);
            const float dx = x.ds[x.tok(b) * items + it].x;
#pragma unroll
            for (int r = 0; r < R; r++) {
                uint4 lo, hi;
                lo.x = fp4x4_to_i8(q[r].x & 0x0f0f0f0fu); lo.y = fp4x4_to_i8(q[r].y & 0x0f0f0f0fu);
                lo.z = fp4x4_to_i8(q[r].z & 0x0f0f0f0fu); lo.w = fp4x4_to_i8(q[r].w & 0x0f0f0f0fu);
                hi.x = fp4x4_to_i8((q[r].x >> 4) & 0x0f0f0f0fu); hi.y = fp4x4_to_i8((q[r].y >> 4) & 0x0f0f0f0fu);
                hi.z = fp4x4_to_i8((q[r].z >> 4) & 0x0f0f0f0fu); hi.w = fp4x4_to_i8((q[r].w >> 4) & 0x0f0f0f0fu);
                acc[r][b] += d[r] * dx * (float)(dot16(lo, x0) + dot16(hi, x1));
            }
        }
    }
}

template <int R, int NB, int WT>
__device__ __forceinline__ void dot_float(const WDesc& w, int row0, const XRef<NB>& x, float (&acc)[R][NB], int lane) {
    const int K = w.k;
    constexpr int EPI = (WT == WT_F32) ? 4 : 8;      // elements per 16-byte item
    const int items = K / EPI;
    const char* base = (const char*)w.p0;
    const size_t rowb = (size_t)K * (WT == WT_F32 ? 4 : 2);
    for (int it = lane; it < items; it += 32) {
        uint4 q[R];
#pragma unroll
        for (int r = 0; r < R; r++) q[r] = ldg16(base + (size_t)min(row0 + r, w.n - 1) * rowb + (size_t)it * 16);
#pragma unroll
        for (int b = 0; b < NB; b++) {
            float xv[EPI];
            const float4* xp = (const float4*)(x.f + x.tok(b) * K + it * EPI);
#pragma unroll
            for (int i = 0; i < EPI / 4; i++) {
                const float4 t = xp[i];
                xv[4 * i] = t.x; xv[4 * i + 1] = t.y; xv[4 * i + 2] = t.z; xv[4 * i + 3] = t.w;
            }
#pragma unroll
            for (int r = 0; r < R; r++) {
                const uint32_t* u = &q[r].x;
                float t = 0.f;
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    if (WT == WT_F32) {
                        t += __uint_as_float(u[i]) * xv[i];
                    } else if (WT == WT_BF16) {
                        t += __uint_as_float(u[i] << 16) * xv[2 * i] + __uint_as_float(u[i] & 0xffff0000u) * xv[2 * i + 1];
                    } else {
                        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&u[i]));
                        t += f.x * xv[2 * i] + f.y * xv[2 * i + 1];
                    }
                }
                acc[r][b] += t;
            }
        }
    }
}

template <int R, int NB>
__device__ __forceinline__ void dot_rows(const WDesc& w, int row0, const XRef<NB>& x, float (&acc)[R][NB], int lane) {
    switch (w.type) {
        case WT_Q4_K: dot_q4k<R, NB>(w, row0, x, acc, lane, false); break;
        case WT_Q5_K: dot_q4k<R, NB>(w, row0, x, acc, lane, true); break;
        case WT_Q6_K: dot_q6k<R, NB>(w, row0, x, acc, lane); break;
        case WT_Q8_0: dot_q8_0<R, NB>(w, row0, x, acc, lane); break;
        case WT_Q4_0: dot_q4_0<R, NB>(w, row0, x, acc, lane); break;
        case WT_MXFP4: dot_mxfp4<R, NB>(w, row0, x, acc, lane); break;
        case WT_BF16: dot_float<R, NB, WT_BF16>(w, row0, x, acc, lane); break;
        case WT_F16: dot_float<R, NB, WT_F16>(w, row0, x, acc, lane); break;
        default: dot_float<R, NB, WT_F32>(w, row0, x, acc, lane); break;
    }
#pragma unroll
    for (int r = 0; r < R; r++)
#pragma unroll
        for (int b = 0; b < NB; b++) acc[r][b] = warp_sum(acc[r][b]);
}

// ---------------------------------------------------------------------------------------------
// y[b, off + row] (+)= W[row, :] . x[b, :] + bias[row]    for up to four weight segments sharing x
// ---------------------------------------------------------------------------------------------
template <int R, int NB>
__global__ void __launch_bounds__(256) gemv_kernel(const __grid_constant__ GemvArgs a) {
    const int lane = threadIdx.x & 31;
    int g = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    int s = 0;
    for (; s < a.nseg; s++) {
        const int groups = (a.seg[s].n + R - 1) / R;
        if (g < groups) break;
        g -= groups;
    }
    pdl_launch();
    if (s >= a.nseg) return;
    const WDesc& w = a.seg[s];
    const int row0 = g * R;
    float acc[R][NB];
#pragma unroll
    for (int r = 0; r < R; r++)
#pragma unroll
        for (int b = 0; b < NB; b++) acc[r][b] = 0.f;
    pdl_wait();
    XRef<NB> x{a.xq, a.xds, a.xf, w.k, a.nb};
    dot_rows<R, NB>(w, row0, x, acc, lane);
    if (lane == 0) {
#pragma unroll
        for (int r = 0; r < R; r++) {
            const int row = row0 + r;
            if (row >= w.n) break;
            const float bias = w.bias ? w.bias[row] : 0.f;
#pragma unroll
            for (int b = 0; b < NB; b++) {
                if (b >= a.nb) break;
                float* o = a.out + (size_t)b * a.ldo + w.out_off + row;
                const float v = acc[r][b] + bias;
                *o = a.accumulate ? *o + v : v;
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Gated FFN front half: h = act(Wg x + bg) * (Wu x + bu), re-quantised to int8 blocks of 32
// ---------------------------------------------------------------------------------------------
struct GluArgs {
    WDesc gate, up;       // same n, k
    int nb;
    const int8_t* xq;
    const float2* xds;
    const float* xf;
    int act;              // 0 silu, 1 gelu_tanh, 2 clamped swiglu (alpha, limit)
    float alpha, limit;
    int8_t* hq;           // [nb][n]
    float2* hds;          // [nb][n/32]
    float* hf;            // [nb][n] or null
};

__device__ __forceinline__ float glu_act(float g, float u, int act, float alpha, float limit) {
    if (act == 0) return g / (1.f + __expf(-g)) * u;
    if (act == 1) {
        const float t = tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g));
        return 0.5f * g * (1.f + t) * u;
    }
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return g / (1.f + __expf(-alpha * g)) * (u + 1.f);
}

template <int NB>
__global__ void __launch_bounds__(256) gemv_glu_quant_kernel(const __grid_constant__ GluArgs a) {
    __shared__ float sh[NB][32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int tile0 = blockIdx.x * 32;
    pdl_launch();
    pdl_wait();
    XRef<NB> x{a.xq, a.xds, a.xf, a.gate.k, a.nb};
#pragma unroll
    for (int pass = 0; pass < 2; pass++) {
        const int row0 = tile0 + warp * 4 + pass * 2;
        float ag[2][NB], au[2][NB];
#pragma unroll
        for (int r = 0; r < 2; r++)
#pragma unroll
            for (int b = 0; b < NB; b++) ag[r][b] = au[r][b] = 0.f;
        if (row0 < a.gate.n) {
            dot_rows<2, NB>(a.gate, row0, x, ag, lane);
            dot_rows<2, NB>(a.up, row0, x, au, lane);
        }
        if (lane == 0) {
#pragma unroll
            for (int r = 0; r < 2; r++) {
                const int row = row0 + r;
                const bool ok = row < a.gate.n;
                const float bg = (ok && a.gate.bias) ? a.gate.bias[row] : 0.f;
                const float bu = (ok && a.up.bias) ? a.up.bias[row] : 0.f;
#pragma unroll
                for (int b = 0; b < NB; b++)
                    sh[b][warp * 4 + pass * 2 + r] = ok ? glu_act(ag[r][b] + bg, au[r][b] + bu, a.act, a.alpha, a.limit) : 0.f;
            }
        }
    }
    __syncthreads();
    for (int b = warp; b < a.nb; b += 8) {
        const float v = sh[b][lane];
        const float amax = warp_max(fabsf(v));
        const float d = amax / 127.f;
        const int q = d > 0.f ? __float2int_rn(v / d) : 0;
        const float s = d * warp_sum((float)q);
        const int col = tile0 + lane;
        if (col < a.gate.n) {
            a.hq[(size_t)b * a.gate.n + col] = (int8_t)q;
            if (a.hf) a.hf[(size_t)b * a.gate.n + col] = v;
        }
        if (lane == 0) a.hds[(size_t)b * (a.gate.n >> 5) + blockIdx.x] = make_float2(d, s);
    }
}

// ---------------------------------------------------------------------------------------------
// host launchers
// ---------------------------------------------------------------------------------------------
static cudaError_t launch_pdl(const void* fn, dim3 grid, dim3 block, void** args, cudaStream_t st, int pdl) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = 0;
    cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = pdl ? 1 : 0;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    return cudaLaunchKernelExC(&cfg, fn, args);
}

template <int R>
static const void* pick_gemv(int nb) {
    if (nb <= 1) return (const void*)gemv_kernel<R, 1>;
    if (nb <= 2) return (const void*)gemv_kernel<R, 2>;
    if (nb <= 4) return (const void*)gemv_kernel<R, 4>;
    return (const void*)gemv_kernel<R, 8>;
}

// Runs y = W x for 1..8 tokens.  Returns a cudaError_t value.
B2_API int b2_gemv(const GemvArgs* a, int pdl, cudaStream_t st) {
    if (a->nb < 1 || a->nb > 8 || a->nseg < 1 || a->nseg > 4) return (int)cudaErrorInvalidValue;
    long rows = 0;
    for (int s = 0; s < a->nseg; s++) rows += a->seg[s].n;
    // rows per warp: keep at least ~2 waves of warps on 148 SMs for small matrices
    const bool small = rows <= 8192 || a->nb > 4;
    const int R = small ? 2 : 4;
    long groups = 0;
    for (int s = 0; s < a->nseg; s++) groups += (a->seg[s].n + R - 1) / R;
    const int wpb = 8;
    dim3 grid((unsigned)((groups + wpb - 1) / wpb)), block(wpb * 32);
    GemvArgs copy = *a;
    void* args[] = {&copy};
    const void* fn = small ? pick_gemv<2>(a->nb) : pick_gemv<4>(a->nb);
    return (int)launch_pdl(fn, grid, block, args, st, pdl);
}

B2_API int b2_gemv_glu_quant(const GluArgs* a, int pdl, cudaStream_t st) {
    if (a->nb < 1 || a->nb > 8 || a->gate.n != a->up.n || a->gate.k != a->up.k || (a->gate.n & 31)) return (int)cudaErrorInvalidValue;
    dim3 grid(a->gate.n / 32), block(256);
    GluArgs copy = *a;
    void* args[] = {&copy};
    const void* fn = a->nb <= 1 ? (const void*)gemv_glu_quant_kernel<1>
                   : a->nb <= 2 ? (const void*)gemv_glu_quant_kernel<2>
                   : a->nb <= 4 ? (const void*)gemv_glu_quant_kernel<4>
                                : (const void*)gemv_glu_quant_kernel<8>;
    return (int)launch_pdl(fn, grid, block, args, st, pdl);
}
