// Per-format partial dot products shared by the decode GEMV kernels.
//
// A weight is described by up to four plane pointers and their row pitches (bytes).  Every function
// accumulates, for R consecutive rows and NB tokens, the contribution of the items
//   it = it0, it0 + step, ...  (< items of a row)
// handled by the calling lane; the caller reduces across lanes / warps.  Row and token base
// pointers are formed once, outside the item loop, and all loads of a trip are issued before the
// first use.  The kernels are bound by instruction issue as much as by memory, so the per-item work
// is kept to: nibble masks, dp4a, two int->float conversions and a handful of FMAs per row.
#pragma once
#include "common.cuh"

struct Planes {
    const uint8_t* p[4];
    uint32_t rb[4];       // row pitch in bytes
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

__device__ __forceinline__ int dot16(const uint4& w, const int4& x) {
    int s = __dp4a((int)w.x, x.x, 0);
    s = __dp4a((int)w.y, x.y, s);
    s = __dp4a((int)w.z, x.z, s);
    return __dp4a((int)w.w, x.w, s);
}

#define NIB_LO(d, s) d.x = s.x & 0x0f0f0f0fu; d.y = s.y & 0x0f0f0f0fu; d.z = s.z & 0x0f0f0f0fu; d.w = s.w & 0x0f0f0f0fu
#define NIB_HI(d, s) d.x = (s.x >> 4) & 0x0f0f0f0fu; d.y = (s.y >> 4) & 0x0f0f0f0fu; d.z = (s.z >> 4) & 0x0f0f0f0fu; d.w = (s.w >> 4) & 0x0f0f0f0fu

// unsigned weights x signed activations, accumulating
__device__ __forceinline__ int dp4a_us(uint32_t w, int x, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(w), "r"(x), "r"(c));
    return d;
}
__device__ __forceinline__ int dot16_us(const uint4& w, const int4& x, int c) {
    c = dp4a_us(w.x, x.x, c);
    c = dp4a_us(w.y, x.y, c);
    c = dp4a_us(w.z, x.z, c);
    return dp4a_us(w.w, x.w, c);
}

// Q4_K (and Q5_K when HAS_QH).  Planes: p0 = nibbles [K/2], p1 = scale bytes, 16 per super-block laid out
// as four words {sc(2j), sc(2j+1), min(2j), min(2j+1)} (the 6-bit table is unpacked once at load time),
// p2 = {half d, half dmin} per super-block, p3 = fifth bits [K/8] (Q5_K only).
// Item = one 64-element group = 32 contiguous nibble bytes = two sub-blocks.  The high nibbles are used
// in place (value * 16, unsigned dp4a) and the factor 1/16 is folded into the sub-block scale.
template <int R, int NB, bool HAS_QH>
__device__ __forceinline__ void dot_q4k(const Planes& w, int row0, int rmax, const XRef<NB>& x, float (&acc)[R][NB], int it0, int step) {
    const int K = x.k, items = K >> 6;
    const uint8_t* qp[R];
    const uint8_t* sp[R];
    const uint8_t* dp[R];
    const uint8_t* bp[R];
#pragma unroll
    for (int r = 0; r < R; r++) {
        const int row = min(row0 + r, rmax);
        qp[r] = w.p[0] + (size_t)row * w.rb[0];
        sp[r] = w.p[1] + (size_t)row * w.rb[1];
        dp[r] = w.p[2] + (size_t)row * w.rb[2];
        bp[r] = HAS_QH ? w.p[3] + (size_t)row * w.rb[3] : nullptr;
    }
    const int8_t* xq[NB];
    const float2* xd[NB];
#pragma unroll
    for (int b = 0; b < NB; b++) {
        xq[b] = x.q + x.tok(b) * K;
        xd[b] = x.ds + x.tok(b) * (K >> 5);
    }
    for (int it = it0; it < items; it += step) {
        const int sb = it >> 2;
        uint4 qa[R], qb[R];
        uint32_t sm[R], dd[R];
#pragma unroll
        for (int r = 0; r < R; r++) {
            qa[r] = ldg16(qp[r] + it * 32);
            qb[r] = ldg16(qp[r] + it * 32 + 16);
            sm[r] = __ldg((const uint32_t*)(sp[r] + it * 4));
            dd[r] = __ldg((const uint32_t*)(dp[r] + sb * 4));
        }
        int4 x0[NB], x1[NB], x2[NB], x3[NB];
        float2 dlo[NB], dhi[NB];
#pragma unroll
        for (int b = 0; b < NB; b++) {
            const int4* xp = (const int4*)(xq[b] + it * 64);
            x0[b] = xp[0]; x1[b] = xp[1]; x2[b] = xp[2]; x3[b] = xp[3];
            dlo[b] = xd[b][it * 2];
            dhi[b] = xd[b][it * 2 + 1];
        }
#pragma unroll
        for (int r = 0; r < R; r++) {
            const float2 df = __half22float2(*reinterpret_cast<const __half2*>(&dd[r]));
            const float dl = df.x * (float)(sm[r] & 0xff), dh = df.x * (float)((sm[r] >> 8) & 0xff) * (HAS_QH ? 1.f : 0.0625f);
            const float ml = df.y * (float)((sm[r] >> 16) & 0xff), mh = df.y * (float)(sm[r] >> 24);
            uint4 la, lb, ha, hb;
            NIB_LO(la, qa[r]); NIB_LO(lb, qb[r]);
            if (HAS_QH) {   // fifth bit of sub-block i is bit i of qh[l], l = 0..31
                const int j = it & 3, s = 2 * j;
                NIB_HI(ha, qa[r]); NIB_HI(hb, qb[r]);
                const uint4 ba = ldg16(bp[r] + sb * 32), bb = ldg16(bp[r] + sb * 32 + 16);
                la.x |= ((ba.x >> s) & 0x01010101u) << 4; la.y |= ((ba.y >> s) & 0x01010101u) << 4;
                la.z |= ((ba.z >> s) & 0x01010101u) << 4; la.w |= ((ba.w >> s) & 0x01010101u) << 4;
                lb.x |= ((bb.x >> s) & 0x01010101u) << 4; lb.y |= ((bb.y >> s) & 0x01010101u) << 4;
                lb.z |= ((bb.z >> s) & 0x01010101u) << 4; lb.w |= ((bb.w >> s) & 0x01010101u) << 4;
                ha.x |= ((ba.x >> (s + 1)) & 0x01010101u) << 4; ha.y |= ((ba.y >> (s + 1)) & 0x01010101u) << 4;
                ha.z |= ((ba.z >> (s + 1)) & 0x01010101u) << 4; ha.w |= ((ba.w >> (s + 1)) & 0x01010101u) << 4;
                hb.x |= ((bb.x >> (s + 1)) & 0x01010101u) << 4; hb.y |= ((bb.y >> (s + 1)) & 0x01010101u) << 4;
                hb.z |= ((bb.z >> (s + 1)) & 0x01010101u) << 4; hb.w |= ((bb.w >> (s + 1)) & 0x01010101u) << 4;
            } else {
                ha.x = qa[r].x & 0xf0f0f0f0u; ha.y = qa[r].y & 0xf0f0f0f0u; ha.z = qa[r].z & 0xf0f0f0f0u; ha.w = qa[r].w & 0xf0f0f0f0u;
                hb.x = qb[r].x & 0xf0f0f0f0u; hb.y = qb[r].y & 0xf0f0f0f0u; hb.z = qb[r].z & 0xf0f0f0f0u; hb.w = qb[r].w & 0xf0f0f0f0u;
            }
#pragma unroll
            for (int b = 0; b < NB; b++) {
                const int sl = dot16_us(lb, x1[b], dot16_us(la, x0[b], 0));
                const int sh = dot16_us(hb, x3[b], dot16_us(ha, x2[b], 0));
                acc[r][b] += (dl * dlo[b].x) * (float)sl + (dh * dhi[b].x) * (float)sh - ml * dlo[b].y - mh * dhi[b].y;
            }
        }
    }
}

// Q6_K: p0 = ql, p1 = qh, p2 = int8 scales, p3 = half d.  Item = 64 weights: 16 values of each of
// the four 32-element quarters of one 128-element half.
template <int R, int NB>
__device__ __forceinline__ void dot_q6k(const Planes& w, int row0, int rmax, const XRef<NB>& x, float (&acc)[R][NB], int it0, int step) {
    const int K = x.k, items = K >> 6;
    const uint8_t* lp[R];
    const uint8_t* hp[R];
    const uint8_t* sp[R];
    const uint8_t* dp[R];
#pragma unroll
    for (int r = 0; r < R; r++) {
        const int row = min(row0 + r, rmax);
        lp[r] = w.p[0] + (size_t)row * w.rb[0];
        hp[r] = w.p[1] + (size_t)row * w.rb[1];
        sp[r] = w.p[2] + (size_t)row * w.rb[2];
        dp[r] = w.p[3] + (size_t)row * w.rb[3];
    }
    const int8_t* xq[NB];
    const float2* xd[NB];
#pragma unroll
    for (int b = 0; b < NB; b++) {
        xq[b] = x.q + x.tok(b) * K;
        xd[b] = x.ds + x.tok(b) * (K >> 5);
    }
    for (int it = it0; it < items; it += step) {
        const int sb = it >> 2, n = (it >> 1) & 1, c = it & 1;
        uint4 a[R], bq[R], hq[R];
        uint2 s8[R];
        float d[R];
#pragma unroll
        for (int r = 0; r < R; r++) {
            const uint8_t* base = lp[r] + sb * 128 + 64 * n + 16 * c;
            a[r] = ldg16(base);
            bq[r] = ldg16(base + 32);
            hq[r] = ldg16(hp[r] + sb * 64 + 32 * n + 16 * c);
            s8[r] = __ldg((const uint2*)(sp[r] + sb * 16 + 8 * n));
            d[r] = __half2float(__ldg((const __half*)(dp[r] + sb * 2)));
        }
        const int xoff = sb * 256 + 128 * n + 16 * c;
        int4 xv[NB][4];
        float dx[NB][4];
#pragma unroll
        for (int b = 0; b < NB; b++)
#pragma unroll
            for (int qd = 0; qd < 4; qd++) {
                xv[b][qd] = *(const int4*)(xq[b] + xoff + 32 * qd);
                dx[b][qd] = xd[b][sb * 8 + 4 * n + qd].x;
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
            // scales of the four quarters: bytes c, c+2, c+4, c+6 of the 8-byte group
            const uint32_t lo = s8[r].x >> (8 * c), hi = s8[r].y >> (8 * c);
            const float sc0 = d[r] * (float)(int8_t)(lo & 0xff), sc1 = d[r] * (float)(int8_t)((lo >> 16) & 0xff);
            const float sc2 = d[r] * (float)(int8_t)(hi & 0xff), sc3 = d[r] * (float)(int8_t)((hi >> 16) & 0xff);
#pragma unroll
            for (int b = 0; b < NB; b++) {
                acc[r][b] += (sc0 * dx[b][0]) * (float)dot16(v[0], xv[b][0]) + (sc1 * dx[b][1]) * (float)dot16(v[1], xv[b][1])
                           + (sc2 * dx[b][2]) * (float)dot16(v[2], xv[b][2]) + (sc3 * dx[b][3]) * (float)dot16(v[3], xv[b][3]);
            }
        }
    }
}

// Q8_0: p0 = int8, p1 = half d per 32.  Item = one block.
template <int R, int NB>
__device__ __forceinline__ void dot_q8_0(const Planes& w, int row0, int rmax, const XRef<NB>& x, float (&acc)[R][NB], int it0, int step) {
    const int K = x.k, items = K >> 5;
    const uint8_t* qp[R];
    const uint8_t* dp[R];
#pragma unroll
    for (int r = 0; r < R; r++) {
        const int row = min(row0 + r, rmax);
        qp[r] = w.p[0] + (size_t)row * w.rb[0];
        dp[r] = w.p[1] + (size_t)row * w.rb[1];
    }
#pragma unroll 2
    for (int it = it0; it < items; it += step) {
        uint4 a[R], bq[R];
        float d[R];
#pragma unroll
        for (int r = 0; r < R; r++) {
            a[r] = ldg16(qp[r] + it * 32);
            bq[r] = ldg16(qp[r] + it * 32 + 16);
            d[r] = __half2float(__ldg((const __half*)(dp[r] + it * 2)));
        }
#pragma unroll
        for (int b = 0; b < NB; b++) {
            const int4* xp = (const int4*)(x.q + x.tok(b) * K + it * 32);
            const int4 x0 = xp[0], x1 = xp[1];
            const float dx = x.ds[x.tok(b) * items + it].x;
#pragma unroll
            for (int r = 0; r < R; r++) acc[r][b] += d[r] * dx * (float)(dot16(a[r], x0) + dot16(bq[r], x1));
        }
    }
}

// Q4_0: p0 = nibbles, p1 = half d per 32; values are q - 8
template <int R, int NB>
__device__ __forceinline__ void dot_q4_0(const Planes& w, int row0, int rmax, const XRef<NB>& x, float (&acc)[R][NB], int it0, int step) {
    const int K = x.k, items = K >> 5;
    const uint8_t* qp[R];
    const uint8_t* dp[R];
#pragma unroll
    for (int r = 0; r < R; r++) {
        const int row = min(row0 + r, rmax);
        qp[r] = w.p[0] + (size_t)row * w.rb[0];
        dp[r] = w.p[1] + (size_t)row * w.rb[1];
    }
#pragma unroll 2
    for (int it = it0; it < items; it += step) {
        uint4 q[R];
        float d[R];
#pragma unroll
        for (int r = 0; r < R; r++) {
            q[r] = ldg16(qp[r] + it * 16);
            d[r] = __half2float(__ldg((const __half*)(dp[r] + it * 2)));
        }
#pragma unroll
        for (int b = 0; b < NB; b++) {
            const int4* xp = (const int4*)(x.q + x.tok(b) * K + it * 32);
            const int4 x0 = xp[0], x1 = xp[1];
            const float2 ds = x.ds[x.tok(b) * items + it];
#pragma unroll
            for (int r = 0; r < R; r++) {
                uint4 lo, hi;
                NIB_LO(lo, q[r]);
                NIB_HI(hi, q[r]);
                acc[r][b] += d[r] * (ds.x * (float)(dot16(lo, x0) + dot16(hi, x1)) - 8.f * ds.y);
            }
        }
    }
}

// MXFP4: p0 = nibbles, p1 = e8m0 per 32.
// A 32-bit word of the nibble plane holds eight E2M1 codes, and a code is already a byte-permute selector: its three magnitude
// bits index a table of the eight magnitudes (times two, as int8), and its sign bit is the selector's "replicate the top bit"
// flag, which turns the looked-up byte into 0x00 because no magnitude has its top bit set.  So prmt(table, word) gives the
// magnitudes of the positive codes of four nibbles and zero for the negative ones, prmt(table, word ^ 0x8888) the reverse; the dot
// product is dp4a(positive part) - dp4a(negative part).  No selector is assembled and no byte is negated.  The four nibbles of a
// half word are the codes of columns (j, 16 + j, j + 1, 17 + j): the activation bytes are brought into that order once per block
// and token and shared by the rows a thread works on.
__device__ __forceinline__ int prmt_b32(uint32_t a, uint32_t b, uint32_t sel) {      // PTX prmt, default mode: selector bit 3 = replicate the byte's top bit
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return (int)d;
}

template <int R, int NB>
__device__ __forceinline__ void dot_mxfp4(const Planes& w, int row0, int rmax, const XRef<NB>& x, float (&acc)[R][NB], int it0, int step) {
    const int K = x.k, items = K >> 5;
    constexpr uint32_t MAG_LO = 0x03020100u, MAG_HI = 0x0c080604u;      // 2 x {0, 0.5, 1, 1.5} and 2 x {2, 3, 4, 6}
    const uint8_t* qp[R];
    const uint8_t* ep[R];
#pragma unroll
    for (int r = 0; r < R; r++) {
        const int row = min(row0 + r, rmax);
        qp[r] = w.p[0] + (size_t)row * w.rb[0];
        ep[r] = w.p[1] + (size_t)row * w.rb[1];
    }
#pragma unroll 2
    for (int it = it0; it < items; it += step) {
        uint4 q[R];
        float d[R];
#pragma unroll
        for (int r = 0; r < R; r++) {
            q[r] = ldg16(qp[r] + it * 16);
            d[r] = 0.5f * e8m0_to_float(__ldg(ep[r] + it));
        }
#pragma unroll
        for (int b = 0; b < NB; b++) {
            const int4* xp = (const int4*)(x.q + x.tok(b) * K + it * 32);
            const int4 xl = xp[0], xh = xp[1];
            const int xlo[4] = {xl.x, xl.y, xl.z, xl.w}, xhi[4] = {xh.x, xh.y, xh.z, xh.w};
            int xa[4], xb[4];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                xa[i] = (int)__byte_perm((uint32_t)xlo[i], (uint32_t)xhi[i], 0x5140);      // columns 4i, 16 + 4i, 4i + 1, 17 + 4i
                xb[i] = (int)__byte_perm((uint32_t)xlo[i], (uint32_t)xhi[i], 0x7362);      // columns 4i + 2, 18 + 4i, 4i + 3, 19 + 4i
            }
            const float dx = x.ds[x.tok(b) * items + it].x;
#pragma unroll
            for (int r = 0; r < R; r++) {
                const uint32_t qw[4] = {q[r].x, q[r].y, q[r].z, q[r].w};
                int sp = 0, sn = 0;
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const uint32_t lo = qw[i], hi = qw[i] >> 16;
                    sp = __dp4a(prmt_b32(MAG_LO, MAG_HI, lo), xa[i], sp);
                    sn = __dp4a(prmt_b32(MAG_LO, MAG_HI, lo ^ 0x8888u), xa[i], sn);
                    sp = __dp4a(prmt_b32(MAG_LO, MAG_HI, hi), xb[i], sp);
                    sn = __dp4a(prmt_b32(MAG_LO, MAG_HI, hi ^ 0x8888u), xb[i], sn);
                }
                acc[r][b] += d[r] * dx * (float)(sp - sn);
            }
        }
    }
}

// f32 / f16 / bf16 weights against fp32 activations
template <int R, int NB, int WT>
__device__ __forceinline__ void dot_float(const Planes& w, int row0, int rmax, const XRef<NB>& x, float (&acc)[R][NB], int it0, int step) {
    const int K = x.k;
    constexpr int EPI = (WT == WT_F32) ? 4 : 8;      // elements per 16-byte item
    const int items = K / EPI;
    const uint8_t* qp[R];
#pragma unroll
    for (int r = 0; r < R; r++) qp[r] = w.p[0] + (size_t)min(row0 + r, rmax) * w.rb[0];
#pragma unroll 2
    for (int it = it0; it < items; it += step) {
        uint4 q[R];
#pragma unroll
        for (int r = 0; r < R; r++) q[r] = ldg16(qp[r] + (size_t)it * 16);
        float xv[NB][EPI];
#pragma unroll
        for (int b = 0; b < NB; b++) {
            const float4* xp = (const float4*)(x.f + x.tok(b) * K + it * EPI);
#pragma unroll
            for (int i = 0; i < EPI / 4; i++) {
                const float4 t = xp[i];
                xv[b][4 * i] = t.x; xv[b][4 * i + 1] = t.y; xv[b][4 * i + 2] = t.z; xv[b][4 * i + 3] = t.w;
            }
        }
#pragma unroll
        for (int r = 0; r < R; r++) {
            const uint32_t* u = &q[r].x;
            float wv[EPI];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                if (WT == WT_F32) {
                    wv[i] = __uint_as_float(u[i]);
                } else if (WT == WT_BF16) {
                    wv[2 * i] = __uint_as_float(u[i] << 16);
                    wv[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
                } else {
                    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&u[i]));
                    wv[2 * i] = f.x;
                    wv[2 * i + 1] = f.y;
                }
            }
#pragma unroll
            for (int b = 0; b < NB; b++) {
                float t = 0.f;
#pragma unroll
                for (int i = 0; i < EPI; i++) t += wv[i] * xv[b][i];
                acc[r][b] += t;
            }
        }
    }
}

template <int R, int NB>
__device__ __forceinline__ void dot_any(int type, const Planes& w, int row0, int rmax, const XRef<NB>& x, float (&acc)[R][NB],
                                        int it0, int step) {
    switch (type) {
        case WT_Q4_K: dot_q4k<R, NB, false>(w, row0, rmax, x, acc, it0, step); break;
        case WT_Q5_K: dot_q4k<R, NB, true>(w, row0, rmax, x, acc, it0, step); break;
        case WT_Q6_K: dot_q6k<R, NB>(w, row0, rmax, x, acc, it0, step); break;
        case WT_Q8_0: dot_q8_0<R, NB>(w, row0, rmax, x, acc, it0, step); break;
        case WT_Q4_0: dot_q4_0<R, NB>(w, row0, rmax, x, acc, it0, step); break;
        case WT_MXFP4: dot_mxfp4<R, NB>(w, row0, rmax, x, acc, it0, step); break;
        case WT_BF16: dot_float<R, NB, WT_BF16>(w, row0, rmax, x, acc, it0, step); break;
        case WT_F16: dot_float<R, NB, WT_F16>(w, row0, rmax, x, acc, it0, step); break;
        default: dot_float<R, NB, WT_F32>(w, row0, rmax, x, acc, it0, step); break;
    }
}

// Items per row as the dot functions count them (used by the launcher to size the row-length split).
__host__ __device__ inline int items_per_row(int type, int k) {
    switch (type) {
        case WT_Q4_K: case WT_Q5_K: case WT_Q6_K: return k / 64;
        case WT_Q8_0: case WT_Q4_0: case WT_MXFP4: return k / 32;
        case WT_F32: return k / 4;
        default: return k / 8;
    }
}

// Row pitches (bytes) of the planes of a [n][k] weight of the given encoding; returns the plane count.
__host__ __device__ inline int plane_pitches(int type, int k, uint32_t rb[4]) {
    rb[0] = rb[1] = rb[2] = rb[3] = 0;
    switch (type) {
        case WT_F32: rb[0] = 4u * k; return 1;
        case WT_F16: case WT_BF16: rb[0] = 2u * k; return 1;
        case WT_Q8_0: rb[0] = k; rb[1] = k / 32 * 2; return 2;
        case WT_Q4_0: rb[0] = k / 2; rb[1] = k / 32 * 2; return 2;
        case WT_MXFP4: rb[0] = k / 2; rb[1] = k / 32; return 2;
        case WT_Q4_K: rb[0] = k / 2; rb[1] = k / 256 * 16; rb[2] = k / 256 * 4; return 3;
        case WT_Q5_K: rb[0] = k / 2; rb[1] = k / 256 * 16; rb[2] = k / 256 * 4; rb[3] = k / 8; return 4;
        case WT_Q6_K: rb[0] = k / 2; rb[1] = k / 4; rb[2] = k / 16; rb[3] = k / 256 * 2; return 4;
    }
    return 0;
}
