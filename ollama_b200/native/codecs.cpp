// GGML block codecs on the host: the work the reference hands to its external quantiser binary
// (server/quantization.go shells out to llama-quantize) and to ggml's CPU dequantisers at load time.
//
// Block layouts (sizes: fs/ggml/ggml.go:442-513):
//   Q8_0   half d | int8 q[32]
//   Q4_0   half d | u8 qs[16]            x[i] = d*((qs[i]&15)-8), x[i+16] = d*((qs[i]>>4)-8)
//   Q4_K   half d, half dmin | u8 scales[12] (8 x 6-bit scale, 8 x 6-bit min) | u8 qs[128]
//   Q5_K   half d, half dmin | u8 scales[12] | u8 qh[32] | u8 qs[128]
//   Q6_K   u8 ql[128] | u8 qh[64] | int8 scales[16] | half d
//   MXFP4  u8 e8m0 | u8 qs[16]           x = e2m1(q) * 2^(e-127), low nibbles = elements 0..15
//
// The quantisers make the same choices, in the same fp32 operation order, as the tensor-op codecs of
// ollama_b200/gguf/quants.py, so both produce identical bytes (compile with -ffp-contract=off).
// Blocks are independent; the entry points split them over hardware threads.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

#define B2H_API extern "C" __attribute__((visibility("default")))

namespace {

inline float half_to_float(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1f, man = h & 0x3ffu, bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {      // subnormal: renormalise
            exp = 127 - 15 + 1;
            while (!(man & 0x400u)) {
                man <<= 1;
                exp--;
            }
            bits = sign | (exp << 23) | ((man & 0x3ffu) << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7f800000u | (man << 13);
    } else {
        bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

inline uint16_t float_to_half(float f) {      // round to nearest even, overflow to infinity
    uint32_t x;
    memcpy(&x, &f, 4);
    const uint32_t sign = (x >> 16) & 0x8000u;
    x &= 0x7fffffffu;
    if (x >= 0x7f800000u) return (uint16_t)(sign | 0x7c00u | (x > 0x7f800000u ? 0x200u : 0));
    if (x >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u);               // rounds to >= 65520
    if (x < 0x38800000u) {                                                    // subnormal half (or zero)
        if (x < 0x33000000u) return (uint16_t)sign;                          // < 2^-25
        const int shift = 126 - (int)(x >> 23);                              // 14..24
        const uint32_t man = (x & 0x7fffffu) | 0x800000u;
        const uint32_t q = man >> shift, rem = man & ((1u << shift) - 1), half = 1u << (shift - 1);
        return (uint16_t)(sign | (q + ((rem > half || (rem == half && (q & 1))) ? 1 : 0)));
    }
    const uint32_t exp = (x >> 23) - 112, man = x & 0x7fffffu;
    uint32_t h = (exp << 10) | (man >> 13);
    const uint32_t rem = man & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (h & 1))) h++;
    return (uint16_t)(sign | h);
}

inline float round_half(float f) { return half_to_float(float_to_half(f)); }
inline uint16_t ld16(const uint8_t* p) { return (uint16_t)(p[0] | (p[1] << 8)); }
inline void st16(uint8_t* p, uint16_t v) {
    p[0] = (uint8_t)v;
    p[1] = (uint8_t)(v >> 8);
}
inline float rne(float x) { return nearbyintf(x); }
// NaN (a block that holds non-finite values) clamps to the lower bound, so that the integer conversions that follow are defined
inline float clampf(float x, float lo, float hi) { return x >= lo ? (x <= hi ? x : hi) : lo; }

template <class F>
void parallel_blocks(int64_t n, F f) {
    unsigned nt = std::thread::hardware_concurrency();
    if (nt == 0) nt = 1;
    nt = (unsigned)std::min<int64_t>(nt, std::max<int64_t>(1, n / 4096));
    if (nt <= 1) {
        f(0, n);
        return;
    }
    std::vector<std::thread> th;
    const int64_t per = (n + nt - 1) / nt;
    for (unsigned t = 0; t < nt; t++) {
        const int64_t lo = t * per, hi = std::min(n, lo + per);
        if (lo < hi) th.emplace_back([=] { f(lo, hi); });
    }
    for (auto& t : th) t.join();
}

// 6-bit scale/min table of Q4_K / Q5_K
inline void scale_min_k4(const uint8_t* s, int j, int& sc, int& m) {
    if (j < 4) {
        sc = s[j] & 63;
        m = s[j + 4] & 63;
    } else {
        sc = (s[j + 4] & 0xf) | ((s[j - 4] >> 6) << 4);
        m = (s[j + 4] >> 4) | ((s[j] >> 6) << 4);
    }
}

const float kMxfp4[16] = {0.f, 0.5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f, -0.f, -0.5f, -1.f, -1.5f, -2.f, -3.f, -4.f, -6.f};

// ---- dequantisers: one block -> block_size floats ---------------------------------------------------
void deq_q8_0(const uint8_t* b, float* y) {
    const float d = half_to_float(ld16(b));
    for (int i = 0; i < 32; i++) y[i] = d * (float)(int8_t)b[2 + i];
}
void deq_q4_0(const uint8_t* b, float* y) {
    const float d = half_to_float(ld16(b));
    for (int i = 0; i < 16; i++) {
        y[i] = d * (float)((int)(b[2 + i] & 15) - 8);
        y[i + 16] = d * (float)((int)(b[2 + i] >> 4) - 8);
    }
}
void deq_q4_k(const uint8_t* b, float* y) {
    const float d = half_to_float(ld16(b)), dmin = half_to_float(ld16(b + 2));
    const uint8_t* sc = b + 4;
    const uint8_t* qs = b + 16;
    for (int j = 0; j < 4; j++) {      // 64 elements: low nibbles then high nibbles of 32 bytes
        int s0, m0, s1, m1;
        scale_min_k4(sc, 2 * j, s0, m0);
        scale_min_k4(sc, 2 * j + 1, s1, m1);
        const float d0 = d * (float)s0, n0 = dmin * (float)m0, d1 = d * (float)s1, n1 = dmin * (float)m1;
        for (int l = 0; l < 32; l++) {
            y[64 * j + l] = d0 * (float)(qs[32 * j + l] & 15) - n0;
            y[64 * j + 32 + l] = d1 * (float)(qs[32 * j + l] >> 4) - n1;
        }
    }
}
void deq_q5_k(const uint8_t* b, float* y) {
    const float d = half_to_float(ld16(b)), dmin = half_to_float(ld16(b + 2));
    const uint8_t* sc = b + 4;
    const uint8_t* qh = b + 16;
    const uint8_t* qs = b + 48;
    for (int j = 0; j < 4; j++) {
        int s0, m0, s1, m1;
        scale_min_k4(sc, 2 * j, s0, m0);
        scale_min_k4(sc, 2 * j + 1, s1, m1);
        const float d0 = d * (float)s0, n0 = dmin * (float)m0, d1 = d * (float)s1, n1 = dmin * (float)m1;
        for (int l = 0; l < 32; l++) {
            const int lo = (qs[32 * j + l] & 15) | (((qh[l] >> (2 * j)) & 1) << 4);
            const int hi = (qs[32 * j + l] >> 4) | (((qh[l] >> (2 * j + 1)) & 1) << 4);
            y[64 * j + l] = d0 * (float)lo - n0;
            y[64 * j + 32 + l] = d1 * (float)hi - n1;
        }
    }
}
void deq_q6_k(const uint8_t* b, float* y) {
    const uint8_t* ql = b;
    const uint8_t* qh = b + 128;
    const int8_t* sc = (const int8_t*)(b + 192);
    const float d = half_to_float(ld16(b + 208));
    for (int h = 0; h < 2; h++) {      // 128 elements per half
        for (int l = 0; l < 32; l++) {
            const int is = l / 16;
            const int q1 = (int)((ql[64 * h + l] & 15) | (((qh[32 * h + l] >> 0) & 3) << 4)) - 32;
            const int q2 = (int)((ql[64 * h + l + 32] & 15) | (((qh[32 * h + l] >> 2) & 3) << 4)) - 32;
            const int q3 = (int)((ql[64 * h + l] >> 4) | (((qh[32 * h + l] >> 4) & 3) << 4)) - 32;
            const int q4 = (int)((ql[64 * h + l + 32] >> 4) | (((qh[32 * h + l] >> 6) & 3) << 4)) - 32;
            y[128 * h + l] = d * (float)sc[8 * h + is] * (float)q1;
            y[128 * h + l + 32] = d * (float)sc[8 * h + is + 2] * (float)q2;
            y[128 * h + l + 64] = d * (float)sc[8 * h + is + 4] * (float)q3;
            y[128 * h + l + 96] = d * (float)sc[8 * h + is + 6] * (float)q4;
        }
    }
}
void deq_mxfp4(const uint8_t* b, float* y) {
    const float s = ldexpf(1.0f, (int)b[0] - 127);
    for (int i = 0; i < 16; i++) {
        y[i] = kMxfp4[b[1 + i] & 15] * s;
        y[i + 16] = kMxfp4[b[1 + i] >> 4] * s;
    }
}

// ---- quantisers: block_size floats -> one block ----------------------------------------------------
void q_q8_0(const float* x, uint8_t* b) {
    float amax = 0.f;
    for (int i = 0; i < 32; i++) amax = std::max(amax, fabsf(x[i]));
    const float d = amax / 127.0f, inv = d > 0.f ? 1.0f / d : 0.f;
    st16(b, float_to_half(d));
    for (int i = 0; i < 32; i++) b[2 + i] = (uint8_t)(int8_t)clampf(rne(x[i] * inv), -127.f, 127.f);
}
void q_q4_0(const float* x, uint8_t* b) {
    float mx = 0.f, amax = -1.f;
    for (int i = 0; i < 32; i++)
        if (fabsf(x[i]) > amax) {      // first occurrence of the largest magnitude keeps its sign
            amax = fabsf(x[i]);
            mx = x[i];
        }
    const float d = mx / -8.0f, inv = d != 0.f ? 1.0f / d : 0.f;
    st16(b, float_to_half(d));
    uint8_t q[32];
    for (int i = 0; i < 32; i++) q[i] = (uint8_t)clampf(floorf(x[i] * inv + 8.5f), 0.f, 15.f);
    for (int i = 0; i < 16; i++) b[2 + i] = (uint8_t)(q[i] | (q[i + 16] << 4));
}
void q_q4_k(const float* x, uint8_t* b) {
    float scale[8], mins[8];
    float smax = 0.f, mmax = 0.f;
    for (int j = 0; j < 8; j++) {
        float mn = x[32 * j], mx = x[32 * j];
        for (int l = 1; l < 32; l++) {
            mn = std::min(mn, x[32 * j + l]);
            mx = std::max(mx, x[32 * j + l]);
        }
        mn = std::min(mn, 0.f);
        scale[j] = (mx - mn) / 15.0f;
        mins[j] = -mn;
        smax = j == 0 ? scale[j] : std::max(smax, scale[j]);
        mmax = j == 0 ? mins[j] : std::max(mmax, mins[j]);
    }
    const float d = round_half(smax / 63.0f), dmin = round_half(mmax / 63.0f);
    const float inv_d = d > 0.f ? 1.0f / d : 0.f, inv_dm = dmin > 0.f ? 1.0f / dmin : 0.f;
    int sc[8], m[8];
    uint8_t q[256];
    for (int j = 0; j < 8; j++) {
        const float scf = clampf(rne(scale[j] * inv_d), 0.f, 63.f), mf = clampf(rne(mins[j] * inv_dm), 0.f, 63.f);
        sc[j] = (int)scf;
        m[j] = (int)mf;
        const float eff = d * scf, inv_eff = eff > 0.f ? 1.0f / eff : 0.f, off = dmin * mf;
        for (int l = 0; l < 32; l++) q[32 * j + l] = (uint8_t)clampf(rne((x[32 * j + l] + off) * inv_eff), 0.f, 15.f);
    }
    st16(b, float_to_half(d));
    st16(b + 2, float_to_half(dmin));
    uint8_t* s = b + 4;
    for (int j = 0; j < 4; j++) {
        s[j] = (uint8_t)((sc[j] & 63) | ((sc[j + 4] >> 4) << 6));
        s[j + 4] = (uint8_t)((m[j] & 63) | ((m[j + 4] >> 4) << 6));
        s[j + 8] = (uint8_t)((sc[j + 4] & 15) | ((m[j + 4] & 15) << 4));
    }
    uint8_t* qs = b + 16;
    for (int j = 0; j < 4; j++)
        for (int l = 0; l < 32; l++) qs[32 * j + l] = (uint8_t)(q[64 * j + l] | (q[64 * j + 32 + l] << 4));
}
void q_q6_k(const float* x, uint8_t* b) {
    float s[16];
    float smax = 0.f, sabs = -1.f;
    for (int j = 0; j < 16; j++) {
        float mx = 0.f, amax = -1.f;
        for (int l = 0; l < 16; l++)
            if (fabsf(x[16 * j + l]) > amax) {
                amax = fabsf(x[16 * j + l]);
                mx = x[16 * j + l];
            }
        s[j] = mx / -32.0f;
        if (fabsf(s[j]) > sabs) {
            sabs = fabsf(s[j]);
            smax = s[j];
        }
    }
    const float d = round_half(smax / -128.0f), inv_d = d != 0.f ? 1.0f / d : 0.f;
    int q[256];
    int8_t sc[16];
    for (int j = 0; j < 16; j++) {
        const float scf = clampf(rne(s[j] * inv_d), -128.f, 127.f);
        sc[j] = (int8_t)scf;
        const float eff = d * scf, inv_eff = eff != 0.f ? 1.0f / eff : 0.f;
        for (int l = 0; l < 16; l++) q[16 * j + l] = (int)clampf(rne(x[16 * j + l] * inv_eff), -32.f, 31.f) + 32;
    }
    uint8_t* ql = b;
    uint8_t* qh = b + 128;
    for (int h = 0; h < 2; h++)
        for (int l = 0; l < 32; l++) {
            const int q1 = q[128 * h + l], q2 = q[128 * h + 32 + l], q3 = q[128 * h + 64 + l], q4 = q[128 * h + 96 + l];
            ql[64 * h + l] = (uint8_t)((q1 & 15) | ((q3 & 15) << 4));
            ql[64 * h + 32 + l] = (uint8_t)((q2 & 15) | ((q4 & 15) << 4));
            qh[32 * h + l] = (uint8_t)((q1 >> 4) | ((q2 >> 4) << 2) | ((q3 >> 4) << 4) | ((q4 >> 4) << 6));
        }
    memcpy(b + 192, sc, 16);
    st16(b + 208, float_to_half(d));
}

struct Codec {
    int type, block, bytes;
    void (*deq)(const uint8_t*, float*);
    void (*quant)(const float*, uint8_t*);
};
// ids are GGML type numbers (fs/ggml/ggml.go): Q4_0 2, Q8_0 8, Q4_K 12, Q5_K 13, Q6_K 14, MXFP4 39
const Codec kCodecs[] = {
    {2, 32, 18, deq_q4_0, q_q4_0},   {8, 32, 34, deq_q8_0, q_q8_0},   {12, 256, 144, deq_q4_k, q_q4_k},
    {13, 256, 176, deq_q5_k, nullptr}, {14, 256, 210, deq_q6_k, q_q6_k}, {39, 32, 17, deq_mxfp4, nullptr},
};
const Codec* find(int type) {
    for (const Codec& c : kCodecs)
        if (c.type == type) return &c;
    return nullptr;
}

}  // namespace

// 1 when this library decodes (what = 0) or encodes (what = 1) the GGML type.
B2H_API int b2h_codec_supported(int type, int what) {
    const Codec* c = find(type);
    return c && (what == 0 ? c->deq != nullptr : c->quant != nullptr);
}

// src: n_blocks blocks of `type`; dst: n_blocks * block_size floats.  Returns 0, or -1 for an unknown type.
B2H_API int b2h_dequantize(int type, const uint8_t* src, float* dst, int64_t n_blocks) {
    const Codec* c = find(type);
    if (!c || !c->deq || n_blocks < 0) return -1;
    parallel_blocks(n_blocks, [=](int64_t lo, int64_t hi) {
        for (int64_t i = lo; i < hi; i++) c->deq(src + i * c->bytes, dst + i * c->block);
    });
    return 0;
}

// src: n_blocks * block_size floats; dst: n_blocks blocks.  Returns 0, or -1 when the type has no encoder here.
B2H_API int b2h_quantize(int type, const float* src, uint8_t* dst, int64_t n_blocks) {
    const Codec* c = find(type);
    if (!c || !c->quant || n_blocks < 0) return -1;
    parallel_blocks(n_blocks, [=](int64_t lo, int64_t hi) {
        for (int64_t i = lo; i < hi; i++) c->quant(src + i * c->block, dst + i * c->bytes);
    });
    return 0;
}
