// Stand-alone exerciser of the host helpers, meant to be built with -fsanitize=address,undefined (see sanitize.py):
// every codec decodes random bytes (any bit pattern is a legal block) and round-trips random floats including the
// extremes (zeros, infinities, NaN, denormals, huge values); the BPE merge loop runs random words against a random merge
// table, including empty words and merges that refer to ids outside the table.  Output buffers are allocated at their
// exact size, so that a write past the end is caught.  Exit code 0 = clean.
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <limits>
#include <random>
#include <vector>

extern "C" {
int b2h_codec_supported(int type, int what);
int b2h_dequantize(int type, const uint8_t* src, float* dst, int64_t n_blocks);
int b2h_quantize(int type, const float* src, uint8_t* dst, int64_t n_blocks);
void* b2h_bpe_new(const int32_t* triples, int32_t n_merges);
void b2h_bpe_free(void* h);
int b2h_bpe_encode(const void* h, const int32_t* syms, const int64_t* word_off, int32_t n_words, int32_t* out, int64_t* out_off);
}

namespace {
struct Shape {
    int type, block, bytes;
};
const Shape kShapes[] = {{2, 32, 18}, {8, 32, 34}, {12, 256, 144}, {13, 256, 176}, {14, 256, 210}, {39, 32, 17}};

int fail(const char* what, int type) {
    std::fprintf(stderr, "selftest: %s (type %d)\n", what, type);
    return 1;
}
}  // namespace

int main() {
    std::mt19937_64 rng(20240611);
    const float specials[] = {0.0f, -0.0f, 1.0f, -1.0f, 65504.0f, 1e30f, -1e30f, 1e-30f, std::numeric_limits<float>::denorm_min(),
                              std::numeric_limits<float>::infinity(), -std::numeric_limits<float>::infinity(), std::nanf("")};
    for (const Shape& s : kShapes) {
        if (!b2h_codec_supported(s.type, 0)) return fail("decoder missing", s.type);
        for (int64_t n : {int64_t(0), int64_t(1), int64_t(3), int64_t(257)}) {
            std::vector<uint8_t> blocks((size_t)n * s.bytes);
            for (auto& b : blocks) b = (uint8_t)rng();
            std::vector<float> out((size_t)n * s.block);
            if (b2h_dequantize(s.type, blocks.data(), out.data(), n)) return fail("decode refused", s.type);
            if (!b2h_codec_supported(s.type, 1)) continue;
            std::vector<float> in((size_t)n * s.block);
            std::normal_distribution<float> g(0.0f, 3.0f);
            for (size_t i = 0; i < in.size(); i++) in[i] = (rng() % 17 == 0) ? specials[rng() % (sizeof(specials) / sizeof(float))] : g(rng);
            std::vector<uint8_t> enc((size_t)n * s.bytes);
            if (b2h_quantize(s.type, in.data(), enc.data(), n)) return fail("encode refused", s.type);
            if (b2h_dequantize(s.type, enc.data(), out.data(), n)) return fail("decode of own blocks refused", s.type);
            // a block of ordinary values must come back close to what went in
            std::vector<float> plain((size_t)s.block), back((size_t)s.block);
            std::vector<uint8_t> one((size_t)s.bytes);
            for (auto& v : plain) v = g(rng);
            b2h_quantize(s.type, plain.data(), one.data(), 1);
            b2h_dequantize(s.type, one.data(), back.data(), 1);
            double err = 0, ref = 0;
            for (int i = 0; i < s.block; i++) err += (back[i] - plain[i]) * (back[i] - plain[i]), ref += plain[i] * plain[i];
            if (!(err <= 0.02 * ref)) return fail("round trip too far off", s.type);
        }
        if (b2h_dequantize(s.type, nullptr, nullptr, -1) != -1) return fail("negative count accepted", s.type);
    }
    if (b2h_codec_supported(9999, 0) || b2h_dequantize(9999, nullptr, nullptr, 0) != -1) return fail("unknown type accepted", 9999);

    for (int round = 0; round < 50; round++) {
        const int n_merges = (int)(rng() % 200);
        std::vector<int32_t> triples((size_t)n_merges * 3);
        for (int i = 0; i < n_merges; i++) {
            triples[3 * i] = (int32_t)(rng() % 64);
            triples[3 * i + 1] = (int32_t)(rng() % 64);
            triples[3 * i + 2] = (int32_t)(rng() % 100000) - 10;      // merged ids are opaque to the loop, odd ones included
        }
        void* h = b2h_bpe_new(triples.data(), n_merges);
        const int n_words = (int)(rng() % 20);
        std::vector<int64_t> off(n_words + 1, 0);
        std::vector<int32_t> syms;
        for (int w = 0; w < n_words; w++) {
            const int len = (int)(rng() % 40);                        // empty words too
            for (int i = 0; i < len; i++) syms.push_back((int32_t)(rng() % 64));
            off[w + 1] = (int64_t)syms.size();
        }
        std::vector<int32_t> out(syms.size());
        std::vector<int64_t> out_off(n_words + 1);
        if (b2h_bpe_encode(h, syms.data(), off.data(), n_words, out.data(), out_off.data())) return fail("bpe refused", round);
        for (int w = 0; w < n_words; w++)
            if (out_off[w + 1] - out_off[w] > off[w + 1] - off[w] || out_off[w + 1] < out_off[w]) return fail("bpe grew a word", round);
        b2h_bpe_free(h);
    }
    if (b2h_bpe_encode(nullptr, nullptr, nullptr, 0, nullptr, nullptr) != -1) return fail("null table accepted", 0);
    std::puts("selftest: ok");
    return 0;
}
