// Byte-pair merge loop of the BPE tokenizer on the host.  In the reference stack tokenisation happens inside the
// llama.cpp server (llm/llama_server.go:257-277 only forwards text); here the regex pre-tokeniser stays in Python and
// the merges of all words of a prompt run in one call.
//
// A merge table is a list of (left id, right id, merged id) in rank order.  A word arrives as the ids of its
// initial symbols (one per byte of the UTF-8 text after the GPT-2 byte-to-unicode map).  Each round takes the
// adjacent pair of lowest rank and merges all of its occurrences from left to right, which is the order the
// Python implementation (ollama_b200/text/tokenizer.py) uses, so both give the same ids.
#include <cstdint>
#include <unordered_map>
#include <vector>

#define B2H_API extern "C" __attribute__((visibility("default")))

namespace {
struct Merge {
    int32_t rank, merged;
};
struct BpeTable {
    std::unordered_map<uint64_t, Merge> pairs;
};
inline uint64_t key(int32_t a, int32_t b) { return ((uint64_t)(uint32_t)a << 32) | (uint32_t)b; }
}  // namespace

// triples: n_merges x {left, right, merged}.  Later duplicates of a pair are ignored (the first one has the lower rank).
B2H_API void* b2h_bpe_new(const int32_t* triples, int32_t n_merges) {
    auto* t = new BpeTable();
    t->pairs.reserve((size_t)n_merges * 2);
    for (int32_t i = 0; i < n_merges; i++)
        t->pairs.emplace(key(triples[3 * i], triples[3 * i + 1]), Merge{i, triples[3 * i + 2]});
    return t;
}

B2H_API void b2h_bpe_free(void* h) { delete static_cast<BpeTable*>(h); }

// syms: concatenated initial symbol ids of n_words words; word_off[n_words + 1] delimits them.
// out receives the merged ids of every word back to back (never more than the input), out_off[n_words + 1] their bounds.
B2H_API int b2h_bpe_encode(const void* h, const int32_t* syms, const int64_t* word_off, int32_t n_words, int32_t* out, int64_t* out_off) {
    if (!h || n_words < 0) return -1;
    const BpeTable& t = *static_cast<const BpeTable*>(h);
    std::vector<int32_t> cur, nxt;
    int64_t o = 0;
    out_off[0] = 0;
    for (int32_t w = 0; w < n_words; w++) {
        cur.assign(syms + word_off[w], syms + word_off[w + 1]);
        while (cur.size() > 1) {
            int32_t best = INT32_MAX, merged = -1, a = 0, b = 0;
            for (size_t i = 0; i + 1 < cur.size(); i++) {
                auto it = t.pairs.find(key(cur[i], cur[i + 1]));
                if (it != t.pairs.end() && it->second.rank < best) {
                    best = it->second.rank;
                    merged = it->second.merged;
                    a = cur[i];
                    b = cur[i + 1];
                }
            }
            if (merged < 0) break;
            nxt.clear();
            for (size_t i = 0; i < cur.size();) {
                if (i + 1 < cur.size() && cur[i] == a && cur[i + 1] == b) {
                    nxt.push_back(merged);
                    i += 2;
                } else {
                    nxt.push_back(cur[i]);
                    i += 1;
                }
            }
            cur.swap(nxt);
        }
        for (int32_t id : cur) out[o++] = id;
        out_off[w + 1] = o;
    }
    return 0;
}
