// Token sampling on the device: penalties -> top-k -> top-p -> min-p -> temperature -> draw.
//
// One CTA per sequence works on that sequence's row of logits (fp32 [vocab], left on the device by the LM-head
// GEMV), so the only bytes that cross to the host per step are the sampled ids.  The filter chain has the order
// of the reference's sampler chain (penalties, top-k, top-p, min-p, temperature, distribution draw; llama.cpp's
// common sampler as configured by llm/llama_server.go, and x/mlxrunner/sample/sample.go:822-871):
//   1. repetition / frequency / presence penalties on the ids of the recent-token window (in place),
//   2. the k largest logits by radix selection: four 8-bit passes over order-preserving keys find the k-th
//      largest key, then the candidates are gathered and sorted (bitonic, <= 256 entries) in shared memory,
//   3. nucleus cut on the softmax of the candidates at temperature 1 (a candidate stays while the mass before
//      it is below top_p), min-p cut relative to the best candidate,
//   4. softmax at the requested temperature and an inverse-CDF draw with a uniform number supplied by the
//      host's seeded generator (so that a seed reproduces the same tokens).
// The candidate list and its final probabilities can be written out for inspection / log-probabilities.
#include "common.cuh"

constexpr int SAMPLE_MAX_K = 256;
constexpr int SAMPLE_THREADS = 1024;

struct SampleRow {
    int n_hist;            // entries of the penalty list of this sequence
    int hist_off;          // offset into hist_ids / hist_counts
    float u;               // uniform draw in [0, 1)
};

struct SampleArgs {
    float* logits;         // [rows][ld] (penalties are applied in place)
    int ld, vocab;
    const SampleRow* rows; // [rows]
    const int* hist_ids;   // distinct recent token ids, all sequences back to back
    const int* hist_counts;
    float repeat_penalty, freq_penalty, presence_penalty;
    int top_k;             // 1..256
    float top_p, min_p, temperature;
    int* out_token;        // [rows]
    float* out_prob;       // [rows] probability of the drawn token (null: not wanted)
    int* cand_idx;         // [rows][256] or null
    float* cand_prob;      // [rows][256] or null
    int* cand_n;           // [rows] or null
};

namespace {

__device__ __forceinline__ uint32_t key_of(float v) {          // larger float <-> larger key; NaN sorts lowest
    if (v != v) return 0u;
    const uint32_t b = __float_as_uint(v);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__global__ void __launch_bounds__(SAMPLE_THREADS) sample_kernel(const __grid_constant__ SampleArgs a) {
    __shared__ unsigned hist[256];
    __shared__ unsigned s_prefix, s_need, s_count, s_ties;
    __shared__ float cv[SAMPLE_MAX_K];
    __shared__ int ci[SAMPLE_MAX_K];
    __shared__ int tie_idx[32];
    const int tid = threadIdx.x, row = blockIdx.x;
    float* lg = a.logits + (size_t)row * a.ld;
    const SampleRow r = a.rows[row];

    // 1. penalties
    for (int i = tid; i < r.n_hist; i += SAMPLE_THREADS) {
        const int id = a.hist_ids[r.hist_off + i];
        if (id < 0 || id >= a.vocab) continue;
        float v = lg[id];
        if (a.repeat_penalty != 1.f) v = v <= 0.f ? v * a.repeat_penalty : v / a.repeat_penalty;
        v -= (float)a.hist_counts[r.hist_off + i] * a.freq_penalty + a.presence_penalty;
        lg[id] = v;
    }
    __syncthreads();

    // 2. radix select: the key of the k-th largest logit, 8 bits at a time from the top
    const int k = min(a.top_k, a.vocab);
    if (tid == 0) { s_prefix = 0u; s_need = (unsigned)k; }
    for (int pass = 0; pass < 4; pass++) {
        const int shift = 24 - 8 * pass;
        if (tid < 256) hist[tid] = 0u;
        __syncthreads();
        const unsigned prefix = s_prefix;
        const unsigned mask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
        for (int i = tid; i < a.vocab; i += SAMPLE_THREADS) {
            const uint32_t key = key_of(lg[i]);
            if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 0xffu], 1u);
        }
        __syncthreads();
        if (tid == 0) {
            unsigned need = s_need, b = 255;
            for (;; b--) {                       // walk the buckets from the largest digit down
                if (hist[b] >= need || b == 0) break;
                need -= hist[b];
            }
            s_need = need;
            s_prefix = prefix | (b << shift);
        }
        __syncthreads();
    }
    const uint32_t kth = s_prefix;               // exactly the k-th largest key; s_need of the entries equal to it are wanted
    const unsigned ties_wanted = s_need;
    if (tid == 0) s_count = 0u;
    if (tid < SAMPLE_MAX_K) { cv[tid] = -INFINITY; ci[tid] = 0x7fffffff; }
    __syncthreads();
    if (tid == 0) s_ties = 0u;
    __syncthreads();
    for (int i = tid; i < a.vocab; i += SAMPLE_THREADS) {
        const float v = lg[i];
        const uint32_t key = key_of(v);
        if (key > kth) {
            const unsigned p = atomicAdd(&s_count, 1u);
            if (p < SAMPLE_MAX_K) { cv[p] = v; ci[p] = i; }
        } else if (key == kth) {
            const unsigned p = atomicAdd(&s_ties, 1u);
            if (p < 32) tie_idx[p] = i;
        }
    }
    __syncthreads();
    const unsigned n_above = min(s_count, (unsigned)SAMPLE_MAX_K);
    const unsigned n_ties = s_ties;
    if (n_ties <= 32) {
        // the usual case (a handful of equal logits at the threshold): take the lowest ids among them
        if (tid == 0) {
            for (unsigned x = 1; x < n_ties; x++) {           // insertion sort of at most 32 ids
                const int v = tie_idx[x];
                int y = (int)x - 1;
                for (; y >= 0 && tie_idx[y] > v; y--) tie_idx[y + 1] = tie_idx[y];
                tie_idx[y + 1] = v;
            }
            for (unsigned x = 0; x < ties_wanted && x < n_ties && n_above + x < SAMPLE_MAX_K; x++) {
                cv[n_above + x] = lg[tie_idx[x]];
                ci[n_above + x] = tie_idx[x];
            }
        }
    } else if (tid < 32) {
        // many equal logits at the threshold (e.g. masked rows): ordered scan, lowest ids first
        unsigned taken = 0;
        for (int base = 0; base < a.vocab && taken < ties_wanted; base += 32) {
            const int i = base + tid;
            const bool hit = i < a.vocab && key_of(lg[i]) == kth;
            const unsigned m = __ballot_sync(0xffffffffu, hit);
            const unsigned before = __popc(m & ((1u << tid) - 1u));
            if (hit && taken + before < ties_wanted && n_above + taken + before < SAMPLE_MAX_K) {
                cv[n_above + taken + before] = lg[i];
                ci[n_above + taken + before] = i;
            }
            taken += __popc(m);
        }
    }
    __syncthreads();
    const int n = min(k, SAMPLE_MAX_K);

    // sort the candidates: value descending, id ascending among equals (bitonic over 256 slots, padded with -inf)
    for (int size = 2; size <= SAMPLE_MAX_K; size <<= 1) {
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            if (tid < SAMPLE_MAX_K) {
                const int j = tid ^ stride;
                if (j > tid) {
                    const bool up = (tid & size) == 0;
                    const float v0 = cv[tid], v1 = cv[j];
                    const int i0 = ci[tid], i1 = ci[j];
                    const bool first_after = v0 < v1 || (v0 == v1 && i0 > i1);      // element tid belongs after element j
                    if (first_after == up) { cv[tid] = v1; cv[j] = v0; ci[tid] = i1; ci[j] = i0; }
                }
            }
            __syncthreads();
        }
    }

    // 3./4. filters and draw: warp 0, candidates strided over its lanes
    if (tid < 32) {
        const float vmax = cv[0];
        float e[SAMPLE_MAX_K / 32];
        float sum = 0.f;
#pragma unroll
        for (int j = 0; j < SAMPLE_MAX_K / 32; j++) {
            const int c = j * 32 + tid;
            e[j] = c < n ? __expf(cv[c] - vmax) : 0.f;
            sum += e[j];
        }
        sum = warp_sum(sum);
        int keep = n;
        if (a.top_p > 0.f && a.top_p < 1.f) {        // keep candidate c while the mass of candidates before it is below top_p
            float run = 0.f;                         // mass before block j
            int cut = n;
#pragma unroll
            for (int j = 0; j < SAMPLE_MAX_K / 32; j++) {
                float incl = e[j];                   // inclusive scan inside the block of 32
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const float t = __shfl_up_sync(0xffffffffu, incl, o);
                    if (tid >= o) incl += t;
                }
                const float before = (run + incl - e[j]) / sum;
                const int c = j * 32 + tid;
                const bool drop = c < n && c > 0 && before >= a.top_p;
                const unsigned m = __ballot_sync(0xffffffffu, drop);
                if (m && cut == n) cut = j * 32 + __ffs(m) - 1;
                run += __shfl_sync(0xffffffffu, incl, 31);
            }
            keep = min(keep, cut);
        }
        if (a.min_p > 0.f) {                          // relative to the best candidate (e = 1 there); the ratio is scale-free
            int cut = keep;
#pragma unroll
            for (int j = 0; j < SAMPLE_MAX_K / 32; j++) {
                const int c = j * 32 + tid;
                const bool drop = c < keep && c > 0 && e[j] < a.min_p;
                const unsigned m = __ballot_sync(0xffffffffu, drop);
                if (m && cut == keep) cut = j * 32 + __ffs(m) - 1;
            }
            keep = cut;
        }
        keep = max(keep, 1);
        const float it = 1.f / fmaxf(a.temperature, 1e-6f);
        float tsum = 0.f;
#pragma unroll
        for (int j = 0; j < SAMPLE_MAX_K / 32; j++) {
            const int c = j * 32 + tid;
            e[j] = c < keep ? __expf((cv[c] - vmax) * it) : 0.f;
            tsum += e[j];
        }
        tsum = warp_sum(tsum);
        // inverse CDF
        const float target = r.u * tsum;
        float run = 0.f;
        int chosen = keep - 1;
        bool found = false;
#pragma unroll
        for (int j = 0; j < SAMPLE_MAX_K / 32; j++) {
            float incl = e[j];
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const float t = __shfl_up_sync(0xffffffffu, incl, o);
                if (tid >= o) incl += t;
            }
            const int c = j * 32 + tid;
            const unsigned m = __ballot_sync(0xffffffffu, c < keep && run + incl > target);
            if (m && !found) { chosen = j * 32 + __ffs(m) - 1; found = true; }
            run += __shfl_sync(0xffffffffu, incl, 31);
        }
        if (tid == 0) {
            a.out_token[row] = ci[chosen];
            if (a.cand_n) a.cand_n[row] = keep;
        }
#pragma unroll
        for (int j = 0; j < SAMPLE_MAX_K / 32; j++) {
            const int c = j * 32 + tid;
            if (c == chosen && a.out_prob) a.out_prob[row] = e[j] / tsum;
            if (a.cand_idx) a.cand_idx[(size_t)row * SAMPLE_MAX_K + c] = c < keep ? ci[c] : -1;
            if (a.cand_prob) a.cand_prob[(size_t)row * SAMPLE_MAX_K + c] = c < keep ? e[j] / tsum : 0.f;
        }
    }
}

}  // namespace

// top_k must be in 1..256 (larger candidate sets take the host path).  Returns a cudaError_t value.
B2_API int b2_sample(const SampleArgs* a, int rows, cudaStream_t st) {
    if (rows < 1 || a->top_k < 1 || a->top_k > SAMPLE_MAX_K || a->vocab < 1 || a->ld < a->vocab) return (int)cudaErrorInvalidValue;
    SampleArgs copy = *a;
    sample_kernel<<<rows, SAMPLE_THREADS, 0, st>>>(copy);
    return (int)cudaGetLastError();
}
