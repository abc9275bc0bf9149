// Streaming quantised matrix-vector kernel for decode steps of 1..32 tokens, sm_100a.
//
// In the reference stack this is ggml's mmvq family (one launch per matrix, dp4a dot products).  Here a
// decode matrix is a linear byte stream of which every SM pulls its share at HBM speed:
//
//   * Weights are re-laid out at load time into "units": 16 rows x 256 columns (one K-quant super-block of
//     each of 16 rows), stored in exactly the order the lanes of a warp load their tensor-core A fragments,
//     followed by the 16 rows' scales.  Units of one 16-row tile are contiguous, tiles follow each other, so
//     any range of units is one contiguous byte range (Q6_K: 3360 B per unit, the GGUF size; Q4_K: 2368 B, 64 more than
//     GGUF because the packed 6-bit scale table is stored as bytes).
//   * The launch is persistent and split by warp: warp w of the W warps of the grid owns units [w U / W, (w + 1) U / W)
//     of the launch's U units, whatever matrix rows they belong to (stream-K), so every warp of every SM streams
//     the same number of bytes for every matrix shape, from one contiguous range.  A unit is requested with six to
//     eight streaming 16-byte loads per lane (each warp instruction covers 512 contiguous bytes) straight into
//     registers; the registers of a chunk are re-requested for the next unit as soon as the chunk has been used,
//     so every warp keeps about one unit in flight and an SM with 16 to 24 warps 40 to 80 KB.  The first unit is
//     requested before the grid-dependency wait, because weights do not depend on the previous kernel.
//     (A shared-memory ring filled by cp.async.bulk from one producer warp measured 0.63 of the copy bandwidth on
//     the LM head at one CTA per SM, whatever the ring depth or the arithmetic; CTA-wide reductions after every
//     16-row tile spent a third of the issue slots in barrier stalls.)
//   * One token: dp4a on the unit layout, the four lanes that share a row are added with two shuffles.  Two to 32
//     tokens: the codes become int8 A fragments with two logic ops per register, the activations (int8, one scale
//     per 256-block of a token) are the B fragments, mma.sync m16n8k32 / m16n8k16 produces the per-sub-block integer
//     sums, and the 6-bit sub-block scales are applied with integer multiply-adds.  Q4_K minima are one extra
//     MMA per sub-block whose A fragment is the replicated minimum (one token: block sums from the quantiser).
//   * A warp that has all 16 units of a 16-row tile finishes the rows from its registers: store, add to the residual
//     stream, gated activation of interleaved gate/up rows, or (value, epoch) stores to the peers of a
//     tensor-parallel group.  A tile that is split between warps is finished by the warp that holds its first unit;
//     the others hand their partial sums over through a small workspace and a flag (bounded wait, fixed
//     summation order).  A warp meets a split tile first (it computes it at the start of its range), so the warp
//     that finishes a tile at the end of its own range finds the partial sums waiting.
//   * The activations are quantised by the CTA itself while its first units are in flight: the kernel
//     reads the fp32 rows (optionally RMS-normalising them first), so a decode layer needs no separate
//     norm / quantise launch.  Inputs too large for shared memory come pre-quantised from b2_quant256.
#include "comm.cuh"

constexpr int SK_WARPS = 8;
constexpr int SK_THREADS = SK_WARPS * 32;
constexpr int SK_UNIT_Q4K = 2368;       // 2048 nibble bytes + 16 x (8 scales + 8 minima) + 16 x (half d, half dmin)
constexpr int SK_UNIT_Q6K = 3360;       // 3072 code bytes + 16 x 16 int8 scales + 16 x half d
constexpr int SK_WS_FLOATS = 16 * 32;   // workspace floats per warp (16 rows x up to 32 tokens)

struct SkSeg {
    const uint8_t* w;     // units of this matrix: [n / 16][k / 256][unit bytes]
    const float* bias;    // [n] or null
    int type;             // WT_Q4_K or WT_Q6_K
    int n;                // rows (multiple of 16)
    int out_off;          // column of row 0 in the output row
    int unit0;            // index of the first unit of this matrix in the launch
};

struct SkArgs {
    SkSeg seg[4];
    int nseg;
    int k;                // row length (multiple of 256)
    int nb;               // tokens, 1..32
    int total_units;
    // input, one of: fp32 rows that the kernel normalises / quantises itself, or int8 + scales from b2_quant256
    const float* x;       // [nb][ldx] or null
    int ldx;
    const float* norm_w;  // RMSNorm weight [k], or null: quantise x as it is
    float eps;
    const int8_t* xq;     // [nb][k]; one token: in the one-token word order of b2_quant256
    const float* xd;      // [nb][k / 256]
    const int16_t* xbs;   // [nb][k / 32] sums of the int8 values of every 32-block (used by the one-token path for Q4_K minima)
    // output
    int mode;             // 0: out = y, 1: out += y, 2: out[b][i] = act(y[2i], y[2i+1]) (interleaved gate/up rows)
    float* out;
    int ldo;
    int act;
    float alpha, limit;
    // split tiles
    float* ws;            // [groups][SK_WS_FLOATS]
    unsigned* flags;      // [groups], zero between launches
    int* status;          // KStatus, written when a bounded wait gives up
    // shared memory offsets and work split (filled in by the launcher)
    int off_red, off_xq, off_xd, off_xbs, off_ring;
    int ring, slot_bytes; // units per warp ring (2..4) and bytes per slot
    int wpt_log2;         // warps of a CTA that share one range of units: 1 << wpt_log2
    int n_groups;         // ranges the launch's units are divided into
    CommSend cm;          // cm.n_dst > 0: the result goes to every rank of the group as (value, epoch) pairs (pitch ldo)
};

constexpr int SK_MAX_PHASES = 4;
constexpr int SK_MAX_DYN_SMEM = 224 * 1024;     // 227 KB per CTA less the kernel's static shared memory (the argument copy)

// Several products in one launch, each reading what the one before it wrote (attention output -> FFN -> next layer's
// Q/K/V, say).  All CTAs of the launch are resident at once; between two phases they meet at a barrier in global memory,
// and every warp's ring keeps requesting weights across that barrier, so the memory stream does not stop while the
// CTAs exchange the few kilobytes of activations.
struct SkChain {
    SkArgs ph[SK_MAX_PHASES];
    int n;
    unsigned* bar;        // two counters (arrivals, exits), zero between launches; unused when n == 1
    int tune;             // experiments: bits 0-1 = units per warp requested before the inputs are read (0: ring - 1), bit 2 = no requests across a phase end
    unsigned long long* trace;   // optional: [grid][16] nanosecond time stamps of thread 0 (launch, inputs ready, per phase: quantised, done)
};

struct Quant256Args {
    const float* x;       // [nb][ldx]
    int ldx;
    const float* norm_w;  // or null
    float eps;
    int k;
    int8_t* xq;           // [nb][k]
    float* xd;            // [nb][k / 256]
    int16_t* xbs;         // [nb][k / 32]
    int perm;             // 1: the one-token word order inside every 256-block (the input of a one-token b2_gemv_sk)
};

namespace {

constexpr unsigned long long SK_WAIT_NS = 1000000000ull;      // a wait on another warp gives up after a second of wall clock

__device__ __forceinline__ void mma_u8s8_k32(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_s8s8_k16(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a0), "r"(a1), "r"(b0));
}
__device__ __forceinline__ int dp4a_us(uint32_t w, uint32_t x, int c) {      // unsigned weights x signed activations
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(w), "r"(x), "r"(c));
    return d;
}
__device__ __forceinline__ int dp4a_ss(uint32_t w, uint32_t x, int c) {
    int d;
    asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(w), "r"(x), "r"(c));
    return d;
}
// two signed 16-bit values of `a` times bytes 0 and 1 (unsigned) of `b`
__device__ __forceinline__ int dp2a_lo_su(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp2a.lo.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ unsigned ld_acquire_gpu_u32(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_gpu_u32(unsigned* p, unsigned v) {
    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int unit_bytes(int type) { return type == WT_Q6_K ? SK_UNIT_Q6K : SK_UNIT_Q4K; }

// byte `b` of `w` zero-extended / replicated into all four bytes / sign-extended (b is a compile-time constant after unrolling)
__device__ __forceinline__ int byte_u(uint32_t w, int b) { return (int)__byte_perm(w, 0, 0x4440 | b); }
__device__ __forceinline__ uint32_t byte_rep(uint32_t w, int b) { return __byte_perm(w, 0, b * 0x1111); }
__device__ __forceinline__ int byte_s(uint32_t w, int b) {
    int d;      // selector nibbles 1..3 carry the replicate-sign bit
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(w), "r"(0u), "r"((uint32_t)(0x8880 | b | (b << 4) | (b << 8) | (b << 12))));
    return d;
}

// A warp's private ring of units in shared memory, filled with cp.async (16 bytes per lane and instruction, no register
// destination, so the bytes in flight do not cost registers).  A lane copies pieces lane, lane + 32, ... of the unit; its own
// code chunks are exactly the pieces it copied, the scales behind them were copied by other lanes of the warp.
// Weights pass through L2 once: they are marked evict-first so that gigabytes of them per token do not push the activations,
// the norm weights and the kernel's own code out of L2 (without the hint every phase start paid HBM latency several times).
__device__ __forceinline__ uint64_t stream_policy() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ void cp_async16(void* dst_smem, const void* src, uint64_t policy) {
    asm volatile("cp.async.cg.shared.global.L2::cache_hint [%0], [%1], 16, %2;" ::"r"((uint32_t)__cvta_generic_to_shared(dst_smem)), "l"(src),
                 "l"(policy) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// The units of one warp in the order it meets them, across the phases of a launch: inside every tile segment of its group's
// range the 2^l2 warps of the group take equal contiguous runs.
struct Walker {
    const uint8_t* p;     // the unit's bytes
    int u, ub;            // unit index, end of the warp's run in the current segment
    int seg_end;          // end of the current segment
    int type;
    bool valid;
    int ph;               // phase the unit belongs to, and that phase's split as seen by this warp:
    int l2, wi, ghi, kts;
};

// Activation operand: int8 [token][k] read as words, one scale per (token, 256-block), int16 sums of the 32-blocks.
struct XOp {
    const uint32_t* q;    // shared or global
    const float* d;
    const uint32_t* bs;   // pairs of int16 block sums
    int kw;               // words per token row
    int nkb;              // 256-blocks per token
    int nb;
};

// ---------------------------------------------------------------------------------------------------------------------
// One token.  The tensor-core tiles would idle seven of their eight columns, and the legacy integer MMA path of this GPU
// runs at about the rate of dp4a anyway, so a single token uses dp4a on the same unit layout.  Lane (g, t) holds, for rows
// g and g + 8, the codes of columns 4 t .. 4 t + 3 and 16 + 4 t .. of every sub-block; the four t lanes of a row are added
// at the end.  The quantiser stores the activations of one token so that the 16 words of a lane are contiguous.
//
// Q4_K unit bytes: [pair p of sub-blocks][lane][4 words]: word i of lane (g, t) holds, for row g + 8 (i & 1), the four GGUF
// nibble bytes 32 p + 16 (i >> 1) + 4 t .. + 3 (low nibbles = sub-block 2p, high nibbles = sub-block 2p + 1); then per row
// 8 scales + 8 minima; then per row (d, dmin).
// ---------------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ void unit_q4k_one(const uint8_t* sp, int lane, const XOp& x, int kt, float& vg_out, float& vh_out) {
    const int g = lane >> 2, t = lane & 3;
    const uint4* q = reinterpret_cast<const uint4*>(sp);
    const uint4* xw4 = reinterpret_cast<const uint4*>(x.q + kt * 64 + t * 16);      // this lane's 16 activation words, contiguous
    const uint4 sg = reinterpret_cast<const uint4*>(sp + 2048)[g], sh = reinterpret_cast<const uint4*>(sp + 2048)[g + 8];
    int lo_g = 0, hi_g = 0, lo_h = 0, hi_h = 0;
#pragma unroll
    for (int p = 0; p < 4; p++) {
        const uint4 w = q[p * 32 + lane], xv = xw4[p];
        const int a_g = dp4a_us(w.z & 0x0f0f0f0fu, xv.y, dp4a_us(w.x & 0x0f0f0f0fu, xv.x, 0));
        const int b_g = dp4a_us(w.z & 0xf0f0f0f0u, xv.w, dp4a_us(w.x & 0xf0f0f0f0u, xv.z, 0));
        const int a_h = dp4a_us(w.w & 0x0f0f0f0fu, xv.y, dp4a_us(w.y & 0x0f0f0f0fu, xv.x, 0));
        const int b_h = dp4a_us(w.w & 0xf0f0f0f0u, xv.w, dp4a_us(w.y & 0xf0f0f0f0u, xv.z, 0));
        const uint32_t scg = p < 2 ? sg.x : sg.y, sch = p < 2 ? sh.x : sh.y;
        const int bl = (2 * p) & 3, bh = bl + 1;
        lo_g += byte_u(scg, bl) * a_g;
        hi_g += byte_u(scg, bh) * b_g;
        lo_h += byte_u(sch, bl) * a_h;
        hi_h += byte_u(sch, bh) * b_h;
    }
    // minima of sub-blocks 2 t and 2 t + 1 (whole 32-element sums), one pair per t lane
    const uint32_t bs = x.bs[kt * 4 + t];
    uint32_t mg = t < 2 ? sg.z : sg.w, mh = t < 2 ? sh.z : sh.w;
    if (t & 1) {
        mg >>= 16;
        mh >>= 16;
    }
    const float xd = x.d[kt];
    const float2 dg = __half22float2(reinterpret_cast<const __half2*>(sp + 2304)[g]);
    const float2 dh = __half22float2(reinterpret_cast<const __half2*>(sp + 2304)[g + 8]);
    vg_out += xd * (dg.x * ((float)lo_g + 0.0625f * (float)hi_g) - dg.y * (float)dp2a_lo_su(bs, mg, 0));
    vh_out += xd * (dh.x * ((float)lo_h + 0.0625f * (float)hi_h) - dh.y * (float)dp2a_lo_su(bs, mh, 0));
}

// Q6_K unit bytes: [chunk 0..5][lane][4 words] = 24 words per lane; words 3G .. 3G + 2 of group G hold registers r0..r2 in
// bits 7..2 of every byte (the 6-bit code q - 32 in two's complement, so the byte is 4 (q - 32) as int8) and two bits each of
// register r3 in bits 1..0.  r0 / r1 = rows g / g + 8 of 16-wide sub-block 2G, r2 / r3 = the same rows of sub-block 2G + 1;
// byte b of a register is column 4 t + b of the sub-block.  Then per row 16 int8 scales, then per row half d.
__device__ __forceinline__ void unit_q6k_one(const uint8_t* sp, int lane, const XOp& x, int kt, float& vg_out, float& vh_out) {
    const int g = lane >> 2, t = lane & 3;
    const uint4* q = reinterpret_cast<const uint4*>(sp);
    const uint4* xw4 = reinterpret_cast<const uint4*>(x.q + kt * 64 + t * 16);
    const uint4 sg4 = reinterpret_cast<const uint4*>(sp + 3072)[g], sh4 = reinterpret_cast<const uint4*>(sp + 3072)[g + 8];
    const uint32_t sg[4] = {sg4.x, sg4.y, sg4.z, sg4.w}, sh[4] = {sh4.x, sh4.y, sh4.z, sh4.w};
    int acc_g = 0, acc_h = 0;
#pragma unroll
    for (int half = 0; half < 2; half++) {      // twelve code words and eight activation words at a time
        uint32_t W[12], xw[8];
#pragma unroll
        for (int c = 0; c < 3; c++) {
            const uint4 v = q[(3 * half + c) * 32 + lane];
            W[4 * c] = v.x; W[4 * c + 1] = v.y; W[4 * c + 2] = v.z; W[4 * c + 3] = v.w;
        }
#pragma unroll
        for (int c = 0; c < 2; c++) {
            const uint4 v = xw4[2 * half + c];
            xw[4 * c] = v.x; xw[4 * c + 1] = v.y; xw[4 * c + 2] = v.z; xw[4 * c + 3] = v.w;
        }
#pragma unroll
        for (int G2 = 0; G2 < 4; G2++) {
            const uint32_t w0 = W[3 * G2], w1 = W[3 * G2 + 1], w2 = W[3 * G2 + 2];
            const uint32_t r3 = ((w0 << 6) & 0xc0c0c0c0u) | ((w1 << 4) & 0x30303030u) | ((w2 << 2) & 0x0c0c0c0cu);
            const int j0 = 8 * half + 2 * G2, j1 = j0 + 1;
            acc_g += byte_s(sg[j0 >> 2], j0 & 3) * dp4a_ss(w0 & 0xfcfcfcfcu, xw[2 * G2], 0);
            acc_h += byte_s(sh[j0 >> 2], j0 & 3) * dp4a_ss(w1 & 0xfcfcfcfcu, xw[2 * G2], 0);
            acc_g += byte_s(sg[j1 >> 2], j1 & 3) * dp4a_ss(w2 & 0xfcfcfcfcu, xw[2 * G2 + 1], 0);
            acc_h += byte_s(sh[j1 >> 2], j1 & 3) * dp4a_ss(r3, xw[2 * G2 + 1], 0);
        }
    }
    const float xd = x.d[kt];
    const float dg = __half2float(reinterpret_cast<const __half*>(sp + 3328)[g]), dh = __half2float(reinterpret_cast<const __half*>(sp + 3328)[g + 8]);
    vg_out += xd * dg * 0.25f * (float)acc_g;
    vh_out += xd * dh * 0.25f * (float)acc_h;
}

// ---------------------------------------------------------------------------------------------------------------------
// Two to 32 tokens: NT groups of eight tokens on the tensor cores.
// ---------------------------------------------------------------------------------------------------------------------
template <int NT>
__device__ __forceinline__ void unit_q4k(const uint8_t* sp, int lane, const XOp& x, int kt, float (&facc)[NT][4]) {
    const int g = lane >> 2, t = lane & 3;
    uint4 w[4];
#pragma unroll
    for (int p = 0; p < 4; p++) w[p] = reinterpret_cast<const uint4*>(sp)[p * 32 + lane];
    const uint4 sg = reinterpret_cast<const uint4*>(sp + 2048)[g], sh = reinterpret_cast<const uint4*>(sp + 2048)[g + 8];
    const float2 dg = __half22float2(reinterpret_cast<const __half2*>(sp + 2304)[g]);
    const float2 dh = __half22float2(reinterpret_cast<const __half2*>(sp + 2304)[g + 8]);
#pragma unroll
    for (int n = 0; n < NT; n++) {
        const uint32_t* xb = x.q + (size_t)min(8 * n + g, x.nb - 1) * x.kw + kt * 64 + t;
        uint32_t bf[16];
#pragma unroll
        for (int j = 0; j < 8; j++) {
            bf[2 * j] = xb[j * 8];
            bf[2 * j + 1] = xb[j * 8 + 4];
        }
        // all sixteen products are issued before the first one is used: a warp issues in order, so an early use of a
        // result would hold back the independent products behind it
        int P[8][4], cmA[4] = {0, 0, 0, 0}, cmB[4] = {0, 0, 0, 0};
#pragma unroll
        for (int p = 0; p < 4; p++) {
            const uint32_t mg = p < 2 ? sg.z : sg.w, mh = p < 2 ? sh.z : sh.w;
            const int bl = (2 * p) & 3, bh = bl + 1;
#pragma unroll
            for (int i = 0; i < 4; i++) P[2 * p][i] = P[2 * p + 1][i] = 0;
            mma_u8s8_k32(P[2 * p], w[p].x & 0x0f0f0f0fu, w[p].y & 0x0f0f0f0fu, w[p].z & 0x0f0f0f0fu, w[p].w & 0x0f0f0f0fu, bf[4 * p], bf[4 * p + 1]);
            mma_u8s8_k32(P[2 * p + 1], w[p].x & 0xf0f0f0f0u, w[p].y & 0xf0f0f0f0u, w[p].z & 0xf0f0f0f0u, w[p].w & 0xf0f0f0f0u, bf[4 * p + 2],
                         bf[4 * p + 3]);
            const uint32_t mgl = byte_rep(mg, bl), mhl = byte_rep(mh, bl), mgh = byte_rep(mg, bh), mhh = byte_rep(mh, bh);
            mma_u8s8_k32(cmA, mgl, mhl, mgl, mhl, bf[4 * p], bf[4 * p + 1]);
            mma_u8s8_k32(cmB, mgh, mhh, mgh, mhh, bf[4 * p + 2], bf[4 * p + 3]);
        }
        int lo[4] = {0, 0, 0, 0}, hi[4] = {0, 0, 0, 0};
#pragma unroll
        for (int p = 0; p < 4; p++) {
            const uint32_t scg = p < 2 ? sg.x : sg.y, sch = p < 2 ? sh.x : sh.y;
            const int bl = (2 * p) & 3, bh = bl + 1;
            const int sgl = byte_u(scg, bl), sgh = byte_u(scg, bh), shl = byte_u(sch, bl), shh = byte_u(sch, bh);
            lo[0] += sgl * P[2 * p][0];
            lo[1] += sgl * P[2 * p][1];
            lo[2] += shl * P[2 * p][2];
            lo[3] += shl * P[2 * p][3];
            hi[0] += sgh * P[2 * p + 1][0];
            hi[1] += sgh * P[2 * p + 1][1];
            hi[2] += shh * P[2 * p + 1][2];
            hi[3] += shh * P[2 * p + 1][3];
        }
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const float xd = x.d[min(8 * n + 2 * t + (i & 1), x.nb - 1) * x.nkb + kt];
            const float2 d = i < 2 ? dg : dh;
            facc[n][i] += xd * (d.x * ((float)lo[i] + 0.0625f * (float)hi[i]) - d.y * (float)(cmA[i] + cmB[i]));
        }
    }
}

template <int NT>
__device__ __forceinline__ void unit_q6k(const uint8_t* sp, int lane, const XOp& x, int kt, float (&facc)[NT][4]) {
    const int g = lane >> 2, t = lane & 3;
    uint32_t W[24];
#pragma unroll
    for (int c = 0; c < 6; c++) {
        const uint4 v = reinterpret_cast<const uint4*>(sp)[c * 32 + lane];
        W[4 * c] = v.x; W[4 * c + 1] = v.y; W[4 * c + 2] = v.z; W[4 * c + 3] = v.w;
    }
    const uint4 sg4 = reinterpret_cast<const uint4*>(sp + 3072)[g], sh4 = reinterpret_cast<const uint4*>(sp + 3072)[g + 8];
    const uint32_t sg[4] = {sg4.x, sg4.y, sg4.z, sg4.w}, sh[4] = {sh4.x, sh4.y, sh4.z, sh4.w};
    const float dg = __half2float(reinterpret_cast<const __half*>(sp + 3328)[g]), dh = __half2float(reinterpret_cast<const __half*>(sp + 3328)[g + 8]);
#pragma unroll
    for (int n = 0; n < NT; n++) {
        const uint32_t* xb = x.q + (size_t)min(8 * n + g, x.nb - 1) * x.kw + kt * 64 + t;
        int acc[4] = {0, 0, 0, 0};
#pragma unroll
        for (int half = 0; half < 2; half++) {      // eight sub-blocks at a time: products first, scale multiplies after
            uint32_t bf[8];
#pragma unroll
            for (int j = 0; j < 8; j++) bf[j] = xb[(8 * half + j) * 4];
            int P[8][4];
#pragma unroll
            for (int G2 = 0; G2 < 4; G2++) {
                const int G = 4 * half + G2;
                const uint32_t w0 = W[3 * G], w1 = W[3 * G + 1], w2 = W[3 * G + 2];
                const uint32_t r3 = ((w0 << 6) & 0xc0c0c0c0u) | ((w1 << 4) & 0x30303030u) | ((w2 << 2) & 0x0c0c0c0cu);
#pragma unroll
                for (int i = 0; i < 4; i++) P[2 * G2][i] = P[2 * G2 + 1][i] = 0;
                mma_s8s8_k16(P[2 * G2], w0 & 0xfcfcfcfcu, w1 & 0xfcfcfcfcu, bf[2 * G2]);
                mma_s8s8_k16(P[2 * G2 + 1], w2 & 0xfcfcfcfcu, r3, bf[2 * G2 + 1]);
            }
#pragma unroll
            for (int j2 = 0; j2 < 8; j2++) {
                const int j = 8 * half + j2;
                const int sgj = byte_s(sg[j >> 2], j & 3), shj = byte_s(sh[j >> 2], j & 3);
                acc[0] += sgj * P[j2][0];
                acc[1] += sgj * P[j2][1];
                acc[2] += shj * P[j2][2];
                acc[3] += shj * P[j2][3];
            }
        }
#pragma unroll
        for (int i = 0; i < 4; i++)
            facc[n][i] += x.d[min(8 * n + 2 * t + (i & 1), x.nb - 1) * x.nkb + kt] * (i < 2 ? dg : dh) * 0.25f * (float)acc[i];
    }
}

// RMSNorm (optional) + int8 quantisation with one scale per 256 elements, by the 256 consumer threads of a CTA (or by a
// whole 256-thread CTA of the stand-alone kernel).  Work item = (token, 256-block) pair; warp w takes pairs w, w + 8, ...,
// eight floats per lane, and requests the pairs of a round before it uses the first, so a round costs one trip to L2.
// PR pairs per warp and round (eight floats per lane each).  KEEP: every warp has at most PR pairs and holds them in registers across the barrier that completes the row sums
// (one trip in all); otherwise the rows are read twice.  `ssq` is scratch for one float per pair (at most 256).
template <bool KEEP, int PR>
__device__ __forceinline__ void quantise_pairs(const float* x, int ldx, const float* norm_w, float eps, int k, int nb, int8_t* xq, int ldq,
                                               float* xd, int16_t* xbs, float* ssq, bool perm) {
    const int tid = threadIdx.x & 255, lane = tid & 31, warp = tid >> 5;
    const int nkb = k >> 8, npairs = nb * nkb;
    const int rounds = KEEP ? 1 : (npairs + 8 * PR - 1) / (8 * PR);
    float4 v[PR][2];
    if (norm_w || KEEP) {
        for (int r = 0; r < rounds; r++) {
#pragma unroll
            for (int i = 0; i < PR; i++) {
                const int pair = r * 8 * PR + i * 8 + warp;
                if (pair < npairs) {
                    const int b = pair / nkb, blk = pair - b * nkb;
                    const float* p = x + (size_t)b * ldx + blk * 256 + lane * 8;
                    v[i][0] = __ldcg(reinterpret_cast<const float4*>(p));
                    v[i][1] = __ldcg(reinterpret_cast<const float4*>(p + 4));
                }
            }
            if (norm_w) {
#pragma unroll
                for (int i = 0; i < PR; i++) {
                    const int pair = r * 8 * PR + i * 8 + warp;
                    if (pair < npairs) {
                        const float4 a0 = v[i][0], a1 = v[i][1];
                        float ss = a0.x * a0.x + a0.y * a0.y + a0.z * a0.z + a0.w * a0.w + a1.x * a1.x + a1.y * a1.y + a1.z * a1.z + a1.w * a1.w;
                        ss = warp_sum(ss);
                        if (lane == 0) ssq[pair] = ss;
                    }
                }
            }
        }
        if (norm_w) {
            __syncthreads();
        }
    }
    for (int r = 0; r < rounds; r++) {
        if (!KEEP) {
#pragma unroll
            for (int i = 0; i < PR; i++) {
                const int pair = r * 8 * PR + i * 8 + warp;
                if (pair < npairs) {
                    const int b = pair / nkb, blk = pair - b * nkb;
                    const float* p = x + (size_t)b * ldx + blk * 256 + lane * 8;
                    v[i][0] = __ldcg(reinterpret_cast<const float4*>(p));
                    v[i][1] = __ldcg(reinterpret_cast<const float4*>(p + 4));
                }
            }
        }
#pragma unroll
        for (int i = 0; i < PR; i++) {
            const int pair = r * 8 * PR + i * 8 + warp;
            if (pair >= npairs) continue;
            const int b = pair / nkb, blk = pair - b * nkb;
            const int e0 = blk * 256 + lane * 8;
            float4 v0 = v[i][0], v1 = v[i][1];
            if (norm_w) {
                float s = 0.f;          // the row's sum of squares, added in a fixed order
                for (int j = lane; j < nkb; j += 32) s += ssq[b * nkb + j];
                const float rstd = rsqrtf(warp_sum(s) / (float)k + eps);
                const float4 n0 = *reinterpret_cast<const float4*>(norm_w + e0), n1 = *reinterpret_cast<const float4*>(norm_w + e0 + 4);
                v0.x *= rstd * n0.x; v0.y *= rstd * n0.y; v0.z *= rstd * n0.z; v0.w *= rstd * n0.w;
                v1.x *= rstd * n1.x; v1.y *= rstd * n1.y; v1.z *= rstd * n1.z; v1.w *= rstd * n1.w;
            }
            float amax = fmaxf(fmaxf(fmaxf(fabsf(v0.x), fabsf(v0.y)), fmaxf(fabsf(v0.z), fabsf(v0.w))),
                               fmaxf(fmaxf(fabsf(v1.x), fabsf(v1.y)), fmaxf(fabsf(v1.z), fabsf(v1.w))));
            amax = warp_max(amax);
            const float d = amax / 127.f, id = amax > 0.f ? 127.f / amax : 0.f;
            const int q0 = __float2int_rn(v0.x * id), q1 = __float2int_rn(v0.y * id), q2 = __float2int_rn(v0.z * id), q3 = __float2int_rn(v0.w * id);
            const int q4 = __float2int_rn(v1.x * id), q5 = __float2int_rn(v1.y * id), q6 = __float2int_rn(v1.z * id), q7 = __float2int_rn(v1.w * id);
            uint2 pk;
            pk.x = (uint32_t)(q0 & 0xff) | ((uint32_t)(q1 & 0xff) << 8) | ((uint32_t)(q2 & 0xff) << 16) | ((uint32_t)(q3 & 0xff) << 24);
            pk.y = (uint32_t)(q4 & 0xff) | ((uint32_t)(q5 & 0xff) << 8) | ((uint32_t)(q6 & 0xff) << 16) | ((uint32_t)(q7 & 0xff) << 24);
            if (perm) {
                // one-token layout: inside a 256-block the words of columns 4 t .. 4 t + 3 of all sixteen 16-column groups follow
                // each other ([t][group]); this lane holds group lane / 2, t = 2 (lane & 1) and t + 1
                uint32_t* blkw = reinterpret_cast<uint32_t*>(xq + (size_t)b * ldq + blk * 256);
                blkw[(2 * (lane & 1)) * 16 + (lane >> 1)] = pk.x;
                blkw[(2 * (lane & 1) + 1) * 16 + (lane >> 1)] = pk.y;
            } else {
                *reinterpret_cast<uint2*>(xq + (size_t)b * ldq + e0) = pk;
            }
            if (lane == 0) xd[b * nkb + blk] = d;
            if (xbs) {      // sum of every 32-block = four lanes
                int sum = q0 + q1 + q2 + q3 + q4 + q5 + q6 + q7;
                sum += __shfl_xor_sync(0xffffffffu, sum, 1);
                sum += __shfl_xor_sync(0xffffffffu, sum, 2);
                if ((lane & 3) == 0) xbs[(size_t)b * (k >> 5) + blk * 8 + (lane >> 2)] = (int16_t)sum;
            }
        }
    }
}

template <int PR>
__device__ __forceinline__ void quantise_rows(const float* x, int ldx, const float* norm_w, float eps, int k, int nb, int8_t* xq, int ldq,
                                              float* xd, int16_t* xbs, float* ssq, bool perm) {
    if (nb * (k >> 8) <= 8 * PR) quantise_pairs<true, PR>(x, ldx, norm_w, eps, k, nb, xq, ldq, xd, xbs, ssq, perm);
    else quantise_pairs<false, PR>(x, ldx, norm_w, eps, k, nb, xq, ldq, xd, xbs, ssq, perm);
}

__device__ __forceinline__ void decode_unit(const SkArgs& a, int kts, int u, int& s, int& tile, int& kt) {
    s = 0;
#pragma unroll
    for (int i = 1; i < 4; i++)
        if (i < a.nseg && u >= a.seg[i].unit0) s = i;
    const int l = u - a.seg[s].unit0;
    tile = l / kts;
    kt = l - tile * kts;
}

// Units [lo, hi) of group `gg` of `n_groups`: an equal share of the launch's units.
__device__ __forceinline__ void group_range(int gg, int total, int n_groups, int& lo, int& hi) {
    lo = (int)((long long)gg * total / n_groups);
    hi = (int)((long long)(gg + 1) * total / n_groups);
}

// Points the walker at phase w.ph: this warp's place in that phase's split; returns where its group's range starts.
__device__ __forceinline__ int walker_enter(Walker& w, const SkChain& c, int warp) {
    const SkArgs& a = c.ph[w.ph];
    w.l2 = a.wpt_log2;
    w.kts = a.k >> 8;
    w.wi = warp & ((1 << w.l2) - 1);
    const int gg = blockIdx.x * (SK_WARPS >> w.l2) + (warp >> w.l2);
    int glo = 0;
    w.ghi = 0;
    if (gg < a.n_groups) group_range(gg, a.total_units, a.n_groups, glo, w.ghi);
    return glo;
}

// Moves `w` to this warp's first unit at or after segment start `from` of phase w.ph, or of the next phase that has one.
// Inside a segment (the part of one 16-row tile that lies in the group's range) the 2^l2 warps of the group take equal
// contiguous runs of units.
__device__ __forceinline__ void walker_find(Walker& w, const SkChain& c, int warp, int from) {
    w.valid = false;
    for (;;) {
        const SkArgs& a = c.ph[w.ph];
        int sl = from;
        while (sl < w.ghi) {
            int s, tile, kt;
            decode_unit(a, w.kts, sl, s, tile, kt);
            const int sh = min(w.ghi, sl + (w.kts - kt)), n = sh - sl;
            const int ua = sl + ((w.wi * n) >> w.l2), ub = sl + (((w.wi + 1) * n) >> w.l2);
            if (ua < ub) {
                w.u = ua;
                w.ub = ub;
                w.seg_end = sh;
                w.type = a.seg[s].type;
                w.p = a.seg[s].w + (size_t)(ua - a.seg[s].unit0) * unit_bytes(w.type);
                w.valid = true;
                return;
            }
            sl = sh;
        }
        if (++w.ph >= c.n) return;
        from = walker_enter(w, c, warp);
    }
}
__device__ __forceinline__ void walker_next(Walker& w, const SkChain& c, int warp) {
    if (++w.u < w.ub) w.p += unit_bytes(w.type);
    else walker_find(w, c, warp, w.seg_end);
}

// Request the walker's unit into a ring slot (nothing when the warp has run out of units) and close the copy group.
__device__ __forceinline__ void ring_issue(const Walker& w, uint8_t* slot, int lane, uint64_t policy) {
    if (w.valid) {
        const int pieces = unit_bytes(w.type) >> 4;
        for (int i = lane; i < pieces; i += 32) cp_async16(slot + i * 16, w.p + i * 16, policy);
    }
    cp_async_commit();
}

// All CTAs of the launch meet (bounded wait): `target` arrivals on the counter.  Stores of the phase before are visible to
// loads that bypass L1 after it.
__device__ __forceinline__ void grid_barrier(unsigned* bar, unsigned target, int* status, bool& dead) {
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        atomicAdd(bar, 1u);
        if (!dead) {
            bool ok = ld_acquire_gpu_u32(bar) >= target;
            if (!ok) {
                const unsigned long long t0 = global_ns();
                while (!ok && global_ns() - t0 < SK_WAIT_NS) ok = ld_acquire_gpu_u32(bar) >= target;
            }
            if (!ok) atomicExch(status, (int)KS_TIMEOUT);
        }
    }
    __syncthreads();
}

template <int NT, bool ONE, bool XSMEM>
__global__ void __launch_bounds__(SK_THREADS, NT == 1 ? 2 : 1) gemv_sk_kernel(const __grid_constant__ SkChain c_param) {
    constexpr int FRAG = NT * 4 * 32;           // floats of one warp's accumulator fragment
    extern __shared__ __align__(128) uint8_t smem[];
    // The argument block is more than a kilobyte and is indexed at run time (phase, matrix): read from the constant bank
    // field by field, every first touch of a line is a miss of about a microsecond, one after the other.  All threads copy
    // it to shared memory in one sweep instead.
    __shared__ __align__(16) SkChain c;
    {
        const uint32_t* src = reinterpret_cast<const uint32_t*>(&c_param);
        uint32_t* dst = reinterpret_cast<uint32_t*>(&c);
        for (int i = threadIdx.x; i < (int)(sizeof(SkChain) / 4); i += SK_THREADS) dst[i] = src[i];
    }
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    float* red = reinterpret_cast<float*>(smem + c.ph[0].off_red);
    pdl_launch();
    unsigned long long* tr = c.trace && threadIdx.x == 0 ? c.trace + (size_t)blockIdx.x * 16 : nullptr;
    int tr_n = 0;
    if (tr) tr[tr_n++] = global_ns();

    // Weights do not depend on the previous kernel: the warp's first units are requested before the grid-dependency wait.
    const int R = c.ph[0].ring, slot_bytes = c.ph[0].slot_bytes;      // R - 1 units are in flight while one is computed
    uint8_t* ring = smem + c.ph[0].off_ring + (size_t)warp * R * slot_bytes;
    const uint64_t policy = stream_policy();
    Walker wk;
    wk.ph = 0;
    walker_find(wk, c, warp, walker_enter(wk, c, warp));
    // Requests in flight fill the SM's miss queues: an activation load issued behind R - 1 units per warp waits for the first of
    // them to come back.  So only `pre` units per warp go out before the inputs are loaded; the ring is topped up right after
    // the activation loads have been issued (`held` counts the slots still owed).
    int slot_in = 0, slot_out = 0, held = 0;
    const int pre = (c.tune & 3) == 0 ? R - 1 : min(c.tune & 3, R - 1);
    const bool hold_phases = (c.tune & 4) != 0;
    auto issue = [&](int ph_limit) {        // one ring slot: the walker's unit, unless it belongs to a phase that is held back
        if (wk.valid && wk.ph > ph_limit) {
            held++;
            return;
        }
        ring_issue(wk, ring + slot_in * slot_bytes, lane, policy);
        if (wk.valid) walker_next(wk, c, warp);
        slot_in = slot_in + 1 == R ? 0 : slot_in + 1;
    };
    auto top_up = [&](int ph_limit) {
        while (held > 0 && !(wk.valid && wk.ph > ph_limit)) {
            held--;
            issue(ph_limit);
        }
    };
    for (int i = 0; i < R - 1; i++) {
        if (i < pre) issue(SK_MAX_PHASES);
        else held++;
    }
    if (tr) tr[tr_n++] = global_ns();
    pdl_wait();
    if (tr) tr[tr_n++] = global_ns();
    bool dead = false;                      // a bounded wait gave up: stop waiting, the status word is set
    for (int ph = 0; ph < c.n; ph++) {
        const SkArgs& a = c.ph[ph];
        if (ph > 0) grid_barrier(c.bar, gridDim.x * (unsigned)ph, a.status, dead);
        if (tr) tr[tr_n++] = global_ns();
        const int kts = a.k >> 8;
        // a group of 2^l2 warps of this CTA works through one contiguous range of units, tile segment by tile segment
        const int l2 = a.wpt_log2, wpt = 1 << l2;
        const int gi = warp >> l2, wi = warp & (wpt - 1);
        const int n_groups = a.n_groups, gg = blockIdx.x * (SK_WARPS >> l2) + gi;
        int glo = 0, ghi = 0;
        if (gg < n_groups) group_range(gg, a.total_units, n_groups, glo, ghi);
        unsigned ep = 0;
        if (a.cm.n_dst > 0) ep = comm_next_epoch(a.cm);
        XOp x;
        x.kw = a.k >> 2;
        x.nkb = kts;
        x.nb = a.nb;
        if (XSMEM) {
            float* ssq = reinterpret_cast<float*>(smem);
            int8_t* xq_s = reinterpret_cast<int8_t*>(smem + a.off_xq);
            float* xd_s = reinterpret_cast<float*>(smem + a.off_xd);
            int16_t* xbs_s = reinterpret_cast<int16_t*>(smem + a.off_xbs);
            // token rows are 16 bytes apart from a multiple of 128, so the eight tokens of a B fragment hit different banks
            quantise_rows<2>(a.x, a.ldx, a.norm_w, a.eps, a.k, a.nb, xq_s, a.k + 16, xd_s, ONE ? xbs_s : nullptr, ssq, ONE);
            top_up(SK_MAX_PHASES);
            __syncthreads();
            x.kw = (a.k + 16) >> 2;
            x.q = reinterpret_cast<const uint32_t*>(xq_s);
            x.d = xd_s;
            x.bs = reinterpret_cast<const uint32_t*>(xbs_s);
        } else {
            x.q = reinterpret_cast<const uint32_t*>(a.xq);
            x.d = a.xd;
            x.bs = reinterpret_cast<const uint32_t*>(a.xbs);
            top_up(SK_MAX_PHASES);
        }
        if (tr) tr[tr_n++] = global_ns();

        int u_seg = glo, seg_i = 0;
        while (u_seg < ghi) {
            // one segment: units [u_seg, u_end) of tile `tile` of matrix `s`, starting at k-tile kt0
            int s, tile, kt0;
            decode_unit(a, kts, u_seg, s, tile, kt0);
            const int u_end = min(ghi, u_seg + (kts - kt0)), type = a.seg[s].type, n_seg = u_end - u_seg;
            const int ua = u_seg + ((wi * n_seg) >> l2), ub = u_seg + (((wi + 1) * n_seg) >> l2);
            float facc[NT][4];
    #pragma unroll
            for (int n = 0; n < NT; n++)
    #pragma unroll
                for (int i = 0; i < 4; i++) facc[n][i] = 0.f;
            for (int u = ua; u < ub; u++) {
                // keep the ring full, then wait for the oldest unit: every slot that was asked for has either closed a copy group
                // or is still owed, so all but the R - 1 - held newest groups are complete when the oldest unit is
                issue(hold_phases ? ph : SK_MAX_PHASES);
                const int newer = R - 1 - held;
                if (newer >= 3) cp_async_wait<3>(); else if (newer == 2) cp_async_wait<2>(); else if (newer == 1) cp_async_wait<1>(); else cp_async_wait<0>();
                __syncwarp();
                const uint8_t* sp = ring + slot_out * slot_bytes;
                slot_out = slot_out + 1 == R ? 0 : slot_out + 1;
                const int kt = kt0 + (u - u_seg);
                if (ONE) {
                    if (type == WT_Q6_K) unit_q6k_one(sp, lane, x, kt, facc[0][0], facc[0][2]);
                    else unit_q4k_one(sp, lane, x, kt, facc[0][0], facc[0][2]);
                } else {
                    if (type == WT_Q6_K) unit_q6k<NT>(sp, lane, x, kt, facc);
                    else unit_q4k<NT>(sp, lane, x, kt, facc);
                }
                __syncwarp();      // every lane is done with the slot before a later request overwrites it
            }
            if (ONE) {      // the four t lanes of a row hold partial sums over different columns
                facc[0][0] += __shfl_xor_sync(0xffffffffu, facc[0][0], 1);
                facc[0][2] += __shfl_xor_sync(0xffffffffu, facc[0][2], 1);
                facc[0][0] += __shfl_xor_sync(0xffffffffu, facc[0][0], 2);
                facc[0][2] += __shfl_xor_sync(0xffffffffu, facc[0][2], 2);
            }
            if (l2 > 0) {
                // the warps of the group add their fragments in shared memory (two buffers: a warp can be one segment ahead)
                float* rb = red + (size_t)((seg_i & 1) * SK_WARPS + gi * wpt) * FRAG;
                if (wi != 0) {
    #pragma unroll
                    for (int n = 0; n < NT; n++)
    #pragma unroll
                        for (int i = 0; i < 4; i++)
                            if (!ONE || !(i & 1)) rb[wi * FRAG + (n * 4 + i) * 32 + lane] = facc[n][i];
                }
                asm volatile("bar.sync %0, %1;" ::"r"(1 + gi), "r"(wpt * 32) : "memory");
                if (wi == 0) {
                    for (int w2 = 1; w2 < wpt; w2++)
    #pragma unroll
                        for (int n = 0; n < NT; n++)
    #pragma unroll
                            for (int i = 0; i < 4; i++)
                                if (!ONE || !(i & 1)) facc[n][i] += rb[w2 * FRAG + (n * 4 + i) * 32 + lane];
                }
            }
            const bool starts = kt0 == 0, ends = kt0 + n_seg == kts;
            if (wi == 0 && !starts) {
                // the tile began in an earlier group: hand the partial sums to the group that owns its first unit
                float* wsp = a.ws + (size_t)gg * SK_WS_FLOATS;
    #pragma unroll
                for (int n = 0; n < NT; n++)
    #pragma unroll
                    for (int i = 0; i < 4; i++)
                        if (!ONE || !(i & 1)) wsp[(n * 4 + i) * 32 + lane] = facc[n][i];
                __threadfence();
                __syncwarp();
                if (lane == 0) st_release_gpu_u32(&a.flags[gg], 1u);
            } else if (wi == 0) {
                if (!ends) {
                    const int tile_end = u_seg + kts;
                    for (int c = gg + 1; c < n_groups; c++) {
                        int clo, chi;
                        group_range(c, a.total_units, n_groups, clo, chi);
                        if (clo >= tile_end) break;
                        if (clo == chi) continue;
                        bool ok = true;
                        if (lane == 0 && !dead) {
                            ok = ld_acquire_gpu_u32(&a.flags[c]) != 0u;
                            if (!ok) {
                                const unsigned long long t0 = global_ns();
                                while (!ok && global_ns() - t0 < SK_WAIT_NS) {
                                    __nanosleep(32);
                                    ok = ld_acquire_gpu_u32(&a.flags[c]) != 0u;
                                }
                            }
                            if (!ok) atomicExch(a.status, (int)KS_TIMEOUT);
                        }
                        ok = __shfl_sync(0xffffffffu, ok, 0);
                        if (!ok) {
                            dead = true;
                            continue;
                        }
                        const float* wsp = a.ws + (size_t)c * SK_WS_FLOATS;
    #pragma unroll
                        for (int n = 0; n < NT; n++)
    #pragma unroll
                            for (int i = 0; i < 4; i++)
                                if (!ONE || !(i & 1)) facc[n][i] += __ldcg(wsp + (n * 4 + i) * 32 + lane);
                        __syncwarp();
                        if (lane == 0) a.flags[c] = 0u;
                    }
                }
                // finish the 16 rows: lane (g, t) holds rows g (i < 2) and g + 8 of tokens 8 n + 2 t + (i & 1); one token: every t
                // lane holds the row sums, t = 0 writes row g and t = 1 row g + 8
                const SkSeg& sg = a.seg[s];
                const int row0 = tile * 16;
                if (a.mode == 2 && a.cm.n_dst == 0) {
                    // interleaved rows: even rows are gates, the odd row after each is its up value and lives in lane + 4
    #pragma unroll
                    for (int n = 0; n < NT; n++)
    #pragma unroll
                        for (int i = 0; i < 4; i++) {
                            if (ONE && (i & 1)) continue;
                            const int row = g + 8 * (i >> 1);
                            const float mine = facc[n][i] + (sg.bias ? sg.bias[row0 + row] : 0.f);
                            const float up = __shfl_down_sync(0xffffffffu, mine, 4);
                            const int b = ONE ? 0 : 8 * n + 2 * t + (i & 1);
                            if (!(g & 1) && b < a.nb && (!ONE || t == 0))
                                a.out[(size_t)b * a.ldo + (sg.out_off >> 1) + ((row0 + row) >> 1)] = glu_act(mine, up, a.act, a.alpha, a.limit);
                        }
                } else {
                    const long long poff = a.cm.n_dst > 0 ? comm_parity_off(a.cm, ep) : 0;
    #pragma unroll
                    for (int n = 0; n < NT; n++)
    #pragma unroll
                        for (int i = 0; i < 4; i++) {
                            if (ONE && (i & 1)) continue;
                            if (ONE && t != (i >> 1)) continue;
                            const int row = row0 + g + 8 * (i >> 1);
                            const int b = ONE ? 0 : 8 * n + 2 * t + (i & 1);
                            if (b >= a.nb) continue;
                            const float v = facc[n][i] + (sg.bias ? sg.bias[row] : 0.f);
                            if (a.cm.n_dst > 0) {
                                const long long o = poff + (long long)b * a.ldo + sg.out_off + row;
                                const uint2 pr = make_uint2(__float_as_uint(v), ep);
                                for (int d2 = 0; d2 < a.cm.n_dst; d2++) reinterpret_cast<uint2*>(a.cm.dst[d2])[o] = pr;
                            } else {
                                float* o = a.out + (size_t)b * a.ldo + sg.out_off + row;
                                *o = a.mode == 1 ? *o + v : v;
                            }
                        }
                }
            }
            u_seg = u_end;
            seg_i++;
        }

        if (tr) tr[tr_n++] = global_ns();
    }
    if (c.n > 1) {
        // the last CTA to leave puts the counters back to zero for the next launch
        __syncthreads();
        if (threadIdx.x == 0 && atomicAdd(c.bar + 1, 1u) == gridDim.x - 1) {
            c.bar[0] = 0u;
            c.bar[1] = 0u;
        }
    }
}

// One CTA per token row when the row is normalised first (the row's sum of squares is needed before any element can be
// scaled); without a norm the 256-blocks are independent and a row is spread over gridDim.y CTAs of up to eight blocks each,
// one block per warp, so a 14336-wide row takes one trip to L2 instead of seven.
constexpr int Q256_CHUNK = 8;      // 256-blocks per CTA in the spread form

__global__ void __launch_bounds__(256) quant256_kernel(const __grid_constant__ Quant256Args a) {
    __shared__ float ssq[256];
    pdl_launch();
    pdl_wait();
    const size_t row = blockIdx.x;
    const int blk0 = blockIdx.y * Q256_CHUNK, nkb = a.k >> 8;
    if (gridDim.y == 1) {
        quantise_rows<8>(a.x + row * a.ldx, a.ldx, a.norm_w, a.eps, a.k, 1, a.xq + row * a.k, a.k, a.xd + row * nkb,
                      a.xbs ? a.xbs + row * (a.k >> 5) : nullptr, ssq, a.perm != 0);
        return;
    }
    if (blk0 >= nkb) return;
    const int kc = min(Q256_CHUNK, nkb - blk0) << 8;        // this CTA's slice of the row; norm_w is null here
    quantise_rows<8>(a.x + row * a.ldx + (size_t)blk0 * 256, a.ldx, nullptr, a.eps, kc, 1, a.xq + row * a.k + (size_t)blk0 * 256, a.k,
                  a.xd + row * nkb + blk0, a.xbs ? a.xbs + row * (a.k >> 5) + blk0 * 8 : nullptr, ssq, a.perm != 0);
}

int g_sm_count[64] = {};

int sm_count() {
    int d = 0;
    cudaGetDevice(&d);
    d &= 63;
    if (!g_sm_count[d]) cudaDeviceGetAttribute(&g_sm_count[d], cudaDevAttrMultiProcessorCount, d);
    return g_sm_count[d];
}

template <int NT, bool ONE>
const void* pick_x(bool xsmem) {
    return xsmem ? (const void*)gemv_sk_kernel<NT, ONE, true> : (const void*)gemv_sk_kernel<NT, ONE, false>;
}

cudaError_t launch(const void* fn, dim3 grid, dim3 block, size_t smem, void** args, cudaStream_t st, int pdl) {
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

PerDeviceOnce g_attr[8];

}  // namespace

// Rows of the workspace / flag arrays a caller must provide (one per group of the largest launch).
B2_API int b2_gemv_sk_max_groups() { return 4096; }

// Runs the phases of `in` (y = W x for 1..32 tokens on unit-ordered Q4_K / Q6_K matrices, the same token count in every phase)
// in one launch.  The launch never has more CTAs than are resident at once (groups wait for each other's partial sums, phases
// for each other); max_ctas > 0 lowers that further.  split: 0 = choose, 1..4 = force 1, 2, 4 or 8 warps per group with equal
// shares of units; ring_slots: 0 = choose, 2..4 = units per warp ring.  Returns a cudaError_t value (cudaErrorInvalidValue also
// when a fused fp32 input does not fit into shared memory: the caller then quantises it with b2_quant256).
B2_API int b2_gemv_sk_chain(const SkChain* in, int max_ctas, int split, int ring_slots, int pdl, cudaStream_t st) {
    SkChain c = *in;
    if (c.n < 1 || c.n > SK_MAX_PHASES || (c.n > 1 && !c.bar)) return (int)cudaErrorInvalidValue;
    const int nb = c.ph[0].nb;
    const bool xsmem = c.ph[0].x != nullptr;
    if (nb < 1 || nb > 32) return (int)cudaErrorInvalidValue;
    const int nt = nb <= 8 ? 1 : nb <= 16 ? 2 : 4;
    const bool one = nb == 1;
    int xbytes = 0, slot = 0;
    for (int p = 0; p < c.n; p++) {
        SkArgs& a = c.ph[p];
        if (a.nb != nb || (a.x != nullptr) != xsmem || a.nseg < 1 || a.nseg > 4 || (a.k & 255) || a.k <= 0) return (int)cudaErrorInvalidValue;
        if (!a.ws || !a.flags || !a.status || (!a.x && (!a.xq || !a.xd || (nb == 1 && !a.xbs)))) return (int)cudaErrorInvalidValue;
        if (a.cm.n_dst < 0 || a.cm.n_dst > COMM_MAX_RANKS || (a.cm.n_dst > 0 && (!a.cm.ll || a.mode != 0))) return (int)cudaErrorInvalidValue;
        if (xsmem && (((uintptr_t)a.x & 15) || (a.ldx & 3) || (a.norm_w && ((uintptr_t)a.norm_w & 15)))) return (int)cudaErrorInvalidValue;
        const int kts = a.k >> 8;
        int units = 0;
        for (int s = 0; s < a.nseg; s++) {
            SkSeg& sg = a.seg[s];
            if ((sg.type != WT_Q4_K && sg.type != WT_Q6_K) || (sg.n & 15) || sg.n <= 0 || ((uintptr_t)sg.w & 15)) return (int)cudaErrorInvalidValue;
            if (a.mode == 2 && ((sg.out_off & 1) || (sg.n & 31))) return (int)cudaErrorInvalidValue;
            sg.unit0 = units;
            units += (sg.n >> 4) * kts;
            slot = max(slot, sg.type == WT_Q6_K ? SK_UNIT_Q6K : SK_UNIT_Q4K);
        }
        a.total_units = units;
        if (xsmem) xbytes = max(xbytes, nb * (a.k + 16) + nb * kts * 4 + nb * (a.k >> 5) * 2);
    }
    // shared memory: quantiser scratch | reduction buffers | quantised activations of the running phase | one ring per warp
    int off = 1024;
    const int off_red = off;
    off += 2 * SK_WARPS * nt * 4 * 32 * 4;
    const int off_x = off;
    off += (xbytes + 127) & ~127;
    const int off_ring = off;
    const void* fn = one ? pick_x<1, true>(xsmem) : nt == 1 ? pick_x<1, false>(xsmem) : nt == 2 ? pick_x<2, false>(xsmem) : pick_x<4, false>(xsmem);
    const int which = (one ? 0 : nt == 1 ? 1 : nt == 2 ? 2 : 3) * 2 + (xsmem ? 1 : 0);
    if (g_attr[which].first()) {
        const cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, SK_MAX_DYN_SMEM);
        if (e != cudaSuccess) return (int)e;
    }
    // ring depth: the one that puts most units in flight per SM (CTAs per SM x slots in flight), more CTAs on a tie
    int per_sm = 0, best = 0, ring = 0;
    size_t smem = 0;
    for (int r = (ring_slots > 0 ? ring_slots : 4); r >= (ring_slots > 0 ? ring_slots : 2); r--) {
        const size_t need = (size_t)off + (size_t)SK_WARPS * r * slot;
        if (need > (size_t)SK_MAX_DYN_SMEM) continue;
        int n = 0;
        const cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, fn, SK_THREADS, need);
        if (e != cudaSuccess) return (int)e;
        if (n * (r - 1) > best || (n * (r - 1) == best && n > per_sm)) {
            best = n * (r - 1);
            per_sm = n;
            ring = r;
            smem = need;
        }
    }
    if (per_sm < 1) return (int)cudaErrorInvalidValue;
    int ctas = min(per_sm * sm_count(), b2_gemv_sk_max_groups() / SK_WARPS);
    if (max_ctas > 0) ctas = min(ctas, max_ctas);
    // Work split of a phase.  Few tiles (at most one per resident CTA): a CTA per tile, or per half tile, so that no or one
    // partial sum crosses CTAs.  Many tiles: every warp slot of the GPU streams an equal share, and as many warps share a
    // range as keep a range about one tile long.
    int grid = 1;
    for (int p = 0; p < c.n; p++) {
        SkArgs& a = c.ph[p];
        const int kts = a.k >> 8, units = a.total_units, tiles = units / kts;
        int l2, groups;
        if (split > 0) {
            l2 = min(split - 1, 3);
            groups = min(ctas * (SK_WARPS >> l2), units);
        } else if (tiles <= ctas) {
            l2 = 3;
            const int ks = (2 * tiles <= ctas && !(kts & 1) && (kts >> 1) >= SK_WARPS) ? 2 : 1;
            groups = tiles * ks;
        } else {
            const long long want = ((long long)kts * ctas * SK_WARPS + units - 1) / units;      // warps per tile-long range
            l2 = want <= 1 ? 0 : want <= 2 ? 1 : want <= 4 ? 2 : 3;
            groups = min(ctas * (SK_WARPS >> l2), units);
        }
        a.wpt_log2 = l2;
        a.n_groups = groups;
        const int per_cta = SK_WARPS >> l2;
        grid = max(grid, (groups + per_cta - 1) / per_cta);
        a.off_red = off_red;
        a.off_xq = off_x;
        a.off_xd = off_x + nb * (a.k + 16);
        a.off_xbs = a.off_xd + nb * kts * 4;
        a.off_ring = off_ring;
        a.ring = ring;
        a.slot_bytes = slot;
    }
    void* args[] = {&c};
    return (int)launch(fn, dim3((unsigned)grid), dim3(SK_THREADS), smem, args, st, pdl);
}

// One product: a chain of one phase.
B2_API int b2_gemv_sk(const SkArgs* in, int max_ctas, int split, int ring_slots, int pdl, cudaStream_t st) {
    SkChain c = {};
    c.ph[0] = *in;
    c.n = 1;
    return b2_gemv_sk_chain(&c, max_ctas, split, ring_slots, pdl, st);
}

// int8 quantisation (one scale per 256 elements) of nb fp32 rows, with an optional RMSNorm in front.
B2_API int b2_quant256(const Quant256Args* a, int nb, int pdl, cudaStream_t st) {
    if (nb < 1 || (a->k & 255) || (a->ldx & 3) || ((uintptr_t)a->x & 15)) return (int)cudaErrorInvalidValue;
    Quant256Args copy = *a;
    void* args[] = {&copy};
    const int nkb = a->k >> 8;
    const unsigned chunks = a->norm_w ? 1u : (unsigned)((nkb + Q256_CHUNK - 1) / Q256_CHUNK);
    return (int)launch((const void*)quant256_kernel, dim3((unsigned)nb, chunks), dim3(256), 0, args, st, pdl);
}
