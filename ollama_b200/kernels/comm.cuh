// One-way exchanges between the GPUs of a tensor-parallel group over peer-mapped memory (NVLink).
//
// A producer kernel writes its results straight into buffers that live on the consuming GPUs (plain
// stores to peer addresses from the GEMV / GEMM epilogue), then announces them: every CTA fences and
// takes a ticket; the CTA that takes the last ticket advances this rank's epoch and stores it, with
// release semantics at system scope, into this rank's flag on every destination.  A consumer kernel
// spins (acquire loads, bounded by a wall-clock limit) until every rank's flag has reached the epoch
// it expects and then reads the buffers from its own memory.  The transfer therefore overlaps the
// producer's math tile by tile, the reduction is fused into the consumer, and no separate collective
// kernel runs.  The reference stack performs the same exchanges with NCCL all-reduce calls between
// graph splits (ggml-cuda's split-buffer / multi-device scheduling).
//
// Buffer reuse: destinations that are written once per exchange are double-buffered on the parity of
// the epoch.  A rank can run at most one exchange ahead of the slowest rank (its next consumer waits
// for that rank's flag), so two halves suffice.
//
// Every wait is bounded: after the channel's time limit the waiter records KS_TIMEOUT in the channel's status word
// and carries on (the step's result is then garbage, the host reads the status and fails the request).
#pragma once
#include "common.cuh"

constexpr int COMM_MAX_RANKS = 8;

struct CommChan {                    // one per exchange site, inside every rank's peer-mapped region
    unsigned ticket;                 // CTAs of the running producer that have finished (used by the owning rank only)
    unsigned epoch;                  // exchanges completed by the owning rank as a producer
    int status;                      // KStatus of the owning rank's waits
    unsigned wait_ms;                // limit of one wait in milliseconds (0: 2000)
    unsigned pad0[4];
    unsigned flag[COMM_MAX_RANKS];   // flag[r]: last epoch announced by rank r (written by rank r)
    unsigned pad1[16];               // 128 bytes in all
};

struct CommSend {
    int n_dst;                       // ranks that receive a copy (0: no exchange)
    int rank;                        // this rank
    CommChan* local;                 // this rank's channel
    unsigned* peer_flag[COMM_MAX_RANKS];   // &channel_on_rank_r->flag[rank]
    float* dst[COMM_MAX_RANKS];      // destination base on rank r, already offset to this rank's slab or column range
    long long parity_stride;         // elements between the two halves of a double-buffered destination (0: single buffer)
    int ll;                          // 1: low-latency protocol, dst holds (value, epoch) pairs and nothing is announced (see below)
};

__device__ __forceinline__ unsigned ld_volatile_u32(const unsigned* p) {
    unsigned v;
    asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned ld_acquire_sys_u32(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys_u32(unsigned* p, unsigned v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// Epoch of the exchange the running producer kernel is about to publish (call after the grid-dependency wait).
__device__ __forceinline__ unsigned comm_next_epoch(const CommSend& c) { return ld_volatile_u32(&c.local->epoch) + 1u; }

// Offset (elements) of the destination half used by exchange `e`.
__device__ __forceinline__ long long comm_parity_off(const CommSend& c, unsigned e) { return (e & 1u) ? c.parity_stride : 0ll; }

// Called by every thread of every CTA of a producer kernel after its last peer store.
__device__ __forceinline__ void comm_publish(const CommSend& c, unsigned total_ctas, unsigned e) {
    // The CTA barrier orders every thread's stores before thread 0's fence, and the fence is cumulative, so one
    // system-scope fence per CTA is enough (a fence in every warp costs microseconds once thousands of them queue up).
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();
        const unsigned t = atomicAdd(&c.local->ticket, 1u);
        if (t == total_ctas - 1u) {
            __threadfence();
            *(volatile unsigned*)&c.local->ticket = 0u;
            *(volatile unsigned*)&c.local->epoch = e;
            __threadfence_system();
            for (int r = 0; r < c.n_dst; r++) st_release_sys_u32(c.peer_flag[r], e);
        }
    }
}

// Wait until the first n flags of `ch` have reached epoch e.  Call with threads 0..n-1 of a CTA (others may
// call too; they return at once) and follow it with __syncthreads().  Returns false after the time limit.
__device__ __forceinline__ bool comm_wait_flags(CommChan* ch, int n, unsigned e) {
    if ((int)threadIdx.x >= n) return true;
    const unsigned* f = &ch->flag[threadIdx.x];
    if ((int)(ld_acquire_sys_u32(f) - e) >= 0) return true;
    if (*(volatile int*)&ch->status != 0) return false;      // an earlier wait already ran out: the host clears the status
    const unsigned long long t0 = global_ns();
    const unsigned ms = ld_volatile_u32(&ch->wait_ms);
    const unsigned long long limit = (unsigned long long)(ms ? ms : 2000u) * 1000000ull;
    for (;;) {
        for (int i = 0; i < 64; i++)
            if ((int)(ld_acquire_sys_u32(f) - e) >= 0) return true;
        if (global_ns() - t0 > limit) {
            atomicExch(&ch->status, (int)KS_TIMEOUT);
            return false;
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Low-latency exchange for small messages (decode): every 8-byte word carries a value and the epoch it
// belongs to, so the data is its own flag.  The producer needs no fence, ticket or flag store (an aligned
// 8-byte store arrives whole), and the consumer polls the words it is about to use.  Destinations are
// double-buffered on the epoch's parity, so a stale word carries epoch e - 2 and can never be mistaken
// for a fresh one.  The consumer advances the channel's epoch when its last CTA finishes.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint4 ld_volatile_u4(const void* p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}

// Two consecutive (value, epoch) words; spins (bounded) until both carry epoch e.  Returns false after the time limit.
__device__ __forceinline__ bool ll_read2(const void* p, unsigned e, CommChan* ch, float& v0, float& v1) {
    uint4 w = ld_volatile_u4(p);
    if (w.y != e || w.w != e) {
        if (*(volatile int*)&ch->status != 0) {      // an earlier wait already ran out: do not wait again until the host clears it
            v0 = v1 = 0.f;
            return false;
        }
        const unsigned long long t0 = global_ns();
        const unsigned ms = ld_volatile_u32(&ch->wait_ms);
        const unsigned long long limit = (unsigned long long)(ms ? ms : 2000u) * 1000000ull;
        for (;;) {
            w = ld_volatile_u4(p);
            if (w.y == e && w.w == e) break;
            if (global_ns() - t0 > limit) {
                atomicExch(&ch->status, (int)KS_TIMEOUT);
                v0 = v1 = 0.f;
                return false;
            }
        }
    }
    v0 = __uint_as_float(w.x);
    v1 = __uint_as_float(w.z);
    return true;
}

// Consumer side: called by every thread at the end of the kernel; the last CTA makes `e` the channel's epoch.
__device__ __forceinline__ void ll_consumed(CommChan* ch, unsigned total_ctas, unsigned e) {
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned t = atomicAdd(&ch->ticket, 1u);
        if (t == total_ctas - 1u) {
            *(volatile unsigned*)&ch->ticket = 0u;
            *(volatile unsigned*)&ch->epoch = e;
        }
    }
}

// Adds one rank's partial row (low-latency protocol) to acc: thread `tid` of 256 owns float4 chunks tid + 256 j.
// All loads of the row are issued back to back and only then checked, so a row costs one L2 round trip when the
// data is already there (polling word by word would cost one round trip per word); words that have not arrived
// yet are re-read until the channel's time limit.
template <int MAXJ>
__device__ __forceinline__ void ll_add_row(const uint2* row, int tid, int nchunk, unsigned e, CommChan* ch, float4 (&acc)[MAXJ]) {
    uint4 w0[MAXJ], w1[MAXJ];
    unsigned long long t0 = 0, limit = 0;
    for (;;) {
#pragma unroll
        for (int j = 0; j < MAXJ; j++) {
            const int c = tid + 256 * j;
            if (c < nchunk) {
                w0[j] = ld_volatile_u4(row + 4 * c);
                w1[j] = ld_volatile_u4(row + 4 * c + 2);
            }
        }
        bool pending = false;
#pragma unroll
        for (int j = 0; j < MAXJ; j++) {
            const int c = tid + 256 * j;
            if (c < nchunk) pending |= (w0[j].y != e) | (w0[j].w != e) | (w1[j].y != e) | (w1[j].w != e);
        }
        if (!pending) break;
        if (*(volatile int*)&ch->status != 0) return;           // an earlier wait already ran out: contribute nothing
        if (limit == 0) {
            t0 = global_ns();
            const unsigned ms = ld_volatile_u32(&ch->wait_ms);
            limit = (unsigned long long)(ms ? ms : 2000u) * 1000000ull;
        } else if (global_ns() - t0 > limit) {
            atomicExch(&ch->status, (int)KS_TIMEOUT);
            return;
        }
    }
#pragma unroll
    for (int j = 0; j < MAXJ; j++) {
        const int c = tid + 256 * j;
        if (c < nchunk) {
            acc[j].x += __uint_as_float(w0[j].x); acc[j].y += __uint_as_float(w0[j].z);
            acc[j].z += __uint_as_float(w1[j].x); acc[j].w += __uint_as_float(w1[j].z);
        }
    }
}
