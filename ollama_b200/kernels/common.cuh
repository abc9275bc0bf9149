// Shared helpers for the sm_100a kernels.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define B2_API extern "C" __attribute__((visibility("default")))

// Weight encodings as laid out in device memory after load-time repacking into planes
// (every plane is a dense row-major array, so all accesses are naturally aligned).
enum WType : int {
    WT_F32 = 0,    // p0: float  [N][K]
    WT_F16 = 1,    // p0: half   [N][K]
    WT_BF16 = 2,   // p0: bf16   [N][K]
    WT_Q8_0 = 3,   // p0: int8   [N][K]        p1: half [N][K/32]
    WT_Q4_K = 4,   // p0: u8     [N][K/2]      p1: u8 [N][K/256][16] = 4 x {sc(2j), sc(2j+1), min(2j), min(2j+1)}   p2: {half d, half dmin} [N][K/256]
    WT_Q6_K = 5,   // p0: ql u8  [N][K/2]      p1: qh u8 [N][K/4]   p2: int8 scales [N][K/16]   p3: half d [N][K/256]
    WT_Q5_K = 6,   // p0..p2 as Q4_K           p3: qh u8 [N][K/8]
    WT_MXFP4 = 7,  // p0: u8     [N][K/2]      p1: e8m0 u8 [N][K/32]
    WT_Q4_0 = 8,   // p0: u8     [N][K/2]      p1: half d [N][K/32]
};

struct WDesc {
    const void* p0;
    const void* p1;
    const void* p2;
    const void* p3;
    const float* bias;   // [N] or null
    int type;
    int n;               // rows
    int k;               // row length (elements)
    int out_off;         // column offset of this segment in the output row
};

// Function attributes (dynamic shared memory opt-in) are per device: first() is true once per device and call site.
struct PerDeviceOnce {
    bool done[64] = {};
    bool first() {
        int d = 0;
        cudaGetDevice(&d);
        d &= 63;
        const bool f = !done[d];
        done[d] = true;
        return f;
    }
};

// Status word written by kernels that can give up (bounded waits, bad arguments); 0 = ok.
enum KStatus : int { KS_OK = 0, KS_TIMEOUT = 1, KS_BAD_ARG = 2 };

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

__device__ __forceinline__ uint4 ldg16(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint2 ldg8(const void* p) {
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}

// Programmatic dependent launch: wait for the producer grid / let the consumer grid start early.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ float bf16_bits_to_float(uint32_t lo16) { return __uint_as_float(lo16 << 16); }

__device__ __forceinline__ float e8m0_to_float(uint32_t e) {
    // 2^(e-127); e == 0 denotes 2^-127 (subnormal in fp32)
    return e == 0 ? __uint_as_float(0x00400000u) : __uint_as_float(e << 23);
}

// Gated FFN activation: 0 = SiLU(g) * u, 1 = tanh-GELU(g) * u, 2 = clamped SwiGLU with alpha and limit (gpt-oss).
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
