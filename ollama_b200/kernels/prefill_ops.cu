// Element-wise glue of the prefill path (between tensor-core GEMMs): gated activation on the interleaved
// gate/up GEMM result.  In the reference stack these are ggml-cuda's unary / glu kernels.
#include "common.cuh"

struct GluRowsArgs {
    const __nv_bfloat16* gu;   // [rows][2 * f]: column 2i = gate_i, 2i + 1 = up_i (the row-interleaved gate/up matrix as GEMM output)
    __nv_bfloat16* out;        // [rows][f]
    int f;                     // multiple of 4
    int act;                   // 0 silu, 1 gelu_tanh, 2 clamped swiglu (alpha, limit)
    float alpha, limit;
};

__device__ __forceinline__ float glu_one(float g, float u, int act, float alpha, float limit) {
    if (act == 0) return g / (1.f + __expf(-g)) * u;
    if (act == 1) {
        const float t = tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g));
        return 0.5f * g * (1.f + t) * u;
    }
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return g / (1.f + __expf(-alpha * g)) * (u + 1.f);
}

// one thread = 4 outputs = 8 inputs (one 16-byte load, one 8-byte store)
__global__ void __launch_bounds__(256) glu_rows_kernel(const __grid_constant__ GluRowsArgs a, long long total4) {
    for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < total4; i += (long long)gridDim.x * 256) {
        const uint4 v = *reinterpret_cast<const uint4*>(a.gu + 8 * i);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
        float r[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float2 p = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[j]));
            r[j] = glu_one(p.x, p.y, a.act, a.alpha, a.limit);
        }
        const __nv_bfloat162 lo = __floats2bfloat162_rn(r[0], r[1]), hi = __floats2bfloat162_rn(r[2], r[3]);
        uint2 o;
        o.x = *reinterpret_cast<const uint32_t*>(&lo);
        o.y = *reinterpret_cast<const uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(a.out + 4 * i) = o;
    }
}

// gu and out dense (row pitch 2f and f).  Returns a cudaError_t value.
B2_API int b2_glu_rows(const GluRowsArgs* a, int rows, cudaStream_t st) {
    if (rows < 1 || a->f < 4 || (a->f & 3) || ((uintptr_t)a->gu & 15) || ((uintptr_t)a->out & 7)) return (int)cudaErrorInvalidValue;
    const long long total4 = (long long)rows * a->f / 4;
    const int grid = (int)((total4 + 255) / 256 < 148 * 8 ? (total4 + 255) / 256 : 148 * 8);
    GluRowsArgs copy = *a;
    glu_rows_kernel<<<grid, 256, 0, st>>>(copy, total4);
    return (int)cudaGetLastError();
}
