// Tensor-parallel plumbing: peer-mapped regions (CUDA IPC), flag waits and barriers, and the prefill-side
// "reduce + residual + RMSNorm + all-gather" kernel.
//
// Prefill keeps the residual stream sharded by token rows: rank r owns rows [r * rows_per_rank, ...).  A
// row-parallel GEMM (attention output / FFN down) writes each partial output tile straight into the parts
// buffer of the rank that owns those rows, as bf16 (kernels/gemm_tc.cu, scatter epilogue).  The kernel below then
// sums the partial rows into its shard of the residual stream, normalises, converts to bf16 and stores the
// row into the activation buffer of EVERY rank (peer stores), which is the operand of the next
// column-parallel GEMM.  One kernel therefore plays the parts of reduce-scatter's reduction, the residual add,
// the norm and the all-gather; the reference stack runs these as an NCCL all-reduce followed by separate
// add / norm kernels on every device.
#include <string.h>

#include "comm.cuh"

// ---------------------------------------------------------------------------------------------
// peer-mapped regions
// ---------------------------------------------------------------------------------------------
B2_API int b2_ipc_alloc(size_t bytes, void** ptr, unsigned char* handle64) {
    cudaError_t e = cudaMalloc(ptr, bytes);
    if (e != cudaSuccess) return (int)e;
    e = cudaMemset(*ptr, 0, bytes);
    if (e != cudaSuccess) return (int)e;
    cudaIpcMemHandle_t h;
    e = cudaIpcGetMemHandle(&h, *ptr);
    if (e != cudaSuccess) return (int)e;
    static_assert(sizeof(h) == 64, "IPC handle size");
    memcpy(handle64, &h, 64);
    return (int)cudaDeviceSynchronize();
}

B2_API int b2_ipc_open(const unsigned char* handle64, void** ptr) {
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    return (int)cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess);
}

B2_API int b2_ipc_close(void* ptr) { return (int)cudaIpcCloseMemHandle(ptr); }
B2_API int b2_ipc_free(void* ptr) { return (int)cudaFree(ptr); }

// ---------------------------------------------------------------------------------------------
// waits and barriers
// ---------------------------------------------------------------------------------------------
__global__ void comm_wait_kernel(CommChan* ch, int n) {
    pdl_launch();
    pdl_wait();
    const unsigned e = ld_volatile_u32(&ch->epoch);
    comm_wait_flags(ch, n, e);
}

// Blocks the stream until every rank's flag on `ch` has reached this rank's own epoch on that channel, i.e.
// until every rank has published the exchange this rank published last.
B2_API int b2_comm_wait(CommChan* ch, int n, int pdl, cudaStream_t st) {
    if (n < 1 || n > COMM_MAX_RANKS) return (int)cudaErrorInvalidValue;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(1);
    cfg.blockDim = dim3(32);
    cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = pdl ? 1 : 0;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    void* args[] = {&ch, &n};
    return (int)cudaLaunchKernelExC(&cfg, (const void*)comm_wait_kernel, args);
}

__global__ void comm_barrier_kernel(const __grid_constant__ CommSend cm) {
    __shared__ unsigned s_e;
    if (threadIdx.x == 0) {
        const unsigned e = comm_next_epoch(cm);
        *(volatile unsigned*)&cm.local->epoch = e;
        __threadfence_system();
        for (int r = 0; r < cm.n_dst; r++) st_release_sys_u32(cm.peer_flag[r], e);
        s_e = e;
    }
    __syncthreads();
    comm_wait_flags(cm.local, cm.n_dst, s_e);
}

// All work enqueued before this call on every rank's stream has finished when the kernel returns on any rank.
B2_API int b2_comm_barrier(const CommSend* cm, cudaStream_t st) {
    if (cm->n_dst < 1 || cm->n_dst > COMM_MAX_RANKS) return (int)cudaErrorInvalidValue;
    comm_barrier_kernel<<<1, 32, 0, st>>>(*cm);
    return (int)cudaGetLastError();
}

// Status word of a channel (0 ok, 1 a wait ran out); synchronises the stream it is called on.
B2_API int b2_comm_status(const CommChan* ch, int* status, cudaStream_t st) {
    cudaError_t e = cudaMemcpyAsync(status, &ch->status, sizeof(int), cudaMemcpyDeviceToHost, st);
    if (e != cudaSuccess) return (int)e;
    return (int)cudaStreamSynchronize(st);
}

// ---------------------------------------------------------------------------------------------
// prefill: x_shard += sum(parts);  h = rmsnorm(x_shard) * w  ->  bf16 row on every rank
// ---------------------------------------------------------------------------------------------
struct TpNormGatherArgs {
    float* x;                 // [rows][k] this rank's shard of the residual stream (updated in place)
    const __nv_bfloat16* parts;   // [n_part][part_rows][k] partial rows (bf16) received from the group (n_part = 0: nothing to add)
    int n_part;
    long long part_stride;    // elements between the slabs of two ranks
    CommChan* rs_chan;        // channel the partial rows were announced on
    const float* w;           // [k] norm weight or null
    float eps;
    int k;                    // <= 8192, multiple of 8
    int row0;                 // global index of this rank's first row
    CommSend ag;              // dst[r] = bf16 activation buffer [T][k] on rank r (passed as float*); announces on its own channel
};

__global__ void __launch_bounds__(256) tp_norm_gather_kernel(const __grid_constant__ TpNormGatherArgs a, int rows) {
    constexpr int MAXJ = 8;
    __shared__ float red[8];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nchunk = a.k >> 2;
    const unsigned ep = comm_next_epoch(a.ag);
    if (a.n_part) {
        const unsigned e = ld_volatile_u32(&a.rs_chan->epoch);
        comm_wait_flags(a.rs_chan, a.n_part, e);
        __syncthreads();
    }
    for (int b = blockIdx.x; b < rows; b += gridDim.x) {
        float* x = a.x + (size_t)b * a.k;
        float4 v[MAXJ];
#pragma unroll
        for (int j = 0; j < MAXJ; j++) {
            const int c = tid + 256 * j;
            v[j] = c < nchunk ? *(const float4*)(x + 4 * c) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        if (a.n_part) {
            for (int r = 0; r < a.n_part; r++) {
                const __nv_bfloat16* p = a.parts + r * a.part_stride + (size_t)b * a.k;
#pragma unroll
                for (int j = 0; j < MAXJ; j++) {
                    const int c = tid + 256 * j;
                    if (c < nchunk) {
                        const uint2 t = __ldcg((const uint2*)(p + 4 * c));        // written by a peer: read through L2
                        const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&t.x));
                        const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&t.y));
                        v[j].x += lo.x; v[j].y += lo.y; v[j].z += hi.x; v[j].w += hi.y;
                    }
                }
            }
#pragma unroll
            for (int j = 0; j < MAXJ; j++) {
                const int c = tid + 256 * j;
                if (c < nchunk) *(float4*)(x + 4 * c) = v[j];
            }
        }
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < MAXJ; j++) ss += v[j].x * v[j].x + v[j].y * v[j].y + v[j].z * v[j].z + v[j].w * v[j].w;
        ss = warp_sum(ss);
        __syncthreads();
        if (lane == 0) red[warp] = ss;
        __syncthreads();
        float t = lane < 8 ? red[lane] : 0.f;
        t = warp_sum(t);
        const float inv = rsqrtf(t / (float)a.k + a.eps);
        const size_t grow = (size_t)(a.row0 + b) * a.k;
#pragma unroll
        for (int j = 0; j < MAXJ; j++) {
            const int c = tid + 256 * j;
            if (c >= nchunk) continue;
            float4 y = v[j];
            y.x *= inv; y.y *= inv; y.z *= inv; y.w *= inv;
            if (a.w) {
                const float4 ww = *(const float4*)(a.w + 4 * c);
                y.x *= ww.x; y.y *= ww.y; y.z *= ww.z; y.w *= ww.w;
            }
            const __nv_bfloat162 lo = __floats2bfloat162_rn(y.x, y.y), hi = __floats2bfloat162_rn(y.z, y.w);
            uint2 pk;
            pk.x = *reinterpret_cast<const uint32_t*>(&lo);
            pk.y = *reinterpret_cast<const uint32_t*>(&hi);
            for (int d = 0; d < a.ag.n_dst; d++)
                *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(a.ag.dst[d]) + grow + 4 * (size_t)c) = pk;
        }
    }
    comm_publish(a.ag, gridDim.x, ep);
}

// `rows` may be 0 (a rank that owns no row of a short chunk still has to announce).
B2_API int b2_tp_norm_gather(const TpNormGatherArgs* a, int rows, cudaStream_t st) {
    if (a->k > 8192 || (a->k & 7) || a->n_part < 0 || a->n_part > COMM_MAX_RANKS || a->ag.n_dst < 1 || a->ag.n_dst > COMM_MAX_RANKS)
        return (int)cudaErrorInvalidValue;
    const int grid = rows < 1 ? 1 : (rows < 1184 ? rows : 1184);
    tp_norm_gather_kernel<<<grid, 256, 0, st>>>(*a, rows);
    return (int)cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------
// prefill fallback: scatter rows of a locally computed partial result to their owners
// (used when the producing GEMM has no scatter epilogue for the weight's encoding)
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) tp_scatter_rows_kernel(const float* src, int m, int k, int rows_per_rank, const __grid_constant__ CommSend cm) {
    const unsigned ep = comm_next_epoch(cm);
    const int nchunk = k >> 2;
    for (int row = blockIdx.x; row < m; row += gridDim.x) {
        const int owner = row / rows_per_rank, lrow = row - owner * rows_per_rank;
        __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(cm.dst[owner]) + (size_t)lrow * k;
        const float* s = src + (size_t)row * k;
        for (int c = threadIdx.x; c < nchunk; c += 256) {
            const float4 v = *(const float4*)(s + 4 * c);
            const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
            uint2 pk;
            pk.x = *reinterpret_cast<const uint32_t*>(&lo);
            pk.y = *reinterpret_cast<const uint32_t*>(&hi);
            *(uint2*)(dst + 4 * c) = pk;
        }
    }
    comm_publish(cm, gridDim.x, ep);
}

B2_API int b2_tp_scatter_rows(const float* src, int m, int k, int rows_per_rank, const CommSend* cm, cudaStream_t st) {
    if (m < 1 || (k & 3) || rows_per_rank < 1 || cm->n_dst < 1 || cm->n_dst > COMM_MAX_RANKS || (m + rows_per_rank - 1) / rows_per_rank > cm->n_dst)
        return (int)cudaErrorInvalidValue;
    const int grid = m < 1184 ? m : 1184;
    tp_scatter_rows_kernel<<<grid, 256, 0, st>>>(src, m, k, rows_per_rank, *cm);
    return (int)cudaGetLastError();
}
