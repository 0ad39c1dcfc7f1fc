// Tensor-parallel finish of the MLP block in one kernel over peer memory: the ranks' f32 partial
// products are summed, rounded to f16 like the down projection's store, and added to the residual
// stream -- the all-reduce and the last two passes of Mlp::accumulate (src/mlp.rs:124-146: out = f16(down(hid));
// y += f32(out)) fused.
//
// Every rank holds its partial product in a buffer that all ranks can address (NVLink peer mapping) and
// a small flag array.  Two-shot scheme, one launch per rank, no host round trip:
//   0. a rank tells every peer that its partial is complete (flag "ready");
//   1. rank r owns slice r of the output: it reads that slice from every rank's buffer, adds the
//      values in rank order 0..W-1 (so every element has one summation order whatever the timing),
//      rounds to f16 and writes the result back into slice r of every rank's buffer;
//   2. when all of a rank's CTAs have done that, it tells every peer (flag "done"); a rank that has
//      all W "done" flags adds its own buffer, now holding the reduced values, to its residual stream.
// Flags carry the call's sequence number and only grow, so nothing is reset between calls.  A rank
// leaves the kernel only after every owner has finished reading its buffer, so the next step may
// overwrite the buffer at once.  Short vectors take a one-shot form instead (every rank adds all the
// partials itself after the "ready" flags; see the kernel).  Every wait is bounded: after a second it raises the
// status word and the kernel returns without touching y.
#include "common.cuh"
#include "kernels.h"

namespace smeg {
namespace {

__device__ unsigned g_ar_ctas_done;   // CTAs of this device's launch that finished their slice; zero at rest

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ float4 ld_sys_f4(const float* p) {
    float4 v;
    asm volatile("ld.relaxed.sys.global.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_sys_f4(float* p, float4 v) {
    asm volatile("st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}
__device__ __forceinline__ float round_f16(float x) { return __half2float(__float2half_rn(x)); }

// Waits until *flag >= seq (sequence numbers compared as a signed difference).  One second at most.
__device__ __forceinline__ bool wait_flag(const uint32_t* flag, uint32_t seq) {
    const unsigned long long t0 = global_ns();
    for (;;) {
        if ((int)(ld_acquire_sys(flag) - seq) >= 0) return true;
        if (global_ns() - t0 > 1000000000ull) return false;
        __nanosleep(200);
    }
}

__global__ void __launch_bounds__(256) tp_reduce_finish_kernel(const __grid_constant__ TpReduceArgs p) {
    __shared__ int s_fail, s_last;
    const int tid = threadIdx.x, W = p.world, r = p.rank;
    if (tid == 0) { s_fail = 0; s_last = 0; }
    __syncthreads();

    // ---- 0: my partial (written by the kernel ahead in the stream) is complete: tell every rank ----
    if (blockIdx.x == 0 && tid < W) {
        __threadfence_system();
        st_release_sys(p.flags[tid] + r, p.seq);
    }
    if (tid < W && !wait_flag(p.flags[r] + tid, p.seq)) s_fail = 1;
    __syncthreads();
    if (s_fail) {
        if (tid == 0 && p.status) atomicOr(p.status, STATUS_PEER_TIMEOUT);
        return;
    }

    const size_t nvec = p.len / 4;
    if (p.oneshot) {
        // Short vectors: every rank adds all the partials itself (same rank order, so the same bits everywhere) and
        // needs no second flag round.  The caller alternates between two buffers: a rank overwrites the buffer of
        // step n in step n + 2, after step n + 1's "ready" flags told it that every peer had finished step n.
        for (size_t v = (size_t)blockIdx.x * blockDim.x + tid; v < nvec; v += (size_t)gridDim.x * blockDim.x) {
            float4 acc = ld_sys_f4(p.bufs[0] + 4 * v);
            for (int s = 1; s < W; ++s) {
                const float4 x = ld_sys_f4(p.bufs[s] + 4 * v);
                acc.x = __fadd_rn(acc.x, x.x); acc.y = __fadd_rn(acc.y, x.y);
                acc.z = __fadd_rn(acc.z, x.z); acc.w = __fadd_rn(acc.w, x.w);
            }
            float4 y = reinterpret_cast<float4*>(p.y)[v];
            y.x = __fadd_rn(y.x, round_f16(acc.x)); y.y = __fadd_rn(y.y, round_f16(acc.y));
            y.z = __fadd_rn(y.z, round_f16(acc.z)); y.w = __fadd_rn(y.w, round_f16(acc.w));
            reinterpret_cast<float4*>(p.y)[v] = y;
        }
        return;
    }

    // ---- 1: my slice, in float4 ----
    const size_t per = (nvec + W - 1) / W;
    const size_t v0 = per * r, v1 = min(nvec, v0 + per);
    for (size_t v = v0 + (size_t)blockIdx.x * blockDim.x + tid; v < v1; v += (size_t)gridDim.x * blockDim.x) {
        float4 acc = ld_sys_f4(p.bufs[0] + 4 * v);
        for (int s = 1; s < W; ++s) {
            const float4 x = ld_sys_f4(p.bufs[s] + 4 * v);
            acc.x = __fadd_rn(acc.x, x.x); acc.y = __fadd_rn(acc.y, x.y);
            acc.z = __fadd_rn(acc.z, x.z); acc.w = __fadd_rn(acc.w, x.w);
        }
        acc.x = round_f16(acc.x); acc.y = round_f16(acc.y); acc.z = round_f16(acc.z); acc.w = round_f16(acc.w);
        for (int s = 0; s < W; ++s) st_sys_f4(p.bufs[s] + 4 * v, acc);
    }
    __threadfence_system();
    __syncthreads();
    if (tid == 0) {
        const unsigned old = atomicAdd(&g_ar_ctas_done, 1u);
        s_last = old == gridDim.x - 1;
    }
    __syncthreads();
    if (s_last) {
        // ---- 2: every CTA of this rank has written its part of slice r everywhere ----
        __threadfence_system();
        if (tid < W) st_release_sys(p.flags[tid] + 8 + r, p.seq);
        if (tid == 0) g_ar_ctas_done = 0;
    }
    if (tid < W && !wait_flag(p.flags[r] + 8 + tid, p.seq)) s_fail = 1;
    __syncthreads();
    if (s_fail) {
        if (tid == 0 && p.status) atomicOr(p.status, STATUS_PEER_TIMEOUT);
        return;
    }

    // ---- residual add from my own buffer, which now holds the reduced, rounded values ----
    const float* mine = p.bufs[r];
    for (size_t v = (size_t)blockIdx.x * blockDim.x + tid; v < nvec; v += (size_t)gridDim.x * blockDim.x) {
        const float4 s = ld_sys_f4(mine + 4 * v);
        float4 y = reinterpret_cast<float4*>(p.y)[v];
        y.x = __fadd_rn(y.x, s.x); y.y = __fadd_rn(y.y, s.y); y.z = __fadd_rn(y.z, s.z); y.w = __fadd_rn(y.w, s.w);
        reinterpret_cast<float4*>(p.y)[v] = y;
    }
}

}  // namespace

cudaError_t tp_reduce_finish_launch(const TpReduceArgs& a, int sm_count, cudaStream_t stream) {
    // at most one CTA per SM: the CTAs of a rank meet at the "done" round, so all of them must be resident
    const size_t nvec = a.len / 4;
    size_t ctas = ((a.oneshot ? nvec : nvec / a.world) + 255) / 256;
    if (ctas < 1) ctas = 1;
    if (ctas > (size_t)sm_count) ctas = (size_t)sm_count;
    tp_reduce_finish_kernel<<<(unsigned)ctas, 256, 0, stream>>>(a);
    return cudaGetLastError();
}

}  // namespace smeg
