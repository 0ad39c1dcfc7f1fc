// Causal attention against an f16 key/value cache, and the append into that cache (sm_100a) -- the attention step of
// SelfAttention::accumulate (src/self_attention.rs:189-231) between its two projections:
//   attention_kv_causal_f16 / attention_kv_f16 (src/kernels/kv_attention.rs:29-331): query row i of a block attends to
//   keys 0..=start+i; per head softmax(f16(q * scale) . k) @ v, f32 sums in key / depth order, f32 probabilities
//   exp(s - max), the division by their sum last.  Query head h uses KV head h / (heads / kv_heads).
//   KvCache::extend (:499-520): a block's key and value rows copied to the cache's next positions.
//
// One CTA per (query row, head).  A thread owns keys t, t + 128, ...: its score is the depth-ordered f32 sum the scalar
// statement forms (separately rounded multiply and add), so scores -- and the maximum -- are the reference's bits; the
// probabilities differ from libm's by the device expf, their sum by summation order.  The value pass gives every thread
// one depth and walks the keys in order (the reference's order again), lanes reading consecutive depths of a row.  This is
// the plain form for decode steps and moderate prompts: scores of one (row, head) live in shared memory (up to ~50 k
// keys), nothing is tiled for the tensor cores.
#include "common.cuh"
#include "kernels.h"

namespace smeg {
namespace {

constexpr int kAttnThreads = 128;

__device__ __forceinline__ float block_reduce(float v, float* red, bool is_max) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o; o >>= 1) {
        const float u = __shfl_xor_sync(0xffffffffu, v, o);
        v = is_max ? fmaxf(v, u) : v + u;
    }
    __syncthreads();                                   // red may still be read from the previous reduction
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float r = red[0];
    for (int w = 1; w < kAttnThreads / 32; ++w) r = is_max ? fmaxf(r, red[w]) : r + red[w];
    return r;
}

template <int QF32>
__global__ void __launch_bounds__(kAttnThreads) attn_kv_causal_kernel(const __grid_constant__ AttnArgs p) {
    extern __shared__ __align__(16) float smem_f[];
    const int h = blockIdx.x, i = blockIdx.y, tid = threadIdx.x;
    const int hd = p.head_dim, ld = p.kv_heads * hd, group = p.heads / p.kv_heads;
    const int off = (h / group) * hd;
    const int len = p.start + i + 1;
    float* qh = smem_f;                                // [hd] f16-rounded scaled query
    float* red = qh + hd;                              // [4]
    float* scores = red + 8;                           // [len]
    for (int d = tid; d < hd; d += kAttnThreads) {
        float x;
        if (QF32) x = reinterpret_cast<const float*>(p.q)[(size_t)i * p.q_stride + (size_t)h * hd + d];
        else x = __half2float(__ushort_as_half(reinterpret_cast<const uint16_t*>(p.q)[(size_t)i * p.q_stride + (size_t)h * hd + d]));
        qh[d] = __half2float(__float2half_rn(__fmul_rn(x, p.scale)));
    }
    __syncthreads();
    // ---- scores: s_t = sum_d qh[d] * k[t][d], d ascending ----
    float mx = -INFINITY;
    for (int t = tid; t < len; t += kAttnThreads) {
        const uint4* kr = reinterpret_cast<const uint4*>(p.k + (size_t)t * ld + off);      // head_dim % 8 == 0: 16-byte vectors
        float s = 0.0f;
        for (int c = 0; c < hd / 8; ++c) {
            const uint4 kv = kr[c];
            const uint32_t w[4] = {kv.x, kv.y, kv.z, kv.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[e]));
                s = __fadd_rn(s, __fmul_rn(qh[8 * c + 2 * e], f.x));
                s = __fadd_rn(s, __fmul_rn(qh[8 * c + 2 * e + 1], f.y));
            }
        }
        scores[t] = s;
        mx = fmaxf(mx, s);
    }
    mx = block_reduce(mx, red, true);
    float sum = 0.0f;
    for (int t = tid; t < len; t += kAttnThreads) {
        const float e = expf(__fsub_rn(scores[t], mx));
        scores[t] = e;
        sum += e;
    }
    sum = block_reduce(sum, red, false);               // (its barriers also publish the probabilities)
    // ---- values: out[d] = (sum_t p_t * v[t][d]) / sum, t ascending ----
    for (int d = tid; d < hd; d += kAttnThreads) {
        const uint16_t* vc = p.v + off + d;
        float o = 0.0f;
        for (int t = 0; t < len; ++t) o = __fadd_rn(o, __fmul_rn(scores[t], __half2float(__ushort_as_half(vc[(size_t)t * ld]))));
        p.out[(size_t)i * p.heads * hd + (size_t)h * hd + d] = __fdiv_rn(o, sum);
    }
}

// rows x row_len f16 values from a strided source (the k or v part of projected [q | k | v] rows) to cache rows pos...
__global__ void kv_append_kernel(uint16_t* __restrict__ kc, uint16_t* __restrict__ vc, const uint16_t* __restrict__ src, size_t stride,
                                 size_t k_off, size_t v_off, size_t row_len, size_t pos, size_t rows) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= rows * row_len) return;
    const size_t r = idx / row_len, c = idx - r * row_len;
    kc[(pos + r) * row_len + c] = src[r * stride + k_off + c];
    vc[(pos + r) * row_len + c] = src[r * stride + v_off + c];
}

}  // namespace

cudaError_t attn_kv_causal_launch(const AttnArgs& a, int q_f32, cudaStream_t stream) {
    const size_t smem = ((size_t)a.head_dim + 8 + (size_t)(a.start + a.rows)) * sizeof(float);
    if (smem > 200 * 1024) return cudaErrorInvalidValue;
    cudaError_t e;
    if (q_f32) e = cudaFuncSetAttribute(attn_kv_causal_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    else e = cudaFuncSetAttribute(attn_kv_causal_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return e;
    const dim3 grid(a.heads, a.rows);
    if (q_f32) attn_kv_causal_kernel<1><<<grid, kAttnThreads, smem, stream>>>(a);
    else attn_kv_causal_kernel<0><<<grid, kAttnThreads, smem, stream>>>(a);
    return cudaGetLastError();
}

cudaError_t kv_append_launch(uint16_t* kc, uint16_t* vc, const uint16_t* src, size_t stride, size_t k_off, size_t v_off, size_t row_len,
                             size_t pos, size_t rows, cudaStream_t stream) {
    const size_t total = rows * row_len;
    if (total == 0) return cudaSuccess;
    kv_append_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(kc, vc, src, stride, k_off, v_off, row_len, pos, rows);
    return cudaGetLastError();
}

}  // namespace smeg
