// Element-wise passes of the MLP block, one thread per element (pair).
// Replace the reference's NEON passes (csrc/neon_ops.cc: neon_glu_f16,
// neon_act_f16, neon_add_f16_to_f32, neon_f32_to_f16, neon_f16_to_f32) with the
// arithmetic of their portable statements (glu, src/linear.rs:804-835;
// add_f16, src/convert.rs:37-48).
#include "epilogue.cuh"
#include "kernels.h"

namespace smeg {
namespace {

// glu(): y[i][c0 + j] = f16( act_f32(both[i][2 c0 + j]) * both[i][2 c0 + w + j] ),
// gate and up interleaved 32 columns at a time (last chunk w < 32 wide).
__global__ void glu_kernel(uint16_t* __restrict__ out, const uint16_t* __restrict__ both, size_t m, size_t n,
                           uint32_t act) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= m * n) return;
    const size_t i = idx / n, col = idx % n;
    const size_t c0 = col & ~(size_t)31, j = col & 31;
    const size_t w = n - c0 < 32 ? n - c0 : 32;
    const uint16_t* br = both + i * 2 * n;
    const float g = __half2float(__ushort_as_half(br[2 * c0 + j]));
    const float u = __half2float(__ushort_as_half(br[2 * c0 + w + j]));
    const float a = glu_gate(act, g);
    out[idx] = __half_as_ushort(__float2half_rn(__fmul_rn(a, u)));
}

__global__ void add_f16_to_f32_kernel(float* __restrict__ dst, const uint16_t* __restrict__ src, size_t n) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx < n) dst[idx] = __fadd_rn(dst[idx], __half2float(__ushort_as_half(src[idx])));
}

// y += f32(f16(sum)): the residual add applied to an f32 sum of tensor-parallel
// partial products (the f16 rounding is the store of the down projection).
__global__ void round_add_f32_kernel(float* __restrict__ y, const float* __restrict__ s, size_t n) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx < n) y[idx] = __fadd_rn(y[idx], __half2float(__float2half_rn(s[idx])));
}

__global__ void act_f16_kernel(uint16_t* __restrict__ dst, const uint16_t* __restrict__ src, size_t n, uint32_t act) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx < n) dst[idx] = __half_as_ushort(__float2half_rn(act_apply(act, __half2float(__ushort_as_half(src[idx])), 0.0f)));
}

__global__ void f32_to_f16_kernel(uint16_t* __restrict__ dst, const float* __restrict__ src, size_t n) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx < n) dst[idx] = __half_as_ushort(__float2half_rn(src[idx]));
}
__global__ void f16_to_f32_kernel(float* __restrict__ dst, const uint16_t* __restrict__ src, size_t n) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx < n) dst[idx] = __half2float(__ushort_as_half(src[idx]));
}

// Sum over the 256 threads of a CTA (every thread gets it).
__device__ __forceinline__ float cta_sum(float v, float* sh) {
#pragma unroll
    for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();                       // sh may still be read from the previous call
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = 0.0f;
#pragma unroll
    for (int w = 0; w < 8; ++w) t += sh[w];
    return t;
}

// layer_norm / rms_norm of one row per CTA, f32 in, f16 (and / or f32) out: norm_row, src/nn.rs:126-153
// (the reference's NEON twin is neon_norm_row_f16, csrc/sme_gemm_api.h:221).  Same formula,
// (v - mean) * r * w + b with r = 1 / sqrt(ss / dim + eps), each operation rounded separately; the
// row sums are taken in another order than the reference's eight lanes, so results agree to f32 rounding.
__global__ void __launch_bounds__(256) norm_rows_kernel(uint16_t* __restrict__ y16, float* __restrict__ y32, const float* __restrict__ x,
                                                        const float* __restrict__ weight, const float* __restrict__ bias, size_t dim,
                                                        float eps, int rms) {
    __shared__ float sh[8];
    pdl_launch_dependents();
    pdl_wait();
    const float* xr = x + (size_t)blockIdx.x * dim;
    const float fdim = (float)dim;
    float mean = 0.0f;
    if (!rms) {
        float s = 0.0f;
        for (size_t j = threadIdx.x; j < dim; j += 256) s += xr[j];
        mean = __fdiv_rn(cta_sum(s, sh), fdim);
    }
    float ss = 0.0f;
    for (size_t j = threadIdx.x; j < dim; j += 256) {
        const float d = __fsub_rn(xr[j], mean);
        ss = __fmaf_rn(d, d, ss);
    }
    const float r = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(cta_sum(ss, sh), fdim), eps)));
    for (size_t j = threadIdx.x; j < dim; j += 256) {
        const float o = __fadd_rn(__fmul_rn(__fmul_rn(__fsub_rn(xr[j], mean), r), weight[j]), bias ? bias[j] : 0.0f);
        if (y16) y16[(size_t)blockIdx.x * dim + j] = __half_as_ushort(__float2half_rn(o));
        if (y32) y32[(size_t)blockIdx.x * dim + j] = o;
    }
}

// rms_scales, src/nn.rs:234-248: out[i] = f16(1 / sqrt(mean(x_i^2) + eps)) for each k-wide f16 row.
__global__ void __launch_bounds__(256) rms_scales_kernel(uint16_t* __restrict__ out, const uint16_t* __restrict__ x, size_t k, float eps) {
    __shared__ float sh[8];
    pdl_launch_dependents();
    pdl_wait();
    const uint16_t* xr = x + (size_t)blockIdx.x * k;
    float ss = 0.0f;
    for (size_t j = threadIdx.x; j < k; j += 256) {
        const float v = __half2float(__ushort_as_half(xr[j]));
        ss = __fmaf_rn(v, v, ss);
    }
    const float ms = __fdiv_rn(cta_sum(ss, sh), (float)k);
    if (threadIdx.x == 0) out[blockIdx.x] = __half_as_ushort(__float2half_rn(__fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(ms, eps)))));
}

inline unsigned blocks_for(size_t n) { return (unsigned)((n + 255) / 256); }

}  // namespace

cudaError_t glu_launch(uint16_t* out, const uint16_t* both, size_t m, size_t n, uint32_t act, cudaStream_t s) {
    if (m * n == 0) return cudaSuccess;
    return launch_pdl(glu_kernel, dim3(blocks_for(m * n)), dim3(256), 0, s, out, both, m, n, act);
}
cudaError_t add_f16_to_f32_launch(float* dst, const uint16_t* src, size_t n, cudaStream_t s) {
    if (n == 0) return cudaSuccess;
    return launch_pdl(add_f16_to_f32_kernel, dim3(blocks_for(n)), dim3(256), 0, s, dst, src, n);
}
cudaError_t round_add_f32_launch(float* y, const float* sum, size_t n, cudaStream_t s) {
    if (n == 0) return cudaSuccess;
    round_add_f32_kernel<<<blocks_for(n), 256, 0, s>>>(y, sum, n);
    return cudaGetLastError();
}
cudaError_t norm_rows_launch(uint16_t* y16, float* y32, const float* x, const float* weight, const float* bias, size_t rows, size_t dim,
                             float eps, int rms, cudaStream_t s) {
    if (rows == 0 || dim == 0) return cudaSuccess;
    return launch_pdl(norm_rows_kernel, dim3((unsigned)rows), dim3(256), 0, s, y16, y32, x, weight, bias, dim, eps, rms);
}
cudaError_t rms_scales_launch(uint16_t* out, const uint16_t* x, size_t rows, size_t k, float eps, cudaStream_t s) {
    if (rows == 0 || k == 0) return cudaSuccess;
    return launch_pdl(rms_scales_kernel, dim3((unsigned)rows), dim3(256), 0, s, out, x, k, eps);
}
cudaError_t act_f16_launch(uint16_t* dst, const uint16_t* src, size_t n, uint32_t act, cudaStream_t s) {
    if (n == 0) return cudaSuccess;
    act_f16_kernel<<<blocks_for(n), 256, 0, s>>>(dst, src, n, act);
    return cudaGetLastError();
}
cudaError_t f32_to_f16_launch(uint16_t* dst, const float* src, size_t n, cudaStream_t s) {
    if (n == 0) return cudaSuccess;
    f32_to_f16_kernel<<<blocks_for(n), 256, 0, s>>>(dst, src, n);
    return cudaGetLastError();
}
cudaError_t f16_to_f32_launch(float* dst, const uint16_t* src, size_t n, cudaStream_t s) {
    if (n == 0) return cudaSuccess;
    f16_to_f32_kernel<<<blocks_for(n), 256, 0, s>>>(dst, src, n);
    return cudaGetLastError();
}

}  // namespace smeg
