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
    float a;
    if (act == 3) a = __fdiv_rn(g, __fadd_rn(1.0f, expf(-g)));
    else {
        const float g3 = __fmul_rn(__fmul_rn(__fmul_rn(0.044715f, g), g), g);
        a = __fmul_rn(__fmul_rn(0.5f, g), __fadd_rn(1.0f, tanhf(__fmul_rn(0.7978846f, __fadd_rn(g, g3)))));
    }
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
