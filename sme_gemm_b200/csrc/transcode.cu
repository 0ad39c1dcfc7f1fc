// 2-bit / 1-bit packed weights -> a 4-bit plane for the tensor-core GEMM.
//
// The reference's f16 MOPA path for these weights (matmul_q2_mopa / matmul_q1_mopa,
// src/kernels/lowbit/matmul.rs:100-139) multiplies f16 activations by the weights
// w(d, j) = f16( scale(d / block, j) * value ) with value = codebook[code] or +-1
// (Codes::dequant, src/kernels/lowbit/matmul.rs:178-197; unpack_q2_f16 / unpack_q1_f16,
// csrc/gemm_f16f16_lowbit.h:51-169).  scale is an f16 and |value| <= 127, so the f32
// product is exact and the f16 conversion is the only rounding: exactly what the 4-bit
// dequant does for the signed code `value` with the same per-block scale
// (dequant_rows, src/kernels/q4/weights.rs:232-259).  A weight set whose values all lie
// in [-8, 7] -- the ternary and sign formats do -- therefore has a 4-bit twin with
// bit-identical dequantised weights, and the prefill GEMM of gemm_tc.cu serves it
// unchanged.  This file builds that twin on the device, once per weight set.
#include "kernels.h"
#include "layout.h"

namespace smeg {
namespace {

// One thread per 32-bit word of the 4-bit plane: eight (depth, column) cells.
__global__ void lowbit_to_q4_kernel(LowbitToQ4Args p) {
    const size_t word = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (word >= p.dst_words) return;
    const int ks = (int)(word & 3), lane = (int)((word >> 2) & 31);
    const size_t unit = word >> 7;
    const size_t u = unit % p.ku4, cg = unit / p.ku4;
    const int g = lane >> 2, t = lane & 3;
    const size_t dbase = 64 * u + 32 * (size_t)(ks >> 1) + 8 * (size_t)t + 4 * (size_t)(ks & 1);
    uint32_t out = 0;
#pragma unroll
    for (int nib = 0; nib < 8; ++nib) {
        const int e = ((nib & 1) << 1) | (nib >> 2), hi = (nib >> 1) & 1;
        const size_t d = dbase + (size_t)e, j = 16 * cg + (size_t)g + 8 * (size_t)hi;
        int value = 0;
        if (d < p.k && j < p.n) {
            size_t wb;
            int f;
            if (p.bits == 2) {
                q2_locate(d, j, p.ku_src, &wb, &f);
                const uint32_t w = *reinterpret_cast<const uint32_t*>(p.src + wb);
                const uint32_t code = (w >> (2 * f)) & 3u;
                value = (int)(int8_t)((p.lut >> (8 * code)) & 0xffu);
            } else {
                q1_locate(d, j, p.ku_src, &wb, &f);
                const uint32_t w = *reinterpret_cast<const uint32_t*>(p.src + wb);
                value = ((w >> f) & 1u) ? 1 : -1;
            }
        }
        out |= (uint32_t)((value + 8) & 15) << (4 * nib);
    }
    reinterpret_cast<uint32_t*>(p.dst)[word] = out;
}

// Scale rows [column group][K-block][16]: same slots, the 4-bit plane's own row count and
// column-group padding.
__global__ void lowbit_scales_to_q4_kernel(LowbitToQ4Args p) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= p.dst_scale_elems) return;
    const size_t slot = idx & 15, row = idx >> 4;
    const size_t blk = row % p.nb4, cg = row / p.nb4;
    uint16_t v = 0;
    if (cg < p.n16_src && blk < p.nb_src) v = p.src_scales[(cg * p.nb_src + blk) * 16 + slot];
    p.dst_scales[idx] = v;
}

// A 2-bit codebook with a value outside [-8, 7] has no 4-bit twin: its weights are written out as the dense
// K-major f16 matrix W[n][kd] the tensor-core GEMM takes directly, each f16(scale * value) -- the eager
// dequant of the reference's fallback arm (prepack_f16(Codes::dequant()), src/kernels/lowbit/matmul.rs:347-349).
// One thread per weight.
__global__ void lowbit_to_dense_kernel(LowbitToQ4Args p, uint16_t* dst, size_t kd, int log2_block) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= p.n * kd) return;
    const size_t j = idx / kd, d = idx % kd;
    uint16_t out = 0;
    if (d < p.k) {
        size_t wb;
        int f;
        int value;
        if (p.bits == 2) {
            q2_locate(d, j, p.ku_src, &wb, &f);
            const uint32_t w = *reinterpret_cast<const uint32_t*>(p.src + wb);
            value = (int)(int8_t)((p.lut >> (8 * ((w >> (2 * f)) & 3u))) & 0xffu);
        } else {
            q1_locate(d, j, p.ku_src, &wb, &f);
            const uint32_t w = *reinterpret_cast<const uint32_t*>(p.src + wb);
            value = ((w >> f) & 1u) ? 1 : -1;
        }
        const float s = __half2float(__ushort_as_half(p.src_scales[((j / 16) * p.nb_src + (d >> log2_block)) * 16 + scale_slot((int)(j % 16))]));
        out = __half_as_ushort(__float2half_rn(__fmul_rn(s, (float)value)));   // the f32 product is exact: one rounding
    }
    dst[idx] = out;
}

}  // namespace

cudaError_t lowbit_to_dense_launch(const LowbitToQ4Args& a, uint16_t* dst, size_t kd, int log2_block, cudaStream_t s) {
    const size_t total = a.n * kd;
    if (total) lowbit_to_dense_kernel<<<(unsigned)((total + 255) / 256), 256, 0, s>>>(a, dst, kd, log2_block);
    return cudaGetLastError();
}

cudaError_t lowbit_to_q4_launch(const LowbitToQ4Args& a, cudaStream_t s) {
    if (a.dst_words) lowbit_to_q4_kernel<<<(unsigned)((a.dst_words + 255) / 256), 256, 0, s>>>(a);
    if (a.dst_scale_elems) lowbit_scales_to_q4_kernel<<<(unsigned)((a.dst_scale_elems + 255) / 256), 256, 0, s>>>(a);
    return cudaGetLastError();
}

}  // namespace smeg
