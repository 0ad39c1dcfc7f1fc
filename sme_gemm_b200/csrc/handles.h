// The opaque weight handles of the C ABI (include/smeg_api.h), shared by the
// translation units that implement entry points.
#pragma once
#include <stdint.h>

#include <atomic>
#include <mutex>
#include <vector>

#include "pack.h"

struct smeg_dense;
struct smeg_q4 {
    smeg::PackedDims d;
    unsigned char* codes = nullptr;   // device: packed units
    uint16_t* scales = nullptr;       // device: f16 scale rows
    size_t code_bytes = 0, scale_elems = 0;
    // Affine form (Q4_1: weight = scale * code + min).  The reference's prefill path expands it once to the 16-bit
    // operand type -- round_T(f64(scale) * code + f64(min)), src/kernels/q4/weights.rs:250-256 -- and multiplies dense;
    // this build keeps the logical arrays and runs such weights through dense twins of exactly those values, one per
    // operand type, built on the first call of that type.
    bool affine = false;
    std::vector<uint8_t> h_quants;
    std::vector<uint16_t> h_scales, h_mins;
    mutable std::mutex twin_lock;
    mutable std::atomic<smeg_dense*> twin_f16{nullptr}, twin_bf16{nullptr};
};
struct smeg_lowbit {
    smeg::PackedDims d;
    int bits = 0;                     // 2 or 1
    uint32_t lut = 0;                 // 2-bit codebook, byte c = value of code c
    int8_t codebook[4] = {0, 0, 0, 0};
    unsigned char* codes = nullptr;
    uint16_t* scales = nullptr;
    size_t code_bytes = 0, scale_elems = 0;
    // 4-bit twin for the f16 tensor-core path, built on the first such call (transcode.cu)
    mutable std::mutex twin_lock;
    mutable std::atomic<smeg_q4*> twin{nullptr};
    // dense f16 twin instead, for a 2-bit codebook with a value outside [-8, 7]
    mutable std::atomic<smeg_dense*> twin_dense{nullptr};
};
// Dense 16-bit weights for the Gemm builder: W[n][kd], K-major, kd = k padded to a multiple of 8.
struct smeg_dense {
    size_t n = 0, k = 0, kd = 0;
    int bf16 = 0;
    uint16_t* w = nullptr;            // device
};
struct smeg_mlp {
    const smeg_q4* gate_up;
    const smeg_q4* down;
    uint32_t act;
};
