// The GPU-resident packed weight layouts ("prepack"), shared by the host
// packers and the kernels.  They replace the reference's band-major layouts
// (src/kernels/q4/weights.rs:92-113, src/kernels/lowbit/q2.rs:153-161,
// src/kernels/lowbit/q1.rs:195-201); the logical content -- code(d, j),
// scale(d / block, j) -- is unchanged.
//
// All three formats tile the weight matrix into UNITS of 16 output columns by
// a fixed number of depths; one unit is 512 bytes = one 16-byte vector for each
// of the 32 lanes of a warp, ordered so that a lane's vector is already the
// A-operand fragment of a warp-level tensor-core instruction
// (mma.m16n8k16 for 4-bit, mma.m16n8k32 for 2-/1-bit) with the 16 weight
// columns as the M dimension and up to 8 activation rows as N.  The same vector
// also holds, for two columns, runs of 8 consecutive depths, so the prefill
// kernels can expand it into 16-byte K-major chunks for tcgen05 operands.
//
//   lane = 4*g + t  (g = 0..7, t = 0..3); columns held: c0 = 16*cg + g and c0 + 8.
//
// Q4 (unit = 16 columns x 64 depths; nibble = code + 8, offset binary):
//   word ks (0..3) of the lane's uint4 covers depths
//       d = 64*u + 32*(ks >> 1) + 8*t + 4*(ks & 1) + {0,1,2,3}
//   nibble 0,4 -> column c0   depths d+0, d+1      nibble 1,5 -> column c0   depths d+2, d+3
//   nibble 2,6 -> column c0+8 depths d+0, d+1      nibble 3,7 -> column c0+8 depths d+2, d+3
//
// Q2 (unit = 16 columns x 128 depths; 2-bit field f = 0..15 of a word):
//   word ks covers depths d = 128*u + 32*ks + 8*t + {0..7}
//   field f: column c0 + 8*(f & 1), depth d + (f >> 1)
//
// Q1 (unit = 16 columns x 256 depths; bit b = 0..31 of a word, 1 = +scale):
//   word wd (0..3) bit b: step s = 2*wd + ((b & 7) >> 2) covers depths
//       d = 256*u + 32*s + 8*t + {0..7}
//   column c0 + 8*(b & 1), depth d + 4*((b >> 1) & 1) + (b >> 3)
//
// Units are stored [column group][unit along K][512 B]: everything one column group needs is one
// contiguous run along K, so a CTA streams it with a few large bulk copies.  Q4 pads the column
// groups to a multiple of 8 (128 columns, the tensor-core kernel's tile).
//
// Scales: f16 bit patterns in rows of 16 slots, stored [column group][K-block][16]; column
// c of the group sits in slot 2*(c % 8) + c / 8, so the two columns a lane holds
// (g and g + 8) are one aligned 32-bit word.
// Padding columns / depths hold code 0 (Q4), and padded scales are 0; padded
// activations are staged as 0, so padding never contributes.
#pragma once
#include <stddef.h>
#include <stdint.h>

namespace smeg {

constexpr int kUnitBytes = 512;
constexpr int kQ4UnitDepth = 64;
constexpr int kQ2UnitDepth = 128;
constexpr int kQ1UnitDepth = 256;

#if defined(__CUDACC__)
#define SMEG_HD __host__ __device__
#else
#define SMEG_HD
#endif

inline size_t div_up(size_t a, size_t b) { return (a + b - 1) / b; }

// Slot of column c (0..15) of a column group inside a 16-entry scale row.
#if defined(__CUDACC__)
__host__ __device__
#endif
inline int scale_slot(int c) { return 2 * (c & 7) + (c >> 3); }

// Element offset of the 16-slot scale row of (column group cg, K-block blk); nb = rows per group.
#if defined(__CUDACC__)
__host__ __device__
#endif
inline size_t q4_scale_row(size_t cg, size_t blk, size_t nb) { return (cg * nb + blk) * 16; }
#if defined(__CUDACC__)
__host__ __device__
#endif
inline size_t q4_unit_offset(size_t cg, size_t u, size_t k_units) { return (cg * k_units + u) * 512; }

// --- Q4 ---
// Position of (depth d, column j) inside the packed code array: byte offset of
// the 32-bit word and the nibble index within it.
SMEG_HD inline void q4_locate(size_t d, size_t j, size_t k_units, size_t* word_byte, int* nibble) {
    size_t cg = j / 16, c = j % 16, u = d / 64, r = d % 64;
    int g = (int)(c % 8), hi_col = (int)(c / 8);
    int half = (int)(r / 32), rr = (int)(r % 32);
    int t = rr / 8, q = rr % 8;       // q = 0..7 within the lane's 8-depth run
    int ks = 2 * half + q / 4, e = q % 4;
    int lane = 4 * g + t;
    // e: 0,1 -> low positions (nibble 0/4 or 2/6); 2,3 -> (1/5 or 3/7)
    int nib = (e & 1) * 4 + (e >> 1) + 2 * hi_col;
    *word_byte = ((cg * k_units + u) * 32 + (size_t)lane) * 16 + (size_t)ks * 4;
    *nibble = nib;
}

// --- Q2 ---
SMEG_HD inline void q2_locate(size_t d, size_t j, size_t k_units, size_t* word_byte, int* field) {
    size_t cg = j / 16, c = j % 16, u = d / 128, r = d % 128;
    int g = (int)(c % 8), hi_col = (int)(c / 8);
    int ks = (int)(r / 32), rr = (int)(r % 32);
    int t = rr / 8, q = rr % 8;
    int lane = 4 * g + t;
    *word_byte = ((cg * k_units + u) * 32 + (size_t)lane) * 16 + (size_t)ks * 4;
    *field = 2 * q + hi_col;
}

// --- Q1 ---
SMEG_HD inline void q1_locate(size_t d, size_t j, size_t k_units, size_t* word_byte, int* bit) {
    size_t cg = j / 16, c = j % 16, u = d / 256, r = d % 256;
    int g = (int)(c % 8), hi_col = (int)(c / 8);
    int s = (int)(r / 32), rr = (int)(r % 32);
    int t = rr / 8, q = rr % 8;       // q = 0..7: depth within the lane's run
    int lane = 4 * g + t;
    int wd = s / 2, sh = s % 2;
    // q < 4 -> slot byte q of the "low" register, q >= 4 -> of the "high" one
    int b = 8 * (q % 4) + 4 * sh + 2 * (q / 4) + hi_col;
    *word_byte = ((cg * k_units + u) * 32 + (size_t)lane) * 16 + (size_t)wd * 4;
    *bit = b;
}

}  // namespace smeg
