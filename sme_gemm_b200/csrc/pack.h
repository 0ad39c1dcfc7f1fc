// Host-side weight preparation: quantisers (f32 -> codes + f16 scales), the GPU
// prepack (logical arrays -> unit layout of layout.h) and its inverse, and the
// import of the reference's own band-major arrays.  One-time work at weight
// construction, as in the reference (Q4Weights::quantize / ::with_params,
// Q2Weights::quantize / ::new, Q1Weights::quantize / ::new / ::interleave).
#pragma once
#include <stddef.h>
#include <stdint.h>

#include <vector>

namespace smeg {

// IEEE binary16 <-> binary32 on the host (round to nearest even), bit patterns.
float h2f(uint16_t h);
uint16_t f2h(float f);

struct PackedDims {
    size_t n = 0, k = 0, block = 0;
    size_t n16 = 0;      // column groups of 16
    size_t ku = 0;       // units along K
    size_t nb = 0;       // scale rows stored per column group (covers the padded depth)
    size_t nb_real = 0;  // ceil(k / block)
    int unit_depth = 0;  // 64 (Q4), 128 (Q2), 256 (Q1)
    int log2_block = 0;
};
PackedDims make_dims(size_t n, size_t k, size_t block, int unit_depth);

// ---- quantisers (logical outputs, same formats as the reference's constructors take) ----
void q4_quantize_host(const float* w, int layout, size_t n, size_t k, size_t block, int affine,
                      std::vector<uint8_t>& quants, std::vector<uint16_t>& scales, std::vector<uint16_t>& mins);
int q2_quantize_host(const float* w, int layout, size_t n, size_t k, size_t block, const int8_t codebook[4],
                     std::vector<uint8_t>& codes, std::vector<uint16_t>& scales);
void q1_quantize_host(const float* w, int layout, size_t n, size_t k, size_t block, std::vector<uint8_t>& signs,
                      std::vector<uint16_t>& scales);

// ---- prepack: logical -> unit layout (codes) + [n16][nb][16] scales ----
void q4_pack(const uint8_t* quants, const uint16_t* scales, const PackedDims& d, std::vector<uint8_t>& codes,
             std::vector<uint16_t>& sc);
void q4_unpack(const uint8_t* codes, const uint16_t* sc, const PackedDims& d, uint8_t* quants, uint16_t* scales);
void q2_pack(const uint8_t* codes_in, const uint16_t* scales, const PackedDims& d, std::vector<uint8_t>& codes,
             std::vector<uint16_t>& sc);
void q2_unpack(const uint8_t* codes, const uint16_t* sc, const PackedDims& d, uint8_t* codes_out, uint16_t* scales);
void q1_pack(const uint8_t* signs, int layout, const uint16_t* scales, const PackedDims& d, std::vector<uint8_t>& codes,
             std::vector<uint16_t>& sc);
// signs come back in OutIn bit order (idx = j*k + d)
void q1_unpack(const uint8_t* codes, const uint16_t* sc, const PackedDims& d, uint8_t* signs, uint16_t* scales);

// ---- the reference's band-major arrays -> logical arrays ----
void q4_from_band(const uint8_t* nibbles, const uint16_t* sc_band, const uint16_t* mn_band, size_t n, size_t k,
                  size_t block, std::vector<uint8_t>& quants, std::vector<uint16_t>& scales, std::vector<uint16_t>& mins);
void q2_from_band(const uint8_t* packed, const uint16_t* sc_band, size_t n, size_t k, size_t block,
                  std::vector<uint8_t>& codes, std::vector<uint16_t>& scales);
void q1_from_band(const uint8_t* packed, const uint16_t* sc_band, size_t n, size_t k, size_t block,
                  std::vector<uint8_t>& signs, std::vector<uint16_t>& scales);

// Runs fn(i) for i in [0, count) on the host's cores.
void parallel_for(size_t count, void (*fn)(size_t, void*), void* ctx);

}  // namespace smeg
