// Host-side quantisers and the GPU prepack.  See pack.h and layout.h.
#include "pack.h"

#include <math.h>
#include <string.h>

#include <algorithm>
#include <atomic>
#include <thread>

#include "layout.h"

namespace smeg {

// ------------------------------------------------------------------ helpers

float h2f(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    const uint32_t e = (h >> 10) & 0x1f, mant = h & 0x3ffu;
    uint32_t bits;
    if (e == 0) {
        if (mant == 0) bits = sign;
        else {
            // normalise the subnormal
            int shift = 0;
            uint32_t mm = mant;
            while (!(mm & 0x400u)) { mm <<= 1; ++shift; }
            bits = sign | ((uint32_t)(113 - shift) << 23) | ((mm & 0x3ffu) << 13);
        }
    } else if (e == 31) bits = sign | 0x7f800000u | (mant << 13);
    else bits = sign | ((e + 112) << 23) | (mant << 13);
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

uint16_t f2h(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    const uint16_t sign = (uint16_t)((x >> 16) & 0x8000u);
    const uint32_t ax = x & 0x7fffffffu;
    if (ax >= 0x7f800000u) return sign | (ax > 0x7f800000u ? (uint16_t)(0x7e00u | ((ax >> 13) & 0x3ffu)) : (uint16_t)0x7c00u);
    if (ax >= 0x47800000u) return sign | 0x7c00u;   // >= 65536 rounds to inf (65520..65536 handled below)
    const int e = (int)(ax >> 23) - 127;
    uint32_t sig = (ax & 0x7fffffu) | 0x800000u;    // 24-bit significand
    int drop;                                        // low bits to round away
    uint32_t base;
    if (e >= -14) { drop = 13; base = (uint32_t)(e + 15) << 10; }
    else { drop = 13 + (-14 - e); base = 0; if (drop > 24) return sign; }
    uint32_t kept = sig >> drop;
    const uint32_t rem = sig & ((1u << drop) - 1), half = 1u << (drop - 1);
    if (rem > half || (rem == half && (kept & 1u))) ++kept;
    uint32_t out = base ? base + (kept - 0x400u) : kept;
    if (out >= 0x7c00u) out = 0x7c00u;
    return sign | (uint16_t)out;
}

namespace {
struct PfJob {
    void (*fn)(size_t, void*);
    void* ctx;
    size_t count;
    std::atomic<size_t> next{0};
};
}  // namespace

void parallel_for(size_t count, void (*fn)(size_t, void*), void* ctx) {
    unsigned hw = std::thread::hardware_concurrency();
    size_t nt = std::min<size_t>(hw ? hw : 1, std::min<size_t>(count, 32));
    if (nt <= 1) {
        for (size_t i = 0; i < count; ++i) fn(i, ctx);
        return;
    }
    PfJob job;
    job.fn = fn; job.ctx = ctx; job.count = count;
    auto worker = [&job]() {
        for (;;) {
            const size_t i = job.next.fetch_add(1);
            if (i >= job.count) break;
            job.fn(i, job.ctx);
        }
    };
    std::vector<std::thread> th;
    for (size_t t = 1; t < nt; ++t) th.emplace_back(worker);
    worker();
    for (auto& x : th) x.join();
}

PackedDims make_dims(size_t n, size_t k, size_t block, int unit_depth) {
    PackedDims d;
    d.n = n; d.k = k; d.block = block; d.unit_depth = unit_depth;
    d.n16 = div_up(n, 16);
    if (unit_depth == kQ4UnitDepth) d.n16 = div_up(d.n16, 8) * 8;   // whole 128-column super-groups
    d.ku = div_up(k, (size_t)unit_depth);
    d.nb_real = div_up(k, block);
    d.nb = std::max(d.nb_real, div_up(d.ku * (size_t)unit_depth, block));
    int l = 0;
    while (((size_t)1 << l) < block) ++l;
    d.log2_block = l;
    return d;
}

// ------------------------------------------------------------------ quantisers

// Q4Weights::quantize (src/kernels/q4/quantize.rs:29-81): per (column, K-block)
// scale = f16(m / -8) with m the block's first largest-magnitude value, code =
// clamp(round_half_away(w / scale), -8, 7); affine form spans min..max with 16 codes.
namespace {
struct Q4QCtx {
    const float* w; int layout; size_t n, k, block, nbk; int affine;
    int8_t* code;  // [j][k] signed codes
    uint16_t *scales, *mins;
};
void q4q_col(size_t j, void* p) {
    Q4QCtx& c = *(Q4QCtx*)p;
    auto at = [&](size_t d) { return c.layout == 0 ? c.w[j * c.k + d] : c.w[d * c.n + j]; };
    for (size_t b = 0; b < c.nbk; ++b) {
        const size_t d0 = b * c.block, d1 = std::min(c.k, d0 + c.block);
        uint16_t sc, mn = 0;
        if (c.affine) {
            float lo = INFINITY, hi = -INFINITY;
            for (size_t d = d0; d < d1; ++d) { lo = fminf(lo, at(d)); hi = fmaxf(hi, at(d)); }
            sc = f2h((hi - lo) / 15.0f);
            mn = f2h(lo + 8.0f * h2f(sc));
            c.mins[j * c.nbk + b] = mn;
        } else {
            float big = 0.0f;
            for (size_t d = d0; d < d1; ++d) if (fabsf(at(d)) > fabsf(big)) big = at(d);
            sc = f2h(big / -8.0f);
        }
        c.scales[j * c.nbk + b] = sc;
        const float s = h2f(sc), off = h2f(mn);
        const float inv = s == 0.0f ? 0.0f : 1.0f / s;
        for (size_t d = d0; d < d1; ++d) {
            float r = roundf((at(d) - off) * inv);
            r = r < -8.0f ? -8.0f : (r > 7.0f ? 7.0f : r);
            c.code[j * c.k + d] = (r != r) ? 0 : (int8_t)r;
        }
    }
}
}  // namespace

void q4_quantize_host(const float* w, int layout, size_t n, size_t k, size_t block, int affine,
                      std::vector<uint8_t>& quants, std::vector<uint16_t>& scales, std::vector<uint16_t>& mins) {
    const size_t nbk = div_up(k, block);
    std::vector<int8_t> code(n * k ? n * k : 1);
    scales.assign(n * nbk, 0);
    mins.assign(affine ? n * nbk : 0, 0);
    Q4QCtx c{w, layout, n, k, block, nbk, affine, code.data(), scales.data(), mins.data()};
    parallel_for(n, q4q_col, &c);
    quants.assign((k * n + 1) / 2, 0);
    for (size_t d = 0; d < k; ++d)
        for (size_t j = 0; j < n; ++j) {
            const size_t idx = d * n + j;
            quants[idx / 2] |= (uint8_t)((code[j * k + d] & 0x0f) << (4 * (idx % 2)));
        }
}

// Q2Weights::quantize (src/kernels/lowbit/q2.rs:110-144).
int q2_quantize_host(const float* w, int layout, size_t n, size_t k, size_t block, const int8_t codebook[4],
                     std::vector<uint8_t>& codes, std::vector<uint16_t>& scales) {
    float cb[4], cmax = 0.0f;
    for (int i = 0; i < 4; ++i) { cb[i] = (float)codebook[i]; cmax = fmaxf(cmax, fabsf(cb[i])); }
    if (!(cmax > 0.0f)) return -1;
    const size_t nbk = div_up(k, block);
    codes.assign((k * n + 3) / 4, 0);
    scales.assign(n * nbk, 0);
    for (size_t j = 0; j < n; ++j)
        for (size_t b = 0; b < nbk; ++b) {
            const size_t d0 = b * block, d1 = std::min(k, d0 + block);
            auto at = [&](size_t d) { return layout == 0 ? w[j * k + d] : w[d * n + j]; };
            float amax = 0.0f;
            for (size_t d = d0; d < d1; ++d) amax = fmaxf(amax, fabsf(at(d)));
            const uint16_t sc = f2h(amax / cmax);
            scales[j * nbk + b] = sc;
            const float s = h2f(sc);
            for (size_t d = d0; d < d1; ++d) {
                const float x = at(d);
                int best = 0;
                float bd = fabsf(x - s * cb[0]);
                for (int c = 1; c < 4; ++c) {
                    const float dd = fabsf(x - s * cb[c]);
                    if (dd < bd) { bd = dd; best = c; }
                }
                const size_t idx = d * n + j;
                codes[idx / 4] |= (uint8_t)(best << (2 * (idx % 4)));
            }
        }
    return 0;
}

// Q1Weights::quantize (src/kernels/lowbit/q1.rs:116-144); signs in OutIn bit order.
void q1_quantize_host(const float* w, int layout, size_t n, size_t k, size_t block, std::vector<uint8_t>& signs,
                      std::vector<uint16_t>& scales) {
    const size_t nbk = div_up(k, block);
    signs.assign((k * n + 7) / 8, 0);
    scales.assign(n * nbk, 0);
    for (size_t j = 0; j < n; ++j)
        for (size_t b = 0; b < nbk; ++b) {
            const size_t d0 = b * block, d1 = std::min(k, d0 + block);
            auto at = [&](size_t d) { return layout == 0 ? w[j * k + d] : w[d * n + j]; };
            float sum = 0.0f;
            for (size_t d = d0; d < d1; ++d) sum += fabsf(at(d));
            scales[j * nbk + b] = f2h(sum / (float)(d1 - d0));
            for (size_t d = d0; d < d1; ++d)
                if (at(d) >= 0.0f) {
                    const size_t idx = j * k + d;
                    signs[idx / 8] |= (uint8_t)(1u << (idx % 8));
                }
        }
}

// ------------------------------------------------------------------ prepack

namespace {
size_t scale_row(const PackedDims& d, size_t cg, size_t b) {
    return d.unit_depth == kQ4UnitDepth ? q4_scale_row(cg, b, d.nb) : (cg * d.nb + b) * 16;
}
void pack_scales(const uint16_t* scales, const PackedDims& d, std::vector<uint16_t>& sc) {
    sc.assign(d.n16 * d.nb * 16, 0);
    for (size_t j = 0; j < d.n; ++j)
        for (size_t b = 0; b < d.nb_real; ++b) sc[scale_row(d, j / 16, b) + scale_slot((int)(j % 16))] = scales[j * d.nb_real + b];
}
void unpack_scales(const uint16_t* sc, const PackedDims& d, uint16_t* scales) {
    for (size_t j = 0; j < d.n; ++j)
        for (size_t b = 0; b < d.nb_real; ++b) scales[j * d.nb_real + b] = sc[scale_row(d, j / 16, b) + scale_slot((int)(j % 16))];
}

struct PackCtx {
    const uint8_t* in; int layout; const PackedDims* d; uint8_t* out; int kind;
};
// one column group per call: no two calls touch the same output bytes
void pack_group(size_t cg, void* p) {
    PackCtx& c = *(PackCtx*)p;
    const PackedDims& d = *c.d;
    const size_t j1 = std::min(d.n, (cg + 1) * 16);
    for (size_t j = cg * 16; j < j1; ++j)
        for (size_t dd = 0; dd < d.k; ++dd) {
            size_t wb; int pos;
            if (c.kind == 4) {
                const size_t idx = dd * d.n + j;
                const uint32_t nib = (c.in[idx / 2] >> (4 * (idx % 2))) & 0xfu;   // two's complement code
                q4_locate(dd, j, d.ku, &wb, &pos);
                // the slot was pre-filled with 8 (code 0); replace by code + 8
                uint8_t& byte = c.out[wb + pos / 2];
                const uint8_t v = (uint8_t)((nib ^ 8u) & 0xfu);
                byte = (pos & 1) ? (uint8_t)((byte & 0x0f) | (v << 4)) : (uint8_t)((byte & 0xf0) | v);
            } else if (c.kind == 2) {
                const size_t idx = dd * d.n + j;
                const uint32_t code = (c.in[idx / 4] >> (2 * (idx % 4))) & 3u;
                q2_locate(dd, j, d.ku, &wb, &pos);
                c.out[wb + pos / 4] |= (uint8_t)(code << (2 * (pos % 4)));
            } else {
                const size_t idx = c.layout == 0 ? j * d.k + dd : dd * d.n + j;
                if ((c.in[idx / 8] >> (idx % 8)) & 1u) {
                    q1_locate(dd, j, d.ku, &wb, &pos);
                    c.out[wb + pos / 8] |= (uint8_t)(1u << (pos % 8));
                }
            }
        }
}
}  // namespace

void q4_pack(const uint8_t* quants, const uint16_t* scales, const PackedDims& d, std::vector<uint8_t>& codes,
             std::vector<uint16_t>& sc) {
    codes.assign(d.n16 * d.ku * kUnitBytes, 0x88);   // every nibble = 8 = code 0
    PackCtx c{quants, 0, &d, codes.data(), 4};
    parallel_for(d.n16, pack_group, &c);
    pack_scales(scales, d, sc);
}
void q2_pack(const uint8_t* codes_in, const uint16_t* scales, const PackedDims& d, std::vector<uint8_t>& codes,
             std::vector<uint16_t>& sc) {
    codes.assign(d.n16 * d.ku * kUnitBytes, 0);
    PackCtx c{codes_in, 0, &d, codes.data(), 2};
    parallel_for(d.n16, pack_group, &c);
    pack_scales(scales, d, sc);
}
void q1_pack(const uint8_t* signs, int layout, const uint16_t* scales, const PackedDims& d, std::vector<uint8_t>& codes,
             std::vector<uint16_t>& sc) {
    codes.assign(d.n16 * d.ku * kUnitBytes, 0);
    PackCtx c{signs, layout, &d, codes.data(), 1};
    parallel_for(d.n16, pack_group, &c);
    pack_scales(scales, d, sc);
}

void q4_unpack(const uint8_t* codes, const uint16_t* sc, const PackedDims& d, uint8_t* quants, uint16_t* scales) {
    memset(quants, 0, (d.k * d.n + 1) / 2);
    for (size_t dd = 0; dd < d.k; ++dd)
        for (size_t j = 0; j < d.n; ++j) {
            size_t wb; int pos;
            q4_locate(dd, j, d.ku, &wb, &pos);
            const uint32_t v = (codes[wb + pos / 2] >> (4 * (pos & 1))) & 0xfu;
            const size_t idx = dd * d.n + j;
            quants[idx / 2] |= (uint8_t)(((v ^ 8u) & 0xfu) << (4 * (idx % 2)));
        }
    unpack_scales(sc, d, scales);
}
void q2_unpack(const uint8_t* codes, const uint16_t* sc, const PackedDims& d, uint8_t* codes_out, uint16_t* scales) {
    memset(codes_out, 0, (d.k * d.n + 3) / 4);
    for (size_t dd = 0; dd < d.k; ++dd)
        for (size_t j = 0; j < d.n; ++j) {
            size_t wb; int pos;
            q2_locate(dd, j, d.ku, &wb, &pos);
            const uint32_t v = (codes[wb + pos / 4] >> (2 * (pos % 4))) & 3u;
            const size_t idx = dd * d.n + j;
            codes_out[idx / 4] |= (uint8_t)(v << (2 * (idx % 4)));
        }
    unpack_scales(sc, d, scales);
}
void q1_unpack(const uint8_t* codes, const uint16_t* sc, const PackedDims& d, uint8_t* signs, uint16_t* scales) {
    memset(signs, 0, (d.k * d.n + 7) / 8);
    for (size_t j = 0; j < d.n; ++j)
        for (size_t dd = 0; dd < d.k; ++dd) {
            size_t wb; int pos;
            q1_locate(dd, j, d.ku, &wb, &pos);
            if ((codes[wb + pos / 8] >> (pos % 8)) & 1u) {
                const size_t idx = j * d.k + dd;
                signs[idx / 8] |= (uint8_t)(1u << (idx % 8));
            }
        }
    unpack_scales(sc, d, scales);
}

// ------------------------------------------------------------------ band-major import
// The arrays a reference-side Q4Weights / Q2Weights / Q1Weights holds:
//   Q4: 128-column bands, byte b*k*64 + d*64 + c/2, nibble c%2; scales [band][blk][128]
//       (src/kernels/q4/weights.rs:92-113)
//   Q2: 64-column bands, byte (j/64)*band_bytes + (d/4)*64 + j%64, bits 2*(d%4),
//       band_bytes = ceil16(k)*16 (src/kernels/lowbit/q2.rs:146-161)
//   Q1: byte (j/64)*band_bytes + (d/4)*32 + c/2, bit 4*(c%2) + d%4, band_bytes = ceil16(k)*8
//       (src/kernels/lowbit/q1.rs:188-201)
//   Q2/Q1 scales: (j/64)*nbk*64 + blk*64 + (c/32)*32 + 2*(c%16) + (c%32)/16 (q2.rs:17-20)

void q4_from_band(const uint8_t* nibbles, const uint16_t* sc_band, const uint16_t* mn_band, size_t n, size_t k,
                  size_t block, std::vector<uint8_t>& quants, std::vector<uint16_t>& scales, std::vector<uint16_t>& mins) {
    const size_t nbk = div_up(k, block);
    quants.assign((k * n + 1) / 2, 0);
    scales.assign(n * nbk, 0);
    mins.assign(mn_band ? n * nbk : 0, 0);
    for (size_t d = 0; d < k; ++d)
        for (size_t j = 0; j < n; ++j) {
            const size_t band = j / 128, c = j % 128;
            const uint32_t nib = (nibbles[band * k * 64 + d * 64 + c / 2] >> (4 * (c % 2))) & 0xfu;
            const size_t idx = d * n + j;
            quants[idx / 2] |= (uint8_t)(nib << (4 * (idx % 2)));
        }
    for (size_t j = 0; j < n; ++j)
        for (size_t b = 0; b < nbk; ++b) {
            const size_t src = (j / 128) * nbk * 128 + b * 128 + j % 128;
            scales[j * nbk + b] = sc_band[src];
            if (mn_band) mins[j * nbk + b] = mn_band[src];
        }
}

static size_t lowbit_scale_slot(size_t nbk, size_t blk, size_t j) {
    const size_t c = j % 64;
    return (j / 64) * nbk * 64 + blk * 64 + (c / 32) * 32 + 2 * (c % 16) + (c % 32) / 16;
}

void q2_from_band(const uint8_t* packed, const uint16_t* sc_band, size_t n, size_t k, size_t block,
                  std::vector<uint8_t>& codes, std::vector<uint16_t>& scales) {
    const size_t nbk = div_up(k, block), band_bytes = div_up(k, 16) * 16 * 16;
    codes.assign((k * n + 3) / 4, 0);
    scales.assign(n * nbk, 0);
    for (size_t d = 0; d < k; ++d)
        for (size_t j = 0; j < n; ++j) {
            const uint32_t code = (packed[(j / 64) * band_bytes + (d / 4) * 64 + j % 64] >> (2 * (d % 4))) & 3u;
            const size_t idx = d * n + j;
            codes[idx / 4] |= (uint8_t)(code << (2 * (idx % 4)));
        }
    for (size_t j = 0; j < n; ++j)
        for (size_t b = 0; b < nbk; ++b) scales[j * nbk + b] = sc_band[lowbit_scale_slot(nbk, b, j)];
}

void q1_from_band(const uint8_t* packed, const uint16_t* sc_band, size_t n, size_t k, size_t block,
                  std::vector<uint8_t>& signs, std::vector<uint16_t>& scales) {
    const size_t nbk = div_up(k, block), band_bytes = div_up(k, 16) * 16 * 8;
    signs.assign((k * n + 7) / 8, 0);
    scales.assign(n * nbk, 0);
    for (size_t j = 0; j < n; ++j) {
        const size_t c = j % 64;
        for (size_t d = 0; d < k; ++d)
            if ((packed[(j / 64) * band_bytes + (d / 4) * 32 + c / 2] >> (4 * (c % 2) + d % 4)) & 1u) {
                const size_t idx = j * k + d;
                signs[idx / 8] |= (uint8_t)(1u << (idx % 8));
            }
        for (size_t b = 0; b < nbk; ++b) scales[j * nbk + b] = sc_band[lowbit_scale_slot(nbk, b, j)];
    }
}

}  // namespace smeg
