// Tensor-core GEMM for sm_100a:  C[m][n] = ep( A[m][k] @ dequant(W) ) on the 5th-generation
// tensor cores (tcgen05.mma, accumulators in tensor memory), for prefill-sized m and -- with the
// depth split over several CTAs -- for decode-sized m as well.
//
// Replaces the reference's MOPA paths -- unpack_q4_f16 / unpack_q4_bf16 + run_q4_panels
// (csrc/gemm_f16f16_q4.h:57-117, csrc/gemm_b16b16_q4.h:32-92) and the dense run_panels consumer
// (csrc/gemm_half.h:1093-1169).  As there, every weight is rounded ONCE to the 16-bit operand type
// exactly as the eager dequant rounds it (dequant_rows, src/kernels/q4/weights.rs:232-259) and the
// dense product accumulates in f32.
//
// One CTA owns NW x 128 weight columns (the MMA's M dimension; NW = 1 or 2 accumulator sets) x a
// tile of up to 512 tokens (the MMA's N dimension, one or two instructions of N <= 256) over a
// slice of the depth, walked in 64-deep stages.  Roles (608 threads):
//   warp 16 (tokens)    one TMA tile load per stage (tensor map, 128-byte swizzle) into the
//                       token ring.
//   warp 18 (weights)   the packed units and scale rows of the CTA's column groups into the
//                       packed ring.  A slot covers several stages: a bulk copy costs a couple
//                       of hundred cycles to issue whatever its size, and a column group's
//                       units are contiguous along K, so one copy carries them for all of them.
//   warps 0-15 (dequant) expand the stage's packed units into the K-major, 128-byte-swizzled
//                       MMA operand in the operand ring: a lane's 16-byte vector becomes four
//                       16-byte chunks of 8 consecutive depths.  With one accumulator set the
//                       two halves of the warps take alternate stages.
//   warp 17 (MMA)       one elected thread issues the stage's tcgen05.mma (K = 16 each) and
//                       commits the stage back to the token and operand rings.
// After the last stage the dequant warps drain tensor memory (thread = weight column, registers
// = tokens): the epilogue graph on the rounded product, or -- for the MLP block -- the gated
// product of a gate/up pair, or the residual add.  With the depth split (grid.z > 1) each CTA
// leaves its f32 partial tile in a global workspace and splitk_reduce_kernel, launched right
// behind, adds the slices in slice order (so the result does not depend on arrival order) and stores.
// Every wait is bounded; a timed-out wait raises the status word and the kernel drains and exits.
#include "epilogue.cuh"
#include "kernels.h"
#include "layout.h"
#include "tc_common.cuh"

#include <stdlib.h>

namespace smeg {

namespace {

// Position in a ring of n slots, advanced once per use: slot index, parity of the current round, first round or not.
// (The ring depths are run-time values: computing slot and round from the stage number costs an integer division each,
// and the role loops are latency chains of one warp -- every instruction in them is on the critical path.)
struct RingPos {
    int slot = 0;
    unsigned phase = 0;
    bool wrapped = false;
    __device__ __forceinline__ void next(int n) {
        if (++slot == n) { slot = 0; phase ^= 1u; wrapped = true; }
    }
};

constexpr int kDeqWarps = 16;                    // dequant warps (the first 8 also drain tensor memory)
constexpr int kTcThreads = 32 * (kDeqWarps + 3);   // + token producer, MMA issuer, packed-weight producer
constexpr int kStageK = 64;                       // depths per stage (one 128-byte swizzle row)
constexpr int kWTile = 128 * kStageK * 2;         // one 128-column operand tile per stage: 16 KB

__device__ __forceinline__ uint32_t swz_off(int row, int chunk) {
    // byte offset of 16-byte chunk `chunk` (0..7) of row `row` in a 128B-swizzled K-major tile
    return (uint32_t)((row >> 3) * 1024 + (row & 7) * 128 + ((chunk ^ (row & 7)) << 4));
}

template <int BF16>
__device__ __forceinline__ uint4 scale_chunk(const __half2 (&c)[4], __half s) {
    uint4 out;
    if (BF16) {
        const float sf = __half2float(s);
        uint32_t* o = reinterpret_cast<uint32_t*>(&out);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __half22float2(c[i]);
            __nv_bfloat162 v = __floats2bfloat162_rn(__fmul_rn(f.x, sf), __fmul_rn(f.y, sf));
            o[i] = *reinterpret_cast<uint32_t*>(&v);
        }
    } else {
        const __half2 s2 = __half2half2(s);
        __half2* o = reinterpret_cast<__half2*>(&out);
#pragma unroll
        for (int i = 0; i < 4; ++i) o[i] = __hmul2(c[i], s2);
    }
    return out;
}

// Q4 word -> exact integer codes as f16 pairs: r[0] = col g (d+0,d+1), r[1] = col g+8 (d+0,d+1),
// r[2] = col g (d+2,d+3), r[3] = col g+8 (d+2,d+3).
__device__ __forceinline__ void q4_word_codes(uint32_t w, __half2 (&r)[4]) {
    const uint32_t w8 = w >> 8;
    uint32_t lo0 = lop3_and_or(w, 0x000f000fu, 0x64006400u), hi0 = lop3_and_or(w, 0x00f000f0u, 0x64006400u);
    uint32_t lo1 = lop3_and_or(w8, 0x000f000fu, 0x64006400u), hi1 = lop3_and_or(w8, 0x00f000f0u, 0x64006400u);
    const __half2 off = __halves2half2(__ushort_as_half(0x6408), __ushort_as_half(0x6408));
    const __half2 sc16 = __halves2half2(__ushort_as_half(0x2c00), __ushort_as_half(0x2c00));
    const __half2 off16 = __halves2half2(__ushort_as_half(0xd480), __ushort_as_half(0xd480));
    r[0] = __hsub2(*reinterpret_cast<__half2*>(&lo0), off);
    r[1] = __hsub2(*reinterpret_cast<__half2*>(&lo1), off);
    r[2] = __hfma2(*reinterpret_cast<__half2*>(&hi0), sc16, off16);
    r[3] = __hfma2(*reinterpret_cast<__half2*>(&hi1), sc16, off16);
}

// One packed Q4 unit (16 columns x 64 depths) -> rows 16*cu + {g, g+8} of a swizzled operand tile.
template <int BF16>
__device__ __forceinline__ void dequant_unit_q4(unsigned char* tile, int cu, const uint4 wv, const uint16_t* sc, int ra,
                                                int rb, int g, int t) {
    __half2 w0[4], w1[4], w2[4], w3[4];
    q4_word_codes(wv.x, w0);
    q4_word_codes(wv.y, w1);
    q4_word_codes(wv.z, w2);
    q4_word_codes(wv.w, w3);
    // chunks: (col g, depths 8t..8t+7), (col g, 32+8t..), (col g+8, 8t..), (col g+8, 32+8t..)
    const __half2 lo_a[4] = {w0[0], w0[2], w1[0], w1[2]};
    const __half2 lo_b[4] = {w2[0], w2[2], w3[0], w3[2]};
    const __half2 hi_a[4] = {w0[1], w0[3], w1[1], w1[3]};
    const __half2 hi_b[4] = {w2[1], w2[3], w3[1], w3[3]};
    const uint32_t sa = *reinterpret_cast<const uint32_t*>(sc + ra * 16 + 2 * g);   // (col g, col g+8) of block ra
    const uint32_t sb = *reinterpret_cast<const uint32_t*>(sc + rb * 16 + 2 * g);
    const __half s_lo_a = __ushort_as_half((uint16_t)(sa & 0xffffu)), s_hi_a = __ushort_as_half((uint16_t)(sa >> 16));
    const __half s_lo_b = __ushort_as_half((uint16_t)(sb & 0xffffu)), s_hi_b = __ushort_as_half((uint16_t)(sb >> 16));
    const int row_lo = 16 * cu + g, row_hi = row_lo + 8;
    // chunk order per store keeps the 8 lanes of a quarter warp on distinct banks
    const int ca = (g & 1) ? 4 + t : t, cb = (g & 1) ? t : 4 + t;
    const uint4 v_lo_a = scale_chunk<BF16>(lo_a, s_lo_a), v_lo_b = scale_chunk<BF16>(lo_b, s_lo_b);
    const uint4 v_hi_a = scale_chunk<BF16>(hi_a, s_hi_a), v_hi_b = scale_chunk<BF16>(hi_b, s_hi_b);
    *reinterpret_cast<uint4*>(tile + swz_off(row_lo, ca)) = (g & 1) ? v_lo_b : v_lo_a;
    *reinterpret_cast<uint4*>(tile + swz_off(row_lo, cb)) = (g & 1) ? v_lo_a : v_lo_b;
    *reinterpret_cast<uint4*>(tile + swz_off(row_hi, ca)) = (g & 1) ? v_hi_b : v_hi_a;
    *reinterpret_cast<uint4*>(tile + swz_off(row_hi, cb)) = (g & 1) ? v_hi_a : v_hi_b;
}

__device__ __forceinline__ uint4 lds128(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ void sts128(uint32_t a, uint4 v) {
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(a), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// The same expansion on addresses the caller keeps per lane (the role loop's per-stage work is then the waits, three
// loads, the arithmetic and four stores).  `row` = shared address of the 128-byte row of column g in the operand tile
// (column g + 8 lies 1024 bytes on), `off_first` / `off_second` = swizzled chunk offsets.  Lanes of odd g take the two
// halves of the unit in the other order (the caller swaps the words and scale words), so that the eight lanes of a
// quarter warp hit distinct banks in every store.
template <int BF16>
__device__ __forceinline__ void dequant_unit_q4_at(uint32_t row, uint32_t off_first, uint32_t off_second, const uint4 wv, uint32_t s_first,
                                                   uint32_t s_second) {
    __half2 w0[4], w1[4], w2[4], w3[4];
    q4_word_codes(wv.x, w0);
    q4_word_codes(wv.y, w1);
    q4_word_codes(wv.z, w2);
    q4_word_codes(wv.w, w3);
    const __half2 lo_a[4] = {w0[0], w0[2], w1[0], w1[2]};
    const __half2 lo_b[4] = {w2[0], w2[2], w3[0], w3[2]};
    const __half2 hi_a[4] = {w0[1], w0[3], w1[1], w1[3]};
    const __half2 hi_b[4] = {w2[1], w2[3], w3[1], w3[3]};
    const __half2 sa = *reinterpret_cast<const __half2*>(&s_first), sb = *reinterpret_cast<const __half2*>(&s_second);
    sts128(row + off_first, scale_chunk<BF16>(lo_a, __low2half(sa)));
    sts128(row + off_second, scale_chunk<BF16>(lo_b, __low2half(sb)));
    sts128(row + 1024u + off_first, scale_chunk<BF16>(hi_a, __high2half(sa)));
    sts128(row + 1024u + off_second, scale_chunk<BF16>(hi_b, __high2half(sb)));
}

// The kernel's tensor maps: the token matrix, and for dense weights the weight matrix as well.
template <int DENSE> struct TcMaps { CUtensorMap tok; CUtensorMap c; CUtensorMap w; };
template <> struct TcMaps<0> { CUtensorMap tok; CUtensorMap c; CUtensorMap codes; CUtensorMap scales; };

// The hot forms of the drain -- the gated product of a gate/up pair, the residual add of the down projection, the f32
// partial tile of a depth slice, the plain rounded store -- out of line and on scalar arguments: sixteen accumulators
// per tcgen05.ld, one thread per weight column (TMEM lane), lanes of a warp on consecutive columns of C.
template <int BF16>
__device__ __noinline__ void drain_glu(uint32_t lane_base, int ntok, int j_begin, int j_end, uint16_t* c, int m, int hn, int hcol, int tok0,
                                       uint32_t act, uint32_t stage) {
    // accumulator set 0 = gate, set 1 = up of hidden unit hcol (glu, src/linear.rs:804-835)
    for (int j0 = j_begin; j0 < j_end; j0 += 16) {
        uint32_t rg[16], ru[16];
        tmem_ld16(lane_base + (uint32_t)j0, rg);
        tmem_ld16(lane_base + (uint32_t)(ntok + j0), ru);
        tmem_ld_wait();
        if (stage) {
            // into the staging tile [token][128 columns]: the bulk store clips what lies outside C
#pragma unroll
            for (int j = 0; j < 16; j += 2) {
                const float2 gv = round2_t<BF16>(__uint_as_float(rg[j]), __uint_as_float(rg[j + 1]));
                const float2 uv = round2_t<BF16>(__uint_as_float(ru[j]), __uint_as_float(ru[j + 1]));
                const uint32_t v = pack2_t<BF16>(__fmul_rn(glu_gate(act, gv.x), uv.x), __fmul_rn(glu_gate(act, gv.y), uv.y));
                sts16(stage + (uint32_t)((j0 + j) * 256), (uint16_t)(v & 0xffffu));
                sts16(stage + (uint32_t)((j0 + j + 1) * 256), (uint16_t)(v >> 16));
            }
            continue;
        }
        if (hcol >= hn) continue;
        uint16_t* dst = c + (size_t)(tok0 + j0) * hn + hcol;
        const int left = m - tok0 - j0;
        // two tokens at a time: the roundings are packed conversions (the scalar ones share a quarter-rate pipe with exp2 / rcp)
#pragma unroll
        for (int j = 0; j < 16; j += 2) {
            const float2 gv = round2_t<BF16>(__uint_as_float(rg[j]), __uint_as_float(rg[j + 1]));
            const float2 uv = round2_t<BF16>(__uint_as_float(ru[j]), __uint_as_float(ru[j + 1]));
            const uint32_t v = pack2_t<BF16>(__fmul_rn(glu_gate(act, gv.x), uv.x), __fmul_rn(glu_gate(act, gv.y), uv.y));
            if (j < left) dst[(size_t)j * hn] = (uint16_t)(v & 0xffffu);
            if (j + 1 < left) dst[(size_t)(j + 1) * hn] = (uint16_t)(v >> 16);
        }
    }
}

template <int BF16>
__device__ __noinline__ void drain_residual(uint32_t lane_base, int j_begin, int j_end, float* y, int m, int n, int col, int tok0) {
    for (int j0 = j_begin; j0 < j_end; j0 += 16) {
        uint32_t r[16];
        tmem_ld16(lane_base + (uint32_t)j0, r);
        tmem_ld_wait();
        if (col >= n) continue;
        float* dst = y + (size_t)(tok0 + j0) * n + col;
        const int left = m - tok0 - j0;
        float yv[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) yv[j] = j < left ? dst[(size_t)j * n] : 0.0f;
#pragma unroll
        for (int j = 0; j < 16; j += 2) {
            const float2 v = round2_t<BF16>(__uint_as_float(r[j]), __uint_as_float(r[j + 1]));
            if (j < left) dst[(size_t)j * n] = __fadd_rn(yv[j], v.x);
            if (j + 1 < left) dst[(size_t)(j + 1) * n] = __fadd_rn(yv[j + 1], v.y);
        }
    }
}

__device__ __noinline__ void drain_partial(uint32_t lane_base, int j_begin, int j_end, float* dst, int stride) {
    // partial tile of this depth slice: ws[tile][slice][token][column]
    for (int j0 = j_begin; j0 < j_end; j0 += 16) {
        uint32_t r[16];
        tmem_ld16(lane_base + (uint32_t)j0, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j) dst[(size_t)(j0 + j) * stride] = __uint_as_float(r[j]);
    }
}

template <int BF16>
__device__ __noinline__ void drain_store(uint32_t lane_base, int j_begin, int j_end, uint16_t* c, int m, int n, int col, int tok0, uint32_t stage) {
    for (int j0 = j_begin; j0 < j_end; j0 += 16) {
        uint32_t r[16];
        tmem_ld16(lane_base + (uint32_t)j0, r);
        tmem_ld_wait();
        if (stage) {
#pragma unroll
            for (int j = 0; j < 16; j += 2) {
                const uint32_t v = pack2_t<BF16>(__uint_as_float(r[j]), __uint_as_float(r[j + 1]));
                sts16(stage + (uint32_t)((j0 + j) * 256), (uint16_t)(v & 0xffffu));
                sts16(stage + (uint32_t)((j0 + j + 1) * 256), (uint16_t)(v >> 16));
            }
            continue;
        }
        if (col >= n) continue;
        uint16_t* dst = c + (size_t)(tok0 + j0) * n + col;
        const int left = m - tok0 - j0;
#pragma unroll
        for (int j = 0; j < 16; j += 2) {
            const uint32_t v = pack2_t<BF16>(__uint_as_float(r[j]), __uint_as_float(r[j + 1]));
            if (j < left) dst[(size_t)j * n] = (uint16_t)(v & 0xffffu);
            if (j + 1 < left) dst[(size_t)(j + 1) * n] = (uint16_t)(v >> 16);
        }
    }
}

// The epilogue graphs that fit a FastEp (up to four slots of a scalar or per-column operand or an activation), row-major C.
template <int BF16>
__device__ __noinline__ void drain_fast_ep(uint32_t lane_base, int j_begin, int j_end, uint16_t* c, int m, int n, int col, int tok0, FastEp fe,
                                           uint32_t stage) {
    for (int j0 = j_begin; j0 < j_end; j0 += 16) {
        uint32_t r[16];
        tmem_ld16(lane_base + (uint32_t)j0, r);
        tmem_ld_wait();
        if (col >= n && !stage) continue;
        uint16_t v[16];
        fast_ep_apply16<BF16>(fe, r, v);
        if (stage) {
#pragma unroll
            for (int j = 0; j < 16; ++j) sts16(stage + (uint32_t)((j0 + j) * 256), v[j]);
            continue;
        }
        uint16_t* dst = c + (size_t)(tok0 + j0) * n + col;
        const int left = m - tok0 - j0;
#pragma unroll
        for (int j = 0; j < 16; ++j)
            if (j < left) dst[(size_t)j * n] = v[j];
    }
}

// The drain of a CTA's accumulators, out of line: its sixteen-wide register groups would otherwise set the register
// budget of the role loops above (which then spill inside their per-stage latency chains).
template <int BF16, int DENSE>
__device__ __noinline__ void drain_tile(const GemmTcArgs& p, uint32_t tmem_base, int warp, int lane, int num_stages, uint64_t* acc_full,
                                        volatile int* abort_flag, const EpNodeDev* ep_nodes, int col0, int tok0) {
    const int NW = p.nw;
    // ---- drain: thread = weight column (TMEM lane), registers = tokens.  A warp reaches the
    // lane quarter warp % 4; the token columns are split over 4 (or 2) warps per quarter ----
    const int ntok = p.ntok_pad;                           // a multiple of 32
    const int parts = (ntok % 64 == 0) ? 4 : 2;            // every part is whole groups of 16 tokens
    if (warp < 4 * parts) {
    if (num_stages > 0) mbar_wait(acc_full, 0, abort_flag, p.status, STATUS_TMEM_TIMEOUT);
    tc_fence_after();
    const int q = warp & 3, part = warp >> 2;              // lane quarter, token part
    const uint32_t lane_base = tmem_base + ((uint32_t)(32 * q) << 16);
    const EpNodeDev* nodes = p.ep.n_nodes <= kMaxInlineNodes ? ep_nodes : p.ep.ext;
    const int j_begin = part * (ntok / parts), j_end = j_begin + ntok / parts;
    const int splits = (int)gridDim.z;
    const int tile_id = blockIdx.y * gridDim.x + blockIdx.x;
    float* ws_tile = p.ws + ((size_t)tile_id * splits) * (size_t)(NW * 128) * ntok;

    if (p.glu && splits == 1) {
        // accumulator set 0 = gate, set 1 = up of hidden unit hcol (glu, src/linear.rs:804-835)
        const int hn = p.n >> 1, hcol = blockIdx.x * 128 + 32 * q + lane;
        for (int j0 = j_begin; j0 < j_end; j0 += 16) {
            uint32_t rg[16], ru[16];
            tmem_ld16(lane_base + (uint32_t)j0, rg);
            tmem_ld16(lane_base + (uint32_t)(ntok + j0), ru);
            tmem_ld_wait();
            if (hcol < hn) {
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const float gv = t_to_f32<BF16>(f32_to_t<BF16>(__uint_as_float(rg[j])));
                    const float uv = t_to_f32<BF16>(f32_to_t<BF16>(__uint_as_float(ru[j])));
                    const float a = glu_gate((uint32_t)p.glu, gv);
                    if (tok0 + j0 + j < p.m) p.c[(size_t)(tok0 + j0 + j) * hn + hcol] = f32_to_t<BF16>(__fmul_rn(a, uv));
                }
            }
        }
    } else
    for (int w = 0; w < NW; ++w) {
        const int col = col0 + 128 * w + 32 * q + lane;
        FastEp fe;
        if (p.ep_fast) fast_ep_build<BF16>(nodes, p.ep.n_nodes, col, col < p.n, fe);
        for (int j0 = j_begin; j0 < j_end; j0 += 16) {
            uint32_t r[16];
            if (num_stages > 0) {
                tmem_ld16(lane_base + (uint32_t)(w * ntok + j0), r);
                tmem_ld_wait();
            } else {
#pragma unroll
                for (int j = 0; j < 16; ++j) r[j] = 0u;
            }
            if (splits == 1) {
                if (DENSE && p.beta != 1.0f) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) r[j] = __float_as_uint(__fmul_rn(p.beta, __uint_as_float(r[j])));
                }
                if (col < p.n) {
                    if (p.c32) {
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (tok0 + j0 + j < p.m) p.c32[(size_t)(tok0 + j0 + j) * p.n + col] = __uint_as_float(r[j]);
                    } else if (p.yacc) {
                        float yv[16];
#pragma unroll
                        for (int j = 0; j < 16; ++j) yv[j] = (tok0 + j0 + j < p.m) ? p.yacc[(size_t)(tok0 + j0 + j) * p.n + col] : 0.0f;
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (tok0 + j0 + j < p.m)
                                p.yacc[(size_t)(tok0 + j0 + j) * p.n + col] = __fadd_rn(yv[j], t_to_f32<BF16>(f32_to_t<BF16>(__uint_as_float(r[j]))));
                    } else {
                        uint16_t v[16];
                        if (p.ep_fast) fast_ep_apply16<BF16>(fe, r, v);
                        else if (p.ep.n_nodes == 0) {
#pragma unroll
                            for (int j = 0; j < 16; ++j) v[j] = f32_to_t<BF16>(__uint_as_float(r[j]));
                        } else {
#pragma unroll
                            for (int j = 0; j < 16; ++j)
                                v[j] = (tok0 + j0 + j < p.m) ? ep_store_nodes<BF16>(nodes, p.ep.n_nodes, __uint_as_float(r[j]), (size_t)(tok0 + j0 + j), (size_t)col) : (uint16_t)0;
                        }
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (tok0 + j0 + j < p.m) {
                                if (!DENSE || !p.col_major) p.c[(size_t)(tok0 + j0 + j) * p.n + col] = v[j];
                                else p.c[(size_t)col * p.m + (tok0 + j0 + j)] = v[j];
                            }
                    }
                }
            } else {
                // partial tile of this depth slice: ws[tile][slice][token][column]
                float* dst = ws_tile + ((size_t)blockIdx.z * ntok) * (NW * 128) + (128 * w + 32 * q + lane);
#pragma unroll
                for (int j = 0; j < 16; ++j) dst[(size_t)(j0 + j) * (NW * 128)] = __uint_as_float(r[j]);
            }
        }
    }
    tc_fence_before();

    }   // drain warps
}

template <int BF16, int US, int DENSE, int CG>
__global__ void __launch_bounds__(kTcThreads, 1) gemm_tc_kernel(const __grid_constant__ TcMaps<DENSE> maps, const __grid_constant__ GemmTcArgs p) {
    const CUtensorMap& tmap_tok = maps.tok;
    extern __shared__ unsigned char smem_dyn[];
    // the swizzled operands need 1024-byte aligned tiles: align the window by hand
    unsigned char* smem_raw = smem_dyn + ((1024u - (smem_u32(smem_dyn) & 1023u)) & 1023u);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int NT = p.nt, NK = p.nk, O = p.no, NW = p.nw, PU = p.pu;
    // CG == 2: the CTA is one of a pair (cluster of two along x).  Each CTA expands its own columns and loads half of
    // the token rows; the even CTA issues MMAs of 256 weight columns that read both CTAs' shared memory and write both
    // CTAs' tensor memory, so a CTA moves half the token bytes per flop.
    const uint32_t pair_rank = CG == 2 ? cluster_ctarank() : 0u;
    const bool leader = pair_rank == 0u;
    const int tok_bytes = p.ntok_pad * 128 / CG;               // this CTA's token operand per 64-deep unit (a stage is US units)
    const int rpg = p.rpg;                                     // scale rows (blocks) staged per packed slot
    // packed slot: boxes of [8 NW groups][up to 4 units] (one tiled copy each) covering PU * US units, then [8 NW groups][rpg rows]
    const int k_code = PU * US * kUnitBytes;                   // code bytes per column group and slot
    const int kbox_shift = PU * US >= 4 ? 2 : (PU * US == 2 ? 1 : 0);   // log2(units per code box)
    const int kbox_bytes = 8 * NW * (kUnitBytes << kbox_shift);        // one code box
    const int k_stride = ((8 * NW * (k_code + rpg * 32) + 1023) / 1024) * 1024;
    const int o_stride = NW * US * kWTile;                     // ring O slot: NW x US operand tiles
    const int t_stride = US * tok_bytes;                       // ring T slot: US token tiles
    // a stage holds 8 * NW packed units, one per dequant warp: with only 8 of them the 16
    // warps form two groups that take alternate stages
    const int deq_groups = (8 * NW * US >= kDeqWarps) ? 1 : 2;
    const int deq_wpg = kDeqWarps / deq_groups;

    unsigned char* ring_o = smem_raw;
    unsigned char* ring_t = ring_o + (size_t)O * o_stride;
    unsigned char* ring_k = ring_t + (size_t)NT * t_stride;
    constexpr bool dense = DENSE != 0;                         // dense 16-bit weights: no packed ring, no expansion
    uint64_t* bars = reinterpret_cast<uint64_t*>(ring_k + (dense ? (size_t)0 : (size_t)NK * k_stride));
    uint64_t* t_full = bars;                 // [NT] token tile landed
    uint64_t* t_empty = t_full + NT;         // [NT] the stage's MMAs retired
    uint64_t* k_full = t_empty + NT;         // [NK] packed units + scale rows landed
    uint64_t* k_empty = k_full + NK;         // [NK] every dequant warp is past the slot's stages
    uint64_t* o_full = k_empty + NK;         // [O] operand written
    uint64_t* o_empty = o_full + O;          // [O] MMAs of the stage retired
    uint64_t* acc_full = o_empty + O;        // all MMAs retired
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    EpNodeDev* ep_nodes = reinterpret_cast<EpNodeDev*>(acc_full + 4);

    const int sg0 = blockIdx.x * NW;                           // first 128-column super-group
    const int col0 = blockIdx.x * 128 * NW;
    const int tok0 = blockIdx.y * p.ntok_tile;
    const int stages_all = (p.ku + US - 1) / US;
    const int per_split = (stages_all + (int)gridDim.z - 1) / (int)gridDim.z;
    const int st_begin = blockIdx.z * per_split;
    const int st_end = min(stages_all, st_begin + per_split);
    const int num_stages = max(0, st_end - st_begin);
    const int num_groups = (num_stages + PU - 1) / PU;         // packed-ring slots this CTA consumes

    if (tid == 0) {
        for (int s = 0; s < NT; ++s) {
            mbar_init(&t_full[s], 1);
            mbar_init(&t_empty[s], 1);
        }
        for (int s = 0; s < NK; ++s) {
            mbar_init(&k_full[s], 1);
            mbar_init(&k_empty[s], kDeqWarps);
        }
        for (int s = 0; s < O; ++s) {
            mbar_init(&o_full[s], dense ? 1 : CG * deq_wpg);
            mbar_init(&o_empty[s], 1);
        }
        mbar_init(acc_full, 1);
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (tid < p.ep.n_nodes && p.ep.n_nodes <= kMaxInlineNodes) ep_nodes[tid] = p.ep.nodes[tid];
    if (warp == kDeqWarps + 1) {
        if (CG == 2) {
            tmem_alloc2(tmem_slot, p.tmem_cols);
            tmem_relinquish2();
        } else {
            tmem_alloc(tmem_slot, p.tmem_cols);
            tmem_relinquish();
        }
    }
    if (warp == kDeqWarps && lane == 0) tma_prefetch_desc(&tmap_tok);
    tc_fence_before();
    if (CG == 2) cluster_sync_all();                            // the peer's barriers are initialised before anything signals them
    else __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // the even CTA's "landed" barriers, which both CTAs signal
    const uint32_t t_full_lead = CG == 2 ? mapa_shared(smem_u32(t_full), 0u) : smem_u32(t_full);
    const uint32_t o_full_lead = CG == 2 ? mapa_shared(smem_u32(o_full), 0u) : smem_u32(o_full);

    if (warp == kDeqWarps) {
        // ===================== token producer =====================
        if (lane == 0) {
            RingPos tp;
            for (int i = 0; i < num_stages; ++i, tp.next(NT)) {
                const int slot = tp.slot;
                if (tp.wrapped && !mbar_wait(&t_empty[slot], tp.phase ^ 1u, abort_flag, p.status, STATUS_TMEM_TIMEOUT)) break;
                unsigned char* sb = ring_t + (size_t)slot * t_stride;
                const int u0 = (st_begin + i) * US;
                const int units = min(US, p.ku - u0);
                if (CG == 2) {
                    // the even CTA expects both halves; each CTA loads its half of every MMA's token rows
                    if (leader) mbar_expect_tx(&t_full[slot], (unsigned)(2 * units * tok_bytes));
                    const int half = p.ntok_box / 2;
                    for (int uu = 0; uu < units; ++uu) {
                        const int d0 = (u0 + uu) * kStageK;
                        tma_load_2d_pair(sb + uu * tok_bytes, &tmap_tok, d0, tok0 + (int)pair_rank * half, t_full_lead + 8u * slot);
                        if (p.nmma == 2)
                            tma_load_2d_pair(sb + uu * tok_bytes + tok_bytes / 2, &tmap_tok, d0, tok0 + p.ntok_box + (int)pair_rank * half,
                                             t_full_lead + 8u * slot);
                    }
                } else {
                mbar_expect_tx(&t_full[slot], (unsigned)(units * tok_bytes));
                for (int uu = 0; uu < units; ++uu) {
                    const int d0 = (u0 + uu) * kStageK;
                    tma_load_2d(sb + uu * tok_bytes, &tmap_tok, d0, tok0, &t_full[slot]);
                    if (p.nmma == 2) tma_load_2d(sb + uu * tok_bytes + tok_bytes / 2, &tmap_tok, d0, tok0 + p.ntok_box, &t_full[slot]);
                }
                }
            }
        }
    } else if (warp == kDeqWarps + 2) {
        // ===================== packed-weight producer =====================
        // One slot covers PU stages: issuing a bulk copy costs a couple of hundred cycles whatever its
        // size, so a column group's units of PU stages (contiguous along K) travel as one copy, and so do
        // its scale rows.  Lanes 0-15 issue the code runs, lanes 16-31 the scale rows.
        if constexpr (DENSE != 0) {
            // dense 16-bit weights need no expansion: their K-major tiles go straight into the operand ring
            if (lane == 0) {
                tma_prefetch_desc(&maps.w);
                RingPos op;
                for (int i = 0; i < num_stages; ++i, op.next(O)) {
                    const int os = op.slot;
                    if (op.wrapped && !mbar_wait(&o_empty[os], op.phase ^ 1u, abort_flag, p.status, STATUS_TMEM_TIMEOUT)) break;
                    unsigned char* ob = ring_o + (size_t)os * o_stride;
                    const int u0 = (st_begin + i) * US;
                    const int units = min(US, p.ku - u0);
                    if (CG == 2) {
                        if (leader) mbar_expect_tx(&o_full[os], (unsigned)(2 * NW * units * kWTile));
                        for (int w = 0; w < NW; ++w)
                            for (int uu = 0; uu < units; ++uu)
                                tma_load_2d_pair(ob + (w * US + uu) * kWTile, &maps.w, (u0 + uu) * kStageK, col0 + 128 * w, o_full_lead + 8u * os);
                    } else {
                    mbar_expect_tx(&o_full[os], (unsigned)(NW * units * kWTile));
                    for (int w = 0; w < NW; ++w)
                        for (int uu = 0; uu < units; ++uu)
                            tma_load_2d(ob + (w * US + uu) * kWTile, &maps.w, (u0 + uu) * kStageK, col0 + 128 * w, &o_full[os]);
                    }
                }
            }
        } else {
        if (lane == 0) {
            tma_prefetch_desc(&maps.codes);
            tma_prefetch_desc(&maps.scales);
            RingPos kp;
            for (int gq = 0; gq < num_groups; ++gq, kp.next(NK)) {
                const int slot = kp.slot;
                if (kp.wrapped && !mbar_wait(&k_empty[slot], kp.phase ^ 1u, abort_flag, p.status, STATUS_TMEM_TIMEOUT)) break;
                unsigned char* sb = ring_k + (size_t)slot * k_stride;
                const int u0 = (st_begin + gq * PU) * US;               // first 64-deep unit of the slot
                const int blk0 = (u0 * kStageK) >> p.log2_block;
                // whole boxes always: what lies past the last unit, block or column group arrives as zeros and is never used
                mbar_expect_tx(&k_full[slot], (unsigned)(8 * NW) * (unsigned)(k_code + rpg * 32));
                for (int x = 0; x < PU * US; x += 4)
                    tma_load_2d(sb + (size_t)(x >> 2) * kbox_bytes, &maps.codes, (u0 + x) * (kUnitBytes / 8), sg0 * 8, &k_full[slot]);
                tma_load_2d(sb + (size_t)8 * NW * k_code, &maps.scales, blk0 * 4, sg0 * 8, &k_full[slot]);
            }
        }
        }
    } else if (warp == kDeqWarps + 1) {
        // ===================== MMA issuer =====================
        // The whole warp walks the stages, converged, and one elected lane issues: the descriptors and barrier addresses
        // are then warp-uniform values.  (A loop run by one lane alone measured 10-25 % slower.)
        const uint32_t idesc = umma_idesc(BF16, 128 * CG, p.ntok_box);
        const uint32_t tok_half = (uint32_t)(tok_bytes / 2);
        RingPos tq, oq;
        for (int i = 0; i < (leader ? num_stages : 0); ++i, tq.next(NT), oq.next(O)) {
            const int ts = tq.slot, os = oq.slot;
            if (!__all_sync(0xffffffffu, mbar_wait(&t_full[ts], tq.phase, abort_flag, p.status, STATUS_TMEM_TIMEOUT))) break;
            if (!__all_sync(0xffffffffu, mbar_wait(&o_full[os], oq.phase, abort_flag, p.status, STATUS_TMEM_TIMEOUT))) break;
            tc_fence_after();
            const uint32_t tok_addr = smem_u32(ring_t + (size_t)ts * t_stride);
            const uint32_t w_addr = smem_u32(ring_o + (size_t)os * o_stride);
            const int units = US == 1 ? 1 : min(US, p.ku - (st_begin + i) * US);
            if (elect_one()) {
#pragma unroll
                for (int uu = 0; uu < US; ++uu) {
                    if (uu >= units) break;
                    for (int w = 0; w < NW; ++w) {
                        const uint64_t a_desc0 = umma_desc_sw128(w_addr + (w * US + uu) * kWTile);
                        for (int h = 0; h < p.nmma; ++h) {
                            const uint64_t b_desc0 = umma_desc_sw128(tok_addr + uu * tok_bytes + h * tok_half);
                            const uint32_t d_tmem = tmem_base + (uint32_t)((w * p.nmma + h) * p.ntok_box);
#pragma unroll
                            for (int ks = 0; ks < kStageK / 16; ++ks)
                                if (CG == 2) umma_f16_2(d_tmem, a_desc0 + 2 * ks, b_desc0 + 2 * ks, idesc, (i > 0 || uu > 0 || ks > 0) ? 1u : 0u);
                                else umma_f16(d_tmem, a_desc0 + 2 * ks, b_desc0 + 2 * ks, idesc, (i > 0 || uu > 0 || ks > 0) ? 1u : 0u);
                        }
                    }
                }
                if (CG == 2) {
                    umma_commit2(&o_empty[os]);
                    umma_commit2(&t_empty[ts]);
                } else {
                    umma_commit(&o_empty[os]);
                    umma_commit(&t_empty[ts]);
                }
            }
            __syncwarp();
        }
        if (leader && elect_one()) {
            if (CG == 2) umma_commit2(acc_full);
            else umma_commit(acc_full);
        }
        __syncwarp();
    } else {
        // ===================== dequant warps (0..15), then epilogue =====================
        const int g = lane >> 2, t = lane & 3;
        const int wig = deq_groups == 2 ? (warp & 7) : warp;   // warp within its group
        RingPos dk, dq;                                        // packed ring (advanced once per PU stages), operand ring
        int iu = 0;                                            // stage within its packed slot
        if (US == 1 && !dense) {
            // One unit per warp and stage (8 NW column groups = the warps of a group): everything that does not change
            // from stage to stage is formed here, once.
            const int c = wig;                                  // this warp's column group within the CTA
            // gate/up matrix: gate column groups go to operand tile 0 and the matching up groups to tile 1, so that a
            // thread of the drain holds both values of one hidden unit (chunks of [2 gate | 2 up] groups)
            const int tw = p.glu ? (c >> 1) & 1 : c >> 3, rg = p.glu ? ((c >> 2) << 1) | (c & 1) : c & 7;
            const bool odd = (g & 1) != 0;
            const uint32_t off_first = (uint32_t)(((odd ? 4 + t : t) ^ g) << 4), off_second = (uint32_t)(((odd ? t : 4 + t) ^ g) << 4);
            const uint32_t row_off = (uint32_t)(tw * kWTile + rg * 2048 + g * 128);
            const uint32_t code_off = (uint32_t)(((c << kbox_shift) * kUnitBytes) + lane * 16);
            const uint32_t sc_off = (uint32_t)(8 * NW * k_code + c * rpg * 32 + 4 * g);
            const uint32_t ring_k_a = smem_u32(ring_k), ring_o_a = smem_u32(ring_o);
            const int L = p.log2_block, box_mask = (1 << kbox_shift) - 1;
            int du = st_begin * kStageK, blk0 = du >> L;       // depth of the stage, first scale row of its packed slot
            for (int i = 0; i < num_stages; ++i, du += kStageK, dq.next(O)) {
                const int ks = dk.slot;
                const bool last_of_slot = (iu == PU - 1) || (i == num_stages - 1);
                if (iu == 0) blk0 = du >> L;
                if (deq_groups == 1 || (i & 1) == (warp >> 3)) {
                    const int os = dq.slot;
                    if (dq.wrapped && !__all_sync(0xffffffffu, mbar_wait(&o_empty[os], dq.phase ^ 1u, abort_flag, p.status, STATUS_TMEM_TIMEOUT))) break;
                    if (!__all_sync(0xffffffffu, mbar_wait(&k_full[ks], dk.phase, abort_flag, p.status, STATUS_TMEM_TIMEOUT))) break;
                    const uint32_t pk = ring_k_a + (uint32_t)(ks * k_stride);
                    uint4 wv = lds128(pk + code_off + (uint32_t)((iu >> kbox_shift) * kbox_bytes + (iu & box_mask) * kUnitBytes));
                    const int ra = ((du + 8 * t) >> L) - blk0, rb = ((du + 32 + 8 * t) >> L) - blk0;
                    uint32_t sa = lds32(pk + sc_off + (uint32_t)(ra * 32)), sb = lds32(pk + sc_off + (uint32_t)(rb * 32));
                    if (odd) {
                        uint32_t x = wv.x; wv.x = wv.z; wv.z = x;
                        x = wv.y; wv.y = wv.w; wv.w = x;
                        x = sa; sa = sb; sb = x;
                    }
                    dequant_unit_q4_at<BF16>(ring_o_a + (uint32_t)(os * o_stride) + row_off, off_first, off_second, wv, sa, sb);
                    fence_proxy_async();
                    __syncwarp();
                    if (lane == 0) {
                        if (CG == 2) mbar_arrive_cluster(o_full_lead + 8u * os);
                        else mbar_arrive(&o_full[os]);
                    }
                }
                // a warp that walks past the end of a packed slot releases it, whether it expanded this stage or not
                if (last_of_slot) {
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&k_empty[ks]);
                }
                if (++iu == PU) { iu = 0; dk.next(NK); }
            }
        } else
        for (int i = 0; i < (dense ? 0 : num_stages); ++i, dq.next(O), (++iu == PU ? (iu = 0, dk.next(NK)) : (void)0)) {
            const int ks = dk.slot;
            const bool last_of_slot = (iu == PU - 1) || (i == num_stages - 1);
            if (deq_groups == 2 && (i & 1) != (warp >> 3)) {
                // not this group's stage; a warp that walks past the end of a packed slot still releases it
                if (last_of_slot) {
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&k_empty[ks]);
                }
                continue;
            }
            const int os = dq.slot;
            if (dq.wrapped && !__all_sync(0xffffffffu, mbar_wait(&o_empty[os], dq.phase ^ 1u, abort_flag, p.status, STATUS_TMEM_TIMEOUT))) break;
            if (!__all_sync(0xffffffffu, mbar_wait(&k_full[ks], dk.phase, abort_flag, p.status, STATUS_TMEM_TIMEOUT))) break;
            const int uq = iu * US;                                 // first unit of the stage within the packed slot
            const int u0 = (st_begin + i) * US;                     // first unit of the stage
            const int units = min(US, p.ku - u0);
            const int blk0 = ((st_begin + i - iu) * US * kStageK) >> p.log2_block;    // first scale row of the slot
            const unsigned char* pk = ring_k + (size_t)ks * k_stride;
            const uint16_t* scs = reinterpret_cast<const uint16_t*>(pk + (size_t)8 * NW * k_code);
            unsigned char* ob = ring_o + (size_t)os * o_stride;
            if (US == 1) {
                // work item c = w * 8 + column group
                const int du = u0 * kStageK;                        // depth of the stage
                const int ra = ((du + 8 * t) >> p.log2_block) - blk0, rb = ((du + 32 + 8 * t) >> p.log2_block) - blk0;
                for (int c = wig; c < 8 * NW; c += deq_wpg) {
                    const int cgl = c & 7, w = c >> 3;
                    const uint4 wv = *reinterpret_cast<const uint4*>(pk + (size_t)(uq >> kbox_shift) * kbox_bytes + (((size_t)c << kbox_shift) + (uq & ((1 << kbox_shift) - 1))) * kUnitBytes + lane * 16);
                    // gate/up matrix: gate column groups go to operand tile 0 and the matching up groups to tile 1,
                    // so that a thread of the drain holds both values of one hidden unit
                    int tw = w, rg = cgl;
                    if (p.glu) {
                        tw = (c >> 1) & 1;                         // chunks of [2 gate | 2 up] groups
                        rg = ((c >> 2) << 1) | (c & 1);
                    }
                    dequant_unit_q4<BF16>(ob + tw * kWTile, rg, wv, scs + (size_t)c * rpg * 16, ra, rb, g, t);
                }
            } else {
            // work item = (w * 8 + column group) * US + unit of the stage
            for (int it = wig; it < 8 * NW * US; it += deq_wpg) {
                const int uu = it % US, c = it / US, cgl = c & 7, w = c >> 3;
                if (uu >= units) continue;
                const int du = (u0 + uu) * kStageK;                 // depth of the unit
                const int ra = ((du + 8 * t) >> p.log2_block) - blk0, rb = ((du + 32 + 8 * t) >> p.log2_block) - blk0;
                const int un = uq + uu;
                const uint4 wv = *reinterpret_cast<const uint4*>(pk + (size_t)(un >> kbox_shift) * kbox_bytes + (((size_t)c << kbox_shift) + (un & ((1 << kbox_shift) - 1))) * kUnitBytes + lane * 16);
                // gate/up matrix: gate column groups go to operand tile 0 and the matching up groups to tile 1,
                // so that a thread of the drain holds both values of one hidden unit
                int tw = w, rg = cgl;
                if (p.glu) {
                    tw = (c >> 1) & 1;                             // chunks of [2 gate | 2 up] groups
                    rg = ((c >> 2) << 1) | (c & 1);
                }
                dequant_unit_q4<BF16>(ob + (tw * US + uu) * kWTile, rg, wv, scs + (size_t)c * rpg * 16, ra, rb, g, t);
            }
            }
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) {
                if (CG == 2) mbar_arrive_cluster(o_full_lead + 8u * os);
                else mbar_arrive(&o_full[os]);
            }
            if (last_of_slot) {
                __syncwarp();
                if (lane == 0) mbar_arrive(&k_empty[ks]);
            }
        }

        // ---- drain: thread = weight column (TMEM lane), registers = tokens.  A warp reaches the lane quarter warp % 4;
        // the token columns are split over 4 (or 2) warps per quarter ----
        // the kernel behind in the stream (the depth-split reduce, the tensor-parallel finish) may be scheduled from here
        // on: it waits (griddepcontrol.wait) for this grid to complete before it touches anything
        pdl_launch_dependents();
        const int ntok = p.ntok_pad;                               // a multiple of 32
        const int parts = (ntok % 64 == 0) ? 4 : 2;                // every part is whole groups of 16 tokens
        const int splits = (int)gridDim.z;
        const bool rowmajor_c = !p.c32 && !p.yacc && !p.glu && !(DENSE && (p.col_major || p.beta != 1.0f));
        const bool plain = rowmajor_c && p.ep.n_nodes == 0, fast = rowmajor_c && p.ep.n_nodes > 0 && p.ep_fast;
        if (num_stages > 0 && (splits > 1 || p.glu || p.yacc || plain || fast)) {
            if (warp < 4 * parts) {
                mbar_wait(acc_full, 0, abort_flag, p.status, STATUS_TMEM_TIMEOUT);
                tc_fence_after();
                const int q = warp & 3, part = warp >> 2;              // lane quarter, token part
                const uint32_t lane_base = tmem_base + ((uint32_t)(32 * q) << 16);
                const int j_begin = part * (ntok / parts), j_end = j_begin + ntok / parts;
                // C leaves through shared memory: the rings are idle once the accumulators are complete (every load has
                // landed, every MMA has retired), a thread stores its column of a [token][128 columns] tile there, and one
                // thread sends the tiles off as tiled bulk stores, which clip at the edges of C
                const bool staged = p.c_tma && splits == 1 && (p.glu || plain || fast);
                const uint32_t stage_lane = smem_u32(ring_o) + (uint32_t)((32 * q + lane) * 2);
                if (splits > 1) {
                    const int tile_id = blockIdx.y * gridDim.x + blockIdx.x;
                    float* ws_tile = p.ws + ((size_t)tile_id * splits + blockIdx.z) * (size_t)(NW * 128) * ntok;
                    for (int w = 0; w < NW; ++w)
                        drain_partial(lane_base + (uint32_t)(w * ntok), j_begin, j_end, ws_tile + (128 * w + 32 * q + lane), NW * 128);
                } else if (p.glu) {
                    drain_glu<BF16>(lane_base, ntok, j_begin, j_end, p.c, p.m, p.n >> 1, blockIdx.x * 128 + 32 * q + lane, tok0, (uint32_t)p.glu, staged ? stage_lane : 0u);
                } else if (p.yacc) {
                    for (int w = 0; w < NW; ++w)
                        drain_residual<BF16>(lane_base + (uint32_t)(w * ntok), j_begin, j_end, p.yacc, p.m, p.n, col0 + 128 * w + 32 * q + lane, tok0);
                } else if (fast) {
                    const EpNodeDev* nodes = p.ep.n_nodes <= kMaxInlineNodes ? ep_nodes : p.ep.ext;
                    for (int w = 0; w < NW; ++w) {
                        const int col = col0 + 128 * w + 32 * q + lane;
                        FastEp fe;
                        fast_ep_build<BF16>(nodes, p.ep.n_nodes, col, col < p.n, fe);
                        drain_fast_ep<BF16>(lane_base + (uint32_t)(w * ntok), j_begin, j_end, p.c, p.m, p.n, col, tok0, fe, staged ? stage_lane + (uint32_t)(w * ntok * 256) : 0u);
                    }
                } else {
                    for (int w = 0; w < NW; ++w)
                        drain_store<BF16>(lane_base + (uint32_t)(w * ntok), j_begin, j_end, p.c, p.m, p.n, col0 + 128 * w + 32 * q + lane, tok0, staged ? stage_lane + (uint32_t)(w * ntok * 256) : 0u);
                }
                tc_fence_before();
                if (staged) {
                    fence_proxy_async();
                    named_barrier_sync(1, 128 * parts);
                    if (warp == 0 && lane == 0) {
                        const int tiles_out = p.glu ? 1 : NW;
                        const int x0 = p.glu ? (int)blockIdx.x * 128 : col0;
                        const int rows = ntok > 256 ? ntok / 2 : ntok;          // a box holds at most 256 rows
                        const int ncols = p.glu ? p.n >> 1 : p.n;
                        for (int w = 0; w < tiles_out; ++w)
                            for (int r0 = 0; r0 < ntok; r0 += rows)
                                if (x0 + 128 * w < ncols && tok0 + r0 < p.m)
                                    tma_store_2d(&maps.c, smem_u32(ring_o) + (uint32_t)((w * ntok + r0) * 256), x0 + 128 * w, tok0 + r0);
                        bulk_commit_group();
                        bulk_wait_read_all();
                    }
                }
            }
        } else {
            drain_tile<BF16, DENSE>(p, tmem_base, warp, lane, num_stages, acc_full, abort_flag, ep_nodes, col0, tok0);
        }
    }
    // (every thread reaches this point, also after a timed-out wait: nothing above returns)
    if (CG == 2) cluster_sync_all();                            // neither CTA frees tensor memory or leaves while the other may still use its memory
    else __syncthreads();
    if (warp == kDeqWarps + 1) {
        tc_fence_after();
        if (CG == 2) tmem_dealloc2(tmem_base, p.tmem_cols);
        else tmem_dealloc(tmem_base, p.tmem_cols);
    }
}

// Adds the depth slices of a split GEMM in slice order and stores, for splits deep enough that one CTA per
// tile would spend longer adding than the GEMM spent multiplying.  One block = all columns of a tile x 8 tokens;
// a thread owns one column (for a gate/up matrix: one hidden unit, i.e. a gate and an up column).
template <int BF16>
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const __grid_constant__ GemmTcArgs p, int splits, int col_tiles) {
    pdl_launch_dependents();
    pdl_wait();                                                    // launched while the GEMM ahead of it drains
    const int NW = p.nw, ntok = p.ntok_pad;
    const int tile_id = blockIdx.x, bx = tile_id % col_tiles, by = tile_id / col_tiles;
    const int tok0 = by * p.ntok_tile, j0 = blockIdx.y * 8;
    const int cl = threadIdx.x;                                  // column within the CTA tile
    const float* ws_tile = p.ws + ((size_t)tile_id * splits) * (size_t)(NW * 128) * ntok;
    const EpNodeDev* nodes = p.ep.n_nodes <= kMaxInlineNodes ? p.ep.nodes : p.ep.ext;
    if (p.glu) {
        const int hn = p.n >> 1, hcol = bx * 128 + cl;
        if (cl >= 128 || hcol >= hn) return;
        float ag[8], au[8];
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) ag[jj] = au[jj] = 0.0f;
        for (int z = 0; z < splits; ++z) {
            const float* src = ws_tile + ((size_t)z * ntok + j0) * (NW * 128) + cl;
            float vg[8], vu[8];
#pragma unroll
            for (int jj = 0; jj < 8; ++jj) {
                vg[jj] = __ldcg(src + (size_t)jj * (NW * 128));
                vu[jj] = __ldcg(src + (size_t)jj * (NW * 128) + 128);
            }
#pragma unroll
            for (int jj = 0; jj < 8; ++jj) { ag[jj] += vg[jj]; au[jj] += vu[jj]; }
        }
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) {
            const int tok = tok0 + j0 + jj;
            const float gv = t_to_f32<BF16>(f32_to_t<BF16>(ag[jj])), uv = t_to_f32<BF16>(f32_to_t<BF16>(au[jj]));
            const float a = glu_gate((uint32_t)p.glu, gv);
            if (tok < p.m) p.c[(size_t)tok * hn + hcol] = f32_to_t<BF16>(__fmul_rn(a, uv));
        }
        return;
    }
    const int col = bx * 128 * NW + cl;
    if (cl >= NW * 128 || col >= p.n) return;
    float acc[8], yv[8];
#pragma unroll
    for (int jj = 0; jj < 8; ++jj) acc[jj] = 0.0f;
    if (p.yacc) {
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) yv[jj] = (tok0 + j0 + jj < p.m) ? p.yacc[(size_t)(tok0 + j0 + jj) * p.n + col] : 0.0f;
    }
    for (int z = 0; z < splits; ++z) {
        const float* src = ws_tile + ((size_t)z * ntok + j0) * (NW * 128) + cl;
        float v[8];
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) v[jj] = __ldcg(src + (size_t)jj * (NW * 128));
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) acc[jj] += v[jj];
    }
    FastEp fe;
    if (p.ep_fast) fast_ep_build<BF16>(nodes, p.ep.n_nodes, col, true, fe);
#pragma unroll
    for (int jj = 0; jj < 8; ++jj) {
        const int tok = tok0 + j0 + jj;
        if (tok >= p.m) continue;
        if (p.beta != 1.0f) acc[jj] = __fmul_rn(p.beta, acc[jj]);
        const size_t ci = p.col_major ? (size_t)col * p.m + tok : (size_t)tok * p.n + col;
        if (p.c32) {
            if (p.push_world) {
                const int owner = tok / p.push_rows;
                p.push[owner][((size_t)p.push_rank * p.push_rows + (size_t)(tok - owner * p.push_rows)) * p.n + col] = acc[jj];
            } else {
                p.c32[(size_t)tok * p.n + col] = acc[jj];
            }
        }
        else if (p.yacc) p.yacc[(size_t)tok * p.n + col] = __fadd_rn(yv[jj], t_to_f32<BF16>(f32_to_t<BF16>(acc[jj])));
        else if (p.ep_fast) p.c[ci] = fast_ep_store<BF16>(fe, acc[jj]);
        else p.c[ci] = ep_store_nodes<BF16>(nodes, p.ep.n_nodes, acc[jj], (size_t)tok, (size_t)col);
    }
}

template <int BF16, int US, int DENSE, int CG>
cudaError_t launch_tc(const CUtensorMap& tm, const CUtensorMap& tc, const CUtensorMap& tw, const CUtensorMap& ts, const GemmTcArgs& a, dim3 grid, size_t smem, cudaStream_t stream) {
    auto kern = gemm_tc_kernel<BF16, US, DENSE, CG>;
    static int attr_dev = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (attr_dev != dev) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (e != cudaSuccess) return e;
        attr_dev = dev;
    }
    TcMaps<DENSE> maps;
    maps.tok = tm;
    maps.c = tc;
    if constexpr (DENSE) maps.w = tw;
    else {
        maps.codes = tw;
        maps.scales = ts;
    }
    if (CG == 2) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = grid;
        cfg.blockDim = dim3(kTcThreads);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = stream;
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = 2;
        attr.val.clusterDim.y = 1;
        attr.val.clusterDim.z = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        return cudaLaunchKernelEx(&cfg, kern, maps, a);
    }
    kern<<<grid, kTcThreads, smem, stream>>>(maps, a);
    return cudaGetLastError();
}

}  // namespace

TensorMapEncodeFn tensor_map_encoder() {
    static TensorMapEncodeFn fn = nullptr;
    if (!fn) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = (TensorMapEncodeFn)ptr;
    }
    return fn;
}

bool gemm_tc_supported(int wkind, int m, int k, int log2_block, const void* a) {
    if (wkind != 4 && wkind != 16) return false;
    if (k % 8 != 0 || k == 0 || ((uintptr_t)a & 15) != 0) return false;   // TMA: 16-byte aligned rows
    if (log2_block < 3) return false;                                      // one scale per 8-depth chunk
    if (m < 1) return false;
    return tensor_map_encoder() != nullptr;
}

void gemm_tc_plan(GemmTcArgs& a, int sm_count, dim3* grid, size_t* smem, size_t* ws_floats, size_t* n_counters) {
    // token tiling: equal tiles of at most 512 tokens, padded so that both token halves of the
    // drain (and both MMA halves above 256) are whole groups of 16
    // the fused gate/up form keeps both values of a hidden unit in one CTA: two accumulator sets, at most 256 tokens
    // Above 256 tokens a CTA takes 128 columns x up to 512 tokens (two MMA halves share one expanded weight tile).
    // 256 columns x 256 tokens would ingest less per flop but expands twice the weights per flop and streams them
    // once per token tile: measured 15-20 % slower at 512 tokens.  The fused gate/up form needs both accumulator
    // sets for the gate and up columns and therefore tiles by 256 tokens.
    static const int env_tt = []() { const char* e = getenv("SMEG_TC_TOKEN_TILE"); return e ? atoi(e) : 0; }();
    const bool wide = a.glu != 0 || env_tt == 256;
    const int tiles = wide ? (a.m + 255) / 256 : (a.m + 511) / 512;
    const int tile = (a.m + tiles - 1) / tiles;
    const int pad = (tile + 31) / 32 * 32;
    a.ntok_tile = pad;
    a.ep_fast = fast_ep_eligible(a.ep) ? 1 : 0;
    a.ntok_pad = pad;
    a.nmma = pad > 256 ? 2 : 1;
    a.ntok_box = pad / a.nmma;
    const int col_tiles_1 = (a.n + 127) / 128;
    // two accumulator sets (256 columns per CTA) halve the token traffic when tensor memory has
    // room and there are still enough CTAs to fill the machine
    static const int env_nw = []() { const char* e = getenv("SMEG_TC_NW"); return e ? atoi(e) : 0; }();
    a.nw = (2 * pad <= 512 && pad >= 64 && col_tiles_1 >= 2 * sm_count * 3 / 4) ? 2 : 1;
    if ((env_nw == 1 || env_nw == 2) && env_nw * pad <= 512) a.nw = env_nw;
    if (wide && 2 * pad <= 512) a.nw = 2;
    int cols = 32;
    while (cols < a.nw * pad) cols *= 2;
    a.tmem_cols = cols;
    const int block = 1 << a.log2_block;
    const int col_tiles = (a.n + 128 * a.nw - 1) / (128 * a.nw);
    // depth split: one CTA per SM is resident.  Small token tiles (decode) split until the grid
    // wastes little of its last wave; larger ones only when the column tiles alone cannot fill the
    // machine (each slice costs a workspace round trip of the whole partial tile)
    a.us = (pad <= 64 && !a.wdense) ? 2 : 1;                        // small token tiles: two 64-deep units per stage halve the per-stage hand-offs
    // CTA pairs from 128 tokens up: a CTA then loads half the token rows per flop and the MMAs read half as much shared memory
    static const int env_cg = []() { const char* e = getenv("SMEG_TC_CG"); return e ? atoi(e) : 0; }();
    // (measured at 256 and 512 tokens: 10-20 % faster than single CTAs, whose token tiles leave room for two operand
    // slots only; SMEG_TC_CG = 1 / 2 forces either)
    a.cg = (a.us == 1 && pad >= 128 && col_tiles >= 2 && env_cg != 1) ? 2 : 1;
    const int stages_all = (a.ku + a.us - 1) / a.us;
    int splits = 1;
    {
        const int base = col_tiles * tiles;
        if (pad <= 64 && !a.glu) {
            double best = 0.0;
            for (int s = 1; s <= 16; s *= 2) {
                if (s > 1 && stages_all / s < 8) break;
                const int ctas = base * s;
                const int waves = (ctas + sm_count - 1) / sm_count;
                double eff = (double)ctas / ((double)waves * sm_count);
                if (s > 1) eff *= 0.97;
                if (eff > best + 1e-9) { best = eff; splits = s; }
            }
        } else {
            while (base * splits * 2 <= sm_count && stages_all / (splits * 2) >= 7 && splits < 8) splits *= 2;
        }
    }
    if (a.push_world && splits < 2 && stages_all >= 2) splits = 2;     // the pushing store lives in the depth-split reduce stage
    // shared memory: operand ring (NW x 16 KB per slot), token ring (pad x 128 B per slot) and the packed-weight
    // ring, whose slots cover PU stages each so that one bulk copy moves a column group's units of PU stages
    const int tok_bytes = a.us * pad * 128 / a.cg, o_stride = a.nw * a.us * kWTile;
    const int budget = 214 * 1024;
    static const int env_no = []() { const char* e = getenv("SMEG_TC_NO"); return e ? atoi(e) : 0; }();
    static const int env_pu = []() { const char* e = getenv("SMEG_TC_PU"); return e ? atoi(e) : 0; }();
    const int per_cta_stages = (stages_all + splits - 1) / splits;
    int best_score = -1;
    for (int pu = 8; pu >= 1; pu /= 2) {
        if (env_pu && pu != env_pu) continue;
        const int sdepth = pu * a.us * kStageK;                       // depths covered by a packed slot
        const int rpg = block <= kStageK ? sdepth / block : sdepth / block + 1;
        if (rpg > 64) continue;                                       // the scale rows of a slot travel as one box of at most 256 eight-byte elements
        const int k_stride = ((8 * a.nw * (pu * a.us * kUnitBytes + rpg * 32) + 1023) / 1024) * 1024;
        for (int no = 4; no >= 2; --no) {
            if (env_no >= 2 && env_no <= 4 && no != env_no) continue;
            for (int nk = 4; nk >= 2; --nk) {
                const int left = budget - 2048 - no * o_stride - (a.wdense ? 0 : nk * k_stride);
                if (left < 2 * tok_bytes) continue;
                int nt = left / tok_bytes;
                if (nt > 8) nt = 8;
                // prefer: at least three token slots, then three operand slots (with two, a stage's expansion cannot start
                // before the MMAs two stages back have retired: measured 15 % slower at 512 tokens), then few copies per
                // stage (large PU), then depth
                const int score = (nt >= 3 ? 1000 : 0) + (no >= 3 ? 400 : 0) + (pu > per_cta_stages ? 0 : pu * 50) + nk * 5 + nt;
                if (score > best_score) {
                    best_score = score;
                    a.pu = pu; a.rpg = rpg; a.no = no; a.nk = nk; a.nt = nt;
                }
            }
        }
    }
    const int k_stride = ((8 * a.nw * (a.pu * a.us * kUnitBytes + a.rpg * 32) + 1023) / 1024) * 1024;
    *smem = 1024 + (size_t)a.no * o_stride + (size_t)a.nt * tok_bytes + (a.wdense ? 0 : (size_t)a.nk * k_stride) +
            (size_t)(2 * a.nt + 2 * a.nk + 2 * a.no + 4) * 8 + kMaxInlineNodes * sizeof(EpNodeDev) + 64;
    a.defer = splits >= 2 ? 1 : 0;
    const int grid_x = a.cg == 2 ? (col_tiles + 1) / 2 * 2 : col_tiles;     // whole pairs: a CTA past the last column computes nothing it stores
    *grid = dim3(grid_x, tiles, splits);
    *ws_floats = splits > 1 ? (size_t)grid_x * tiles * splits * (a.nw * 128) * pad : 0;
    *n_counters = splits > 1 ? (size_t)grid_x * tiles : 0;
}

cudaError_t gemm_tc_launch(GemmTcArgs a, int bf16, dim3 grid, size_t smem, cudaStream_t stream) {
    CUtensorMap tm;
    const cuuint64_t gdim[2] = {(cuuint64_t)a.k, (cuuint64_t)a.m};
    const cuuint64_t gstride[1] = {(cuuint64_t)a.k * 2};
    const cuuint32_t box[2] = {(cuuint32_t)kStageK, (cuuint32_t)(a.ntok_box / (a.cg == 2 ? 2 : 1))};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = tensor_map_encoder()(&tm, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (void*)a.a, gdim,
                             gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                             CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
    if (smem > 227 * 1024) return cudaErrorInvalidConfiguration;
    CUtensorMap tw = tm;                                         // unused unless the weights are dense
    if (a.wdense) {
        const cuuint64_t wdim[2] = {(cuuint64_t)a.kd, (cuuint64_t)a.n};
        const cuuint64_t wstride[1] = {(cuuint64_t)a.kd * 2};
        const cuuint32_t wbox[2] = {(cuuint32_t)kStageK, 128};
        r = tensor_map_encoder()(&tw, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (void*)a.wdense, wdim,
                        wstride, wbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
    }
    CUtensorMap ts = tm;                                         // scale rows of packed weights
    if (!a.wdense) {
        // packed codes: one row per column group, ku units of 512 bytes, as 8-byte elements; a box = the CTA's column groups x up to 4 units
        const int box_units = a.pu * a.us >= 4 ? 4 : a.pu * a.us;
        const cuuint64_t cdim[2] = {(cuuint64_t)a.ku * (kUnitBytes / 8), (cuuint64_t)a.n16};
        const cuuint64_t cstride[1] = {(cuuint64_t)a.ku * kUnitBytes};
        const cuuint32_t cbox[2] = {(cuuint32_t)(box_units * (kUnitBytes / 8)), (cuuint32_t)(8 * a.nw)};
        r = tensor_map_encoder()(&tw, CU_TENSOR_MAP_DATA_TYPE_UINT64, 2, (void*)a.codes, cdim, cstride, cbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                 CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
        // scale rows: per column group nb rows of 32 bytes
        const cuuint64_t sdim[2] = {(cuuint64_t)a.nb * 4, (cuuint64_t)a.n16};
        const cuuint64_t sstride[1] = {(cuuint64_t)a.nb * 32};
        const cuuint32_t sbox[2] = {(cuuint32_t)(a.rpg * 4), (cuuint32_t)(8 * a.nw)};
        r = tensor_map_encoder()(&ts, CU_TENSOR_MAP_DATA_TYPE_UINT64, 2, (void*)a.scales, sdim, sstride, sbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                 CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
    }
    if (a.beta == 0.0f && !a.wdense) a.beta = 1.0f;
    // C as a tensor for the bulk stores of the drain: row-major 16-bit rows that start on 16-byte boundaries, and room for a
    // CTA's whole tile in the operand and token rings
    CUtensorMap tc = tm;
    a.c_tma = 0;
    {
        const size_t ncols = a.glu ? (size_t)a.n / 2 : (size_t)a.n;
        const int rows = a.ntok_pad > 256 ? a.ntok_pad / 2 : a.ntok_pad;
        const size_t tile_bytes = (size_t)(a.glu ? 1 : a.nw) * a.ntok_pad * 256;
        const size_t ring_bytes = (size_t)a.no * a.nw * a.us * kWTile + (size_t)a.nt * a.us * a.ntok_pad * 128 / a.cg;
        static const int env_ctma = []() { const char* e = getenv("SMEG_TC_CTMA"); return e ? atoi(e) : 1; }();
        if (env_ctma && a.c && !a.c32 && !a.yacc && !(a.wdense && a.col_major) && grid.z == 1 && ncols % 8 == 0 && ((uintptr_t)a.c & 15) == 0 &&
            tile_bytes <= ring_bytes) {
            const cuuint64_t cdim[2] = {(cuuint64_t)ncols, (cuuint64_t)a.m};
            const cuuint64_t cstride[1] = {(cuuint64_t)ncols * 2};
            const cuuint32_t cbox[2] = {128, (cuuint32_t)rows};
            r = tensor_map_encoder()(&tc, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (void*)a.c, cdim, cstride,
                                     cbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
            a.c_tma = 1;
        }
    }
    cudaError_t e;
    if (a.cg == 2 && a.wdense) e = bf16 ? launch_tc<1, 1, 1, 2>(tm, tc, tw, ts, a, grid, smem, stream) : launch_tc<0, 1, 1, 2>(tm, tc, tw, ts, a, grid, smem, stream);
    else if (a.cg == 2) e = bf16 ? launch_tc<1, 1, 0, 2>(tm, tc, tw, ts, a, grid, smem, stream) : launch_tc<0, 1, 0, 2>(tm, tc, tw, ts, a, grid, smem, stream);
    else if (a.wdense) e = bf16 ? launch_tc<1, 1, 1, 1>(tm, tc, tw, ts, a, grid, smem, stream) : launch_tc<0, 1, 1, 1>(tm, tc, tw, ts, a, grid, smem, stream);
    else if (a.us == 2) e = bf16 ? launch_tc<1, 2, 0, 1>(tm, tc, tw, ts, a, grid, smem, stream) : launch_tc<0, 2, 0, 1>(tm, tc, tw, ts, a, grid, smem, stream);
    else e = bf16 ? launch_tc<1, 1, 0, 1>(tm, tc, tw, ts, a, grid, smem, stream) : launch_tc<0, 1, 0, 1>(tm, tc, tw, ts, a, grid, smem, stream);
    if (e != cudaSuccess || !a.defer || grid.z < 2) return e;
    const dim3 rgrid(grid.x * grid.y, a.ntok_pad / 8);
    if (bf16) return launch_pdl(splitk_reduce_kernel<1>, rgrid, dim3(256), 0, stream, a, (int)grid.z, (int)grid.x);
    return launch_pdl(splitk_reduce_kernel<0>, rgrid, dim3(256), 0, stream, a, (int)grid.z, (int)grid.x);
}

}  // namespace smeg
