// Q4 decode GEMV / small-M GEMM for sm_100a:  C[m][n] = ep( A[m][k] @ dequant(W) ),
// m small (rows are processed in groups of 8 per tensor-core instruction).
//
// Replaces the reference's SME Q4 GEMV (run_q4_gemv1 / run_q4_gemv,
// csrc/gemm_f16f16_q4.h:236-431, and the bf16 twin csrc/gemm_b16b16_q4.h:171-268).
//
// HBM-bound design:
//   * one CTA owns CG groups of 16 output columns for the whole depth K, so no
//     cross-CTA reduction and a column's result never depends on the grid;
//   * a producer warp streams that CTA's packed codes and scales, which are
//     contiguous in the prepacked layout, into a ring of shared-memory stages
//     with cp.async.bulk (TMA engine) + mbarriers: bytes in flight are set by
//     the ring depth, not by registers;
//   * 8 consumer warps split each stage's depth (one 64-deep unit each).  A
//     lane's 16-byte vector is four A fragments of mma.m16n8k16 (16 weight
//     columns x 16 depths) -- nibbles become f16 pairs with one lop3 each, the
//     activations are the 8-wide N operand, accumulation is f32;
//   * per K-block the raw code sums are folded with the f32 block scale
//     (accumulator-side scaling), or -- for bf16 and for blocks below 32 -- each
//     weight is dequantised to exactly the reference's rounded value first;
//   * warps' partial sums are added in a fixed order through shared memory, the
//     epilogue graph runs on the rounded product, C is stored once.
#include <algorithm>
#include <cstdlib>
#include "epilogue.cuh"
#include "kernels.h"
#include "layout.h"

namespace smeg {

namespace {

constexpr int kConsumerWarps = 8;
constexpr int kStageDepth = 64 * kConsumerWarps;  // 512 depths per stage
constexpr int kThreads = 32 * (kConsumerWarps + 1);

__device__ __forceinline__ void mma_f16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1,
                                        const float (&c)[4]) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
                 : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(c[0]), "f"(c[1]), "f"(c[2]), "f"(c[3]));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1,
                                         const float (&c)[4]) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
                 : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(c[0]), "f"(c[1]), "f"(c[2]), "f"(c[3]));
}

// One packed word (8 nibbles, offset binary) -> the four A registers holding
// the exact integer codes as f16 pairs.
__device__ __forceinline__ void decode_word_f16(uint32_t w, uint32_t (&a)[4]) {
    const uint32_t w8 = w >> 8;
    uint32_t lo0 = lop3_and_or(w, 0x000f000fu, 0x64006400u);   // 1024 + u
    uint32_t hi0 = lop3_and_or(w, 0x00f000f0u, 0x64006400u);   // 1024 + 16 u
    uint32_t lo1 = lop3_and_or(w8, 0x000f000fu, 0x64006400u);
    uint32_t hi1 = lop3_and_or(w8, 0x00f000f0u, 0x64006400u);
    const __half2 off = __halves2half2(__ushort_as_half(0x6408), __ushort_as_half(0x6408));      // 1032
    const __half2 sc16 = __halves2half2(__ushort_as_half(0x2c00), __ushort_as_half(0x2c00));     // 1/16
    const __half2 off16 = __halves2half2(__ushort_as_half(0xd480), __ushort_as_half(0xd480));    // -72
    __half2 r0 = __hsub2(*reinterpret_cast<__half2*>(&lo0), off);
    __half2 r1 = __hsub2(*reinterpret_cast<__half2*>(&lo1), off);
    __half2 r2 = __hfma2(*reinterpret_cast<__half2*>(&hi0), sc16, off16);
    __half2 r3 = __hfma2(*reinterpret_cast<__half2*>(&hi1), sc16, off16);
    a[0] = *reinterpret_cast<uint32_t*>(&r0);
    a[1] = *reinterpret_cast<uint32_t*>(&r1);
    a[2] = *reinterpret_cast<uint32_t*>(&r2);
    a[3] = *reinterpret_cast<uint32_t*>(&r3);
}

template <int BF16>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    if (BF16) {
        __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&v);
    }
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Operand-side dequant of one word: every weight becomes T(f32(scale) * code),
// the reference's rounded weight (the f32 product of an f16 scale and a 4-bit
// code is exact, so this is one rounding; dequant_rows,
// src/kernels/q4/weights.rs:250-256).  sc points at this column group's staged
// scale rows [row][16]; d is the depth of the word's first element relative to
// the first staged row's block start.
template <int BF16>
__device__ __forceinline__ void decode_word_scaled(uint32_t w, uint32_t (&a)[4], const uint16_t* sc, int g,
                                                   int d_rel, int log2_block) {
    // nibble -> (column half, depth offset): see layout.h
    float v[8];
#pragma unroll
    for (int nb = 0; nb < 8; ++nb) {
        const int hi_col = (nb >> 1) & 1;
        const int e = ((nb & 1) << 1) | (nb >> 2);   // nib 0,4,1,5 -> e 0,1,2,3
        const int code = (int)((w >> (4 * nb)) & 0xfu) - 8;
        const int row = (d_rel + e) >> log2_block;
        const float s = __half2float(__ushort_as_half(sc[row * 16 + 2 * g + hi_col]));
        v[nb] = s * (float)code;
    }
    a[0] = pack2<BF16>(v[0], v[4]);   // column g,   depths +0,+1
    a[1] = pack2<BF16>(v[2], v[6]);   // column g+8, depths +0,+1
    a[2] = pack2<BF16>(v[1], v[5]);   // column g,   depths +2,+3
    a[3] = pack2<BF16>(v[3], v[7]);   // column g+8, depths +2,+3
}

template <int BF16, int OPSIDE, int MT>
__global__ void __launch_bounds__(kThreads) q4_gemv_kernel(const __grid_constant__ Q4GemvArgs p) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int NS = p.ns, CG = p.cg;
    const int code_bytes = kUnitBytes * kConsumerWarps;       // per cg per stage
    const int scale_bytes = p.rps * 32;                       // per cg per stage
    const int stage_bytes = CG * (code_bytes + scale_bytes);

    // ---- shared memory carve-up ----
    uint64_t* full = reinterpret_cast<uint64_t*>(smem_raw);
    uint64_t* empty = full + NS;
    uint64_t* a_full = empty + NS;                            // [2] activation chunk landed
    uint64_t* a_empty = a_full + 2;                           // [2] activation chunk released
    volatile int* abort_flag = reinterpret_cast<volatile int*>(a_empty + 2);
    unsigned char* stages = smem_raw + 256;
    const int a_stride = p.ka + 8;                            // halves; +16 B keeps LDS.128 conflict-free
    uint16_t* As = reinterpret_cast<uint16_t*>(stages + (size_t)NS * stage_bytes);
    const int kpad = p.k64 * 64;
    const int nchunks = (kpad + p.ka - 1) / p.ka;
    const int nbuf = nchunks > 1 ? 2 : 1;
    const size_t a_buf_halves = (size_t)p.a_rows * a_stride;   // only the rows in play are staged
    float* red = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(As) + nbuf * a_buf_halves * 2);

    const int cg0 = blockIdx.x * CG;                          // first column group of this CTA
    const int ncg = min(CG, p.n16 - cg0);
    const int row0 = blockIdx.y * 8 * MT;                     // first activation row of this CTA
    const int rows_used = min(8 * MT, p.m - row0);
    const int num_stages = (p.k64 + kConsumerWarps - 1) / kConsumerWarps;
    const int stages_per_chunk = p.ka / kStageDepth;

    if (tid == 0) {
        for (int s = 0; s < NS; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], kConsumerWarps);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&a_full[b], 1);
            mbar_init(&a_empty[b], kConsumerWarps);
        }
        *abort_flag = 0;
        fence_barrier_init();
    }
    __syncthreads();
    pdl_launch_dependents();

    if (warp == kConsumerWarps) {
        // ================= producer: stream activations and this CTA's weights =================
        // Issuing a bulk copy costs a few hundred cycles on the issuing thread, so the copies of
        // a round of stages go out from different lanes at once: lane = (stage of the round,
        // copy of the stage), the first CG copies of a stage being the code runs of its column
        // groups and the next CG their scale rows.
        const int per_stage = 2 * CG;
        // a round never spans more stages than the ring has slots (its waits are on stages issued
        // in earlier rounds) nor, with several activation chunks, more than one chunk
        // two stages per round: the first data lands early and the issue still runs ahead of the consumers
        int round_stages = min(min(32 / per_stage, NS), 2);
        if (nchunks > 1) round_stages = min(round_stages, stages_per_chunk);
        const int si = lane / per_stage, j = lane % per_stage;
        // activation chunks that start inside the round at st0: one bulk copy per row, one lane each
        auto send_a = [&](int st0) -> bool {
            if (!p.a_vec_ok) return true;
            for (int st = st0; st < min(num_stages, st0 + round_stages); ++st) {
                if (st % stages_per_chunk != 0) continue;
                const int ch = st / stages_per_chunk, buf = ch & 1;
                const int ka0 = ch * p.ka;
                const unsigned bytes = (unsigned)(min(p.ka, p.k - ka0) * 2);
                bool ok = true;
                if (lane == 0) {
                    if (ch >= 2) ok = mbar_wait(&a_empty[buf], ((ch >> 1) - 1) & 1, abort_flag, p.status);
                    if (ok) mbar_expect_tx(&a_full[buf], rows_used * bytes);
                }
                if (!__all_sync(0xffffffffu, ok)) return false;
                for (int r = lane; r < rows_used; r += 32)
                    bulk_g2s(As + buf * a_buf_halves + (size_t)r * a_stride, p.a + (size_t)(row0 + r) * p.k + ka0, bytes, &a_full[buf]);
            }
            return true;
        };
        for (int st0 = 0; st0 < num_stages; st0 += round_stages) {
            // The first round's weights go out before anything else: they do not depend on the kernel ahead in
            // the stream; the activations may, and follow once that kernel's memory is visible.
            if (st0 != 0 && !send_a(st0)) return;
            const int st = st0 + si;
            const bool active = si < round_stages && st < num_stages;
            const int slot = active ? st % NS : 0;
            const int units = active ? min(kConsumerWarps, p.k64 - st * kConsumerWarps) : 0;
            const int blk0 = (st * kStageDepth) >> p.log2_block;
            const int blk1 = min(p.nb, ((st * kStageDepth + units * 64 - 1) >> p.log2_block) + 1);
            const unsigned cb = units * kUnitBytes, sb = (unsigned)(blk1 - blk0) * 32;
            bool ok = true;
            if (active && j == 0) {
                if (st >= NS) ok = mbar_wait(&empty[slot], ((st / NS) - 1) & 1, abort_flag, p.status);
                if (ok) mbar_expect_tx(&full[slot], ncg * (cb + sb));
            }
            if (!__all_sync(0xffffffffu, ok)) return;
            if (active) {
                unsigned char* sbase = stages + (size_t)slot * stage_bytes;
                const int c = j < CG ? j : j - CG;
                if (c < ncg) {
                    const size_t cgi = cg0 + c;
                    if (j < CG) bulk_g2s(sbase + c * code_bytes, p.codes + q4_unit_offset(cgi, (size_t)st * kConsumerWarps, p.k64), cb, &full[slot]);
                    else bulk_g2s(sbase + CG * code_bytes + c * scale_bytes, p.scales + q4_scale_row(cgi, blk0, p.nb), sb, &full[slot]);
                }
            }
            if (st0 == 0) {
                pdl_wait();
                if (!send_a(0)) return;
            }
        }
        return;
    }

    // ================= consumers =================
    pdl_wait();
    float total[4][MT][4];
#pragma unroll
    for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int r = 0; r < 4; ++r) total[c][mt][r] = 0.0f;
    const float zero4[4] = {0.f, 0.f, 0.f, 0.f};

    for (int ch = 0; ch < nchunks; ++ch) {
        const int ka0 = ch * p.ka;
        const int chunk = min(p.ka, kpad - ka0);               // depths of this chunk (multiple of 64)
        const int buf = ch & (nbuf - 1);
        uint16_t* Ab = As + buf * a_buf_halves;
        const int valid = min(chunk, p.k - ka0);                // depths that exist in A
        if (p.a_vec_ok) {
            if (valid < chunk) {
                // zero the padded tail (the bulk copy writes only the first `valid` depths)
                for (int idx = tid; idx < rows_used * (chunk - valid); idx += 32 * kConsumerWarps)
                    Ab[(size_t)(idx / (chunk - valid)) * a_stride + valid + idx % (chunk - valid)] = 0;
                asm volatile("bar.sync 1, %0;" ::"n"(32 * kConsumerWarps));
            }
            mbar_wait(&a_full[buf], (ch >> 1) & 1, abort_flag, p.status);
        } else {
            // rows of A are not 16-byte aligned: cooperative copy (zero padded)
            asm volatile("bar.sync 1, %0;" ::"n"(32 * kConsumerWarps));
            for (int r = 0; r < rows_used; ++r) {
                const uint16_t* src = p.a + (size_t)(row0 + r) * p.k + ka0;
                for (int d = tid; d < chunk; d += 32 * kConsumerWarps) Ab[(size_t)r * a_stride + d] = d < valid ? src[d] : (uint16_t)0;
            }
            asm volatile("bar.sync 1, %0;" ::"n"(32 * kConsumerWarps));
        }

        const int st_begin = ch * stages_per_chunk, st_end = min(num_stages, st_begin + stages_per_chunk);
        for (int st = st_begin; st < st_end; ++st) {
            const int slot = st % NS;
            mbar_wait(&full[slot], (st / NS) & 1, abort_flag, p.status);
            const int units = min(kConsumerWarps, p.k64 - st * kConsumerWarps);
            if (warp < units) {
                const unsigned char* sbase = stages + (size_t)slot * stage_bytes;
                const int d_unit = st * kStageDepth + warp * 64;            // global depth of this unit
                const int dl = d_unit - ka0;                                // within the staged A chunk
                const int blk0 = (st * kStageDepth) >> p.log2_block;        // first staged scale row
                // activation fragments for this unit, shared by every column group;
                // rows past the batch contribute zeros
                uint4 alo[MT], ahi[MT];
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    alo[mt] = make_uint4(0, 0, 0, 0);
                    ahi[mt] = make_uint4(0, 0, 0, 0);
                    if (8 * mt + g < rows_used) {
                        const uint16_t* ar = Ab + (size_t)(8 * mt + g) * a_stride + dl + 8 * t;
                        alo[mt] = *reinterpret_cast<const uint4*>(ar);
                        ahi[mt] = *reinterpret_cast<const uint4*>(ar + 32);
                    }
                }
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    if (c >= ncg) break;
                    const uint4 wv = *reinterpret_cast<const uint4*>(sbase + c * code_bytes + warp * kUnitBytes + lane * 16);
                    const uint16_t* sc = reinterpret_cast<const uint16_t*>(sbase + CG * code_bytes + c * scale_bytes);
                    const uint32_t words[4] = {wv.x, wv.y, wv.z, wv.w};
                    if (OPSIDE) {
#pragma unroll
                        for (int ks = 0; ks < 4; ++ks) {
                            uint32_t af[4];
                            const int d_word = d_unit + 32 * (ks >> 1) + 8 * t + 4 * (ks & 1);
                            decode_word_scaled<BF16>(words[ks], af, sc, g, d_word - (blk0 << p.log2_block), p.log2_block);
#pragma unroll
                            for (int mt = 0; mt < MT; ++mt) {
                                const uint4& av = (ks >> 1) ? ahi[mt] : alo[mt];
                                const uint32_t b0 = (ks & 1) ? av.z : av.x, b1 = (ks & 1) ? av.w : av.y;
                                if (BF16) mma_bf16(total[c][mt], af, b0, b1, total[c][mt]);
                                else mma_f16(total[c][mt], af, b0, b1, total[c][mt]);
                            }
                        }
                    } else {
                        // accumulator-side scaling: raw code sums per 32-deep half unit,
                        // folded with the f32 block scale (block >= 32 here)
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            uint32_t af0[4], af1[4];
                            decode_word_f16(words[2 * h], af0);
                            decode_word_f16(words[2 * h + 1], af1);
                            const int row = ((d_unit + 32 * h) >> p.log2_block) - blk0;
                            // one 32-bit read: the scales of columns g and g+8 sit side by side
                            const uint32_t sp = *reinterpret_cast<const uint32_t*>(sc + row * 16 + 2 * g);
                            const float2 sf = __half22float2(*reinterpret_cast<const __half2*>(&sp));
#pragma unroll
                            for (int mt = 0; mt < MT; ++mt) {
                                const uint4& av = h ? ahi[mt] : alo[mt];
                                float part[4];
                                mma_f16(part, af0, av.x, av.y, zero4);
                                mma_f16(part, af1, av.z, av.w, part);
                                total[c][mt][0] = fmaf(part[0], sf.x, total[c][mt][0]);
                                total[c][mt][1] = fmaf(part[1], sf.x, total[c][mt][1]);
                                total[c][mt][2] = fmaf(part[2], sf.y, total[c][mt][2]);
                                total[c][mt][3] = fmaf(part[3], sf.y, total[c][mt][3]);
                            }
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[slot]);
        }
        if (p.a_vec_ok && lane == 0) mbar_arrive(&a_empty[buf]);
    }

    // ---- fixed-order reduction over the 8 warps, epilogue, store ----
    // red[warp][c][mt][r][lane]
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        if (c >= CG) break;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int r = 0; r < 4; ++r) red[((((size_t)warp * CG + c) * MT + mt) * 4 + r) * 32 + lane] = total[c][mt][r];
    }
    asm volatile("bar.sync 1, %0;" ::"n"(32 * kConsumerWarps));
    const int per_warp = CG * MT * 128;
    for (int o = tid; o < per_warp; o += 32 * kConsumerWarps) {
        float acc = 0.0f;
#pragma unroll
        for (int w = 0; w < kConsumerWarps; ++w) acc += red[(size_t)w * per_warp + o];
        const int ln = o & 31, r = (o >> 5) & 3, mt = (o >> 7) % MT, c = o / (128 * MT);
        const int col = (cg0 + c) * 16 + (ln >> 2) + 8 * (r >> 1);
        const int row = row0 + 8 * mt + 2 * (ln & 3) + (r & 1);
        if (c < ncg && col < p.n && row < p.m) {
            if (p.c32) p.c32[(size_t)row * p.n + col] = acc;
            else p.c[(size_t)row * p.n + col] = ep_store_value<BF16>(p.ep, acc, (size_t)row, (size_t)col);
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Streaming form for decode-sized calls (m <= 16, all of A in shared memory).
//
// The packed codes are one linear stream of 512-byte units in (column group, depth) order.  The
// list of 16-unit stages -- never crossing a column group -- is cut into one contiguous range per
// CTA, one CTA per SM, so that every SM streams the same number of bytes (within one stage)
// whatever n and k are, through a ring as deep as shared memory allows.  16 consumer warps take one
// unit of each stage; when a column group (or this CTA's share of it) ends they hand their partial
// sums to a store warp through a double-buffered exchange and go on with the next column group,
// so the ring never drains between column groups.  A column group cut by a range boundary is
// summed through global scratch: every CTA of it writes its share, the one that arrives last
// (an atomic counter per column group, left at zero again) adds the shares in range order and
// stores.  No CTA waits for another.
constexpr int kSWarps = 16;
constexpr int kSThreads = 32 * (kSWarps + 2);   // + producer warp + store warp
// UPW = units of a stage each consumer warp takes (1 or 2): a stage is 16 * UPW units.  Two units
// per warp halve the barrier traffic per byte and give the scheduler two independent chains; one
// keeps the ranges balanced when a CTA only gets a handful of stages.

// UPW units of one stage at once, the walk over the units innermost: their chains are independent,
// so the instruction stream alternates between them.
template <int BF16, int OPSIDE, int MT, int UPW>
__device__ __forceinline__ void consume_units(const uint4 (&wv)[UPW], const uint16_t* sc, const uint4 (&alo)[UPW][MT],
                                              const uint4 (&ahi)[UPW][MT], int g, int t, const int (&d_unit)[UPW], int blk0,
                                              int log2_block, float (&total)[MT][4]) {
    const float zero4[4] = {0.f, 0.f, 0.f, 0.f};
    if (OPSIDE) {
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
#pragma unroll
            for (int u = 0; u < UPW; ++u) {
                const uint32_t word = ks == 0 ? wv[u].x : (ks == 1 ? wv[u].y : (ks == 2 ? wv[u].z : wv[u].w));
                uint32_t af[4];
                const int d_word = d_unit[u] + 32 * (ks >> 1) + 8 * t + 4 * (ks & 1);
                decode_word_scaled<BF16>(word, af, sc, g, d_word - (blk0 << log2_block), log2_block);
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    const uint4& av = (ks >> 1) ? ahi[u][mt] : alo[u][mt];
                    const uint32_t b0 = (ks & 1) ? av.z : av.x, b1 = (ks & 1) ? av.w : av.y;
                    if (BF16) mma_bf16(total[mt], af, b0, b1, total[mt]);
                    else mma_f16(total[mt], af, b0, b1, total[mt]);
                }
            }
        }
    } else {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            float part[UPW][MT][4];
            float2 sf[UPW];
#pragma unroll
            for (int u = 0; u < UPW; ++u) {
                uint32_t af0[4], af1[4];
                decode_word_f16(h ? wv[u].z : wv[u].x, af0);
                decode_word_f16(h ? wv[u].w : wv[u].y, af1);
                const int row = ((d_unit[u] + 32 * h) >> log2_block) - blk0;
                // one 32-bit read: the scales of columns g and g+8 sit side by side
                const uint32_t sp = *reinterpret_cast<const uint32_t*>(sc + row * 16 + 2 * g);
                sf[u] = __half22float2(*reinterpret_cast<const __half2*>(&sp));
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    const uint4& av = h ? ahi[u][mt] : alo[u][mt];
                    mma_f16(part[u][mt], af0, av.x, av.y, zero4);
                    mma_f16(part[u][mt], af1, av.z, av.w, part[u][mt]);
                }
            }
#pragma unroll
            for (int u = 0; u < UPW; ++u)
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    total[mt][0] = fmaf(part[u][mt][0], sf[u].x, total[mt][0]);
                    total[mt][1] = fmaf(part[u][mt][1], sf[u].x, total[mt][1]);
                    total[mt][2] = fmaf(part[u][mt][2], sf[u].y, total[mt][2]);
                    total[mt][3] = fmaf(part[u][mt][3], sf[u].y, total[mt][3]);
                }
        }
    }
}

// First stage of CTA b's range, and the CTA whose range holds stage s.
__device__ __forceinline__ int srange_begin(int b, int total, int grid) { return (int)((long long)b * total / grid); }
__device__ __forceinline__ int srange_owner(int s, int total, int grid) {
    return (int)((((long long)s + 1) * grid - 1) / total);
}

template <int BF16, int OPSIDE, int MT, int UPW>
__global__ void __launch_bounds__(kSThreads, 1) q4_gemv_stream_kernel(const __grid_constant__ Q4GemvArgs p) {
    constexpr int kSU = kSWarps * UPW;                               // units per stage
    constexpr int kSCodeBytes = kSU * kUnitBytes;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int NS = p.sns, spc = p.spc;

    uint64_t* full = reinterpret_cast<uint64_t*>(smem_raw);         // [NS] stage landed
    uint64_t* empty = full + NS;                                     // [NS] stage released by the 16 consumer warps
    uint64_t* r_full = empty + NS;                                   // [2] partial sums handed to the store warp
    uint64_t* r_empty = r_full + 2;                                  // [2] ... and read by it
    uint64_t* a_full = r_empty + 2;                                  // activations landed
    volatile int* abort_flag = reinterpret_cast<volatile int*>(a_full + 1);
    unsigned char* ring = smem_raw + 1024;
    const int a_stride = p.k64 * 64 + 8;                             // halves; +16 B keeps LDS.128 conflict-free
    uint16_t* As = reinterpret_cast<uint16_t*>(ring + (size_t)NS * p.sslot);
    float* red = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(As) + (size_t)p.a_rows * a_stride * 2);
    constexpr int kVals = 4 * MT;                                    // values per lane of one column group's tile

    const int s_begin = srange_begin(blockIdx.x, p.stotal, gridDim.x);
    const int s_end = srange_begin(blockIdx.x + 1, p.stotal, gridDim.x);

    if (tid == 0) {
        for (int s = 0; s < NS; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], kSWarps);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&r_full[b], kSWarps);
            mbar_init(&r_empty[b], 1);
        }
        mbar_init(a_full, 1);
        *abort_flag = 0;
        fence_barrier_init();
    }
    // depths past k: the bulk copies write [0, k) of each row only
    {
        const int pad = p.k64 * 64 - p.k;
        for (int idx = tid; idx < p.a_rows * pad; idx += kSThreads) As[(size_t)(idx / pad) * a_stride + p.k + idx % pad] = 0;
    }
    __syncthreads();
    pdl_launch_dependents();

    if (warp == kSWarps) {
        // ================= producer =================
        // The weights do not depend on the kernel ahead in the stream: the ring is filled first, and the
        // activations follow once that kernel's memory is visible (before the first wait on a ring slot).
        bool a_sent = false;
        auto send_a = [&]() {
            pdl_wait();
            if (lane == 0) mbar_expect_tx(a_full, (unsigned)(p.a_rows * p.k * 2));
            __syncwarp();
            for (int r = lane; r < p.a_rows; r += 32)
                bulk_g2s(As + (size_t)r * a_stride, p.a + (size_t)r * p.k, (unsigned)(p.k * 2), a_full);
            a_sent = true;
        };
        // a round of four stages, two lanes each: codes and scale rows go out in parallel
        constexpr int kRound = 4;
        const int si = lane >> 1, j = lane & 1;
        for (int st0 = s_begin; st0 < s_end; st0 += kRound) {
            if (!a_sent && st0 - s_begin + kRound > NS) send_a();
            const int st = st0 + si;
            const bool active = si < kRound && st < s_end;
            const int i = st - s_begin, slot = active ? i % NS : 0;
            const int cg = active ? st / spc : 0;
            const int u0 = active ? (st - cg * spc) * kSU : 0;
            const int units = active ? min(kSU, p.k64 - u0) : 0;
            const int blk0 = (u0 * 64) >> p.log2_block;
            const int blk1 = min(p.nb, (((u0 + units) * 64 - 1) >> p.log2_block) + 1);
            const unsigned cb = units * kUnitBytes, sb = (unsigned)max(blk1 - blk0, 0) * 32;
            bool ok = true;
            if (active && j == 0) {
                if (i >= NS) ok = mbar_wait(&empty[slot], ((i / NS) - 1) & 1, abort_flag, p.status);
                if (ok) mbar_expect_tx(&full[slot], cb + sb);
            }
            if (!__all_sync(0xffffffffu, ok)) return;
            if (active) {
                unsigned char* sbase = ring + (size_t)slot * p.sslot;
                if (j == 0) bulk_g2s(sbase, p.codes + q4_unit_offset((size_t)cg, (size_t)u0, p.k64), cb, &full[slot]);
                else if (sb) bulk_g2s(sbase + kSCodeBytes, p.scales + q4_scale_row((size_t)cg, blk0, p.nb), sb, &full[slot]);
            }
        }
        if (!a_sent) send_a();
        return;
    }

    if (warp == kSWarps + 1) {
        // ================= store warp =================
        pdl_wait();
        int tix = 0;
        for (int st = s_begin; st < s_end; ++tix) {
            const int cg = st / spc;
            const int cg_first = cg * spc, cg_last = cg_first + spc;      // this column group's stages
            const int piece_end = min(s_end, cg_last);
            const int par = tix & 1;
            if (!mbar_wait(&r_full[par], (tix >> 1) & 1, abort_flag, p.status)) return;
            float v[kVals];
            const float* rb = red + (size_t)par * kSWarps * kVals * 32;
#pragma unroll
            for (int q = 0; q < kVals; ++q) {
                float acc = 0.0f;
#pragma unroll
                for (int w = 0; w < kSWarps; ++w) acc += rb[(w * kVals + q) * 32 + lane];
                v[q] = acc;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&r_empty[par]);
            bool store = true;
            if (st != cg_first || piece_end != cg_last) {
                // a cut column group: publish this share; the last CTA to arrive adds them in range order
                const int first_cta = srange_owner(cg_first, p.stotal, gridDim.x);
                const int last_cta = srange_owner(cg_last - 1, p.stotal, gridDim.x);
                const int np = last_cta - first_cta + 1;
                float* mine = p.ws + ((size_t)cg * p.spieces + (blockIdx.x - first_cta)) * (kVals * 32);
#pragma unroll
                for (int q = 0; q < kVals; ++q) mine[q * 32 + lane] = v[q];
                __threadfence();
                __syncwarp();
                int old = 0;
                if (lane == 0) old = atomicAdd(&p.counters[cg], 1);
                old = __shfl_sync(0xffffffffu, old, 0);
                store = old == np - 1;
                if (store) {
                    __threadfence();
                    const float* base = p.ws + (size_t)cg * p.spieces * (kVals * 32);
#pragma unroll
                    for (int q = 0; q < kVals; ++q) v[q] = 0.0f;
                    for (int pc = 0; pc < np; ++pc) {
#pragma unroll
                        for (int q = 0; q < kVals; ++q) v[q] += __ldcg(base + (size_t)pc * (kVals * 32) + q * 32 + lane);
                    }
                    if (lane == 0) p.counters[cg] = 0;
                }
            }
            if (store) {
#pragma unroll
                for (int q = 0; q < kVals; ++q) {
                    const int mt = q >> 2, r = q & 3;
                    const int col = cg * 16 + g + 8 * (r >> 1);
                    const int row = 8 * mt + 2 * t + (r & 1);
                    if (col < p.n && row < p.m) {
                        if (p.c32) p.c32[(size_t)row * p.n + col] = v[q];
                        else p.c[(size_t)row * p.n + col] = ep_store_value<BF16>(p.ep, v[q], (size_t)row, (size_t)col);
                    }
                }
            }
            st = piece_end;
        }
        return;
    }

    // ================= consumers =================
    float total[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int r = 0; r < 4; ++r) total[mt][r] = 0.0f;
    pdl_wait();
    if (!mbar_wait(a_full, 0, abort_flag, p.status)) return;
    int tix = 0;
    int sl = s_begin % spc;
    int slot = 0;
    unsigned phase = 0;
    for (int st = s_begin; st < s_end; ++st) {
        if (!mbar_wait(&full[slot], phase, abort_flag, p.status)) return;
        const int u0 = sl * kSU;
        const int units = min(kSU, p.k64 - u0);
        const unsigned char* sbase = ring + (size_t)slot * p.sslot;
        const int blk0 = (u0 * 64) >> p.log2_block;
        // a unit past the end of a short stage is computed as zero weights at the first unit's depth
        uint4 wv[UPW], alo[UPW][MT], ahi[UPW][MT];
        int d_unit[UPW];
#pragma unroll
        for (int uu = 0; uu < UPW; ++uu) {
            const int ul = warp + uu * kSWarps;
            const bool valid = ul < units;
            d_unit[uu] = (u0 + (valid ? ul : 0)) * 64;
            wv[uu] = make_uint4(0x88888888u, 0x88888888u, 0x88888888u, 0x88888888u);
            if (valid) wv[uu] = *reinterpret_cast<const uint4*>(sbase + ul * kUnitBytes + lane * 16);
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                alo[uu][mt] = make_uint4(0, 0, 0, 0);
                ahi[uu][mt] = make_uint4(0, 0, 0, 0);
                if (8 * mt + g < p.a_rows) {
                    const uint16_t* ar = As + (size_t)(8 * mt + g) * a_stride + d_unit[uu] + 8 * t;
                    alo[uu][mt] = *reinterpret_cast<const uint4*>(ar);
                    ahi[uu][mt] = *reinterpret_cast<const uint4*>(ar + 32);
                }
            }
        }
        if (warp < units)
            consume_units<BF16, OPSIDE, MT, UPW>(wv, reinterpret_cast<const uint16_t*>(sbase + kSCodeBytes), alo, ahi, g, t, d_unit,
                                                 blk0, p.log2_block, total);
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[slot]);
        if (sl == spc - 1 || st == s_end - 1) {
            const int par = tix & 1;
            if (tix >= 2 && !mbar_wait(&r_empty[par], ((tix >> 1) - 1) & 1, abort_flag, p.status)) return;
            float* rb = red + ((size_t)par * kSWarps + warp) * kVals * 32;
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    rb[(mt * 4 + r) * 32 + lane] = total[mt][r];
                    total[mt][r] = 0.0f;
                }
            __syncwarp();
            if (lane == 0) mbar_arrive(&r_full[par]);
            ++tix;
        }
        if (++sl == spc) sl = 0;
        if (++slot == NS) { slot = 0; phase ^= 1u; }
    }
}

template <int BF16, int OPSIDE, int MT>
cudaError_t launch(const Q4GemvArgs& a, dim3 grid, size_t smem, cudaStream_t stream) {
    auto kern = q4_gemv_kernel<BF16, OPSIDE, MT>;
    static int attr_dev = -1;   // the opt-in is per device; set it once (to the maximum) per device
    int dev = 0;
    cudaGetDevice(&dev);
    if (attr_dev != dev) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (e != cudaSuccess) return e;
        attr_dev = dev;
    }
    if (smem > 227 * 1024) return cudaErrorInvalidConfiguration;
    return launch_pdl(kern, grid, dim3(kThreads), smem, stream, a);
}

}  // namespace

// Host-side launcher.  Chooses the column groups per CTA so that the grid has
// at least about two CTAs per SM when the matrix allows it, the ring depth from
// the shared-memory budget, and the activation chunk from the row count.
void q4_gemv_stream_plan(Q4GemvArgs& a, int bf16, int sm_count, size_t* ws_floats, size_t* ncounters) {
    (void)bf16;
    a.sgrid = 0;
    *ws_floats = 0;
    *ncounters = 0;
    // tuning knob, read per call: 0 keeps every call on the column-group-per-CTA kernel, 2 streams small matrices too
    const char* knob = getenv("SMEG_Q4_STREAM");
    const int enabled = knob ? atoi(knob) : 1;
    if (!enabled || !a.a_vec_ok || a.m > 16 || a.k64 <= 0 || a.n16 <= 0 || sm_count <= 0) return;
    const int mt = a.m <= 8 ? 1 : 2;
    // two units per warp and stage when every CTA still gets a dozen stages or more
    const int upw = (long long)a.n16 * ((a.k64 + 2 * kSWarps - 1) / (2 * kSWarps)) >= 12ll * sm_count ? 2 : 1;
    // smaller matrices (under about 200 KB of codes per SM) stay on the column-group-per-CTA kernel: its two
    // CTAs per SM start and finish faster than one deep ring does (SMEG_Q4_STREAM=2 streams them too)
    if (upw == 1 && enabled != 2) return;
    const int su = kSWarps * upw;
    const int block = 1 << a.log2_block, stage_depth = 64 * su;
    a.supw = upw;
    a.srps = block < stage_depth ? stage_depth / block : 1;
    a.sslot = (su * kUnitBytes + a.srps * 32 + 127) / 128 * 128;
    const size_t a_bytes = (size_t)a.m * ((size_t)a.k64 * 64 + 8) * 2;
    const size_t red_bytes = (size_t)2 * kSWarps * 4 * mt * 32 * sizeof(float);
    const size_t budget = 227 * 1024;
    if (1024 + a_bytes + red_bytes + (size_t)4 * a.sslot > budget) return;     // the ring needs at least 4 slots (64 KB in flight)
    a.sns = (int)std::min<size_t>((budget - 1024 - a_bytes - red_bytes) / a.sslot, 48);
    a.spc = (a.k64 + su - 1) / su;
    const long long total = (long long)a.n16 * a.spc;
    if (total > 0x3fffffff) return;
    a.stotal = (int)total;
    const int grid = (int)std::min<long long>(sm_count, total);
    const int minlen = a.stotal / grid;                                         // shortest range, >= 1
    a.spieces = (a.spc + minlen - 1) / minlen + 1;
    a.a_rows = a.m;
    a.sgrid = grid;
    *ws_floats = (size_t)a.n16 * a.spieces * 128 * mt;
    *ncounters = (size_t)a.n16;
}

template <int BF16, int OPSIDE, int MT, int UPW>
static cudaError_t launch_stream_u(const Q4GemvArgs& a, cudaStream_t stream) {
    auto kern = q4_gemv_stream_kernel<BF16, OPSIDE, MT, UPW>;
    static int attr_dev = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (attr_dev != dev) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (e != cudaSuccess) return e;
        attr_dev = dev;
    }
    const size_t smem = 1024 + (size_t)a.sns * a.sslot + (size_t)a.a_rows * ((size_t)a.k64 * 64 + 8) * 2 +
                        (size_t)2 * kSWarps * 4 * MT * 32 * sizeof(float);
    if (smem > 227 * 1024) return cudaErrorInvalidConfiguration;
    return launch_pdl(kern, dim3(a.sgrid), dim3(kSThreads), smem, stream, a);
}

template <int BF16, int OPSIDE, int MT>
static cudaError_t launch_stream(const Q4GemvArgs& a, cudaStream_t stream) {
    return a.supw == 2 ? launch_stream_u<BF16, OPSIDE, MT, 2>(a, stream) : launch_stream_u<BF16, OPSIDE, MT, 1>(a, stream);
}

cudaError_t q4_gemv_launch(Q4GemvArgs a, int bf16, int sm_count, cudaStream_t stream) {
    const int opside = bf16 || a.log2_block < 5;
    if (a.sgrid > 0) {
        if (!a.ws || !a.counters) return cudaErrorInvalidValue;
        const int smt = a.m <= 8 ? 1 : 2;
        if (!bf16 && !opside) return smt == 1 ? launch_stream<0, 0, 1>(a, stream) : launch_stream<0, 0, 2>(a, stream);
        if (!bf16) return smt == 1 ? launch_stream<0, 1, 1>(a, stream) : launch_stream<0, 1, 2>(a, stream);
        return smt == 1 ? launch_stream<1, 1, 1>(a, stream) : launch_stream<1, 1, 2>(a, stream);
    }
    const int mt = a.m <= 8 ? 1 : (a.m <= 16 ? 2 : 4);
    int cg = 4;
    while (cg > 1 && (a.n16 + cg - 1) / cg < 2 * sm_count) cg >>= 1;
    a.cg = cg;
    const int block = 1 << a.log2_block;
    // scale rows staged per stage: a stage starts on a block boundary when the
    // block is shorter than it, and lies inside one block otherwise
    a.rps = block < kStageDepth ? kStageDepth / block : 1;
    const int stage_bytes = cg * (kUnitBytes * kConsumerWarps + a.rps * 32);
    int ns = (48 * 1024) / stage_bytes;
    if (ns > 8) ns = 8;
    if (ns < 2) ns = 2;
    a.ns = ns;
    // activation chunk: whole K when it fits 16 KB for the rows in play, else
    // double-buffered chunks of a whole number of stages
    const int kpad = a.k64 * 64;
    const int rows = 8 * mt;
    const int rows_used = a.m < rows ? a.m : rows;
    int ka = ((kpad + kStageDepth - 1) / kStageDepth) * kStageDepth;
    if (ka == 0) ka = kStageDepth;
    if ((size_t)rows_used * ka * 2 > 32 * 1024) {
        ka = (16 * 1024 / (rows_used * 2)) / kStageDepth * kStageDepth;
        if (ka < kStageDepth) ka = kStageDepth;
    }
    a.ka = ka;
    const int nbuf = kpad > ka ? 2 : 1;
    a.a_rows = rows_used;
    const size_t smem = 256 + (size_t)ns * stage_bytes + (size_t)nbuf * rows_used * (ka + 8) * 2 +
                        (size_t)kConsumerWarps * cg * mt * 128 * sizeof(float);
    dim3 grid((a.n16 + cg - 1) / cg, (a.m + 8 * mt - 1) / (8 * mt));
#define SMEG_Q4_LAUNCH(B, O, M) return launch<B, O, M>(a, grid, smem, stream)
    if (!bf16 && !opside) {
        if (mt == 1) SMEG_Q4_LAUNCH(0, 0, 1);
        if (mt == 2) SMEG_Q4_LAUNCH(0, 0, 2);
        SMEG_Q4_LAUNCH(0, 0, 4);
    } else if (!bf16) {
        if (mt == 1) SMEG_Q4_LAUNCH(0, 1, 1);
        if (mt == 2) SMEG_Q4_LAUNCH(0, 1, 2);
        SMEG_Q4_LAUNCH(0, 1, 4);
    } else {
        if (mt == 1) SMEG_Q4_LAUNCH(1, 1, 1);
        if (mt == 2) SMEG_Q4_LAUNCH(1, 1, 2);
        SMEG_Q4_LAUNCH(1, 1, 4);
    }
#undef SMEG_Q4_LAUNCH
}

}  // namespace smeg
