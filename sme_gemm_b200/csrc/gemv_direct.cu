// Decode GEMV for one to four activation rows, straight from global memory (sm_100a):
//   q4_direct_kernel      C[m][n] = ep( A[m][k] @ dequant(W) ), Q4 weights, f16, K-blocks of 32 and up
//   lowbit_direct_kernel  2-bit / 1-bit weights against int8-quantised activations (matmul_q2 / matmul_q1)
//
// They replace the reference's SME GEMV kernels for the batch sizes a decode step has
// (run_q4_gemv1 / run_q4_gemv, csrc/gemm_f16f16_q4.h:236-431; run_q2_gemv, csrc/gemm_q2.cc:300-404).
//
// A call of this size is a few microseconds long, so what it costs is the time to the first byte
// and the instructions issued per weight, not steady-state bandwidth.  Hence:
//   * no producer warp and no barrier: a packed unit (512 bytes, 16 columns) is one coalesced
//     16-byte asynchronous copy per lane into the lane's own slot of a shared-memory ring
//     (cp.async, a dozen units deep per warp: register loads cannot run that far ahead, a warp
//     has only a handful of scoreboards), and every warp issues its first ring-full as the first
//     thing the kernel does -- before the activations are staged and before the kernel ahead in
//     the stream has finished (the weights do not depend on it).  A lane reads back only what it
//     copied itself, so cp.async.wait_group is all the synchronisation the ring needs;
//   * one CTA owns whole column groups over the whole depth, its eight warps split the depth, so
//     a column's result never depends on the grid and nothing crosses CTAs;
//   * Q4: nibbles become exact f16 integers with one lop3 per pair, and are multiplied into
//     packed f16 sums over 8 depths (HFMA2, as the reference's SME kernel accumulates a K-block
//     in f16, csrc/gemm_f16f16_q4.h:236-341); every 32 depths the pair sums are widened and folded into
//     the f32 total with the block's scale.  Against the f32-accumulating oracle this differs by
//     f16 rounding of four-term partial sums, far inside the 1e-2 bar;
//   * 2-bit / 1-bit: the activation rows are quantised to int8 in shared memory by the CTA itself
//     (one or two rows; bit-exact quantize_row, src/kernels/lowbit/matmul.rs:354-371) or copied from
//     act_quant_kernel's output (three or four rows); codes are expanded in registers (2-bit: byte
//     permute of the 4-entry codebook, 1-bit: {0,1} bytes with sum = 2S - sum(q)), dot products
//     run on dp4a, exact int32 block sums meet in shared memory and one thread per output cell
//     folds them in K order with fmaf((float)sum, scale * sa, total) -- the reference's bits.
#include "epilogue.cuh"
#include "kernels.h"
#include "layout.h"

namespace smeg {
namespace {

constexpr int kDWarps = 8;
constexpr int kDThreads = 32 * kDWarps;

// Per-lane asynchronous copies global -> shared; a lane waits for its own groups only.
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async4(void* smem_dst, const void* gsrc) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// One packed Q4 word (8 nibbles, offset binary) -> the exact integer codes as f16 pairs:
// r[0] = column g (d, d+1), r[1] = column g+8 (d, d+1), r[2] = column g (d+2, d+3), r[3] = column g+8 (d+2, d+3).
__device__ __forceinline__ void q4_codes_h2(uint32_t w, __half2 (&r)[4]) {
    const uint32_t w8 = w >> 8;
    uint32_t lo0 = lop3_and_or(w, 0x000f000fu, 0x64006400u), hi0 = lop3_and_or(w, 0x00f000f0u, 0x64006400u);
    uint32_t lo1 = lop3_and_or(w8, 0x000f000fu, 0x64006400u), hi1 = lop3_and_or(w8, 0x00f000f0u, 0x64006400u);
    const __half2 off = __halves2half2(__ushort_as_half(0x6408), __ushort_as_half(0x6408));      // 1032
    const __half2 sc16 = __halves2half2(__ushort_as_half(0x2c00), __ushort_as_half(0x2c00));     // 1/16
    const __half2 off16 = __halves2half2(__ushort_as_half(0xd480), __ushort_as_half(0xd480));    // -72
    r[0] = __hsub2(*reinterpret_cast<__half2*>(&lo0), off);
    r[1] = __hsub2(*reinterpret_cast<__half2*>(&lo1), off);
    r[2] = __hfma2(*reinterpret_cast<__half2*>(&hi0), sc16, off16);
    r[3] = __hfma2(*reinterpret_cast<__half2*>(&hi1), sc16, off16);
}

__device__ __forceinline__ __half2 as_h2(uint32_t v) { return *reinterpret_cast<__half2*>(&v); }

// ---------------------------------------------------------------------------------------------
// Q4, f16, M rows (1..4), K-blocks >= 32.
// Shared memory: ring [8 warps][PF][32 lanes] of {16 B codes} then {2 x 4 B scales} | A rows
// [M][kpad + 8] f16 | the cross-warp exchange [8 warps][CPC][M][16] f32.
// ---------------------------------------------------------------------------------------------
constexpr int kQ4PF = 8;                                           // units in flight per warp
constexpr size_t kQ4RingBytes = (size_t)kDWarps * kQ4PF * 32 * (16 + 8);

template <int M>
__global__ void __launch_bounds__(kDThreads, M <= 2 ? 3 : 2) q4_direct_kernel(const __grid_constant__ Q4GemvArgs p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    constexpr int PF = kQ4PF;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int kpad = p.k64 * 64, a_stride = kpad + 8;
    uint4* ring_w = reinterpret_cast<uint4*>(smem_raw) + (size_t)warp * PF * 32 + lane;                     // + slot * 32
    uint32_t* ring_s = reinterpret_cast<uint32_t*>(smem_raw + (size_t)kDWarps * PF * 512) + (size_t)warp * PF * 64 + lane;   // + slot * 64 (+ 32)
    uint16_t* As = reinterpret_cast<uint16_t*>(smem_raw + kQ4RingBytes);
    float* red = reinterpret_cast<float*>(smem_raw + kQ4RingBytes + (size_t)M * a_stride * 2);
    const int CPC = p.cg;                                          // most column groups a CTA takes
    // this CTA's column groups: an equal share of all of them
    // (gated form: the share is counted in pairs of a gate group 4q + e and its up group 4q + 2 + e, e = 0, 1 -- the
    // matrix interleaves 32 gate and 32 up columns -- and the CTA walks gate, up, gate, up, ...)
    const int first = (int)blockIdx.x * p.dq + min((int)blockIdx.x, p.dr);
    const int share = p.dq + ((int)blockIdx.x < p.dr ? 1 : 0);
    const int ncg = p.glu ? 2 * share : share;
    auto group_of = [&](int c) -> int {
        if (!p.glu) return first + c;
        const int u = first + (c >> 1);
        return 4 * (u >> 1) + (u & 1) + 2 * (c & 1);
    };
    const int upw = p.dupw;                                        // units per warp: a contiguous run of the depth
    const int u_begin = min(warp * upw, p.k64), u_end = min(u_begin + upw, p.k64);
    const int total = ncg * (u_end - u_begin);                     // units this warp walks, column group by column group

    // load cursor: the unit's codes and the scale words of its two 32-deep halves (columns g, g + 8)
    const unsigned char* lp = p.codes + q4_unit_offset((size_t)group_of(0), (size_t)u_begin, p.k64) + lane * 16;
    const uint16_t* ls = p.scales + q4_scale_row((size_t)group_of(0), 0, p.nb) + 2 * g;
    int lu = u_begin, lc = 0;
    auto issue = [&](int slot) {
        cp_async16(ring_w + slot * 32, lp);
        cp_async4(ring_s + slot * 64, ls + (size_t)((lu * 64) >> p.log2_block) * 16);
        cp_async4(ring_s + slot * 64 + 32, ls + (size_t)((lu * 64 + 32) >> p.log2_block) * 16);
        lp += kUnitBytes;
        if (++lu == u_end) {
            lu = u_begin;
            const int cgn = group_of(++lc);                        // (one past the last group is never loaded from)
            lp = p.codes + q4_unit_offset((size_t)cgn, (size_t)u_begin, p.k64) + lane * 16;
            ls = p.scales + q4_scale_row((size_t)cgn, 0, p.nb) + 2 * g;
        }
    };
#pragma unroll
    for (int i = 0; i < PF; ++i) {
        if (i < total) issue(i);
        cp_async_commit();
    }
    pdl_launch_dependents();
    pdl_wait();                                                    // the activations may come from the kernel ahead

    // ---- stage the activation rows (zero past k) ----
#pragma unroll
    for (int r = 0; r < M; ++r)
    for (int d = tid * 8; d < kpad; d += kDThreads * 8) {
        uint4 v = make_uint4(0, 0, 0, 0);
        if (d + 8 <= p.k) v = *reinterpret_cast<const uint4*>(p.a + (size_t)r * p.k + d);
        else if (d < p.k) {
            __align__(16) uint16_t tmp[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) tmp[e] = d + e < p.k ? p.a[(size_t)r * p.k + d + e] : (uint16_t)0;
            v = *reinterpret_cast<uint4*>(tmp);
        }
        *reinterpret_cast<uint4*>(As + (size_t)r * a_stride + d) = v;
    }
    __syncthreads();

    float tot[M][2];
#pragma unroll
    for (int r = 0; r < M; ++r) tot[r][0] = tot[r][1] = 0.0f;
    int cc = 0, cu = u_begin, slot = 0;                            // compute cursor
    const uint16_t* ap = As + cu * 64 + 8 * t;
    for (int j = 0; j < total; ++j) {
        cp_async_wait<PF - 1>();                                   // this lane's copies of unit j have landed
        const uint4 wv = ring_w[slot * 32];
        const uint32_t sw[2] = {ring_s[slot * 64], ring_s[slot * 64 + 32]};
        const uint32_t words[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            __half2 c0[4], c1[4];
            q4_codes_h2(words[2 * h], c0);
            q4_codes_h2(words[2 * h + 1], c1);
#pragma unroll
            for (int r = 0; r < M; ++r) {
                const uint4 av = *reinterpret_cast<const uint4*>(ap + (size_t)r * a_stride + 32 * h);
                __half2 s0 = __hmul2(c0[0], as_h2(av.x)), s1 = __hmul2(c0[1], as_h2(av.x));
                s0 = __hfma2(c0[2], as_h2(av.y), s0);
                s1 = __hfma2(c0[3], as_h2(av.y), s1);
                s0 = __hfma2(c1[0], as_h2(av.z), s0);
                s1 = __hfma2(c1[1], as_h2(av.z), s1);
                s0 = __hfma2(c1[2], as_h2(av.w), s0);
                s1 = __hfma2(c1[3], as_h2(av.w), s1);
                // (column g, column g + 8): the pair sums of 8 depths, times the block's scales, widened once
                const __half2 sum = __hadd2(__lows2half2(s0, s1), __highs2half2(s0, s1));
                const float2 f = __half22float2(__hmul2(sum, as_h2(sw[h])));
                tot[r][0] += f.x;
                tot[r][1] += f.y;
            }
        }
        if (j + PF < total) issue(slot);
        cp_async_commit();
        slot = slot + 1 == PF ? 0 : slot + 1;
        ap += 64;
        if (++cu == u_end) {
            // end of this warp's share of a column group: the four lanes of a column hold different depths
#pragma unroll
            for (int r = 0; r < M; ++r)
#pragma unroll
                for (int jj = 0; jj < 2; ++jj) {
                    float v = tot[r][jj];
                    v += __shfl_xor_sync(0xffffffffu, v, 1);
                    v += __shfl_xor_sync(0xffffffffu, v, 2);
                    if (t == 0) red[(((size_t)warp * CPC + cc) * M + r) * 16 + g + 8 * jj] = v;
                    tot[r][jj] = 0.0f;
                }
            cu = u_begin;
            ap = As + cu * 64 + 8 * t;
            ++cc;
        }
    }
    cp_async_wait<0>();
    if (total == 0) {
        // a warp with no depth of its own contributes zeros
        for (int o = lane; o < ncg * M * 16; o += 32) red[(size_t)warp * CPC * M * 16 + o] = 0.0f;
    }
    __syncthreads();
    // ---- the warps' shares in warp order, epilogue, store ----
    if (p.glu) {
        // a hidden unit's gate and up sums lie in neighbouring local groups: out = f16(act(f16(gate)) * f16(up)), the
        // arithmetic of the separate gate pass (glu, src/linear.rs:804-835) on the rounded projections
        const int hn = p.n >> 1;
        for (int o = tid; o < share * M * 16; o += kDThreads) {
            const int col16 = o & 15, r = (o >> 4) % M, ul = o / (16 * M);
            float ag = 0.0f, au = 0.0f;
#pragma unroll
            for (int w = 0; w < kDWarps; ++w) {
                ag += red[(((size_t)w * CPC + 2 * ul) * M + r) * 16 + col16];
                au += red[(((size_t)w * CPC + 2 * ul + 1) * M + r) * 16 + col16];
            }
            const float gv = __half2float(__float2half_rn(ag)), uv = __half2float(__float2half_rn(au));
            const int hcol = (first + ul) * 16 + col16;
            if (hcol < hn) p.c[(size_t)r * hn + hcol] = __half_as_ushort(__float2half_rn(__fmul_rn(glu_gate((uint32_t)p.glu, gv), uv)));
        }
        return;
    }
    for (int o = tid; o < ncg * M * 16; o += kDThreads) {
        const int col16 = o & 15, r = (o >> 4) % M, c = o / (16 * M);
        float acc = 0.0f;
#pragma unroll
        for (int w = 0; w < kDWarps; ++w) acc += red[(((size_t)w * CPC + c) * M + r) * 16 + col16];
        const int col = (first + c) * 16 + col16;
        if (col < p.n) {
            if (p.c32) p.c32[(size_t)r * p.n + col] = acc;
            else if (p.yacc) p.yacc[(size_t)r * p.n + col] = __fadd_rn(p.yacc[(size_t)r * p.n + col], __half2float(__float2half_rn(acc)));
            else p.c[(size_t)r * p.n + col] = ep_store_value<0>(p.ep, acc, (size_t)r, (size_t)col);
        }
    }
}

// ---------------------------------------------------------------------------------------------
// 2-bit / 1-bit weights x int8 activations, M rows (1..4).
// Shared memory: ring [8 warps][PF][32 lanes] of 16 B codes | Qs [M][kq + 16] int8 | SAs [M][nb] f32 |
//                QSs [M][nb] i32 | AMX [M][nb] i32 | sums [2][nb][M][16] i32 | staged scale rows.
// ---------------------------------------------------------------------------------------------
constexpr int kLbPF = 8;                                           // units in flight per warp
constexpr size_t kLbRingBytes = (size_t)kDWarps * kLbPF * 512;

__device__ __forceinline__ uint32_t prmt_lut(uint32_t lut, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(lut), "r"(0u), "r"(sel));
    return d;
}

template <int BITS, int M, int BIGBLK>
__global__ void __launch_bounds__(kDThreads, 3) lowbit_direct_kernel(const __grid_constant__ LowbitGemvArgs p) {
    constexpr int UD = BITS == 2 ? kQ2UnitDepth : kQ1UnitDepth;
    constexpr int STEPS = UD / 32;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int kq = p.kq, q_stride = kq + 16, nb = p.nb;
    const int CPC = p.gpt;
    uint4* ring_w = reinterpret_cast<uint4*>(smem_raw) + (size_t)warp * kLbPF * 32 + lane;                  // + slot * 32
    int8_t* Qs = reinterpret_cast<int8_t*>(smem_raw + kLbRingBytes);
    float* SAs = reinterpret_cast<float*>(smem_raw + kLbRingBytes + (size_t)M * q_stride);
    int* QSs = reinterpret_cast<int*>(SAs + (size_t)M * nb);
    int* AMX = QSs + (size_t)M * nb;
    int* sums = AMX + (size_t)M * nb;
    // [ncg][nb][16] when p.dsc; 16-byte aligned for the asynchronous copies
    uint16_t* SCs = reinterpret_cast<uint16_t*>((reinterpret_cast<uintptr_t>(sums + (size_t)2 * nb * M * 16) + 15) & ~(uintptr_t)15);
    const int cg_first = (int)blockIdx.x * p.dq + min((int)blockIdx.x, p.dr);
    const int ncg = p.dq + ((int)blockIdx.x < p.dr ? 1 : 0);
    const int upw = p.dupw;
    const int u_begin = min(warp * upw, p.ku), u_end = min(u_begin + upw, p.ku);
    const int total = ncg * (u_end - u_begin);                     // units this warp walks, column group by column group
    const int block = 1 << p.log2_block;

    constexpr int PF = kLbPF;
    const unsigned char* lp = p.codes + ((size_t)cg_first * p.ku + (size_t)u_begin) * kUnitBytes + lane * 16;   // load cursor
    int lu = u_begin;
    auto issue = [&](int slot) {
        cp_async16(ring_w + slot * 32, lp);
        lp += kUnitBytes;
        if (++lu == u_end) {
            lu = u_begin;
            lp += (size_t)(p.ku - (u_end - u_begin)) * kUnitBytes;
        }
    };
    // the CTA's scale rows ride along with the first units
    if (p.dsc) {
        const uint16_t* src = p.scales + (size_t)cg_first * nb * 16;
        for (int ch = tid; ch < ncg * nb * 2; ch += kDThreads) cp_async16(SCs + ch * 8, src + (size_t)ch * 8);
    }
#pragma unroll
    for (int i = 0; i < PF; ++i) {
        if (i < total) issue(i);
        cp_async_commit();
    }
    pdl_launch_dependents();
    for (int idx = tid; idx < 2 * nb * M * 16; idx += kDThreads) sums[idx] = 0;
    for (int idx = tid; idx < M * nb; idx += kDThreads) { AMX[idx] = 0; QSs[idx] = 0; SAs[idx] = 0.0f; }
    pdl_wait();

    if (p.a != nullptr) {
        // ---- quantize_row (src/kernels/lowbit/matmul.rs:354-371) over the rows, in shared memory ----
        // An item is eight consecutive depths of one row; a thread keeps its items in registers between the
        // two passes (block maxima, then codes), QI items at a time.
        __syncthreads();
        const int nvec = kq / 8;                                   // items per row
        constexpr int QI = 4;
        // eight consecutive depths of one row as f16 bits (zero past k)
        auto load8 = [&](int r, int d) -> uint4 {
            if (p.a_vec_ok && d + 8 <= p.k) return *reinterpret_cast<const uint4*>(p.a + (size_t)r * p.k + d);
            __align__(16) uint16_t h[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) h[e] = d + e < p.k ? p.a[(size_t)r * p.k + d + e] : (uint16_t)0;
            return *reinterpret_cast<uint4*>(h);
        };
        // rows longer than QI * 256 items go in several rounds; a K-block must then lie inside one round
        // (the host only takes this path when it does)
        for (int v0 = 0; v0 < nvec; v0 += QI * kDThreads) {
#pragma unroll
            for (int r = 0; r < M; ++r) {
                uint4 hv[QI];
#pragma unroll
                for (int i = 0; i < QI; ++i) {
                    const int d = (v0 + tid + i * kDThreads) * 8;
                    hv[i] = make_uint4(0, 0, 0, 0);
                    if (d < p.k) hv[i] = load8(r, d);
                }
#pragma unroll
                for (int i = 0; i < QI; ++i) {
                    const int d = (v0 + tid + i * kDThreads) * 8;
                    const uint32_t hw[4] = {hv[i].x, hv[i].y, hv[i].z, hv[i].w};
                    int mx = 0;
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        // |x| as integer bits: ordered like the values, and every NaN is above infinity (padding is 0)
                        const float2 f = __half22float2(as_h2(hw[e] & 0x7fff7fffu));
                        mx = max(mx, max(__float_as_int(f.x), __float_as_int(f.y)));
                    }
                    if (block >= 256) {
                        // a warp's 32 items are 256 consecutive depths: one K-block
                        mx = __reduce_max_sync(0xffffffffu, mx);
                        if (lane == 0 && mx != 0) atomicMax(&AMX[r * nb + (d >> p.log2_block)], mx);
                    } else if (d < p.k) {
                        atomicMax(&AMX[r * nb + (d >> p.log2_block)], mx);
                    }
                }
                __syncthreads();
#pragma unroll
                for (int i = 0; i < QI; ++i) {
                    const int d = (v0 + tid + i * kDThreads) * 8;
                    if (d >= kq) continue;
                    uint32_t lo = 0, hi = 0;
                    if (d < p.k) {
                        const int bl = d >> p.log2_block;
                        const int bits = AMX[r * nb + bl];
                        const float amax = bits > 0x7f800000 ? __int_as_float(0x7fc00000) : __int_as_float(bits);
                        const float inv = amax > 0.0f ? __fdiv_rn(127.0f, amax) : 0.0f;
                        if ((d & (block - 1)) == 0) {
                            const float sa = __fdiv_rn(amax, 127.0f);
                            SAs[r * nb + bl] = sa;
                            if (p.sa_out && blockIdx.x == 0) p.sa_out[(size_t)r * p.nb_real + bl] = sa;
                        }
                        const uint32_t hw[4] = {hv[i].x, hv[i].y, hv[i].z, hv[i].w};
                        int q[8];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const float2 f = __half22float2(as_h2(hw[e]));
                            // round to nearest even, NaN -> 0, then saturate: round_ties_even(x) as i8 (padding is 0)
                            q[2 * e] = max(-128, min(127, __float2int_rn(__fmul_rn(f.x, inv))));
                            q[2 * e + 1] = max(-128, min(127, __float2int_rn(__fmul_rn(f.y, inv))));
                        }
                        lo = __byte_perm(__byte_perm(q[0], q[1], 0x0040), __byte_perm(q[2], q[3], 0x0040), 0x5410);
                        hi = __byte_perm(__byte_perm(q[4], q[5], 0x0040), __byte_perm(q[6], q[7], 0x0040), 0x5410);
                        if (BITS == 1) {
                            const int sq = __dp4a((int)lo, 0x01010101, __dp4a((int)hi, 0x01010101, 0));
                            if (sq != 0) atomicAdd(&QSs[r * nb + bl], sq);
                        }
                        if (p.q_out && blockIdx.x == 0) {
#pragma unroll
                            for (int e = 0; e < 8; ++e)
                                if (d + e < p.k) p.q_out[(size_t)r * p.k + d + e] = (int8_t)q[e];
                        }
                    }
                    *reinterpret_cast<uint2*>(Qs + (size_t)r * q_stride + d) = make_uint2(lo, hi);
                }
            }
        }
    } else {
#pragma unroll
        for (int r = 0; r < M; ++r)
            for (int v = tid; v < kq / 16; v += kDThreads)
                *reinterpret_cast<uint4*>(Qs + (size_t)r * q_stride + v * 16) = *reinterpret_cast<const uint4*>(p.q + (size_t)r * kq + v * 16);
        for (int idx = tid; idx < M * nb; idx += kDThreads) {
            SAs[idx] = p.sa[idx];
            QSs[idx] = p.qsum ? p.qsum[idx] : 0;
        }
    }
    __syncthreads();

    // ---- block sums ----
    int acc[M][2];
#pragma unroll
    for (int r = 0; r < M; ++r) acc[r][0] = acc[r][1] = 0;
    int cu = u_begin;                                              // compute cursor
    int* sb = sums;                                                // the column group's block sums
    // flush: the lanes of a column holding the same block add into one cell
    auto flush = [&](int bl) {
#pragma unroll
        for (int r = 0; r < M; ++r)
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                int v = acc[r][j];
                acc[r][j] = 0;
                if (block >= 32) {
                    v += __shfl_xor_sync(0xffffffffu, v, 1);
                    v += __shfl_xor_sync(0xffffffffu, v, 2);
                    if (t == 0 && v != 0) atomicAdd(&sb[((size_t)bl * M + r) * 16 + g + 8 * j], v);
                } else if (v != 0) {
                    atomicAdd(&sb[((size_t)bl * M + r) * 16 + g + 8 * j], v);
                }
            }
    };
    // One column group at a time: its block sums meet in one of two buffers; when every warp has added its share the
    // cells' owners fold them (and clear the buffer) while the other warps go on with the next column group.
    int slot = 0, j = 0;
    for (int c = 0; c < ncg; ++c) {
        sb = sums + (size_t)(c & 1) * nb * M * 16;
        for (cu = u_begin; cu < u_end; ++cu, ++j) {
            cp_async_wait<PF - 1>();                               // this lane's copy of unit j has landed
            const uint4 wv = ring_w[slot * 32];
            const uint32_t words[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
            for (int s = 0; s < STEPS; ++s) {
                const int d = cu * UD + 32 * s + 8 * t;            // this lane's 8 depths
                const uint32_t w = words[BITS == 2 ? s : (s >> 1)];
                uint32_t af[4];
                if (BITS == 2) {
                    const uint32_t e = w & 0x33333333u, o = (w >> 2) & 0x33333333u;
                    af[0] = prmt_lut(p.lut, e);
                    af[1] = prmt_lut(p.lut, o);
                    af[2] = prmt_lut(p.lut, e >> 16);
                    af[3] = prmt_lut(p.lut, o >> 16);
                } else {
                    const int sh = 4 * (s & 1);
                    af[0] = (w >> (sh + 0)) & 0x01010101u;
                    af[1] = (w >> (sh + 1)) & 0x01010101u;
                    af[2] = (w >> (sh + 2)) & 0x01010101u;
                    af[3] = (w >> (sh + 3)) & 0x01010101u;
                }
#pragma unroll
                for (int r = 0; r < M; ++r) {
                    const uint2 aq = *reinterpret_cast<const uint2*>(Qs + (size_t)r * q_stride + d);
                    acc[r][0] = __dp4a((int)af[0], (int)aq.x, acc[r][0]);
                    acc[r][0] = __dp4a((int)af[2], (int)aq.y, acc[r][0]);
                    acc[r][1] = __dp4a((int)af[1], (int)aq.x, acc[r][1]);
                    acc[r][1] = __dp4a((int)af[3], (int)aq.y, acc[r][1]);
                }
                // end of a K-block for this lane's depths (blocks of 16: lanes t < 2 and t >= 2 differ),
                // or of this warp's share of the column group
                if (!BIGBLK && (((d + 32) >> p.log2_block) != (d >> p.log2_block) || (s == STEPS - 1 && cu == u_end - 1))) flush(d >> p.log2_block);
            }
            // blocks of a whole unit or more: one test per unit
            if (BIGBLK && ((((cu + 1) * UD) & (block - 1)) == 0 || cu == u_end - 1)) flush((cu * UD) >> p.log2_block);
            if (j + PF < total) issue(slot);
            cp_async_commit();
            slot = slot + 1 == PF ? 0 : slot + 1;
        }
        if (c == 0) cp_async_wait<0>();                            // the staged scale rows (first group of copies) as well
        __syncthreads();
        // ---- ordered fold of the column group's cells, epilogue, store ----
        if (tid < M * 16) {
            const int col16 = tid & 15, r = tid >> 4;
            const int col = (cg_first + c) * 16 + col16;
            const uint16_t* sc = (p.dsc ? SCs + (size_t)c * nb * 16 : p.scales + ((size_t)(cg_first + c) * nb) * 16) + scale_slot(col16);
            int* cell = sb + (size_t)r * 16 + col16;
            float tot = 0.0f;
#pragma unroll 4
            for (int bl = 0; bl < p.nb_real; ++bl) {
                int sum = cell[(size_t)bl * M * 16];
                cell[(size_t)bl * M * 16] = 0;
                if (BITS == 1) sum = 2 * sum - QSs[r * nb + bl];
                if (p.sums_out && col < p.n) p.sums_out[((size_t)r * p.n + col) * p.nb_real + bl] = sum;
                const float scale = __half2float(__ushort_as_half(sc[(size_t)bl * 16]));
                tot = fmaf((float)sum, __fmul_rn(scale, SAs[r * nb + bl]), tot);
            }
            if (col < p.n) p.c[(size_t)r * p.n + col] = ep_store_value<0>(p.ep, tot, (size_t)r, (size_t)col);
        }
    }
    cp_async_wait<0>();
}

template <typename K>
cudaError_t opt_in_smem(K kern, size_t smem) {
    if (smem <= 48 * 1024) return cudaSuccess;
    return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
}

// Grid of the one-wave kernels: per_sm CTAs per SM when there are that many column groups, more when a
// CTA would otherwise take more than max_groups of them; *cpc = most column groups of one CTA.
int direct_grid(int n16, int sm_count, int max_groups, int* cpc, int per_sm) {
    int grid = n16 < per_sm * sm_count ? n16 : per_sm * sm_count;
    if ((n16 + grid - 1) / grid > max_groups) grid = (n16 + max_groups - 1) / max_groups;
    if (grid < 1) grid = 1;
    *cpc = (n16 + grid - 1) / grid;
    return grid;
}

}  // namespace

// ---- Q4 ----
bool q4_direct_supported(const Q4GemvArgs& a, int bf16) {
    if (bf16 || a.m < 1 || a.m > 4 || a.log2_block < 5 || a.k64 < 1) return false;
    if (a.k % 8 != 0 || !a.a_vec_ok) return false;                // 128-bit activation loads
    const size_t smem = kQ4RingBytes + (size_t)a.m * ((size_t)a.k64 * 64 + 8) * 2;
    return smem <= 100 * 1024;
}

cudaError_t q4_direct_launch(Q4GemvArgs a, int sm_count, cudaStream_t stream) {
    const int n16 = (a.n + 15) / 16;
    a.n16 = n16;
    // three CTAs per SM when the matrix gives every SM that many, else two (and then never three on one SM
    // while another has one: the shared-memory request is padded past a third of an SM's)
    const int per_sm = (a.m <= 2 && n16 > 2 * sm_count) ? 3 : 2;
    int grid_x;
    if (a.glu) {
        // shares are (gate group, up group) pairs: n16 / 2 of them, at most 8 (16 groups) per CTA
        const int pairs = n16 / 2;
        int cpp = 1;
        grid_x = direct_grid(pairs, sm_count, 8, &cpp, per_sm);
        a.cg = 2 * cpp;
        a.dq = pairs / grid_x; a.dr = pairs % grid_x;
    } else {
        grid_x = direct_grid(n16, sm_count, 16, &a.cg, per_sm);
        a.dq = n16 / grid_x; a.dr = n16 % grid_x;
    }
    a.dupw = (a.k64 + kDWarps - 1) / kDWarps;
    size_t smem = kQ4RingBytes + (size_t)a.m * ((size_t)a.k64 * 64 + 8) * 2 + (size_t)kDWarps * a.cg * a.m * 16 * sizeof(float);
    if (per_sm == 2 && smem < 80 * 1024) smem = 80 * 1024;
    const dim3 grid(grid_x);
    cudaError_t e;
#define SMEG_QD(MM)                                                                   \
    case MM:                                                                          \
        e = opt_in_smem(q4_direct_kernel<MM>, smem);                                  \
        if (e != cudaSuccess) return e;                                               \
        return launch_pdl(q4_direct_kernel<MM>, grid, dim3(kDThreads), smem, stream, a);
    switch (a.m) {
        SMEG_QD(1) SMEG_QD(2) SMEG_QD(3) SMEG_QD(4)
    default: return cudaErrorInvalidValue;
    }
#undef SMEG_QD
}

// ---- 2-bit / 1-bit ----
static bool lowbit_scales_staged(const LowbitGemvArgs& a, int cpc) { return (size_t)cpc * a.nb * 32 <= 16 * 1024; }
static size_t lowbit_direct_smem(const LowbitGemvArgs& a, int cpc) {
    return kLbRingBytes + (size_t)a.m * (a.kq + 16) + (size_t)3 * a.m * a.nb * 4 + (size_t)2 * a.nb * a.m * 16 * 4 +
           (lowbit_scales_staged(a, cpc) ? (size_t)cpc * a.nb * 32 + 16 : 0);
}

bool lowbit_direct_supported(const LowbitGemvArgs& a, bool fused) {
    if (a.m < 1 || a.m > 4 || a.ku < 1 || a.k < 1) return false;
    if (fused && a.m > 2) return false;                          // every CTA repeats the quantisation
    // in-kernel quantisation walks a row in rounds of 8192 depths: a K-block must lie inside one round
    if (fused && a.kq > 8192 && ((1 << a.log2_block) > 8192 || 8192 % (1 << a.log2_block) != 0)) return false;
    return lowbit_direct_smem(a, 1) <= 110 * 1024;
}

cudaError_t lowbit_direct_launch(LowbitGemvArgs a, int bits, int sm_count, cudaStream_t stream) {
    int cpc = 1, maxg = 16;
    int grid_x = direct_grid(a.n16, sm_count, maxg, &cpc, 3);
    while (maxg > 1 && lowbit_direct_smem(a, cpc) > 110 * 1024) grid_x = direct_grid(a.n16, sm_count, --maxg, &cpc, 3);
    a.gpt = cpc;
    a.dq = a.n16 / grid_x; a.dr = a.n16 % grid_x; a.dupw = (a.ku + kDWarps - 1) / kDWarps;
    a.dsc = lowbit_scales_staged(a, cpc) ? 1 : 0;
    const size_t smem = lowbit_direct_smem(a, cpc);
    const dim3 grid(grid_x);
    cudaError_t e;
    const int ud = bits == 2 ? kQ2UnitDepth : kQ1UnitDepth;
    const bool big = (1 << a.log2_block) >= ud;
#define SMEG_LD(BB, MM)                                                                   \
    if (bits == BB && a.m == MM) {                                                        \
        if (big) {                                                                        \
            e = opt_in_smem(lowbit_direct_kernel<BB, MM, 1>, smem);                       \
            if (e != cudaSuccess) return e;                                               \
            return launch_pdl(lowbit_direct_kernel<BB, MM, 1>, grid, dim3(kDThreads), smem, stream, a); \
        }                                                                                 \
        e = opt_in_smem(lowbit_direct_kernel<BB, MM, 0>, smem);                           \
        if (e != cudaSuccess) return e;                                                   \
        return launch_pdl(lowbit_direct_kernel<BB, MM, 0>, grid, dim3(kDThreads), smem, stream, a); \
    }
    SMEG_LD(2, 1) SMEG_LD(2, 2) SMEG_LD(2, 3) SMEG_LD(2, 4)
    SMEG_LD(1, 1) SMEG_LD(1, 2) SMEG_LD(1, 3) SMEG_LD(1, 4)
#undef SMEG_LD
    return cudaErrorInvalidValue;
}

}  // namespace smeg
