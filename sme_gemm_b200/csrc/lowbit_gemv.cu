// 2-bit / 1-bit weights x int8-quantised activations (matmul_q2 / matmul_q1) for sm_100a.
//
// Replaces the reference's SME kernel (q2_quant / run_q2_gemv / Q2_FOLD,
// csrc/gemm_q2.cc:59-97,180-204,300-404) and reproduces the bits of its portable
// statement (quantize_row + reference, src/kernels/lowbit/matmul.rs:354-398):
//   * activations are quantised per (row, K-block) to int8 by act_quant_kernel,
//     bit-exactly (amax with sticky NaN, inv = 127/amax, ties-to-even, saturate);
//   * block sums are exact int32, computed on the int8 tensor cores
//     (mma.m16n8k32.s8: 16 weight columns x 32 depths against up to 8 rows) from
//     codes expanded in registers -- 2-bit through a byte-permute lookup of the
//     4-entry codebook, 1-bit as {0,1} bytes with the exact correction
//     sum = 2*S - sum(q);
//   * each output cell then folds its blocks in K order with
//     total = fmaf((float)sum, scale * sa, total), one thread per cell, so the
//     result does not depend on m, the grid or the split of K over warps;
//   * the epilogue graph runs on the f16-rounded product.
// Weights stream through shared memory with cp.async.bulk + mbarriers exactly
// as in the Q4 kernel.
#include "epilogue.cuh"
#include "kernels.h"
#include "layout.h"

namespace smeg {

namespace {

constexpr int kWarps = 8;
constexpr int kThreadsLb = 32 * (kWarps + 1);
constexpr int kMaxOutPerThread = 8;

__device__ __forceinline__ void mma_s8(int (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t prmt(uint32_t lut, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(lut), "r"(0u), "r"(sel));
    return d;
}

// ---------------------------------------------------------------------------
// Activation quantisation: one CTA per (K-block, row).
// quantize_row, src/kernels/lowbit/matmul.rs:354-371.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(128) act_quant_kernel(ActQuantArgs p) {
    __shared__ float s_max[4];
    __shared__ int s_nan[4];
    __shared__ int s_sum[4];
    const int b = blockIdx.x, row = blockIdx.y, tid = threadIdx.x;
    const size_t block = (size_t)1 << p.log2_block;
    const size_t d0 = (size_t)b * block;
    const size_t d1 = min(d0 + block, (size_t)p.kq);
    const uint16_t* ar = p.a + (size_t)row * p.k;
    int8_t* qr = p.q + (size_t)row * p.kq;

    float mx = 0.0f;
    int has_nan = 0;
    for (size_t d = d0 + tid; d < d1 && d < (size_t)p.k; d += 128) {
        const float x = fabsf(__half2float(__ushort_as_half(ar[d])));
        if (x != x) has_nan = 1;
        else mx = fmaxf(mx, x);
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) {
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        has_nan |= __shfl_xor_sync(0xffffffffu, has_nan, o);
    }
    if ((tid & 31) == 0) { s_max[tid >> 5] = mx; s_nan[tid >> 5] = has_nan; }
    __syncthreads();
    mx = fmaxf(fmaxf(s_max[0], s_max[1]), fmaxf(s_max[2], s_max[3]));
    has_nan = s_nan[0] | s_nan[1] | s_nan[2] | s_nan[3];
    const float amax = has_nan ? __int_as_float(0x7fc00000) : mx;
    const float inv = amax > 0.0f ? __fdiv_rn(127.0f, amax) : 0.0f;

    int local = 0;
    for (size_t d = d0 + tid; d < d1; d += 128) {
        int v = 0;
        if (d < (size_t)p.k) {
            const float r = rintf(__fmul_rn(__half2float(__ushort_as_half(ar[d])), inv));
            if (r != r) v = 0;
            else v = (int)fminf(fmaxf(r, -128.0f), 127.0f);
        }
        qr[d] = (int8_t)v;
        local += v;
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) local += __shfl_xor_sync(0xffffffffu, local, o);
    if ((tid & 31) == 0) s_sum[tid >> 5] = local;
    __syncthreads();
    if (tid == 0) {
        const bool real = d0 < (size_t)p.k;
        p.sa[(size_t)row * p.nbq + b] = real ? __fdiv_rn(amax, 127.0f) : 0.0f;
        if (p.qsum) p.qsum[(size_t)row * p.nbq + b] = s_sum[0] + s_sum[1] + s_sum[2] + s_sum[3];
    }
}

// ---------------------------------------------------------------------------
// The GEMV.  BITS = 2 or 1, MT = groups of 8 rows per CTA.
// ---------------------------------------------------------------------------
template <int BITS, int MT>
__global__ void __launch_bounds__(kThreadsLb) lowbit_gemv_kernel(LowbitGemvArgs p) {
    constexpr int UD = BITS == 2 ? kQ2UnitDepth : kQ1UnitDepth;   // depths per unit
    constexpr int STEPS = UD / 32;                                 // mma k-steps per unit
    constexpr int SD = UD * kWarps;                                // depths per stage
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int NS = p.ns, CG = p.cg, KC = p.kc;
    const int block = 1 << p.log2_block;
    const int bpc = KC >= block ? KC / block : 1;                  // sums rows held per chunk
    const int code_bytes = kUnitBytes * kWarps;
    const int stage_bytes = CG * code_bytes;
    const int rows = 8 * MT;

    uint64_t* full = reinterpret_cast<uint64_t*>(smem_raw);
    uint64_t* empty = full + NS;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(empty + NS);
    unsigned char* stages = smem_raw + 256;
    const int q_stride = KC + 32;                                  // bytes; keeps LDS.64 conflict-free
    int8_t* Qs = reinterpret_cast<int8_t*>(stages + (size_t)NS * stage_bytes);
    uint16_t* Ss = reinterpret_cast<uint16_t*>(Qs + (size_t)rows * q_stride);          // [CG][bpc][16] scales
    float* SAs = reinterpret_cast<float*>(Ss + (size_t)CG * bpc * 16);                 // [rows][bpc]
    int* QSs = reinterpret_cast<int*>(SAs + (size_t)rows * bpc);                       // [rows][bpc]
    int* sums = QSs + (size_t)rows * bpc;                                              // [bpc][CG][rows][16]

    const int cg0 = blockIdx.x * CG;
    const int ncg = min(CG, p.n16 - cg0);
    const int row0 = blockIdx.y * rows;
    const int num_chunks = (p.kq + KC - 1) / KC;
    const int stages_total = (p.ku + kWarps - 1) / kWarps;

    if (tid == 0) {
        for (int s = 0; s < NS; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], kWarps);
        }
        *abort_flag = 0;
        fence_barrier_init();
    }
    __syncthreads();

    if (warp == kWarps) {
        // ================= producer =================
        if (lane == 0) {
            int st = 0;
            for (int ch = 0; ch < num_chunks; ++ch) {
                const int d0 = ch * KC;
                const int st_end = min(stages_total, (d0 + KC) / SD);
                for (; st < st_end; ++st) {
                    const int slot = st % NS;
                    if (st >= NS) mbar_wait(&empty[slot], ((st / NS) - 1) & 1, abort_flag, p.status);
                    const int units = min(kWarps, p.ku - st * kWarps);
                    mbar_expect_tx(&full[slot], ncg * units * kUnitBytes);
                    unsigned char* sbase = stages + (size_t)slot * stage_bytes;
                    for (int c = 0; c < ncg; ++c)
                        bulk_g2s(sbase + c * code_bytes,
                                 p.codes + (((size_t)(cg0 + c) * p.ku + (size_t)st * kWarps) * kUnitBytes),
                                 units * kUnitBytes, &full[slot]);
                }
            }
        }
        return;
    }

    // ================= consumers =================
    float total[kMaxOutPerThread];
#pragma unroll
    for (int i = 0; i < kMaxOutPerThread; ++i) total[i] = 0.0f;
    const int n_out = CG * 16 * rows;            // output cells of this CTA
    int acc[4][MT][4];

    int st = 0;
    for (int ch = 0; ch < num_chunks; ++ch) {
        const int d0 = ch * KC;
        const int chunk = min(KC, p.kq - d0);
        const int blk0 = d0 >> p.log2_block;                     // first block (row of scales) of the chunk
        const bool block_starts = (d0 & (block - 1)) == 0;       // always true when block <= KC
        asm volatile("bar.sync 1, %0;" ::"n"(32 * kWarps));
        // ---- stage q, sa, qsum, scales; clear the sums ----
        {
            const int vec_per_row = chunk / 16;
            for (int idx = tid; idx < rows * vec_per_row; idx += 32 * kWarps) {
                const int r = idx / vec_per_row, v = idx % vec_per_row;
                uint4 val = make_uint4(0, 0, 0, 0);
                if (row0 + r < p.m) val = *reinterpret_cast<const uint4*>(p.q + (size_t)(row0 + r) * p.kq + d0 + v * 16);
                *reinterpret_cast<uint4*>(Qs + (size_t)r * q_stride + v * 16) = val;
            }
            const int nblk = min(bpc, p.nb - blk0);
            for (int idx = tid; idx < rows * bpc; idx += 32 * kWarps) {
                const int r = idx / bpc, bl = idx % bpc;
                const bool ok = row0 + r < p.m && bl < nblk;
                SAs[idx] = ok ? p.sa[(size_t)(row0 + r) * p.nb + blk0 + bl] : 0.0f;
                QSs[idx] = (ok && p.qsum) ? p.qsum[(size_t)(row0 + r) * p.nb + blk0 + bl] : 0;
            }
            for (int idx = tid; idx < CG * bpc * 16; idx += 32 * kWarps) {
                const int c = idx / (bpc * 16), rem = idx % (bpc * 16);
                const int bl = rem / 16, col = rem % 16;
                Ss[idx] = (c < ncg && bl < nblk) ? p.scales[((size_t)(cg0 + c) * p.nb + blk0 + bl) * 16 + col] : (uint16_t)0;
            }
            if (block_starts)
                for (int idx = tid; idx < bpc * n_out; idx += 32 * kWarps) sums[idx] = 0;
        }
        asm volatile("bar.sync 1, %0;" ::"n"(32 * kWarps));

        const int st_end = min(stages_total, (d0 + chunk + SD - 1) / SD);
        for (; st < st_end; ++st) {
            const int slot = st % NS;
            mbar_wait(&full[slot], (st / NS) & 1, abort_flag, p.status);
            const int units = min(kWarps, p.ku - st * kWarps);
            if (warp < units) {
                const unsigned char* sbase = stages + (size_t)slot * stage_bytes;
                const int d_unit = st * SD + warp * UD;             // global depth of this unit
                const int dl = d_unit - d0;                         // within the staged chunk
#pragma unroll
                for (int c = 0; c < 4; ++c)
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                        for (int r = 0; r < 4; ++r) acc[c][mt][r] = 0;

                uint4 wv[4];
#pragma unroll
                for (int c = 0; c < 4; ++c)
                    if (c < ncg) wv[c] = *reinterpret_cast<const uint4*>(sbase + c * code_bytes + warp * kUnitBytes + lane * 16);

#pragma unroll
                for (int s = 0; s < STEPS; ++s) {
                    // activation fragment of this 32-deep step: 8 int8 of row g at depth 8t
                    uint2 bq[MT];
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt)
                        bq[mt] = *reinterpret_cast<const uint2*>(Qs + (size_t)(8 * mt + g) * q_stride + dl + 32 * s + 8 * t);
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        if (c >= ncg) break;
                        uint32_t af[4];
                        if (BITS == 2) {
                            const uint32_t w = s == 0 ? wv[c].x : (s == 1 ? wv[c].y : (s == 2 ? wv[c].z : wv[c].w));
                            const uint32_t e = w & 0x33333333u, o = (w >> 2) & 0x33333333u;
                            af[0] = prmt(p.lut, e);
                            af[1] = prmt(p.lut, o);
                            af[2] = prmt(p.lut, e >> 16);
                            af[3] = prmt(p.lut, o >> 16);
                        } else {
                            const int wd = s >> 1, sh = 4 * (s & 1);
                            const uint32_t w = wd == 0 ? wv[c].x : (wd == 1 ? wv[c].y : (wd == 2 ? wv[c].z : wv[c].w));
                            af[0] = (w >> (sh + 0)) & 0x01010101u;
                            af[1] = (w >> (sh + 1)) & 0x01010101u;
                            af[2] = (w >> (sh + 2)) & 0x01010101u;
                            af[3] = (w >> (sh + 3)) & 0x01010101u;
                        }
                        if (block >= 32) {
#pragma unroll
                            for (int mt = 0; mt < MT; ++mt) mma_s8(acc[c][mt], af, bq[mt].x, bq[mt].y);
                        } else {
                            // 16-deep blocks: a step covers two; lanes t < 2 feed the
                            // first, t >= 2 the second, and each is flushed separately
#pragma unroll
                            for (int hb = 0; hb < 2; ++hb) {
                                const bool mine = (t >> 1) == hb;
                                int a2[MT][4];
#pragma unroll
                                for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
                                    for (int r = 0; r < 4; ++r) a2[mt][r] = 0;
                                    mma_s8(a2[mt], af, mine ? bq[mt].x : 0u, mine ? bq[mt].y : 0u);
                                    const int bl = ((d_unit + 32 * s + 16 * hb) >> p.log2_block) - blk0;
                                    int* dst = sums + (((size_t)bl * CG + c) * rows + 8 * mt) * 16;
                                    atomicAdd(dst + (2 * t) * 16 + g, a2[mt][0]);
                                    atomicAdd(dst + (2 * t + 1) * 16 + g, a2[mt][1]);
                                    atomicAdd(dst + (2 * t) * 16 + g + 8, a2[mt][2]);
                                    atomicAdd(dst + (2 * t + 1) * 16 + g + 8, a2[mt][3]);
                                }
                            }
                        }
                    }
                    // flush at the end of a block (or of the unit)
                    if (block >= 32) {
                        const int d_end = d_unit + 32 * (s + 1);
                        if ((d_end & (block - 1)) == 0 || s == STEPS - 1) {
                            const int bl = (block <= KC) ? (((d_end - 1) >> p.log2_block) - blk0) : 0;
#pragma unroll
                            for (int c = 0; c < 4; ++c) {
                                if (c >= ncg) break;
#pragma unroll
                                for (int mt = 0; mt < MT; ++mt) {
                                    int* dst = sums + (((size_t)bl * CG + c) * rows + 8 * mt) * 16;
                                    atomicAdd(dst + (2 * t) * 16 + g, acc[c][mt][0]);
                                    atomicAdd(dst + (2 * t + 1) * 16 + g, acc[c][mt][1]);
                                    atomicAdd(dst + (2 * t) * 16 + g + 8, acc[c][mt][2]);
                                    atomicAdd(dst + (2 * t + 1) * 16 + g + 8, acc[c][mt][3]);
#pragma unroll
                                    for (int r = 0; r < 4; ++r) acc[c][mt][r] = 0;
                                }
                            }
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[slot]);
        }
        asm volatile("bar.sync 1, %0;" ::"n"(32 * kWarps));

        // ---- ordered fold of the blocks completed by this chunk ----
        const bool block_ends = block <= KC || ((d0 + chunk) & (block - 1)) == 0 || ch == num_chunks - 1;
        if (block_ends) {
            const int nblk = block <= KC ? min(bpc, p.nb_real - blk0) : (blk0 < p.nb_real ? 1 : 0);
#pragma unroll
            for (int i = 0; i < kMaxOutPerThread; ++i) {
                const int o = tid + i * 32 * kWarps;
                if (o >= n_out) break;
                const int col = o & 15, r = (o >> 4) % rows, c = o / (16 * rows);
                float tot = total[i];
                for (int bl = 0; bl < nblk; ++bl) {
                    int s = sums[(((size_t)bl * CG + c) * rows + r) * 16 + col];
                    if (BITS == 1) s = 2 * s - QSs[r * bpc + bl];
                    if (p.sums_out) {
                        const int gr = row0 + r, gc = (cg0 + c) * 16 + col;
                        if (c < ncg && gr < p.m && gc < p.n) p.sums_out[((size_t)gr * p.n + gc) * p.nb_real + blk0 + bl] = s;
                    }
                    const float sc = __half2float(__ushort_as_half(Ss[(c * bpc + bl) * 16 + scale_slot(col)]));
                    tot = fmaf((float)s, __fmul_rn(sc, SAs[r * bpc + bl]), tot);
                }
                total[i] = tot;
            }
        }
    }

    // ---- epilogue + store ----
#pragma unroll
    for (int i = 0; i < kMaxOutPerThread; ++i) {
        const int o = tid + i * 32 * kWarps;
        if (o >= n_out) break;
        const int col = o & 15, r = (o >> 4) % rows, c = o / (16 * rows);
        const int gr = row0 + r, gc = (cg0 + c) * 16 + col;
        if (c < ncg && gr < p.m && gc < p.n)
            p.c[(size_t)gr * p.n + gc] = ep_store_value<0>(p.ep, total[i], (size_t)gr, (size_t)gc);
    }
}

template <int BITS, int MT>
cudaError_t launch_lb(const LowbitGemvArgs& a, dim3 grid, size_t smem, cudaStream_t stream) {
    auto kern = lowbit_gemv_kernel<BITS, MT>;
    static int attr_dev = -1;   // the opt-in is per device; set it once (to the maximum) per device
    int dev = 0;
    cudaGetDevice(&dev);
    if (attr_dev != dev) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (e != cudaSuccess) return e;
        attr_dev = dev;
    }
    if (smem > 227 * 1024) return cudaErrorInvalidConfiguration;
    kern<<<grid, kThreadsLb, smem, stream>>>(a);
    return cudaGetLastError();
}

size_t lowbit_smem(int bits, int ns, int cg, int mt, int kc, int block) {
    const int rows = 8 * mt;
    const int bpc = kc >= block ? kc / block : 1;
    (void)bits;
    return 256 + (size_t)ns * cg * kUnitBytes * kWarps + (size_t)rows * (kc + 32) + (size_t)cg * bpc * 16 * 2 +
           (size_t)rows * bpc * 8 + (size_t)bpc * cg * 16 * rows * 4 + 64;
}

}  // namespace

cudaError_t act_quant_launch(const ActQuantArgs& a, cudaStream_t stream) {
    if (a.m == 0 || a.nbq == 0) return cudaSuccess;
    dim3 grid(a.nbq, a.m);
    act_quant_kernel<<<grid, 128, 0, stream>>>(a);
    return cudaGetLastError();
}

cudaError_t lowbit_gemv_launch(LowbitGemvArgs a, int bits, int sm_count, cudaStream_t stream) {
    const int ud = bits == 2 ? kQ2UnitDepth : kQ1UnitDepth;
    const int sd = ud * kWarps;
    const int block = 1 << a.log2_block;
    int mt = a.m <= 8 ? 1 : (a.m <= 16 ? 2 : 4);
    int cg = 4;
    while (cg > 1 && (a.n16 + cg - 1) / cg < 2 * sm_count) cg >>= 1;
    // K chunk: a power-of-two number of stages, at most 32 KB of int8 activations
    int kc = sd;
    while (kc * 2 <= 4096 / mt * 1 && kc < a.kq) kc *= 2;
    if (kc < sd) kc = sd;
    const size_t budget = 200 * 1024;
    int ns = 4;
    for (;;) {
        ns = cg >= 4 ? 3 : (cg == 2 ? 4 : 6);
        const int n_out = cg * 16 * 8 * mt;
        if (lowbit_smem(bits, ns, cg, mt, kc, block) <= budget && n_out <= kMaxOutPerThread * 32 * kWarps) break;
        if (kc > sd) { kc /= 2; continue; }
        if (cg > 1) { cg >>= 1; continue; }
        if (mt > 1) { mt >>= 1; continue; }
        return cudaErrorInvalidConfiguration;
    }
    a.ns = ns; a.cg = cg; a.kc = kc;
    const size_t smem = lowbit_smem(bits, ns, cg, mt, kc, block);
    dim3 grid((a.n16 + cg - 1) / cg, (a.m + 8 * mt - 1) / (8 * mt));
    if (bits == 2) {
        if (mt == 1) return launch_lb<2, 1>(a, grid, smem, stream);
        if (mt == 2) return launch_lb<2, 2>(a, grid, smem, stream);
        return launch_lb<2, 4>(a, grid, smem, stream);
    }
    if (mt == 1) return launch_lb<1, 1>(a, grid, smem, stream);
    if (mt == 2) return launch_lb<1, 2>(a, grid, smem, stream);
    return launch_lb<1, 4>(a, grid, smem, stream);
}

}  // namespace smeg

// ---------------------------------------------------------------------------
// smeg_matmul_lowbit_static_dev: the 2-bit / 1-bit GEMV for callers that must
// not allocate device memory.
//
// The ordinary entry point takes the scratch for the quantised activations
// (int8 codes, per-block scales, per-block code sums) from the stream-ordered
// allocator on every call.  Some callers cannot do that: code running inside a
// latency-critical serving loop that has frozen its memory map, a host that
// pre-reserved all of HBM for weights and KV cache and leaves the allocator
// nothing, or a plug-in sandbox that is simply not allowed to call cudaMalloc.
// For them this variant keeps that scratch in a fixed array that is part of the
// library image: it exists on every GPU that loads the library, from load until
// the process exits, whether the entry point is ever called or not.
//
// Limits (rejected with rc = -4 beyond them): at most kStaticRows activation
// rows, padded depth at most kStaticDepth, at most kStaticBlocks K-blocks per
// row, and an epilogue graph of at most 16 nodes.
//
// The array is shared by every call on the device and keeps whatever the last
// call left in it.  Nothing in it has to start at zero: each call rewrites the
// region it reads (all codes, scales and sums of its rows) before the GEMV
// kernel, ordered by the stream.  Two calls that overlap on the GPU (different
// streams, or different host threads on different streams) race on the array and
// give wrong results; serialise them on one stream.
//
// The first call on a device looks up the array's device address (host code
// cannot use the array's name as a pointer: on the host that name is only a
// stand-in symbol) and raises the kernels' shared-memory limit; make that first
// call before any stream capture.
// ---------------------------------------------------------------------------
#include <mutex>

#include "../../include/smeg_api.h"
#include "handles.h"

namespace {

constexpr size_t kStaticRows = 8;
constexpr size_t kStaticDepth = 16384;
constexpr size_t kStaticBlocks = 1024;
constexpr size_t kStaticQBytes = kStaticRows * kStaticDepth;               // int8 codes
constexpr size_t kStaticSaBytes = kStaticRows * kStaticBlocks * 4;         // f32 scales / i32 sums
constexpr size_t kStaticBytes = kStaticQBytes + 2 * kStaticSaBytes + 256;  // + the status word's slot

static __device__ __align__(256) unsigned char g_lowbit_static_scratch[kStaticBytes];

struct StaticSetup {
    bool ready = false;
    unsigned char* base = nullptr;   // device address of g_lowbit_static_scratch on this device
    int sm_count = 0;
};
std::mutex g_static_mu;
StaticSetup g_static[64];

// Once per device, with that device current.
int static_setup(StaticSetup** out) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -5;
    std::lock_guard<std::mutex> lk(g_static_mu);
    StaticSetup& s = g_static[dev];
    if (!s.ready) {
        int major = 0;
        if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess || major != 10) return -5;
        if (cudaDeviceGetAttribute(&s.sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return -5;
        void* ptr = nullptr;
        if (cudaGetSymbolAddress(&ptr, g_lowbit_static_scratch) != cudaSuccess || !ptr) return -6;
        s.base = static_cast<unsigned char*>(ptr);
        // the status word lives in the array's last 256 bytes and starts at zero
        if (cudaMemset(s.base + kStaticQBytes + 2 * kStaticSaBytes, 0, 256) != cudaSuccess) return -6;
        s.ready = true;
    }
    *out = &s;
    return 0;
}

}  // namespace

extern "C" int smeg_matmul_lowbit_static_dev(const smeg_lowbit* w, const uint16_t* a, uint16_t* c, size_t m,
                                              const ep_desc16* ep, void* stream_v) {
    using namespace smeg;
    if (!w) return -4;
    cudaStream_t stream = (cudaStream_t)stream_v;
    const size_t n = w->d.n, k = w->d.k;
    if (m == 0 || n == 0) return 0;
    if (!c || (k && !a) || n > 0x7fffffffu || k > 0x7fffffffu) return -4;
    const size_t kq = w->d.ku * (size_t)w->d.unit_depth, nb = w->d.nb;
    if (m > kStaticRows || kq > kStaticDepth || nb > kStaticBlocks) return -4;   // beyond the fixed scratch
    if (ep && ep->n_nodes > (uint32_t)kMaxInlineNodes) return -4;               // a longer graph would need a device buffer
    StaticSetup* st = nullptr;
    int rc = static_setup(&st);
    if (rc) return rc;

    ActQuantArgs aq;
    aq.a = a;
    aq.q = reinterpret_cast<int8_t*>(st->base);
    aq.sa = reinterpret_cast<float*>(st->base + kStaticQBytes);
    aq.qsum = w->bits == 1 ? reinterpret_cast<int32_t*>(st->base + kStaticQBytes + kStaticSaBytes) : nullptr;
    aq.m = (int)m; aq.k = (int)k; aq.kq = (int)kq; aq.nbq = (int)nb; aq.log2_block = w->d.log2_block;

    LowbitGemvArgs g;
    memset(&g, 0, sizeof(g));
    if (ep && ep->n_nodes && ep->nodes) {
        for (uint32_t i = 0; i < ep->n_nodes; ++i) {
            const EpNode& s = ep->nodes[i];
            if (s.op > 24u) return -4;
            g.ep.nodes[i].op = (s.op & 0xffu) | ((s.aux & 0xffu) << 8);
            g.ep.nodes[i].scalar = s.scalar;
            g.ep.nodes[i].ptr = static_cast<const uint16_t*>(s.ptr);
            g.ep.nodes[i].ld = s.ld == 0 ? n : s.ld;
        }
        g.ep.n_nodes = (int)ep->n_nodes;
    }
    g.codes = w->codes; g.scales = w->scales; g.q = aq.q; g.sa = aq.sa; g.qsum = aq.qsum; g.c = c;
    g.m = (int)m; g.n = (int)n; g.k = (int)k; g.kq = (int)kq;
    g.n16 = (int)w->d.n16; g.ku = (int)w->d.ku; g.nb = (int)nb; g.nb_real = (int)w->d.nb_real;
    g.log2_block = w->d.log2_block; g.lut = w->lut;
    g.status = reinterpret_cast<unsigned*>(st->base + kStaticQBytes + 2 * kStaticSaBytes);
    if (act_quant_launch(aq, stream) != cudaSuccess) return -6;
    if (lowbit_gemv_launch(g, w->bits, st->sm_count, stream) != cudaSuccess) return -6;
    return 0;
}
