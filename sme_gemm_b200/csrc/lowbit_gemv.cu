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

constexpr int kWarps = 8;                 // units per stage
constexpr int kCWarps = 16;               // consumer warps: two per unit, each taking every other column group
constexpr int kThreadsLb = 32 * (kCWarps + 1);

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
    pdl_launch_dependents();
    pdl_wait();
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
        if (p.qh) {
            // qh_perm: depths of a group of four in the order 0 2 1 3 (the fragment order of lowbit_mma_kernel);
            // 2: also scaled by position in a group of eight -- 2^8 2^8 2^0 2^0 2^6 2^6 2^-2 2^-2, all exact in f16
            const size_t pos = p.qh_perm ? ((d & ~(size_t)3) | ((d & 1) << 1) | ((d >> 1) & 1)) : d;
            float fv = (float)v;
            if (p.qh_perm == 2) {
                const int e = (int)(pos & 7) >> 1;
                fv *= e == 0 ? 256.0f : (e == 1 ? 1.0f : (e == 2 ? 64.0f : 0.25f));
            }
            p.qh[(size_t)row * p.kq + pos] = __half_as_ushort(__float2half_rn(fv));
        }
        local += v;
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) local += __shfl_xor_sync(0xffffffffu, local, o);
    if ((tid & 31) == 0) s_sum[tid >> 5] = local;
    __syncthreads();
    if (tid == 0) {
        const bool real = d0 < (size_t)p.k;
        const float sa = real ? __fdiv_rn(amax, 127.0f) : 0.0f;
        const int qsum = s_sum[0] + s_sum[1] + s_sum[2] + s_sum[3];
        p.sa[(size_t)row * p.nbq + b] = sa;
        if (p.qsum) p.qsum[(size_t)row * p.nbq + b] = qsum;
        if (p.sa_t) p.sa_t[(size_t)b * p.mpad + row] = sa;
        if (p.qsum_t) p.qsum_t[(size_t)b * p.mpad + row] = (float)qsum;
    }
}

// ---------------------------------------------------------------------------
// The GEMV.  BITS = 2 or 1, MT = groups of 8 rows per CTA, NCG = most column groups per task,
// B16 = 16-deep K-blocks (two per MMA step).
//
// One CTA per SM, persistent over TASKS: a task is `gpt` adjacent column groups (16 columns
// each) over the whole depth.  Everything the CTA reads from global memory goes through the
// bulk-copy engine, in the order it is needed -- a plain load issued while tens of KB of
// copies are queued waits behind them: first the activation rows (when the call passes f16
// activations), then per stage the packed units of the task (8 units = one per consumer warp,
// for every column group) and, with the first stage of a fold chunk, its scale rows.  The
// copies of a round of stages are issued from different lanes at once.  The 8 consumer warps
//   1. quantise the activation rows to int8 in shared memory while the first weights are in
//      flight (or copy rows that act_quant_kernel prepared, for depths too long to stage),
//   2. run the int8 MMAs of their unit of each stage and add the exact block sums into a
//      shared int32 array covering one fold chunk of the depth,
//   3. after each fold chunk, fold every output cell's blocks in K order (one thread per
//      cell), and at the end of the task run the epilogue and store.
// ---------------------------------------------------------------------------
template <int BITS, int MT, int NCG, int B16, int DP>
__global__ void __launch_bounds__(kThreadsLb, 1) lowbit_gemv_kernel(const __grid_constant__ LowbitGemvArgs p) {
    constexpr int UD = BITS == 2 ? kQ2UnitDepth : kQ1UnitDepth;   // depths per unit
    constexpr int STEPS = UD / 32;                                 // mma k-steps per unit
    constexpr int SD = UD * kWarps;                                // depths per stage
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int uw = warp & (kWarps - 1), chalf = warp >> 3;         // consumer warp: unit of the stage, half of the column groups
    const int NS = p.ns, GPT = p.gpt, KC = p.kc, KQ = p.kqc;
    const int block = 1 << p.log2_block;
    const int bpc = KC >= block ? KC / block : 1;                  // sums rows held per fold chunk
    const int nbq = (KQ + block - 1) / block;                      // activation-scale rows per staged chunk
    const int code_bytes = kUnitBytes * kWarps;
    const int stage_bytes = GPT * code_bytes;
    const int rows = 8 * MT;
    const int row0 = blockIdx.y * rows;
    const int rows_used = min(rows, p.m - row0);
    const int RS = p.rows_s;                                       // rows kept in the sums array
    const bool fused = p.a != nullptr;

    uint64_t* full = reinterpret_cast<uint64_t*>(smem_raw);
    uint64_t* empty = full + NS;
    uint64_t* a_full = empty + NS;
    uint64_t* s_empty = a_full + 1;                                // [2] scale buffer read by its fold
    volatile int* abort_flag = reinterpret_cast<volatile int*>(s_empty + 2);
    unsigned char* stages = smem_raw + 256;
    const int q_stride = KQ + 32;                                  // bytes; keeps LDS.64 conflict-free
    int8_t* Qs = reinterpret_cast<int8_t*>(stages + (size_t)NS * stage_bytes);
    uint16_t* Ss = reinterpret_cast<uint16_t*>(Qs + (size_t)rows * q_stride);          // [2][GPT][bpc][16] scales
    float* SAs = reinterpret_cast<float*>(Ss + (size_t)2 * GPT * bpc * 16);            // [rows][nbq]
    int* QSs = reinterpret_cast<int*>(SAs + (size_t)rows * nbq);                       // [rows][nbq]
    int* AMX = QSs + (size_t)rows * nbq;                                               // [rows][nbq] amax bits, then 127/amax
    // the f16 rows are dead once quantised, before the first block sum is written: same storage
    int* sums = reinterpret_cast<int*>((reinterpret_cast<uintptr_t>(AMX + (size_t)rows * nbq) + 127) & ~(uintptr_t)127);   // [bpc][GPT][RS][16]
    const uint16_t* Abuf = reinterpret_cast<const uint16_t*>(sums);                    // [rows_used][KQ] f16
    // running f32 totals of the task's output cells, [GPT][RS][16], behind whichever of the two is larger
    float* TOT = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(sums) + p.u_bytes);

    const int num_qchunks = (p.kq + KQ - 1) / KQ;
    const int stages_total = (p.ku + kWarps - 1) / kWarps;
    const int fc_stages = KC / SD;                                 // stages per fold chunk
    const int my_tasks = ((int)blockIdx.x < p.ntasks) ? (p.ntasks - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;

    if (tid == 0) {
        for (int s = 0; s < NS; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], kCWarps);
        }
        mbar_init(a_full, 1);
        mbar_init(&s_empty[0], kCWarps);
        mbar_init(&s_empty[1], kCWarps);
        *abort_flag = 0;
        fence_barrier_init();
    }
    __syncthreads();
    pdl_launch_dependents();

    if (warp == kCWarps) {
        // ================= producer =================
        // The first round of weights goes out at once (it does not depend on the kernel ahead in the stream);
        // the activation rows follow when that kernel's memory is visible: one bulk copy per row, one lane each.
        auto send_a = [&]() {
            pdl_wait();
            if (!fused) return;
            if (lane == 0) mbar_expect_tx(a_full, (unsigned)rows_used * (unsigned)p.k * 2u);
            __syncwarp();
            for (int r = lane; r < rows_used; r += 32)
                bulk_g2s(const_cast<uint16_t*>(Abuf) + (size_t)r * KQ, p.a + (size_t)(row0 + r) * p.k, (unsigned)p.k * 2u, a_full);
        };
        // lane = (stage of the round, copy): copies 0-7 are the code runs of the task's column
        // groups, 8-15 their scale rows (first stage of a fold chunk only); a round never holds
        // more stages than the ring has slots
        const int si = lane >> 4, j = lane & 15;
        const int round_stages = min(2, NS);
        const int total_seq = my_tasks * stages_total;
        for (int seq0 = 0; seq0 < total_seq; seq0 += round_stages) {
            const int seq = seq0 + si;
            const bool active = si < round_stages && seq < total_seq;
            const int ti = active ? seq / stages_total : 0, st = active ? seq % stages_total : 0;
            const int task = (int)blockIdx.x + ti * (int)gridDim.x;
            const int cg0 = task * GPT;
            const int ncg = min(GPT, p.n16 - cg0);
            const int slot = seq % NS;
            const int units = min(kWarps, p.ku - st * kWarps);
            const bool fc_first = st % fc_stages == 0;
            const int fseq = ti * ((stages_total + fc_stages - 1) / fc_stages) + st / fc_stages;   // fold chunks so far
            const int blk0 = (st * SD) >> p.log2_block;
            const int nrows = min(bpc, p.nb - blk0);
            bool ok = true;
            if (active && j == 0) {
                if (seq >= NS) ok = mbar_wait(&empty[slot], ((seq / NS) - 1) & 1, abort_flag, p.status);
                // the scale buffer of this parity was last read by the fold two chunks back
                if (ok && fc_first && fseq >= 2) ok = mbar_wait(&s_empty[fseq & 1], ((fseq >> 1) - 1) & 1, abort_flag, p.status);
                if (ok) mbar_expect_tx(&full[slot], ncg * units * kUnitBytes + (fc_first ? ncg * nrows * 32 : 0));
            }
            if (!__all_sync(0xffffffffu, ok)) return;
            if (active) {
                if (j < ncg)
                    bulk_g2s(stages + (size_t)slot * stage_bytes + j * code_bytes,
                             p.codes + (((size_t)(cg0 + j) * p.ku + (size_t)st * kWarps) * kUnitBytes), units * kUnitBytes, &full[slot]);
                else if (fc_first && j >= 8 && j - 8 < ncg)
                    bulk_g2s(Ss + ((size_t)(fseq & 1) * GPT + (j - 8)) * bpc * 16,
                             p.scales + ((size_t)(cg0 + j - 8) * p.nb + blk0) * 16, nrows * 32, &full[slot]);
            }
            if (seq0 == 0) send_a();
        }
        if (total_seq == 0) send_a();
        return;
    }

    // ================= consumers =================
    pdl_wait();
    // rows past the batch feed zeros to the MMAs
    for (int idx = tid; idx < (rows - rows_used) * (q_stride / 4); idx += 32 * kCWarps)
        reinterpret_cast<uint32_t*>(Qs + (size_t)rows_used * q_stride)[idx] = 0u;

    int acc[NCG / 2][DP ? 2 : MT][4];                                  // DP (= most rows): [column g | g + 8][row]
    int staged_qc = -1;
    int seq = 0;                                                   // stage counter of this CTA's ring
    int fseq = 0;                                                  // fold-chunk counter (scale buffer parity)

    for (int ti = 0; ti < my_tasks; ++ti) {
        const int task = (int)blockIdx.x + ti * (int)gridDim.x;
        const int cg0 = task * GPT;
        const int ncg = min(GPT, p.n16 - cg0);
        const int n_out = ncg * 16 * RS;                           // output cells of this task
        for (int o = tid; o < n_out; o += 32 * kCWarps) TOT[o] = 0.0f;   // read back by the same thread only

        int st = 0;
        for (int qc = 0; qc < num_qchunks; ++qc) {
            const int dq0 = qc * KQ;
            const int qchunk = min(KQ, p.kq - dq0);
            const int blkq0 = dq0 >> p.log2_block;                   // first block of the staged chunk
            // ---- the chunk's activations: int8 codes, per-block scales, per-block code sums ----
            if (staged_qc != qc) {
                staged_qc = qc;
                asm volatile("bar.sync 1, %0;" ::"n"(32 * kCWarps));  // the previous chunk's readers are done
                if (fused) {
                    // quantize_row (src/kernels/lowbit/matmul.rs:354-371) over the staged f16 rows (whole depth)
                    for (int idx = tid; idx < rows * nbq; idx += 32 * kCWarps) { AMX[idx] = 0; QSs[idx] = 0; }
                    mbar_wait(a_full, 0, abort_flag, p.status);
                    asm volatile("bar.sync 1, %0;" ::"n"(32 * kCWarps));
                    // items: 8 consecutive depths of one row; consecutive lanes take consecutive items, so the
                    // lanes of one K-block are an aligned run of seg = min(32, block / 8) lanes
                    const int nvec = qchunk / 8;
                    const int total_items = rows_used * nvec;
                    const float inv_nvec = 1.0f / (float)nvec;
                    int seg = min(32, block >> 3);
                    if (nvec % seg) seg = 16;                        // the staged depth is whole units: a multiple of 16 items
                    const int iters = (total_items + 32 * kCWarps - 1) / (32 * kCWarps);
                    for (int it = 0; it < iters; ++it) {
                        const int idx = tid + it * 32 * kCWarps;
                        const bool in = idx < total_items;
                        int r = in ? (int)(((float)idx + 0.5f) * inv_nvec) : 0;
                        if (r * nvec > idx) --r;
                        if ((r + 1) * nvec <= idx) ++r;
                        const int v = idx - r * nvec, d = 8 * v;
                        int mx = 0;
                        if (in && d < p.k) {
                            const uint4 hv = *reinterpret_cast<const uint4*>(Abuf + (size_t)r * KQ + d);
                            const uint32_t hw[4] = {hv.x, hv.y, hv.z, hv.w};
                            // |x| as integer bits: ordered like the values, and every NaN is above infinity
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&hw[i]));
                                mx = max(mx, max(__float_as_int(fabsf(f.x)), __float_as_int(fabsf(f.y))));
                            }
                        }
                        // nvec is a multiple of seg, so a run never crosses a row
                        for (int o = 1; o < seg; o <<= 1) mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
                        if (in && d < p.k && (lane & (seg - 1)) == 0) atomicMax(&AMX[r * nbq + (d >> p.log2_block)], mx);
                    }
                    asm volatile("bar.sync 1, %0;" ::"n"(32 * kCWarps));
                    for (int idx = tid; idx < rows_used * nbq; idx += 32 * kCWarps) {
                        const int r = idx / nbq, bl = idx % nbq;
                        const int bits = AMX[idx];
                        const float amax = bits > 0x7f800000 ? __int_as_float(0x7fc00000) : __int_as_float(bits);
                        const bool real = ((size_t)bl << p.log2_block) < (size_t)p.k;
                        const float sa = real ? __fdiv_rn(amax, 127.0f) : 0.0f;
                        SAs[idx] = sa;
                        AMX[idx] = __float_as_int(amax > 0.0f ? __fdiv_rn(127.0f, amax) : 0.0f);
                        if (p.sa_out && blockIdx.x == 0 && real) p.sa_out[(size_t)(row0 + r) * p.nb_real + bl] = sa;
                    }
                    asm volatile("bar.sync 1, %0;" ::"n"(32 * kCWarps));
                    for (int it = 0; it < iters; ++it) {
                        const int idx = tid + it * 32 * kCWarps;
                        const bool in = idx < total_items;
                        int r = in ? (int)(((float)idx + 0.5f) * inv_nvec) : 0;
                        if (r * nvec > idx) --r;
                        if ((r + 1) * nvec <= idx) ++r;
                        const int v = idx - r * nvec, d = 8 * v;
                        uint32_t lo = 0, hi = 0;
                        int sum = 0;
                        const int bl = d >> p.log2_block;
                        if (in && d < p.k) {
                            const uint4 hv = *reinterpret_cast<const uint4*>(Abuf + (size_t)r * KQ + d);
                            const uint32_t hw[4] = {hv.x, hv.y, hv.z, hv.w};
                            const float inv = __int_as_float(AMX[r * nbq + bl]);
                            int q[8];
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&hw[i]));
                                // round to nearest even, NaN -> 0, then saturate: round_ties_even(x) as i8
                                q[2 * i] = max(-128, min(127, __float2int_rn(__fmul_rn(f.x, inv))));
                                q[2 * i + 1] = max(-128, min(127, __float2int_rn(__fmul_rn(f.y, inv))));
                            }
                            lo = __byte_perm(__byte_perm(q[0], q[1], 0x0040), __byte_perm(q[2], q[3], 0x0040), 0x5410);
                            hi = __byte_perm(__byte_perm(q[4], q[5], 0x0040), __byte_perm(q[6], q[7], 0x0040), 0x5410);
                            if (BITS == 1) sum = __dp4a((int)lo, 0x01010101, __dp4a((int)hi, 0x01010101, 0));
                            if (p.q_out && blockIdx.x == 0) *reinterpret_cast<uint2*>(p.q_out + (size_t)(row0 + r) * p.k + d) = make_uint2(lo, hi);
                        }
                        if (BITS == 1) {
                            for (int o = 1; o < seg; o <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
                            if (in && d < p.k && (lane & (seg - 1)) == 0 && sum != 0) atomicAdd(&QSs[r * nbq + bl], sum);
                        }
                        if (in) *reinterpret_cast<uint2*>(Qs + (size_t)r * q_stride + d) = make_uint2(lo, hi);
                    }
                } else {
                    const int vec_per_row = qchunk / 16;
                    for (int idx = tid; idx < rows_used * vec_per_row; idx += 32 * kCWarps) {
                        const int r = idx / vec_per_row, v = idx % vec_per_row;
                        *reinterpret_cast<uint4*>(Qs + (size_t)r * q_stride + v * 16) =
                            *reinterpret_cast<const uint4*>(p.q + (size_t)(row0 + r) * p.kq + dq0 + v * 16);
                    }
                    const int nblkq = min(nbq, p.nb - blkq0);
                    for (int idx = tid; idx < rows_used * nbq; idx += 32 * kCWarps) {
                        const int r = idx / nbq, bl = idx % nbq;
                        const bool ok = bl < nblkq;
                        SAs[idx] = ok ? p.sa[(size_t)(row0 + r) * p.nb + blkq0 + bl] : 0.0f;
                        QSs[idx] = (ok && p.qsum) ? p.qsum[(size_t)(row0 + r) * p.nb + blkq0 + bl] : 0;
                    }
                }
            }

            const int st_qend = min(stages_total, (dq0 + qchunk + SD - 1) / SD);
            while (st < st_qend) {
                // ---- one fold chunk: KC depths from stage st ----
                const int d0 = st * SD;
                const int chunk = min(KC, p.kq - d0);
                const int blk0 = d0 >> p.log2_block;                     // first block (row of scales) of the fold chunk
                const int blr = block <= KQ ? blk0 - blkq0 : 0;          // ... relative to the staged activation scales
                const bool block_starts = (d0 & (block - 1)) == 0;       // always true when block <= KC
                const uint16_t* Sc = Ss + (size_t)(fseq & 1) * GPT * bpc * 16;
                asm volatile("bar.sync 1, %0;" ::"n"(32 * kCWarps));      // quantised rows visible; previous fold done
                if (block_starts)
                    for (int idx = tid; idx < bpc * GPT * RS * 16; idx += 32 * kCWarps) sums[idx] = 0;
                asm volatile("bar.sync 1, %0;" ::"n"(32 * kCWarps));

                const int st_end = min(st_qend, st + fc_stages);
                for (; st < st_end; ++st, ++seq) {
                    const int slot = seq % NS;
                    mbar_wait(&full[slot], (seq / NS) & 1, abort_flag, p.status);
                    const int units = min(kWarps, p.ku - st * kWarps);
                    if (uw < units) {
                        const unsigned char* sbase = stages + (size_t)slot * stage_bytes;
                        const int d_unit = st * SD + uw * UD;             // global depth of this unit
                        const int dl = d_unit - dq0;                        // within the staged activations
#pragma unroll
                        for (int ci = 0; ci < NCG / 2; ++ci)
#pragma unroll
                            for (int mt = 0; mt < (DP ? 2 : MT); ++mt)
#pragma unroll
                                for (int r = 0; r < 4; ++r) acc[ci][mt][r] = 0;

                        uint4 wv[NCG / 2];
#pragma unroll
                        for (int ci = 0; ci < NCG / 2; ++ci)
                            if (2 * ci + chalf < ncg) wv[ci] = *reinterpret_cast<const uint4*>(sbase + (2 * ci + chalf) * code_bytes + uw * kUnitBytes + lane * 16);

                        // rolled on purpose: the body is large once the column groups are unrolled, and a fully
                        // unrolled unit did not fit the instruction cache
#pragma unroll 1
                        for (int s = 0; s < STEPS; ++s) {
                            if (DP) {
                                // at most four rows: dot products on the integer units instead of the tensor cores
                                // (an int8 mma.sync issues about once per 85 cycles per scheduler on this part).
                                // The lane's bytes are columns g and g + 8 at depths 8t .. 8t + 7.
                                uint2 aq[DP ? DP : 1];
#pragma unroll
                                for (int r = 0; r < DP; ++r)
                                    aq[r] = r < RS ? *reinterpret_cast<const uint2*>(Qs + (size_t)r * q_stride + dl + 32 * s + 8 * t) : make_uint2(0u, 0u);
                                const int wsel = BITS == 2 ? s : (s >> 1);
                                const int sh = 4 * (s & 1);
#pragma unroll
                                for (int ci = 0; ci < NCG / 2; ++ci) {
                                    const int c = 2 * ci + chalf;
                                    if (c >= ncg) break;
                                    uint32_t af[4];
                                    const uint32_t w = wsel == 0 ? wv[ci].x : (wsel == 1 ? wv[ci].y : (wsel == 2 ? wv[ci].z : wv[ci].w));
                                    if (BITS == 2) {
                                        const uint32_t e = w & 0x33333333u, o = (w >> 2) & 0x33333333u;
                                        af[0] = prmt(p.lut, e);
                                        af[1] = prmt(p.lut, o);
                                        af[2] = prmt(p.lut, e >> 16);
                                        af[3] = prmt(p.lut, o >> 16);
                                    } else {
                                        af[0] = (w >> (sh + 0)) & 0x01010101u;
                                        af[1] = (w >> (sh + 1)) & 0x01010101u;
                                        af[2] = (w >> (sh + 2)) & 0x01010101u;
                                        af[3] = (w >> (sh + 3)) & 0x01010101u;
                                    }
#pragma unroll
                                    for (int r = 0; r < DP; ++r) {
                                        acc[ci][0][r] = __dp4a((int)af[0], (int)aq[r].x, acc[ci][0][r]);
                                        acc[ci][0][r] = __dp4a((int)af[2], (int)aq[r].y, acc[ci][0][r]);
                                        acc[ci][1][r] = __dp4a((int)af[1], (int)aq[r].x, acc[ci][1][r]);
                                        acc[ci][1][r] = __dp4a((int)af[3], (int)aq[r].y, acc[ci][1][r]);
                                    }
                                }
                                // flush at the end of a block (or of the unit): the four lanes holding the depth
                                // slices of a column add into the same cell
                                const int d_end = d_unit + 32 * (s + 1);
                                if (B16 || (d_end & (block - 1)) == 0 || s == STEPS - 1) {
                                    const int bl = B16 ? (((d_unit + 32 * s + 16 * (t >> 1)) >> p.log2_block) - blk0)
                                                       : ((block <= KC) ? (((d_end - 1) >> p.log2_block) - blk0) : 0);
                                    int* dst0 = sums + (size_t)bl * GPT * RS * 16 + g;
#pragma unroll
                                    for (int ci = 0; ci < NCG / 2; ++ci) {
                                        const int c = 2 * ci + chalf;
                                        if (c >= ncg) break;
#pragma unroll
                                        for (int r = 0; r < DP; ++r) {
                                            if (r < RS) {
                                                atomicAdd(dst0 + (c * RS + r) * 16, acc[ci][0][r]);
                                                atomicAdd(dst0 + (c * RS + r) * 16 + 8, acc[ci][1][r]);
                                            }
                                            acc[ci][0][r] = 0;
                                            acc[ci][1][r] = 0;
                                        }
                                    }
                                }
                                continue;
                            }
                            // activation fragment of this 32-deep step: 8 int8 of row g at depth 8t
                            uint2 bq[MT];
#pragma unroll
                            for (int mt = 0; mt < MT; ++mt)
                                bq[mt] = *reinterpret_cast<const uint2*>(Qs + (size_t)(8 * mt + g) * q_stride + dl + 32 * s + 8 * t);
                            const int wsel = BITS == 2 ? s : (s >> 1);
                            const int sh = 4 * (s & 1);
#pragma unroll
                            for (int ci = 0; ci < NCG / 2; ++ci) {
                                const int c = 2 * ci + chalf;
                                if (c >= ncg) break;
                                uint32_t af[4];
                                const uint32_t w = wsel == 0 ? wv[ci].x : (wsel == 1 ? wv[ci].y : (wsel == 2 ? wv[ci].z : wv[ci].w));
                                if (BITS == 2) {
                                    const uint32_t e = w & 0x33333333u, o = (w >> 2) & 0x33333333u;
                                    af[0] = prmt(p.lut, e);
                                    af[1] = prmt(p.lut, o);
                                    af[2] = prmt(p.lut, e >> 16);
                                    af[3] = prmt(p.lut, o >> 16);
                                } else {
                                    af[0] = (w >> (sh + 0)) & 0x01010101u;
                                    af[1] = (w >> (sh + 1)) & 0x01010101u;
                                    af[2] = (w >> (sh + 2)) & 0x01010101u;
                                    af[3] = (w >> (sh + 3)) & 0x01010101u;
                                }
                                if (!B16) {
#pragma unroll
                                    for (int mt = 0; mt < MT; ++mt) mma_s8(acc[ci][mt], af, bq[mt].x, bq[mt].y);
                                } else {
                                    // 16-deep blocks: a step covers two; lanes t < 2 feed the
                                    // first, t >= 2 the second, and each is flushed separately
#pragma unroll 1
                                    for (int hb = 0; hb < 2; ++hb) {
                                        const bool mine = (t >> 1) == hb;
#pragma unroll
                                        for (int mt = 0; mt < MT; ++mt) {
                                            int a2[4] = {0, 0, 0, 0};
                                            mma_s8(a2, af, mine ? bq[mt].x : 0u, mine ? bq[mt].y : 0u);
                                            const int bl = ((d_unit + 32 * s + 16 * hb) >> p.log2_block) - blk0;
                                            int* dst = sums + ((size_t)bl * GPT + c) * RS * 16;
                                            const int r0 = 8 * mt + 2 * t;
                                            if (r0 < RS) {
                                                atomicAdd(dst + r0 * 16 + g, a2[0]);
                                                atomicAdd(dst + r0 * 16 + g + 8, a2[2]);
                                            }
                                            if (r0 + 1 < RS) {
                                                atomicAdd(dst + (r0 + 1) * 16 + g, a2[1]);
                                                atomicAdd(dst + (r0 + 1) * 16 + g + 8, a2[3]);
                                            }
                                        }
                                    }
                                }
                            }
                            // flush at the end of a block (or of the unit)
                            if (!B16) {
                                const int d_end = d_unit + 32 * (s + 1);
                                if ((d_end & (block - 1)) == 0 || s == STEPS - 1) {
                                    const int bl = (block <= KC) ? (((d_end - 1) >> p.log2_block) - blk0) : 0;
#pragma unroll
                                    for (int ci = 0; ci < NCG / 2; ++ci) {
                                        const int c = 2 * ci + chalf;
                                        if (c >= ncg) break;
#pragma unroll
                                        for (int mt = 0; mt < MT; ++mt) {
                                            int* dst = sums + ((size_t)bl * GPT + c) * RS * 16;
                                            const int r0 = 8 * mt + 2 * t;
                                            if (r0 < RS) {
                                                atomicAdd(dst + r0 * 16 + g, acc[ci][mt][0]);
                                                atomicAdd(dst + r0 * 16 + g + 8, acc[ci][mt][2]);
                                            }
                                            if (r0 + 1 < RS) {
                                                atomicAdd(dst + (r0 + 1) * 16 + g, acc[ci][mt][1]);
                                                atomicAdd(dst + (r0 + 1) * 16 + g + 8, acc[ci][mt][3]);
                                            }
#pragma unroll
                                            for (int r = 0; r < 4; ++r) acc[ci][mt][r] = 0;
                                        }
                                    }
                                }
                            }
                        }
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&empty[slot]);
                }
                asm volatile("bar.sync 1, %0;" ::"n"(32 * kCWarps));

                // ---- ordered fold of the blocks completed by this fold chunk ----
                const bool block_ends = block <= KC || ((d0 + chunk) & (block - 1)) == 0 || st == stages_total;
                if (block_ends) {
                    const int nfold = block <= KC ? min(bpc, p.nb_real - blk0) : (blk0 < p.nb_real ? 1 : 0);
#pragma unroll 1
                    for (int o = tid; o < n_out; o += 32 * kCWarps) {
                        const int col = o & 15, r = (o >> 4) % RS, c = o / (16 * RS);
                        if (r >= rows_used) continue;
                        float tot = TOT[o];
#pragma unroll 4
                        for (int bl = 0; bl < nfold; ++bl) {
                            int s = sums[(((size_t)bl * GPT + c) * RS + r) * 16 + col];
                            if (BITS == 1) s = 2 * s - QSs[r * nbq + blr + bl];
                            if (p.sums_out) {
                                const int gr = row0 + r, gc = (cg0 + c) * 16 + col;
                                if (gc < p.n) p.sums_out[((size_t)gr * p.n + gc) * p.nb_real + blk0 + bl] = s;
                            }
                            const float sc = __half2float(__ushort_as_half(Sc[(c * bpc + bl) * 16 + scale_slot(col)]));
                            tot = fmaf((float)s, __fmul_rn(sc, SAs[r * nbq + blr + bl]), tot);
                        }
                        TOT[o] = tot;
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&s_empty[fseq & 1]);
                ++fseq;
            }
        }

        // ---- epilogue + store ----
#pragma unroll 1
        for (int o = tid; o < n_out; o += 32 * kCWarps) {
            const int col = o & 15, r = (o >> 4) % RS, c = o / (16 * RS);
            const int gr = row0 + r, gc = (cg0 + c) * 16 + col;
            if (r < rows_used && gc < p.n)
                p.c[(size_t)gr * p.n + gc] = ep_store_value<0>(p.ep, TOT[o], (size_t)gr, (size_t)gc);
        }
    }
}

template <int BITS, int MT, int NCG, int B16, int DP>
cudaError_t launch_lb(const LowbitGemvArgs& a, dim3 grid, size_t smem, cudaStream_t stream) {
    auto kern = lowbit_gemv_kernel<BITS, MT, NCG, B16, DP>;
    static int attr_dev = -1;   // the opt-in is per device; set it once (to the maximum) per device
    int dev = 0;
    cudaGetDevice(&dev);
    if (attr_dev != dev) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (e != cudaSuccess) return e;
        attr_dev = dev;
    }
    if (smem > 227 * 1024) return cudaErrorInvalidConfiguration;
    return launch_pdl(kern, grid, dim3(kThreadsLb), smem, stream, a);
}

// bytes of the region shared by the staged f16 rows and the block sums
size_t lowbit_u_bytes(int gpt, int rows_s, int kc, int kqc, int block, bool fused) {
    const int bpc = kc >= block ? kc / block : 1;
    const size_t sums = (size_t)bpc * gpt * 16 * rows_s * 4;
    const size_t abuf = fused ? (size_t)rows_s * kqc * 2 : 0;
    return ((sums > abuf ? sums : abuf) + 127) / 128 * 128;
}
size_t lowbit_smem(int ns, int gpt, int mt, int rows_s, int kc, int kqc, int block, bool fused) {
    const int rows = 8 * mt;
    const int bpc = kc >= block ? kc / block : 1;
    const int nbq = (kqc + block - 1) / block;
    return 256 + (size_t)ns * gpt * kUnitBytes * kWarps + (size_t)rows * (kqc + 32) + (size_t)2 * gpt * bpc * 32 +
           (size_t)rows * nbq * 12 + 128 + lowbit_u_bytes(gpt, rows_s, kc, kqc, block, fused) + (size_t)gpt * rows_s * 64 + 64;
}

}  // namespace

cudaError_t act_quant_launch(const ActQuantArgs& a, cudaStream_t stream) {
    if (a.m == 0 || a.nbq == 0) return cudaSuccess;
    dim3 grid(a.nbq, a.m);
    return launch_pdl(act_quant_kernel, grid, dim3(128), 0, stream, a);
}

// Picks rows per CTA, column groups per task, the staged activation chunk, the fold chunk and the
// ring depth.  `fused`: the kernel stages and quantises the f16 rows itself, which needs the
// whole depth in one staged chunk; returns false if no configuration fits shared memory.
bool lowbit_gemv_plan(LowbitGemvArgs& a, int bits, int sm_count, bool fused, dim3* grid, size_t* smem, int* mt_out) {
    const int ud = bits == 2 ? kQ2UnitDepth : kQ1UnitDepth;
    const int sd = ud * kWarps;
    const int block = 1 << a.log2_block;
    const int stages_total = (a.ku + kWarps - 1) / kWarps;
    const int kq_pad = stages_total * sd;
    const size_t budget = 212 * 1024;
    for (int mt = a.m <= 8 ? 1 : (a.m <= 16 ? 2 : 4); mt >= 1; mt >>= 1) {
        const int ncg_max = mt == 1 ? 8 : 4;
        const int rows = 8 * mt;
        const int rows_s = a.m < rows ? a.m : rows;
        const int row_tiles = (a.m + rows - 1) / rows;
        const int target_x = sm_count / row_tiles > 0 ? sm_count / row_tiles : 1;   // one CTA per SM
        int gpt0 = (a.n16 + target_x - 1) / target_x;
        if (gpt0 > ncg_max) gpt0 = ncg_max;
        if (gpt0 < 1) gpt0 = 1;
        // staged activation chunk: the whole depth when its int8 rows fit 72 KB, else a power-of-two number of stages
        int kqc = kq_pad;
        if ((size_t)rows * (kq_pad + 32) > 72 * 1024) {
            if (fused) continue;
            kqc = sd;
            while ((size_t)rows * (2 * kqc + 32) <= 64 * 1024 && 2 * kqc < kq_pad) kqc *= 2;
        }
        int kc_max = sd;
        while (kc_max * 2 <= kqc && kc_max < 8192) kc_max *= 2;
        const int want = stages_total < 8 ? stages_total : 8;
        const int needs[3] = {want < 4 ? want : 4, want < 2 ? want : 2, 1};
        for (int gpt = gpt0; gpt >= 1; --gpt) {
            // a deep ring matters more than a long fold chunk
            for (int ni = 0; ni < 3; ++ni) {
                for (int kc = kc_max; kc >= sd; kc /= 2) {
                    int ns = want;
                    while (ns >= 1 && lowbit_smem(ns, gpt, mt, rows_s, kc, kqc, block, fused) > budget) --ns;
                    if (ns < needs[ni] || ns < 1) continue;
                    a.ns = ns; a.gpt = gpt; a.kc = kc; a.kqc = kqc; a.rows_s = rows_s;
                    a.u_bytes = (int)lowbit_u_bytes(gpt, rows_s, kc, kqc, block, fused);
                    a.ntasks = (a.n16 + gpt - 1) / gpt;
                    *grid = dim3(a.ntasks < target_x ? a.ntasks : target_x, row_tiles);
                    *smem = lowbit_smem(ns, gpt, mt, rows_s, kc, kqc, block, fused);
                    *mt_out = mt;
                    return true;
                }
            }
        }
    }
    return false;
}

cudaError_t lowbit_gemv_launch(LowbitGemvArgs a, int bits, int sm_count, cudaStream_t stream) {
    dim3 grid;
    size_t smem = 0;
    int mt = 1;
    if (!lowbit_gemv_plan(a, bits, sm_count, a.a != nullptr, &grid, &smem, &mt)) return cudaErrorInvalidConfiguration;
    const bool b16 = a.log2_block < 5;
#define SMEG_LB(B, M, N)                                                   \
    do {                                                                   \
        if (b16) return launch_lb<B, M, N, 1, 0>(a, grid, smem, stream);   \
        return launch_lb<B, M, N, 0, 0>(a, grid, smem, stream);            \
    } while (0)
    // up to four rows: the dot-product path
#define SMEG_LB_DP(B, D)                                                   \
    do {                                                                   \
        if (b16) return launch_lb<B, 1, 8, 1, D>(a, grid, smem, stream);   \
        return launch_lb<B, 1, 8, 0, D>(a, grid, smem, stream);            \
    } while (0)
    if (mt == 1 && a.rows_s <= 4) {
        if (bits == 2) {
            if (a.rows_s == 1) SMEG_LB_DP(2, 1);
            if (a.rows_s == 2) SMEG_LB_DP(2, 2);
            SMEG_LB_DP(2, 4);
        }
        if (a.rows_s == 1) SMEG_LB_DP(1, 1);
        if (a.rows_s == 2) SMEG_LB_DP(1, 2);
        SMEG_LB_DP(1, 4);
    }
#undef SMEG_LB_DP
    if (bits == 2) {
        if (mt == 1) SMEG_LB(2, 1, 8);
        if (mt == 2) SMEG_LB(2, 2, 4);
        SMEG_LB(2, 4, 4);
    }
    if (mt == 1) SMEG_LB(1, 1, 8);
    if (mt == 2) SMEG_LB(1, 2, 4);
    SMEG_LB(1, 4, 4);
#undef SMEG_LB
}

// Whether lowbit_gemv_launch can take f16 activations (a.a) for this shape, i.e. stage and quantise
// them in the kernel; otherwise the caller runs act_quant_kernel first and passes q / sa / qsum.
bool lowbit_gemv_fuses_quant(LowbitGemvArgs a, int bits, int sm_count) {
    dim3 grid;
    size_t smem = 0;
    int mt = 1;
    return lowbit_gemv_plan(a, bits, sm_count, true, &grid, &smem, &mt);
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

// Reads and clears the status word of the fixed array on the current device (0 if the entry point
// was never used there).  Called by smeg_last_status after it has synchronised the device; allocates nothing.
unsigned smeg_static_take_status() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
    unsigned char* base = nullptr;
    {
        std::lock_guard<std::mutex> lk(g_static_mu);
        if (!g_static[dev].ready) return 0;
        base = g_static[dev].base;
    }
    unsigned v = 0;
    unsigned char* word = base + kStaticQBytes + 2 * kStaticSaBytes;
    if (cudaMemcpy(&v, word, sizeof(v), cudaMemcpyDeviceToHost) != cudaSuccess) return ~0u;
    if (v) cudaMemset(word, 0, sizeof(unsigned));
    return v;
}

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
    memset(&aq, 0, sizeof(aq));
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
