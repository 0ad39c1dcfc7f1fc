// 2-bit / 1-bit weights x int8-quantised activations on the 5th-generation tensor cores
// (tcgen05.mma, accumulators in tensor memory): matmul_q2 / matmul_q1 above a handful of rows, up to
// prefill-sized batches.
//
// Replaces the reference's SME kernel for these batch sizes (q2_core / run_q2_gemv / Q2_FOLD,
// csrc/gemm_q2.cc:180-204,300-404, which walks the rows in groups of five) and reproduces the bits
// of its portable statement (reference, src/kernels/lowbit/matmul.rs:376-398): every K-block's sum
// is an exact int32, and an output cell folds its blocks in K order with
// total = fmaf((float)sum, scale * sa, total).
//
// The block sums are integer dot products, formed EXACTLY on the f16 tensor-core path: the int8
// activation codes travel as f16 integers (act_quant_kernel writes them so), a weight travels as
// the f16 whose bit pattern is a small unsigned integer u (u * 2^-24: the sign bit itself for
// 1-bit weights, codebook value + 128 for 2-bit ones), products of such numbers are exact, and an
// f32 accumulator holds their sum exactly while it stays below 2^24 units -- which a run of at
// most 256 depths guarantees (255 * 128 * 256 < 2^24).  A K-block longer than that is accumulated
// in runs of 256 depths whose integer sums are added in the fold.  (tcgen05.mma.kind::i8 gives the
// same integers, and an earlier form of this kernel used it, but the int8 tensor path of this
// part sustains only ~135 TOP/s against ~1500 TFLOP/s for f16.)  The 1-bit form does not even move
// its sign bits: bit b of a half word is the f16 number 2^(b-24) for b < 12, so an operand register
// is the packed word under one mask, and act_quant_kernel leaves the codes of the matching depths
// in the matching order, scaled by the inverse power of two (2^8, 1, 2^6, 2^-2: still exact f16
// numbers); the sums of a lane's two columns then carry 2^-16 and 2^-15, which the fold undoes.
//
// One CTA owns 128 weight columns (the MMA's M dimension) x a tile of up to 128 activation rows (the
// MMA's N dimension) over the whole depth, walked in 64-deep stages.  Roles (640 threads):
//   warp 16 (rows)      one TMA tile load per stage of the activation codes (tensor map, 128-byte
//                       swizzle, rows past m read as zero).
//   warp 18 (weights)   the packed units of the CTA's 8 column groups, 512 depths per bulk copy.
//   warps 0-7 (expand)  four pairs taking the stages in turn, a warp four column groups of its
//                       stage: 2-bit codes through a byte-permute lookup of the offset codebook,
//                       sign bits as they are, widened to 16 bits and written as the K-major,
//                       128-byte-swizzled operand.
//   warp 17 (MMA)       one elected thread issues the stage's four K = 16 instructions.  A run's
//                       steps accumulate into one of a ring of accumulators in tensor memory
//                       (512 columns / row tile); the run's last step commits it to the fold warps.
//   warp 19 (scales)    per K-block the operands of the fold -- the rows' activation scales and code
//                       sums, the column groups' scale rows -- into a small ring, so that no fold
//                       warp ever waits for a global load.
//   warps 8-15 (fold)   thread = weight column: read a finished run per row (tcgen05.ld), release
//                       the accumulator, and at the end of a K-block fold the block's integer into
//                       the running f32 total with the block's scale (K-blocks of one run: without
//                       leaving floating point, the integer being exact there; 128-row tiles: totals
//                       in tensor memory); after the last block the epilogue graph runs on the
//                       f16-rounded product and C is stored.
// Every wait is bounded; a timed-out wait raises the status word and the kernel drains and exits.
#include "epilogue.cuh"
#include "kernels.h"
#include "layout.h"
#include "tc_common.cuh"

namespace smeg {
namespace {

constexpr int kLtThreads = 32 * 20;
constexpr int kLtStage = 64;                     // depths per stage (one 128-byte swizzle row of f16)
constexpr int kLtATile = 128 * 128;              // expanded weights of a stage: 16 KB
constexpr int kLtNA = 6, kLtNB = 6, kLtNK = 3;   // ring depths: operand, rows, packed
constexpr int kLtSlotStages = 8;                 // stages of one packed-ring slot (512 depths)
constexpr int kLtNF = 8;                         // ring depth of the fold operands (K-blocks)
constexpr int kLtRun = 256;                      // most depths summed in one accumulator

__device__ __forceinline__ uint32_t prmt2(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}
// Four bytes -> four 16-bit values with zero high bytes (f16 bit patterns u * 2^-24).
__device__ __forceinline__ uint2 widen4(uint32_t v) { return make_uint2(prmt2(v, 0u, 0x4140u), prmt2(v, 0u, 0x4342u)); }
// (tcgen05.ld / tcgen05.st are whole-warp instructions: never under a condition that differs between lanes)
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&r)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr));
}
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&r)[8]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                 : "memory");
}
// 32 consecutive columns of the warp's lanes in one instruction
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr));
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
                 : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// TPW = rows one fold warp takes (16 or 32), DW = fold warps per lane quarter (1 or 2): the row
// tile of a CTA is TPW * DW rows.
// FAST: K-blocks of one run (256 depths or fewer) and no debug output -- the fold stays in floating point.
// FAST == 2 (TPW 32, DW 2): a tile of 128 rows, so that the weights are expanded half as often; a fold warp then takes
// 32 rows of either 64-row half, and the running totals live in tensor memory (columns 384..511: lane = weight column,
// column = row) beside three accumulators instead of in registers.
template <int BITS, int TPW, int DW, int FAST>
__global__ void __launch_bounds__(kLtThreads, 1) lowbit_tc_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ LowbitTcArgs p) {
    constexpr int NT = FAST == 2 ? 128 : TPW * DW;             // rows per CTA tile
    constexpr int ACC_STRIDE = NT < 32 ? 32 : NT;              // tensor-memory columns between accumulators
    constexpr int NACC = FAST == 2 ? 3 : 512 / ACC_STRIDE;
    constexpr int TOT_COL = 384;                               // FAST == 2: first column of the running totals
    constexpr int NA = FAST == 2 ? 5 : kLtNA, NB = NA;         // ring depths: operand, rows (both tiles are 16 KB at 128 rows)
    constexpr int UPS = BITS == 2 ? 4 : 2;                     // packed units per slot and column group (512 depths)
    constexpr int SPU = BITS == 2 ? 2 : 4;                     // stages per unit
    constexpr int KSLOT = 8 * UPS * kUnitBytes;                // bytes of a packed slot
    constexpr int BTILE = NT * 128;
    extern __shared__ unsigned char smem_dyn[];
    unsigned char* smem_raw = smem_dyn + ((1024u - (smem_u32(smem_dyn) & 1023u)) & 1023u);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    unsigned char* ring_a = smem_raw;                                          // [NA][16 KB]
    unsigned char* ring_b = ring_a + (size_t)NA * kLtATile;                 // [NB][BTILE], tiles 1024-byte aligned
    constexpr int BSLOT = (BTILE + 1023) / 1024 * 1024;
    unsigned char* ring_k = ring_b + (size_t)NB * BSLOT;                    // [NK][KSLOT]
    uint64_t* bars = reinterpret_cast<uint64_t*>(ring_k + (size_t)kLtNK * KSLOT);
    uint64_t* a_full = bars;                      // [NA] operand written (the stage's two expand warps)
    uint64_t* a_empty = a_full + NA;           // [NA] the stage's MMAs retired
    uint64_t* b_full = a_empty + NA;           // [NB] row tile landed
    uint64_t* b_empty = b_full + NB;           // [NB] the stage's MMAs retired
    uint64_t* k_full = b_empty + NB;           // [NK] packed units landed
    uint64_t* k_empty = k_full + kLtNK;           // [NK] every stage of the slot has been expanded
    uint64_t* acc_full = k_empty + kLtNK;         // [NACC] a K-block's sums are complete
    uint64_t* acc_empty = acc_full + NACC;        // [NACC] ... and read by every fold warp
    uint64_t* f_full = acc_empty + NACC;          // [NF] fold operands of a K-block landed
    uint64_t* f_empty = f_full + kLtNF;           // [NF] ... and read by every fold warp
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(f_empty + kLtNF);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    // fold-operand ring: per K-block [NT f32 activation scales][NT i32 code sums][8 column groups x 16 f16 scales]
    constexpr int FSLOT = NT * 8 + 256;
    unsigned char* ring_f = reinterpret_cast<unsigned char*>(bars) + 1024;

    const int col0 = blockIdx.x * 128, cg0 = blockIdx.x * 8;
    const int tok0 = blockIdx.y * NT;
    const int block = 1 << p.log2_block;
    const int log2_run = min(p.log2_block, 8);                 // an accumulator sums a run of min(block, 256) depths
    const int run = 1 << log2_run;
    // depths that belong to a real K-block and are staged (>= k: what lies past k multiplies zero activations)
    const int k_end = (int)min((long long)p.nb_real << p.log2_block, (long long)p.kq);
    const int stages = (k_end + kLtStage - 1) / kLtStage;
    const int slots = (stages + kLtSlotStages - 1) / kLtSlotStages;

    if (tid == 0) {
        for (int s = 0; s < NA; ++s) { mbar_init(&a_full[s], 2); mbar_init(&a_empty[s], 1); }
        for (int s = 0; s < NB; ++s) { mbar_init(&b_full[s], 1); mbar_init(&b_empty[s], 1); }
        for (int s = 0; s < kLtNK; ++s) { mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 2 * kLtSlotStages); }
        for (int s = 0; s < NACC; ++s) { mbar_init(&acc_full[s], 1); mbar_init(&acc_empty[s], 4 * DW); }
        for (int s = 0; s < kLtNF; ++s) { mbar_init(&f_full[s], 1); mbar_init(&f_empty[s], 4 * DW); }
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 17) {
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
    }
    if (warp == 16 && lane == 0) tma_prefetch_desc(&tmap_q);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 16) {
        // ===================== row producer =====================
        if (lane == 0) {
            for (int i = 0; i < stages; ++i) {
                const int slot = i % NB;
                if (i >= NB && !mbar_wait_poll(&b_empty[slot], ((i / NB) - 1) & 1, abort_flag, p.status, STATUS_TMEM_TIMEOUT)) break;
                mbar_expect_tx(&b_full[slot], (unsigned)BTILE);
                tma_load_2d(ring_b + (size_t)slot * BSLOT, &tmap_q, i * kLtStage, tok0, &b_full[slot]);   // x in f16 elements
            }
        }
    } else if (warp == 18) {
        // ===================== packed-weight producer: lane c = column group c of the CTA =====================
        for (int gq = 0; gq < slots; ++gq) {
            const int slot = gq % kLtNK;
            if (gq >= kLtNK && !__all_sync(0xffffffffu, mbar_wait_poll(&k_empty[slot], ((gq / kLtNK) - 1) & 1, abort_flag, p.status, STATUS_TMEM_TIMEOUT))) break;
            const int u0 = gq * UPS;
            const int units = min(UPS, p.ku - u0);
            if (lane == 0) mbar_expect_tx(&k_full[slot], (unsigned)(8 * units * kUnitBytes));
            __syncwarp();
            if (lane < 8) {
                const size_t cgi = (size_t)min(cg0 + lane, p.n16 - 1);         // a tail group re-reads the last one
                bulk_g2s(ring_k + (size_t)slot * KSLOT + (size_t)lane * UPS * kUnitBytes,
                         p.codes + (cgi * p.ku + (size_t)u0) * kUnitBytes, units * kUnitBytes, &k_full[slot]);
            }
            __syncwarp();
        }
    } else if (warp == 19) {
        // ===================== fold-operand producer: lane 0 the rows' scales, lane 1 their code sums, lanes 2-9 a column group's scale row =====================
        for (int blk = 0; blk < p.nb_real; ++blk) {
            const int fs = blk % kLtNF;
            if (blk >= kLtNF && !__all_sync(0xffffffffu, mbar_wait_poll(&f_empty[fs], ((blk / kLtNF) - 1) & 1, abort_flag, p.status, STATUS_TMEM_TIMEOUT))) break;
            unsigned char* dst = ring_f + (size_t)fs * FSLOT;
            if (lane == 0) mbar_expect_tx(&f_full[fs], (unsigned)(NT * 8 + 8 * 32));
            __syncwarp();
            if (lane == 0) bulk_g2s(dst, p.sa_t + (size_t)blk * p.mpad + tok0, NT * 4, &f_full[fs]);
            else if (lane == 1) bulk_g2s(dst + NT * 4, p.qsum_t + (size_t)blk * p.mpad + tok0, NT * 4, &f_full[fs]);
            else if (lane >= 2 && lane < 10) {
                const size_t cgi = (size_t)min(cg0 + lane - 2, p.n16 - 1);
                bulk_g2s(dst + NT * 8 + (lane - 2) * 32, p.scales + (cgi * p.nb + (size_t)blk) * 16, 32, &f_full[fs]);
            }
            __syncwarp();
        }
    } else if (warp == 17) {
        // ===================== MMA issuer =====================
        const uint32_t idesc = umma_idesc(0, 128, NT);
        for (int i = 0; i < stages; ++i) {
            const int as = i % NA, bs = i % NB;
            if (!__all_sync(0xffffffffu, mbar_wait_poll(&b_full[bs], (i / NB) & 1, abort_flag, p.status, STATUS_TMEM_TIMEOUT))) break;
            if (!__all_sync(0xffffffffu, mbar_wait_poll(&a_full[as], (i / NA) & 1, abort_flag, p.status, STATUS_TMEM_TIMEOUT))) break;
            tc_fence_after();
            const uint64_t a_desc0 = umma_desc_sw128(smem_u32(ring_a + (size_t)as * kLtATile));
            const uint64_t b_desc0 = umma_desc_sw128(smem_u32(ring_b + (size_t)bs * BSLOT));
            // the runs that begin in this stage take the next accumulators of the ring once the fold warps have read
            // their last use: wait for those first, then issue the whole stage from one thread
            bool ok = true;
#pragma unroll
            for (int ks = 0; ks < kLtStage / 16; ++ks) {
                const int depth = i * kLtStage + 16 * ks;
                const int ri = depth >> log2_run;
                if (depth < k_end && (depth & (run - 1)) == 0 && ri >= NACC && ok)
                    ok = __all_sync(0xffffffffu, mbar_wait_poll(&acc_empty[ri % NACC], ((ri / NACC) - 1) & 1, abort_flag, p.status, STATUS_TMEM_TIMEOUT));
            }
            if (!ok) break;
            tc_fence_after();
            if (elect_one()) {
#pragma unroll
                for (int ks = 0; ks < kLtStage / 16; ++ks) {
                    const int depth = i * kLtStage + 16 * ks;
                    if (depth >= k_end) break;                             // padding past the last real K-block
                    const int buf = (depth >> log2_run) % NACC;             // the accumulator of the depth's run
                    const bool first = (depth & (run - 1)) == 0;
                    const bool last = ((depth + 16) & (run - 1)) == 0 || depth + 16 >= k_end;
                    umma_f16(tmem_base + (uint32_t)(buf * ACC_STRIDE), a_desc0 + 2 * ks, b_desc0 + 2 * ks, idesc, first ? 0u : 1u);
                    if (last) umma_commit(&acc_full[buf]);
                }
                umma_commit(&a_empty[as]);
                umma_commit(&b_empty[bs]);
            }
            __syncwarp();
        }
    } else if (warp < 8) {
        // ===================== expand warps: four pairs of warps take the stages in turn =====================
        // A warp's trip through one stage (waits, loads, expansion, stores, fence, arrival) is a chain of
        // latencies several hundred cycles long however little it computes, so a stage is not spread over
        // all eight warps: pair (stage % 4) expands it, each warp four column groups with independent
        // instruction chains, and four stages are in flight at once.
        const int g = lane >> 2, t = lane & 3;
        const int pair = warp >> 1, half = warp & 1;
        for (int i = pair; i < stages; i += 4) {
            const int gq = i / kLtSlotStages, si = i % kLtSlotStages, ks_slot = gq % kLtNK, as = i % NA;
            if (i >= NA && !__all_sync(0xffffffffu, mbar_wait_poll(&a_empty[as], ((i / NA) - 1) & 1, abort_flag, p.status, STATUS_TMEM_TIMEOUT))) break;
            if (!__all_sync(0xffffffffu, mbar_wait_poll(&k_full[ks_slot], (gq / kLtNK) & 1, abort_flag, p.status, STATUS_TMEM_TIMEOUT))) break;
            unsigned char* at = ring_a + (size_t)as * kLtATile;
            const int h = si % SPU;                                            // 64-deep part of the unit
            const unsigned char* pk = ring_k + (size_t)ks_slot * KSLOT + (si / SPU) * kUnitBytes + lane * 16;
            uint4 wv[4];
#pragma unroll
            for (int cc = 0; cc < 4; ++cc) wv[cc] = *reinterpret_cast<const uint4*>(pk + (size_t)(4 * half + cc) * UPS * kUnitBytes);
#pragma unroll
            for (int cc = 0; cc < 4; ++cc) {
                const int row_lo = 16 * (4 * half + cc) + g, row_hi = row_lo + 8;
                // 8 depths (16 bytes) of a 32-deep step land in chunk 4 * step + t of the row
                const uint32_t off_lo = (uint32_t)((row_lo >> 3) * 1024 + (row_lo & 7) * 128);
                const uint32_t off_hi = (uint32_t)((row_hi >> 3) * 1024 + (row_hi & 7) * 128);
                const uint32_t sw_lo = (uint32_t)(row_lo & 7), sw_hi = (uint32_t)(row_hi & 7);
                // 2-bit: words 2 h, 2 h + 1 (32 depths each); 1-bit: word h (its two 4-bit halves are the two steps)
                const uint32_t w0 = BITS == 2 ? (h ? wv[cc].z : wv[cc].x) : (h == 0 ? wv[cc].x : (h == 1 ? wv[cc].y : (h == 2 ? wv[cc].z : wv[cc].w)));
                const uint32_t w1 = h ? wv[cc].w : wv[cc].y;
#pragma unroll
                for (int s = 0; s < 2; ++s) {
                    // 32-deep step s of the stage: depths 8 t .. 8 t + 7 of columns g (lo) and g + 8 (hi)
                    uint32_t lo03 = 0, lo47 = 0, hi03 = 0, hi47 = 0;           // 2-bit: four bytes each: u of depths +0..3 / +4..7
                    if (BITS == 2) {
                        const uint32_t w = s ? w1 : w0;
                        const uint32_t e = w & 0x33333333u, o = (w >> 2) & 0x33333333u;
                        lo03 = prmt2(p.lut, 0u, e); lo47 = prmt2(p.lut, 0u, e >> 16);
                        hi03 = prmt2(p.lut, 0u, o); hi47 = prmt2(p.lut, 0u, o >> 16);
                    }
                    const uint32_t chunk = (uint32_t)(4 * s + t);
                    if (BITS == 1) {
                        // A sign bit stays where it lies in its half word: bit b of an f16 is the number 2^(b-24) for
                        // b < 12, and act_quant_kernel has left the codes of a run of eight depths in the order
                        // 0 2 1 3 4 6 5 7, scaled by 2^8 2^8 1 1 2^6 2^6 2^-2 2^-2: every product of column g is
                        // u q 2^-16 and of column g + 8 (one bit higher) u q 2^-15.  One AND per register.
                        const uint32_t v = w0 >> (4 * s);
                        *reinterpret_cast<uint4*>(at + off_lo + ((chunk ^ sw_lo) << 4)) =
                            make_uint4(v & 0x00010001u, v & 0x01000100u, v & 0x00040004u, v & 0x04000400u);
                        *reinterpret_cast<uint4*>(at + off_hi + ((chunk ^ sw_hi) << 4)) =
                            make_uint4(v & 0x00020002u, v & 0x02000200u, v & 0x00080008u, v & 0x08000800u);
                        continue;
                    }
                    const uint2 l0 = widen4(lo03), l1 = widen4(lo47), h0 = widen4(hi03), h1 = widen4(hi47);
                    *reinterpret_cast<uint4*>(at + off_lo + ((chunk ^ sw_lo) << 4)) = make_uint4(l0.x, l0.y, l1.x, l1.y);
                    *reinterpret_cast<uint4*>(at + off_hi + ((chunk ^ sw_hi) << 4)) = make_uint4(h0.x, h0.y, h1.x, h1.y);
                }
            }
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&a_full[as]);
                mbar_arrive(&k_empty[ks_slot]);        // one arrival per warp and stage: a full slot collects 16
            }
        }
    } else if (warp < 16) {
        // ===================== fold warps: thread = weight column, registers = rows =====================
        const int dw = warp - 8, q = dw & 3, part = dw >> 2;
        if (part < DW) {
            const int cl = 32 * q + lane;                                   // column within the CTA tile
            const int col = col0 + cl;
            const uint32_t lane_base = tmem_base + ((uint32_t)(32 * q) << 16) + (uint32_t)(part * TPW);
            const int row0 = tok0 + part * TPW;                             // first activation row of this warp
            const int sc_off = NT * 8 + (cl >> 4) * 32 + scale_slot(cl & 15) * 2;   // this column's scale inside a fold slot
            // what turns an accumulator into S = sum u q: 2-bit sums are scaled by 2^-24, 1-bit by 2^-16 (columns g of a
            // column group) or 2^-15 (columns g + 8)
            const float unscale = BITS == 2 ? 16777216.0f : ((cl & 8) ? 32768.0f : 65536.0f);
            if (FAST == 2) {
                // ---- 128 rows: rows 32 part .. 32 part + 31 of either 64-row half, totals in tensor memory ----
                const uint32_t acc_base = tmem_base + ((uint32_t)(32 * q) << 16);
                const uint32_t tot_base = acc_base + (uint32_t)TOT_COL;
                {
                    const uint32_t z[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
#pragma unroll
                    for (int pass = 0; pass < 2; ++pass)
#pragma unroll
                        for (int j0 = 0; j0 < 32; j0 += 8) tmem_st8(tot_base + (uint32_t)(64 * pass + 32 * part + j0), z);
                    tmem_st_wait();
                }
                bool ok = true;
                for (int blk = 0; blk < p.nb_real && ok; ++blk) {              // one run per block: run counter = blk
                    const int fs = blk % kLtNF, buf = blk % NACC;
                    ok = mbar_wait_poll(&acc_full[buf], (blk / NACC) & 1, abort_flag, p.status, STATUS_TMEM_TIMEOUT);
                    if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
                    ok = mbar_wait_poll(&f_full[fs], (blk / kLtNF) & 1, abort_flag, p.status, STATUS_TMEM_TIMEOUT);
                    if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
                    tc_fence_after();
                    const unsigned char* fo = ring_f + (size_t)fs * FSLOT;
                    const float scale = __half2float(__ushort_as_half(*reinterpret_cast<const uint16_t*>(fo + sc_off)));
#pragma unroll
                    for (int pass = 0; pass < 2; ++pass) {
                        const int ro = 64 * pass + 32 * part;                  // first row of this pass within the tile
                        const float* sa = reinterpret_cast<const float*>(fo) + ro;
                        const float* qf = reinterpret_cast<const float*>(fo + NT * 4) + ro;
#pragma unroll
                        for (int hf = 0; hf < 2; ++hf) {
                            // sixteen accumulator values and their totals: two loads in flight, one wait
                            uint32_t av[16], tt[16];
                            if (pass == 0 && hf == 0) tmem_st_wait();              // the totals stored in the block before
                            tmem_ld16(acc_base + (uint32_t)(buf * ACC_STRIDE + ro + 16 * hf), av);
                            tmem_ld16(tot_base + (uint32_t)(ro + 16 * hf), tt);
                            tmem_ld_wait();
                            if (pass == 1 && hf == 1) {
                                // the accumulator has been read: hand it back to the MMA warp
                                tc_fence_before();
                                __syncwarp();
                                if (lane == 0) mbar_arrive(&acc_empty[buf]);
                            }
#pragma unroll
                            for (int j0 = 0; j0 < 16; j0 += 4) {
                                const float4 s0 = *reinterpret_cast<const float4*>(sa + 16 * hf + j0);
                                const float4 q0 = *reinterpret_cast<const float4*>(qf + 16 * hf + j0);
                                const float sv[4] = {s0.x, s0.y, s0.z, s0.w};
                                const float qv[4] = {q0.x, q0.y, q0.z, q0.w};
#pragma unroll
                                for (int j = 0; j < 4; ++j) {
                                    const float a = __uint_as_float(av[j0 + j]);
                                    const float sumf = BITS == 1 ? fmaf(a, 2.0f * unscale, -qv[j]) : fmaf(a, unscale, __fmul_rn(qv[j], -128.0f));
                                    tt[j0 + j] = __float_as_uint(fmaf(sumf, __fmul_rn(scale, sv[j]), __uint_as_float(tt[j0 + j])));
                                }
                            }
                            tmem_st16(tot_base + (uint32_t)(ro + 16 * hf), tt);
                        }
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&f_empty[fs]);
                }
                tmem_st_wait();
                if (ok) {                                                      // (warp-uniform: the tensor-memory loads take whole warps)
#pragma unroll
                    for (int pass = 0; pass < 2; ++pass)
#pragma unroll
                        for (int j0 = 0; j0 < 32; j0 += 8) {
                            uint32_t tt[8];
                            tmem_ld8(tot_base + (uint32_t)(64 * pass + 32 * part + j0), tt);
                            tmem_ld_wait();
#pragma unroll
                            for (int j = 0; j < 8; ++j) {
                                const int row = tok0 + 64 * pass + 32 * part + j0 + j;
                                if (row < p.m && col < p.n)
                                    p.c[(size_t)row * p.n + col] = ep_store_value<0>(p.ep, __uint_as_float(tt[j]), (size_t)row, (size_t)col);
                            }
                        }
                }
            } else {
            float tot[TPW];
#pragma unroll
            for (int j = 0; j < TPW; ++j) tot[j] = 0.0f;
            bool ok = true;
            const int rpb = block >> log2_run;                              // runs per K-block
            int ri = 0;                                                     // run counter
            for (int blk = 0; blk < p.nb_real && ok; ++blk) {
                const int fs = blk % kLtNF;
                if (FAST) {
                    // One run per block: the accumulator holds S / unscale exactly, so the block's integer sum as a
                    // float -- what (float)sum is -- comes from one exact fused multiply-add, without the two
                    // conversions: 2 S - sum(q) = fma(acc, 2 unscale, -sum(q)); S - 128 sum(q) = fma(acc, unscale, -128 sum(q)).
                    const int buf = ri % NACC;
                    ok = mbar_wait_poll(&acc_full[buf], (ri / NACC) & 1, abort_flag, p.status, STATUS_TMEM_TIMEOUT);
                    if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
                    tc_fence_after();
                    uint32_t av[TPW];                                          // every load in flight before the one wait
                    if constexpr (TPW == 32) {
                        tmem_ld32(lane_base + (uint32_t)(buf * ACC_STRIDE), av);
                    } else {
#pragma unroll
                        for (int j0 = 0; j0 < TPW; j0 += 8) {
                            uint32_t r[8];
                            tmem_ld8(lane_base + (uint32_t)(buf * ACC_STRIDE + j0), r);
#pragma unroll
                            for (int j = 0; j < 8; ++j) av[j0 + j] = r[j];
                        }
                    }
                    tmem_ld_wait();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&acc_empty[buf]);
                    ++ri;
                    ok = mbar_wait_poll(&f_full[fs], (blk / kLtNF) & 1, abort_flag, p.status, STATUS_TMEM_TIMEOUT);
                    if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
                    const unsigned char* fo = ring_f + (size_t)fs * FSLOT;
                    const float scale = __half2float(__ushort_as_half(*reinterpret_cast<const uint16_t*>(fo + sc_off)));
                    const float* sa = reinterpret_cast<const float*>(fo) + part * TPW;
                    const float* qf = reinterpret_cast<const float*>(fo + NT * 4) + part * TPW;
#pragma unroll
                    for (int j0 = 0; j0 < TPW; j0 += 4) {
                        const float4 s0 = *reinterpret_cast<const float4*>(sa + j0);
                        const float4 q0 = *reinterpret_cast<const float4*>(qf + j0);
                        const float sv[4] = {s0.x, s0.y, s0.z, s0.w};
                        const float qv[4] = {q0.x, q0.y, q0.z, q0.w};
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const float a = __uint_as_float(av[j0 + j]);
                            const float sumf = BITS == 1 ? fmaf(a, 2.0f * unscale, -qv[j]) : fmaf(a, unscale, __fmul_rn(qv[j], -128.0f));
                            tot[j0 + j] = fmaf(sumf, __fmul_rn(scale, sv[j]), tot[j0 + j]);
                        }
                    }
                } else {
                int sblk[TPW];                                              // the block's integer sums
#pragma unroll
                for (int j = 0; j < TPW; ++j) sblk[j] = 0;
                // runs of this block that hold staged depths
                const int runs = min(rpb, (k_end - (blk << p.log2_block) + run - 1) >> log2_run);
                for (int rr = 0; rr < runs; ++rr, ++ri) {
                    const int buf = ri % NACC;
                    ok = mbar_wait_poll(&acc_full[buf], (ri / NACC) & 1, abort_flag, p.status, STATUS_TMEM_TIMEOUT);
                    if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
                    tc_fence_after();
#pragma unroll
                    for (int j0 = 0; j0 < TPW; j0 += 8) {
                        uint32_t r[8];
                        tmem_ld8(lane_base + (uint32_t)(buf * ACC_STRIDE + j0), r);
                        tmem_ld_wait();
                        // the accumulator holds (sum of u * q) / unscale exactly
#pragma unroll
                        for (int j = 0; j < 8; ++j) sblk[j0 + j] += __float2int_rn(__uint_as_float(r[j]) * unscale);
                    }
                    // the accumulator is in registers: hand it back to the MMA warp
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&acc_empty[buf]);
                }
                if (!ok) break;
                ok = mbar_wait_poll(&f_full[fs], (blk / kLtNF) & 1, abort_flag, p.status, STATUS_TMEM_TIMEOUT);
                if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
                const unsigned char* fo = ring_f + (size_t)fs * FSLOT;
                const float scale = __half2float(__ushort_as_half(*reinterpret_cast<const uint16_t*>(fo + sc_off)));
                const float* sa = reinterpret_cast<const float*>(fo) + part * TPW;
                const float* qs = reinterpret_cast<const float*>(fo + NT * 4) + part * TPW;
#pragma unroll
                for (int j0 = 0; j0 < TPW; j0 += 4) {
                    const float4 s0 = *reinterpret_cast<const float4*>(sa + j0);
                    const float4 q0 = *reinterpret_cast<const float4*>(qs + j0);
                    const float sv[4] = {s0.x, s0.y, s0.z, s0.w};
                    const int qv[4] = {__float2int_rn(q0.x), __float2int_rn(q0.y), __float2int_rn(q0.z), __float2int_rn(q0.w)};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        // 1-bit: u is the sign bit, value = 2 u - 1; 2-bit: u = value + 128
                        const int sum = BITS == 1 ? 2 * sblk[j0 + j] - qv[j] : sblk[j0 + j] - 128 * qv[j];
                        if (p.sums_out && col < p.n && row0 + j0 + j < p.m)
                            p.sums_out[((size_t)(row0 + j0 + j) * p.n + col) * p.nb_real + blk] = sum;
                        tot[j0 + j] = fmaf((float)sum, __fmul_rn(scale, sv[j]), tot[j0 + j]);
                    }
                }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&f_empty[fs]);
            }
            if (ok && col < p.n) {
#pragma unroll
                for (int j = 0; j < TPW; ++j) {
                    const int row = row0 + j;
                    if (row < p.m) p.c[(size_t)row * p.n + col] = ep_store_value<0>(p.ep, tot[j], (size_t)row, (size_t)col);
                }
            }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 17) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

template <int BITS, int TPW, int DW, int FAST>
cudaError_t launch_lt(const CUtensorMap& tm, const LowbitTcArgs& a, dim3 grid, size_t smem, cudaStream_t stream) {
    auto kern = lowbit_tc_kernel<BITS, TPW, DW, FAST>;
    static int attr_dev = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (attr_dev != dev) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (e != cudaSuccess) return e;
        attr_dev = dev;
    }
    kern<<<grid, kLtThreads, smem, stream>>>(tm, a);
    return cudaGetLastError();
}

}  // namespace

bool lowbit_tc_supported(int bits, int m, int k, int log2_block) {
    if (bits != 1 && bits != 2) return false;
    if (m < 1 || k < 1 || log2_block < 4) return false;           // an MMA step is 16 deep: K-blocks of 16 and up
    if (log2_block > 16) return false;                             // a block's sum of activation codes travels as a float
    return tensor_map_encoder() != nullptr;
}

// an MMA of 128 weight columns takes 16 rows or more
int lowbit_tc_row_tile(int m) { return m <= 16 ? 16 : (m <= 32 ? 32 : 64); }
// ... and 128 rows where the floating-point fold applies, the rows fill more than one 64-row tile and at most one
// K-block begins per 64-deep stage: the MMA warp takes the accumulators of every run that begins in a stage before it
// issues the stage, and the 128-row form has a ring of three (smaller blocks would wait for their own stage)
static int lt_row_tile(int m, int fast, int log2_block) { return fast && m > 64 && log2_block >= 6 ? 128 : lowbit_tc_row_tile(m); }

cudaError_t lowbit_tc_launch(LowbitTcArgs a, cudaStream_t stream) {
    // blocks of one run and no debug output: the floating-point fold
    const int fast = a.log2_block <= 8 && a.sums_out == nullptr ? 1 : 0;
    const int nt = lt_row_tile(a.m, fast, a.log2_block);
    const int nab = nt == 128 ? 5 : kLtNA;                         // ring depths of the kernel's NA, NB
    CUtensorMap tm;
    const cuuint64_t gdim[2] = {(cuuint64_t)a.kq, (cuuint64_t)a.m};
    const cuuint64_t gstride[1] = {(cuuint64_t)a.kq * 2};
    const cuuint32_t box[2] = {(cuuint32_t)kLtStage, (cuuint32_t)nt};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = tensor_map_encoder()(&tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (void*)a.qh, gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                      CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
    const int ups = a.bits == 2 ? 4 : 2;
    const int bslot = (nt * 128 + 1023) / 1024 * 1024;
    const size_t smem = 1024 + (size_t)nab * kLtATile + (size_t)nab * bslot + (size_t)kLtNK * 8 * ups * kUnitBytes +
                        1024 + (size_t)kLtNF * (nt * 8 + 256) + 64;
    const dim3 grid((a.n + 127) / 128, (a.m + nt - 1) / nt);
#define SMEG_LT(B, F)                                                                  \
    if (a.bits == B && fast == F) {                                                    \
        if (nt == 16) return launch_lt<B, 16, 1, F>(tm, a, grid, smem, stream);        \
        if (nt == 32) return launch_lt<B, 16, 2, F>(tm, a, grid, smem, stream);        \
        if (nt == 128) return launch_lt<B, 32, 2, 2 * F>(tm, a, grid, smem, stream);   \
        return launch_lt<B, 32, 2, F>(tm, a, grid, smem, stream);                      \
    }
    SMEG_LT(2, 0) SMEG_LT(2, 1)
    SMEG_LT(1, 0) SMEG_LT(1, 1)
#undef SMEG_LT
    return cudaErrorInvalidValue;
}

}  // namespace smeg
