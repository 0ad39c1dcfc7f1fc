// Prefill GEMM for sm_100a:  C[m][n] = ep( A[m][k] @ dequant(W) ) for large m, on the
// 5th-generation tensor cores (tcgen05.mma, accumulators in tensor memory).
//
// Replaces the reference's MOPA paths -- unpack_q4_f16 / unpack_q4_bf16 +
// run_q4_panels (csrc/gemm_f16f16_q4.h:57-117, csrc/gemm_b16b16_q4.h:32-92), the
// 1-/2-bit unpack_q{1,2}_f16 + lowbit_panels (csrc/gemm_f16f16_lowbit.h:51-169) and
// the dense run_panels consumer (csrc/gemm_half.h:1093-1169).  As there, every
// weight is rounded ONCE to the 16-bit operand type exactly as the eager dequant
// rounds it (dequant_rows, src/kernels/q4/weights.rs:232-259; Codes::dequant,
// src/kernels/lowbit/matmul.rs:178-197) and the dense product accumulates in f32.
//
// One CTA owns 128 weight columns (the MMA's M dimension) x a tile of up to 512
// tokens (the MMA's N dimension, one or two instructions of N <= 256), over the
// whole depth.  Per 64-deep stage:
//   warp 4 (producer)   TMA: the token tile (tensor map, 128-byte swizzle) and this
//                       CTA's 4 KB of packed weight units + their scales (bulk copies)
//   warps 0-3 (dequant) expand the packed units into the K-major, 128-byte-swizzled
//                       shared-memory operand: each lane turns its 16-byte vector
//                       into four 16-byte chunks of 8 consecutive depths
//   warp 5 (MMA)        one elected thread issues 4 (x1 or x2) tcgen05.mma of K = 16
//                       and commits the stage back to the producer
// After the last stage warps 0-3 drain the accumulators from tensor memory
// (thread = weight column, registers = tokens), run the epilogue graph on the
// rounded product and store C.  Every wait is bounded.
#include "epilogue.cuh"
#include "kernels.h"
#include "layout.h"
#include "tc_common.cuh"

namespace smeg {

namespace {

constexpr int kTcThreads = 192;
constexpr int kColsPerCta = 128;       // weight columns per CTA (UMMA M)
constexpr int kStageK = 64;            // depths per stage (one 128-byte swizzle row of 16-bit values)
constexpr int kWBytes = kColsPerCta * kStageK * 2;   // dequantised weight operand per stage: 16 KB

// WKIND: 4 = Q4 units, 2 = 2-bit units, 1 = 1-bit units, 16 = dense 16-bit weights (already K-major tiles)
template <int WKIND>
struct WSrc {
    static constexpr int unit_depth = WKIND == 4 ? 64 : (WKIND == 2 ? 128 : 256);
    // packed bytes of 128 columns x 64 depths
    static constexpr int stage_bytes = WKIND == 4 ? 4096 : (WKIND == 2 ? 2048 : 1024);
};

__device__ __forceinline__ uint32_t swz_off(int row, int chunk) {
    // byte offset of 16-byte chunk `chunk` (0..7) of row `row` in a 128B-swizzled K-major tile
    return (uint32_t)((row >> 3) * 1024 + (row & 7) * 128 + ((chunk ^ (row & 7)) << 4));
}

template <int BF16>
__device__ __forceinline__ uint4 scale_chunk(const __half2 (&c)[4], float s_f32, __half2 s_h2) {
    uint4 out;
    if (BF16) {
        uint32_t* o = reinterpret_cast<uint32_t*>(&out);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __half22float2(c[i]);
            __nv_bfloat162 v = __floats2bfloat162_rn(__fmul_rn(f.x, s_f32), __fmul_rn(f.y, s_f32));
            o[i] = *reinterpret_cast<uint32_t*>(&v);
        }
    } else {
        __half2* o = reinterpret_cast<__half2*>(&out);
#pragma unroll
        for (int i = 0; i < 4; ++i) o[i] = __hmul2(c[i], s_h2);
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

template <int BF16, int WKIND>
__global__ void __launch_bounds__(kTcThreads, 1) gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_tok, GemmTcArgs p) {
    extern __shared__ unsigned char smem_dyn[];
    // the swizzled operands need 1024-byte aligned tiles: align the window by hand
    unsigned char* smem_raw = smem_dyn + ((1024u - (smem_u32(smem_dyn) & 1023u)) & 1023u);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int NS = p.ns;
    const int tok_bytes = p.ntok_pad * 128;                    // token operand per stage
    constexpr int pk_bytes = WSrc<WKIND>::stage_bytes;         // packed weights per stage
    const int sc_rows = p.sc_rows;                             // scale rows (blocks) staged per stage
    const int sc_bytes = 8 * sc_rows * 32;                     // 8 column groups x rows x 16 halves
    const int stage_stride = kWBytes + tok_bytes + ((pk_bytes + sc_bytes + 1023) / 1024) * 1024;

    // carve-up: [stages: W operand | token operand | packed + scales] then barriers
    unsigned char* stages = smem_raw;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem_raw + (size_t)NS * stage_stride);
    uint64_t* full = bars;                 // packed weights + tokens landed
    uint64_t* deq = bars + NS;             // dequantised operand written (128 arrivals)
    uint64_t* empty = bars + 2 * NS;       // MMAs of the stage retired
    uint64_t* acc_full = bars + 3 * NS;    // all MMAs retired
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3 * NS + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    EpNodeDev* ep_nodes = reinterpret_cast<EpNodeDev*>(bars + 3 * NS + 4);

    const int cg0 = blockIdx.x * 8;                            // first 16-column group
    const int col0 = blockIdx.x * kColsPerCta;
    const int tok0 = blockIdx.y * p.ntok_tile;
    const int num_stages = (p.k + kStageK - 1) / kStageK;

    if (tid == 0) {
        for (int s = 0; s < NS; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&deq[s], 128);
            mbar_init(&empty[s], 1);
        }
        mbar_init(acc_full, 1);
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (tid < p.ep.n_nodes && p.ep.n_nodes <= kMaxInlineNodes) ep_nodes[tid] = p.ep.nodes[tid];
    if (warp == 5) {
        tmem_alloc(tmem_slot, p.tmem_cols);
        tmem_relinquish();
    }
    if (warp == 4 && lane == 0) tma_prefetch_desc(&tmap_tok);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 4) {
        // ===================== producer =====================
        if (lane == 0) {
            for (int st = 0; st < num_stages; ++st) {
                const int slot = st % NS;
                if (st >= NS && !mbar_wait(&empty[slot], ((st / NS) - 1) & 1, abort_flag, p.status, STATUS_TMEM_TIMEOUT)) break;
                unsigned char* sb = stages + (size_t)slot * stage_stride;
                const int d0 = st * kStageK;
                const int blk0 = d0 >> p.log2_block;
                const int blk1 = min(p.nb, ((d0 + kStageK - 1) >> p.log2_block) + 1);
                const int rows = blk1 - blk0;
                // packed units of this stage: for unit depths above 64 a unit spans several
                // stages and is copied as a whole by the stage that starts it
                constexpr int UD = WSrc<WKIND>::unit_depth;
                const bool copy_units = (d0 % UD) == 0;
                const unsigned pk = copy_units ? 8u * kUnitBytes : 0u;
                mbar_expect_tx(&full[slot], (unsigned)tok_bytes + pk + 8u * rows * 32u);
                // tokens: one or two boxes of ntok_box rows
                tma_load_2d(sb + kWBytes, &tmap_tok, d0, tok0, &full[slot]);
                if (p.nmma == 2) tma_load_2d(sb + kWBytes + tok_bytes / 2, &tmap_tok, d0, tok0 + p.ntok_box, &full[slot]);
                unsigned char* pkdst = sb + kWBytes + tok_bytes;
                for (int c = 0; c < 8; ++c) {
                    const size_t cgi = (size_t)min(cg0 + c, p.n16 - 1);     // clamp: tail groups re-read the last one
                    if (copy_units)
                        bulk_g2s(pkdst + c * kUnitBytes, p.codes + (cgi * p.ku + (size_t)(d0 / UD)) * kUnitBytes, kUnitBytes, &full[slot]);
                    bulk_g2s(pkdst + 8 * kUnitBytes + c * sc_rows * 32, p.scales + (cgi * p.nb + blk0) * 16, rows * 32, &full[slot]);
                }
            }
        }
    } else if (warp == 5) {
        // ===================== MMA issuer =====================
        if (lane == 0) {
            const uint32_t idesc = umma_idesc(BF16, kColsPerCta, p.ntok_box);
            for (int st = 0; st < num_stages; ++st) {
                const int slot = st % NS;
                const unsigned ph = (st / NS) & 1;
                if (!mbar_wait(&full[slot], ph, abort_flag, p.status, STATUS_TMEM_TIMEOUT)) break;
                if (!mbar_wait(&deq[slot], ph, abort_flag, p.status, STATUS_TMEM_TIMEOUT)) break;
                tc_fence_after();
                unsigned char* sb = stages + (size_t)slot * stage_stride;
                const uint64_t a_desc = umma_desc_sw128(smem_u32(sb));
                const uint64_t b_desc = umma_desc_sw128(smem_u32(sb + kWBytes));
#pragma unroll
                for (int ks = 0; ks < kStageK / 16; ++ks) {
                    const uint32_t accum = (st > 0 || ks > 0) ? 1u : 0u;
                    umma_f16(tmem_base, a_desc + 2 * ks, b_desc + 2 * ks, idesc, accum);
                    if (p.nmma == 2)
                        umma_f16(tmem_base + p.ntok_box, a_desc + 2 * ks, b_desc + (uint64_t)((tok_bytes / 2) >> 4) + 2 * ks, idesc, accum);
                }
                umma_commit(&empty[slot]);
            }
            umma_commit(acc_full);
        }
    } else {
        // ===================== dequant warps (0..3), then epilogue =====================
        const int g = lane >> 2, t = lane & 3;
        // this thread's packed vector: column groups 2*warp and 2*warp+1 of the CTA
        for (int st = 0; st < num_stages; ++st) {
            const int slot = st % NS;
            const unsigned ph = (st / NS) & 1;
            unsigned char* sb = stages + (size_t)slot * stage_stride;
            if (st >= NS) {
                // the dequantised operand of this slot is being read by MMAs until empty[] flips
                if (!mbar_wait(&empty[slot], ((st / NS) - 1) & 1, abort_flag, p.status, STATUS_TMEM_TIMEOUT)) break;
            }
            if (!mbar_wait(&full[slot], ph, abort_flag, p.status, STATUS_TMEM_TIMEOUT)) break;
            const int d0 = st * kStageK;
            const int blk0 = d0 >> p.log2_block;
            const unsigned char* pk = sb + kWBytes + tok_bytes;
            const uint16_t* scs = reinterpret_cast<const uint16_t*>(pk + 8 * kUnitBytes);
            if (WKIND == 4) {
#pragma unroll
                for (int cc = 0; cc < 2; ++cc) {
                    const int c = 2 * warp + cc;
                    const uint4 wv = *reinterpret_cast<const uint4*>(pk + c * kUnitBytes + lane * 16);
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
                    const int ra = ((d0 + 8 * t) >> p.log2_block) - blk0, rb = ((d0 + 32 + 8 * t) >> p.log2_block) - blk0;
                    const uint16_t* sc = scs + c * sc_rows * 16;
                    const __half s_lo_a = __ushort_as_half(sc[ra * 16 + 2 * g]), s_lo_b = __ushort_as_half(sc[rb * 16 + 2 * g]);
                    const __half s_hi_a = __ushort_as_half(sc[ra * 16 + 2 * g + 1]), s_hi_b = __ushort_as_half(sc[rb * 16 + 2 * g + 1]);
                    const int row_lo = 16 * c + g, row_hi = row_lo + 8;
                    // chunk order per store keeps the 8 lanes of a quarter warp on distinct banks
                    const int ca = (g & 1) ? 4 + t : t, cb = (g & 1) ? t : 4 + t;
                    const uint4 v_lo_a = scale_chunk<BF16>(lo_a, __half2float(s_lo_a), __half2half2(s_lo_a));
                    const uint4 v_lo_b = scale_chunk<BF16>(lo_b, __half2float(s_lo_b), __half2half2(s_lo_b));
                    const uint4 v_hi_a = scale_chunk<BF16>(hi_a, __half2float(s_hi_a), __half2half2(s_hi_a));
                    const uint4 v_hi_b = scale_chunk<BF16>(hi_b, __half2float(s_hi_b), __half2half2(s_hi_b));
                    *reinterpret_cast<uint4*>(sb + swz_off(row_lo, ca)) = (g & 1) ? v_lo_b : v_lo_a;
                    *reinterpret_cast<uint4*>(sb + swz_off(row_lo, cb)) = (g & 1) ? v_lo_a : v_lo_b;
                    *reinterpret_cast<uint4*>(sb + swz_off(row_hi, ca)) = (g & 1) ? v_hi_b : v_hi_a;
                    *reinterpret_cast<uint4*>(sb + swz_off(row_hi, cb)) = (g & 1) ? v_hi_a : v_hi_b;
                }
            }
            fence_proxy_async();
            mbar_arrive(&deq[slot]);
        }

        // ---- epilogue: thread = weight column (TMEM lane), registers = tokens ----
        mbar_wait(acc_full, 0, abort_flag, p.status, STATUS_TMEM_TIMEOUT);
        tc_fence_after();
        const int col = col0 + 32 * warp + lane;
        const uint32_t lane_base = tmem_base + ((uint32_t)(32 * warp) << 16);
        const EpNodeDev* nodes = p.ep.n_nodes <= kMaxInlineNodes ? ep_nodes : p.ep.ext;
        for (int j0 = 0; j0 < p.ntok_pad; j0 += 16) {
            uint32_t r[16];
            tmem_ld16(lane_base + (uint32_t)j0, r);
            tmem_ld_wait();
            if (num_stages == 0) {
#pragma unroll
                for (int j = 0; j < 16; ++j) r[j] = 0u;
            }
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const int tok = tok0 + j0 + j;
                if (tok < p.m && col < p.n) {
                    const float acc = __uint_as_float(r[j]);
                    if (p.c32) p.c32[(size_t)tok * p.n + col] = acc;
                    else p.c[(size_t)tok * p.n + col] = ep_store_nodes<BF16>(nodes, p.ep.n_nodes, acc, (size_t)tok, (size_t)col);
                }
            }
        }
        tc_fence_before();
    }
    __syncthreads();
    if (warp == 5) {
        tc_fence_after();
        tmem_dealloc(tmem_base, p.tmem_cols);
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)ptr;
    }
    return fn;
}

template <int BF16, int WKIND>
cudaError_t launch_tc(const CUtensorMap& tm, const GemmTcArgs& a, dim3 grid, size_t smem, cudaStream_t stream) {
    auto kern = gemm_tc_kernel<BF16, WKIND>;
    static int attr_dev = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (attr_dev != dev) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (e != cudaSuccess) return e;
        attr_dev = dev;
    }
    kern<<<grid, kTcThreads, smem, stream>>>(tm, a);
    return cudaGetLastError();
}

}  // namespace

bool gemm_tc_supported(int wkind, int m, int k, int log2_block, const void* a) {
    if (wkind != 4) return false;
    if (k % 8 != 0 || k == 0 || ((uintptr_t)a & 15) != 0) return false;   // TMA: 16-byte aligned rows
    if (log2_block < 3) return false;                                      // one scale per 8-depth chunk
    if (m < 1) return false;
    return encode_fn() != nullptr;
}

cudaError_t gemm_tc_launch(GemmTcArgs a, int bf16, int wkind, cudaStream_t stream) {
    // token tiling: equal tiles of at most 512 tokens, padded to the MMA's N granularity
    const int tiles = (a.m + 511) / 512;
    int tile = (a.m + tiles - 1) / tiles;
    int pad = tile > 256 ? (tile + 31) / 32 * 32 : (tile + 15) / 16 * 16;
    a.ntok_tile = pad;
    a.ntok_pad = pad;
    a.nmma = pad > 256 ? 2 : 1;
    a.ntok_box = pad / a.nmma;
    int cols = 32;
    while (cols < pad) cols *= 2;
    a.tmem_cols = cols;
    const int block = 1 << a.log2_block;
    a.sc_rows = block >= kStageK ? 1 : kStageK / block;
    const int pk_bytes = wkind == 4 ? 4096 : (wkind == 2 ? 2048 : 1024);
    const int stage_stride = kWBytes + pad * 128 + ((pk_bytes + 8 * a.sc_rows * 32 + 1023) / 1024) * 1024;
    int ns = (int)((220 * 1024 - 2048) / stage_stride);
    if (ns > 8) ns = 8;
    if (ns < 2) return cudaErrorInvalidConfiguration;
    a.ns = ns;
    const size_t smem = 1024 + (size_t)ns * stage_stride + (3 * ns + 4) * 8 + kMaxInlineNodes * sizeof(EpNodeDev) + 64;

    CUtensorMap tm;
    const cuuint64_t gdim[2] = {(cuuint64_t)a.k, (cuuint64_t)a.m};
    const cuuint64_t gstride[1] = {(cuuint64_t)a.k * 2};
    const cuuint32_t box[2] = {(cuuint32_t)kStageK, (cuuint32_t)a.ntok_box};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = encode_fn()(&tm, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (void*)a.a, gdim,
                             gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                             CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
    dim3 grid((a.n + kColsPerCta - 1) / kColsPerCta, tiles);
    if (bf16) return launch_tc<1, 4>(tm, a, grid, smem, stream);
    return launch_tc<0, 4>(tm, a, grid, smem, stream);
}

}  // namespace smeg
