// Internal launch interfaces between the C-ABI layer (api.cu) and the kernels.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include "epilogue.cuh"

namespace smeg {

// ---- Q4 GEMV (q4_gemv.cu) ----
struct Q4GemvArgs {
    const unsigned char* codes;   // packed units, [n16][k64][512 B]
    const uint16_t* scales;       // f16 bits, [n16][nb][16]
    const uint16_t* a;            // activations, row-major m x k (T bits)
    uint16_t* c;                  // output, row-major m x n (T bits)
    float* c32;                   // if set: raw f32 accumulators go here instead (no rounding, no epilogue)
    // direct kernel only -- the fused forms of the MLP block at decode size:
    int glu;                      // SMEG_ACT_SILU / _GELU: W is a gate/up matrix (32 gate columns, 32 up columns, ...) and c (m x n/2)
                                  // receives f16(act(f16(gate)) * f16(up)); a CTA then owns (gate group, up group) pairs
    float* yacc;                  // if set: y[m][n] += f32(f16(acc)) instead of storing c (the residual add)
    int m, n, k;
    int n16, k64, nb;             // column groups, 64-deep units, staged scale rows per group
    int log2_block;
    int ns, cg, rps, ka, a_rows;  // filled in by the launcher
    int dq, dr, dupw;             // direct kernel: column groups per CTA (quotient, remainder), units per warp
    int a_vec_ok;                 // rows of `a` are 16-byte aligned (k % 8 == 0 and base aligned)
    // streaming form (q4_gemv_stream_plan): the (column group, 16-unit stage) list is cut into one
    // contiguous range per CTA; a column group cut by a range boundary is summed through ws
    int sgrid;                    // CTAs of the streaming kernel; 0 = the column-group-per-CTA kernel runs
    int spc, stotal, spieces;     // stages per column group, stages in all, most CTAs one column group spans
    int sns, sslot, srps, supw;   // ring slots, bytes per slot, scale rows staged per slot, units per warp and stage
    float* ws;                    // [n16][spieces][8 * MT rows][16] partial sums of cut column groups
    int* counters;                // one per column group, zero between launches
    unsigned* status;
    EpParams ep;
};
// Chooses the streaming form when the call fits it (fills the s* fields; *ws_floats / *ncounters = the
// scratch the caller must provide in ws / counters).  Leaves sgrid = 0 otherwise.
void q4_gemv_stream_plan(Q4GemvArgs& a, int bf16, int sm_count, size_t* ws_floats, size_t* ncounters);
cudaError_t q4_gemv_launch(Q4GemvArgs a, int bf16, int sm_count, cudaStream_t stream);
// One to four rows, f16, K-blocks of 32 and up: plain 128-bit loads, packed f16 multiply-adds (gemv_direct.cu).
bool q4_direct_supported(const Q4GemvArgs& a, int bf16);
cudaError_t q4_direct_launch(Q4GemvArgs a, int sm_count, cudaStream_t stream);

// Launch with programmatic stream serialisation allowed: when the kernel ahead in the stream has let
// its dependents go (griddepcontrol.launch_dependents in every CTA, or its end), this kernel's CTAs
// may start while that one drains.  Every kernel launched this way executes griddepcontrol.wait
// (pdl_wait) in every thread before its first access to memory another kernel may have written, and
// before its first store; what it does earlier (barrier set-up, weight prefetch) overlaps the tail of
// its predecessor.  SMEG_PDL=0 launches plainly.
bool pdl_enabled();
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}

// ---- activation int8 quantisation + 2-bit / 1-bit GEMV (lowbit_gemv.cu) ----
struct ActQuantArgs {
    const uint16_t* a;    // m x k f16 bits
    int8_t* q;            // m x kq int8 (kq = k padded to the unit depth, pad = 0)
    float* sa;            // m x nbq per-block activation scales (amax / 127), padded blocks 0
    int32_t* qsum;        // m x nbq per-block sums of q (1-bit path only; may be null)
    int m, k, kq, nbq, log2_block;
    uint16_t* qh;         // optional: the codes as f16 integers, m x kq, for the tensor-core kernels
    int qh_perm;          // qh holds every run of 8 depths in the order 0 2 1 3 4 6 5 7 (B fragments of the mma kernel); 2: and scaled by 2^8 2^8 1 1 2^6 2^6 2^-2 2^-2 (its 1-bit form)
    float* sa_t;          // optional: the same scales as nbq x mpad (block-major), for the tensor-core kernel
    float* qsum_t;        // optional: the same sums as nbq x mpad floats (exact: |sum| <= 128 * block < 2^24)
    int mpad;
};
cudaError_t act_quant_launch(const ActQuantArgs& a, cudaStream_t stream);

struct LowbitGemvArgs {
    const unsigned char* codes;   // packed units [n16][ku][512 B]
    const uint16_t* scales;       // f16 bits [n16][nb][16]
    const uint16_t* a;            // m x k f16 activations: the kernel quantises them itself (else q / sa / qsum)
    int a_vec_ok;                 // rows of a are 16-byte aligned
    const int8_t* q;              // m x kq
    const float* sa;              // m x nb
    const int32_t* qsum;          // m x nb (1-bit; the mma kernel reads it for 2-bit weights too)
    const uint16_t* qh;           // mma kernel: the codes as f16, (m rounded up to 8) x kq with zero rows past m, runs of 8 depths in fragment order
    uint16_t* c;                  // m x n f16 bits
    int32_t* sums_out;            // optional debug: m x n x nb_real exact block sums
    int8_t* q_out;                // optional debug (with a): m x k int8 codes
    float* sa_out;                // optional debug (with a): m x nb_real activation scales
    int m, n, k, kq;
    int n16, ku, nb, nb_real;     // column groups, units along K, block rows staged / real
    int log2_block;
    uint32_t lut;                 // 2-bit codebook, byte c = value of code c
    int ns, gpt, kc, kqc;         // launcher-filled: ring depth, column groups per task, fold chunk, staged activation chunk
    int ntasks, rows_s, u_bytes;  // launcher-filled: tasks along n, rows kept in the shared sums, bytes of the sums / f16-rows region
    int dq, dr, dupw, dsc;        // direct kernel: column groups per CTA (quotient, remainder), units per warp, scales staged in shared memory
    unsigned* status;
    EpParams ep;
};
cudaError_t lowbit_gemv_launch(LowbitGemvArgs a, int bits, int sm_count, cudaStream_t stream);
bool lowbit_gemv_fuses_quant(LowbitGemvArgs a, int bits, int sm_count);
// One to four rows: plain 128-bit loads and dp4a (gemv_direct.cu).  fused: the kernel quantises the f16 rows
// itself (a.a set, at most two rows); otherwise a.q / a.sa / a.qsum come from act_quant_kernel.
bool lowbit_direct_supported(const LowbitGemvArgs& a, bool fused);
cudaError_t lowbit_direct_launch(LowbitGemvArgs a, int bits, int sm_count, cudaStream_t stream);
// Up to sixteen rows on warp-level tensor-core instructions, exact block sums (lowbit_mma.cu); a.q / a.sa / a.qsum from
// act_quant_kernel (a.qsum for 2-bit weights as well).
bool lowbit_mma_supported(const LowbitGemvArgs& a, int sm_count);
cudaError_t lowbit_mma_launch(LowbitGemvArgs a, int bits, int sm_count, cudaStream_t stream);

// ---- 2-bit / 1-bit x int8 activations, exact block sums on tcgen05 kind::f16 (lowbit_tc.cu) ----
struct LowbitTcArgs {
    const unsigned char* codes;   // packed units [n16][ku][512 B]
    const uint16_t* scales;       // f16 bits [n16][nb][16]
    const uint16_t* qh;           // m x kq activation codes as f16 integers (act_quant_kernel)
    const float* sa_t;            // nb x mpad activation scales, block-major
    const float* qsum_t;          // nb x mpad per-block sums of q, as floats
    int mpad;                     // m rounded up to a multiple of 128
    uint16_t* c;                  // m x n f16 bits
    int32_t* sums_out;            // optional debug: m x n x nb_real exact block sums
    int m, n, k, kq;
    int n16, ku, nb, nb_real;
    int log2_block, bits;
    uint32_t lut;                 // 2-bit codebook, byte c = value of code c + 128
    unsigned* status;
    EpParams ep;
};
bool lowbit_tc_supported(int bits, int m, int k, int log2_block);
cudaError_t lowbit_tc_launch(LowbitTcArgs a, cudaStream_t stream);

// cuTensorMapEncodeTiled through the runtime's driver entry point lookup (gemm_tc.cu); null if unavailable.
typedef CUresult (*TensorMapEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                      const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                      CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
TensorMapEncodeFn tensor_map_encoder();

// ---- prefill GEMM on tcgen05 (gemm_tc.cu) ----
struct GemmTcArgs {
    const unsigned char* codes;   // packed units [n16][ku][512 B]
    const uint16_t* scales;       // f16 bits [n16][nb][16]
    const uint16_t* a;            // tokens, row-major m x k (T bits), 16-byte aligned rows
    uint16_t* c;                  // m x n (T bits)
    float* c32;                   // if set: raw f32 accumulators instead
    float* yacc;                  // if set: y[m][n] += f32(T(acc)) instead of storing C (the MLP's residual add)
    int glu;                      // 0, or SMEG_ACT_SILU / _GELU: W is a gate/up matrix interleaved 32 columns at a time and
                                  // C (m x n/2) receives T(act(T(gate)) * T(up))
    const uint16_t* wdense;       // if set: dense weights W[n][kd] (T bits, K-major, kd = k padded to 8) instead of codes / scales
    int kd;                       // row length of wdense
    float beta;                   // the product is scaled by beta before the store rounding (dense builder; 1 elsewhere)
    int col_major;                // store C column-major: c[i + j * m]
    int m, n, k;
    int n16, ku, nb, log2_block;
    int ntok_tile, ntok_pad, ntok_box, nmma, tmem_cols;                // planner-filled
    int ep_fast;                  // the graph runs as a per-thread FastEp (see epilogue.cuh)
    int nt, nk, no, nw;           // ring depths (tokens / packed / operand), accumulator sets per CTA
    int us;                       // 64-deep units per stage (2 for small token tiles)
    // Tensor-parallel push (with c32 set): the f32 result rows go straight into their owner rank's receive area instead of
    // c32 -- row i belongs to rank i / push_rows and lands in slot push_rank of that rank's area, push[owner] +
    // (push_rank * push_rows + i % push_rows) * n -- by plain stores to peer-mapped memory from splitk_reduce_kernel.
    float* push[8];
    int push_world, push_rank, push_rows;
    int c_tma;                    // launcher-filled: C leaves through shared memory and tiled bulk stores (16-byte aligned rows of C)
    int cg;                       // CTAs per MMA: 2 = pairs of CTAs (a cluster of two along x) run MMAs of 256 weight columns
    int pu;                       // stages covered by one packed-ring slot
    int rpg;                      // scale rows staged per packed-ring slot
    int defer;                    // the depth slices are added by splitk_reduce_kernel after the GEMM instead of by the last CTA
    float* ws;                    // split-depth workspace [tile][slice][token][column]
    int* counters;                // one per output tile, zero between launches
    unsigned* status;
    EpParams ep;
};
bool gemm_tc_supported(int wkind, int m, int k, int log2_block, const void* a);
void gemm_tc_plan(GemmTcArgs& a, int sm_count, dim3* grid, size_t* smem, size_t* ws_floats, size_t* n_counters);
cudaError_t gemm_tc_launch(GemmTcArgs a, int bf16, dim3 grid, size_t smem, cudaStream_t stream);

// ---- 2-bit / 1-bit weights -> 4-bit plane for the tensor-core GEMM (transcode.cu) ----
struct LowbitToQ4Args {
    const unsigned char* src;       // packed 2-bit / 1-bit units
    const uint16_t* src_scales;     // [n16_src][nb_src][16]
    unsigned char* dst;             // packed 4-bit units [n16 (padded)][ku4][512]
    uint16_t* dst_scales;           // [n16 (padded)][nb4][16]
    size_t n, k;
    size_t ku_src, n16_src, nb_src; // source units along K, column groups, scale rows
    size_t ku4, nb4;                // 4-bit plane: units along K, scale rows
    size_t dst_words, dst_scale_elems;
    int bits;                       // 2 or 1
    uint32_t lut;                   // 2-bit codebook, byte c = value of code c
};
cudaError_t lowbit_to_q4_launch(const LowbitToQ4Args& a, cudaStream_t s);
// Dense K-major f16 weights W[n][kd] of a 2-bit / 1-bit set (for codebooks the 4-bit plane cannot hold).
cudaError_t lowbit_to_dense_launch(const LowbitToQ4Args& a, uint16_t* dst, size_t kd, int log2_block, cudaStream_t s);

// ---- element-wise model ops (elementwise.cu) ----
cudaError_t glu_launch(uint16_t* out, const uint16_t* both, size_t m, size_t n, uint32_t act, cudaStream_t s);
cudaError_t add_f16_to_f32_launch(float* dst, const uint16_t* src, size_t n, cudaStream_t s);
cudaError_t act_f16_launch(uint16_t* dst, const uint16_t* src, size_t n, uint32_t act, cudaStream_t s);
cudaError_t f32_to_f16_launch(uint16_t* dst, const float* src, size_t n, cudaStream_t s);
cudaError_t f16_to_f32_launch(float* dst, const uint16_t* src, size_t n, cudaStream_t s);
cudaError_t norm_rows_launch(uint16_t* y16, float* y32, const float* x, const float* weight, const float* bias, size_t rows, size_t dim,
                             float eps, int rms, cudaStream_t s);
cudaError_t rms_scales_launch(uint16_t* out, const uint16_t* x, size_t rows, size_t k, float eps, cudaStream_t s);
cudaError_t round_add_f32_launch(float* y, const float* partial_sum, size_t n, cudaStream_t s);

// ---- tensor-parallel sum + f16 rounding + residual add over peer memory (tp_reduce.cu) ----
constexpr int kTpReadyWords = 8;                                   // "ready" from rank s at [s]
constexpr int kTpMaxGrid = 160;                                    // most CTAs of the kernel
constexpr int kTpFlagWords = kTpReadyWords + 8 * kTpMaxGrid;       // "done" from owner s, CTA b at [8 + s * kTpMaxGrid + b]
// ---- causal attention against an f16 KV cache (attention.cu) ----
struct AttnArgs {
    float* out;            // [rows][heads][head_dim] f32
    const void* q;         // rows of heads * head_dim queries, f16 bits or f32, q_stride elements apart
    size_t q_stride;
    const uint16_t* k;     // cache rows of kv_heads * head_dim f16 bits
    const uint16_t* v;
    int start, rows;       // query row i attends to keys 0..=start+i
    int heads, kv_heads, head_dim;
    float scale;
};
cudaError_t attn_kv_causal_launch(const AttnArgs& a, int q_f32, cudaStream_t stream);
cudaError_t kv_append_launch(uint16_t* kc, uint16_t* vc, const uint16_t* src, size_t stride, size_t k_off, size_t v_off, size_t row_len,
                             size_t pos, size_t rows, cudaStream_t stream);

struct TpReduceArgs {
    float* bufs[8];        // every rank's buffer, peer-mapped into this process: len f32 partial sums, then len f16 results
    uint32_t* flags[8];    // every rank's flag array (kTpFlagWords words, zero before the first call)
    float* y;              // this rank's residual stream, len floats
    int rank, world;       // world <= 8
    size_t len;            // multiple of 4
    uint32_t seq;          // call number, the same on every rank, growing by one per call from 1
    int oneshot;           // every rank sums everything itself (short vectors; the caller double-buffers bufs)
    int pushed;            // the partials of this rank's slice are already here: bufs[rank] holds world slots of slice floats (rank order)
    size_t slice;          // pushed: floats per slot (rows per rank x row length)
    size_t res_off;        // offset (floats) of the f16 result area in a buffer: len, or world * slice when pushed
    unsigned* status;
};
cudaError_t tp_reduce_finish_launch(const TpReduceArgs& a, int sm_count, cudaStream_t stream);

}  // namespace smeg
