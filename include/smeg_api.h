/*
 * smeg_api.h -- C ABI of the B200 (sm_100a) implementation of sme-gemm's
 * weight-quantised matmul hot path.
 *
 * This header stands where csrc/sme_gemm_api.h stands in the reference: it is
 * the single list of exported symbols, and src/ffi.rs would bind exactly these.
 * Citations are file:line inside the reference project.
 *
 * Conventions (same as the reference, ARCHITECTURE.md:838-844):
 *   - every function returns int: 0 = ran and wrote its outputs; non-zero =
 *     argument / allocation / device failure and the outputs are untouched.
 *     There is no CPU fallback behind a non-zero return.
 *   - matrices are row-major and contiguous; 16-bit floats are passed as
 *     uint16_t bit patterns (f16 or bf16 as the entry point says).
 *   - m == 0 or n == 0 returns 0 without touching anything.
 *   - the caller owns every buffer; weights are immutable after creation and
 *     may be shared by concurrent calls from many host threads.
 *   - functions ending in _dev take DEVICE pointers (activations, outputs and
 *     every EpNode.ptr) plus a CUDA stream (cudaStream_t passed as void*) and
 *     only enqueue work; all others take HOST pointers, copy in and out, and
 *     return after the result is in host memory.
 */
#ifndef SMEG_API_H
#define SMEG_API_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- epilogue op-graph: byte-identical to csrc/epilogue.h:136-236 ---------- */

enum smeg_ep_op {            /* enum ep_op, csrc/epilogue.h:173-200 */
    SMEG_OP_ADD_SCALAR = 0, SMEG_OP_MUL_SCALAR = 1, SMEG_OP_ADD_ROW = 2, SMEG_OP_MUL_ROW = 3,
    SMEG_OP_ADD_COL = 4, SMEG_OP_MUL_COL = 5, SMEG_OP_ADD_TENSOR = 6, SMEG_OP_MUL_TENSOR = 7,
    SMEG_OP_ACT = 8, SMEG_OP_MAX_SCALAR = 9, SMEG_OP_MIN_SCALAR = 10, SMEG_OP_SUB_SCALAR = 11,
    SMEG_OP_SUB_ROW = 12, SMEG_OP_SUB_COL = 13, SMEG_OP_SUB_TENSOR = 14, SMEG_OP_DIV_SCALAR = 15,
    SMEG_OP_DIV_ROW = 16, SMEG_OP_DIV_COL = 17, SMEG_OP_DIV_TENSOR = 18, SMEG_OP_MAX_ROW = 19,
    SMEG_OP_MAX_COL = 20, SMEG_OP_MAX_TENSOR = 21, SMEG_OP_MIN_ROW = 22, SMEG_OP_MIN_COL = 23,
    SMEG_OP_MIN_TENSOR = 24
};
enum smeg_ep_act {           /* enum ep_act, csrc/epilogue.h:136-166 */
    SMEG_ACT_NONE = 0, SMEG_ACT_RELU = 1, SMEG_ACT_GELU = 2, SMEG_ACT_SILU = 3, SMEG_ACT_TANH = 4,
    SMEG_ACT_SIGMOID = 5, SMEG_ACT_LEAKY_RELU = 6, SMEG_ACT_RELU6 = 7, SMEG_ACT_HARDSIGMOID = 8,
    SMEG_ACT_HARDSWISH = 9, SMEG_ACT_ABS = 10, SMEG_ACT_NEG = 11, SMEG_ACT_SQUARE = 12,
    SMEG_ACT_SIGN = 13, SMEG_ACT_SQRT = 14, SMEG_ACT_SOFTSIGN = 15, SMEG_ACT_RECIP = 16,
    SMEG_ACT_RSQRT = 17, SMEG_ACT_EXP = 18, SMEG_ACT_LOG = 19, SMEG_ACT_ELU = 20, SMEG_ACT_SELU = 21,
    SMEG_ACT_SOFTPLUS = 22, SMEG_ACT_MISH = 23, SMEG_ACT_GELU_EXACT = 24
};

/* One ordered op-graph node (csrc/epilogue.h:214-229; Rust mirror
 * src/epilogue/mod.rs:148-185).  32 bytes, offsets 0/4/8/16/24.  `ptr`
 * operands are in the GEMM's 16-bit type.  The node array is already resolved
 * as src/exec/scalar.rs:28-53 does: TENSOR `ld == 0` means n, and a named
 * trailing activation arrives as a final ACT node. */
typedef struct {
    uint32_t op;      /* enum smeg_ep_op */
    uint32_t aux;     /* activation kind for SMEG_OP_ACT */
    float scalar;     /* *_SCALAR operand; alpha of leaky_relu / elu */
    const void *ptr;  /* ROW (length m) / COL (length n) / TENSOR (m rows, stride ld) operand */
    size_t ld;        /* TENSOR row stride in elements */
} EpNode;

/* csrc/epilogue.h:233-236.  NULL or n_nodes == 0 means identity. */
typedef struct {
    uint32_t n_nodes;
    const EpNode *nodes;
} ep_desc16;

/* ---- library ---------------------------------------------------------------- */

/* Version string of this library. */
const char *smeg_version(void);
/* SM count and total device memory of the current CUDA device; non-zero if no
 * usable sm_100 device is present. */
int smeg_device_info(int *sm_count, size_t *hbm_bytes);
/* Reads and clears the device status word (bit 0: a shared-memory barrier wait
 * gave up, bit 1: a tensor-memory pipeline wait gave up, bit 2: a peer wait gave
 * up).  Synchronises the device.  0 = no kernel ever abandoned a wait. */
unsigned smeg_last_status(void);
/* SME_GEMM_TRACE twin (src/warm.rs:115-179): when on (or env SMEG_TRACE=1) every
 * host-pointer entry prints "smeg: <kernel> MxNxK <us>" to stderr. */
void smeg_trace(int on);

/* ---- weight handles: device-resident, prepacked ------------------------------ */

typedef struct smeg_q4 smeg_q4;          /* Q4Weights, src/kernels/q4/weights.rs:26-37 */
typedef struct smeg_lowbit smeg_lowbit;  /* Q2Weights / Q1Weights, src/kernels/lowbit/q2.rs:31-38, q1.rs:23-30 */
typedef struct smeg_mlp smeg_mlp;        /* Mlp (gated), src/mlp.rs:56-92 */
typedef struct smeg_dense smeg_dense;    /* Packed<f16> / Packed<bf16>, src/element.rs */

#define SMEG_LAYOUT_OUT_IN 0             /* WeightLayout::OutIn: w[j*k + d] */
#define SMEG_LAYOUT_IN_OUT 1             /* WeightLayout::InOut: w[d*n + j] */

/* Q4Weights::with_params (src/kernels/q4/weights.rs:63-123).  quants: ceil(k*n/2)
 * bytes, weight idx = d*n + j in nibble idx%2 (low first), signed 4-bit codes;
 * scales (and mins, NULL for Q4_0): n*ceil(k/block) f16 bits at [j*nbk + blk].
 * block: power of two.  Returns -1 for a bad block size (csrc/gemm_f16f16_q4.h:474).
 * The affine form (Q4_1, mins != NULL: weight = scale * code + min) is kept as given and runs through dense twins
 * of the reference's expanded weights -- round_T(f64(scale) * code + f64(min)), src/kernels/q4/weights.rs:250-256 --
 * one per operand type, built on the first call of that type (2 bytes per weight of device memory each).  The
 * fused forms of the MLP block (smeg_mlp_create) take Q4_0 handles only and return -3 for an affine one. */
int smeg_q4_create(const uint8_t *quants, const uint16_t *scales, const uint16_t *mins, size_t n,
                   size_t k, size_t block, smeg_q4 **out);
/* Q4Weights::quantize (src/kernels/q4/quantize.rs:29-81). */
int smeg_q4_quantize(const float *w, int layout, size_t n, size_t k, size_t block, int affine,
                     smeg_q4 **out);
/* From the band-major arrays a reference-side Q4Weights holds
 * (src/kernels/q4/weights.rs:92-113). */
int smeg_q4_from_band(const uint8_t *nibbles, const uint16_t *scales, const uint16_t *mins, size_t n,
                      size_t k, size_t block, smeg_q4 **out);
void smeg_q4_destroy(smeg_q4 *w);
size_t smeg_q4_n(const smeg_q4 *w);
size_t smeg_q4_k(const smeg_q4 *w);
size_t smeg_q4_block(const smeg_q4 *w);
/* Inverse of smeg_q4_create: reads the prepacked device arrays back into the
 * logical layout (pack then unpack is the identity; counterpart of the
 * reference's pack round-trip tests, src/kernels/q4/weights.rs:425-463). */
int smeg_q4_unpack(const smeg_q4 *w, uint8_t *quants, uint16_t *scales);
/* Bytes of device memory the prepacked weights occupy (codes + scales). */
size_t smeg_q4_device_bytes(const smeg_q4 *w);

/* Q2Weights::new (src/kernels/lowbit/q2.rs:48-84): codes four to a byte, weight
 * idx = d*n + j at bits 2*(idx%4); scales [j*nbk + blk]; block a power of two in
 * 16..65536 (-1 otherwise); codebook: the four int8 values of the codes. */
int smeg_q2_create(const uint8_t *codes, const uint16_t *scales, size_t n, size_t k, size_t block,
                   const int8_t codebook[4], smeg_lowbit **out);
/* Q2Weights::quantize (src/kernels/lowbit/q2.rs:110-144); -2 for an all-zero codebook. */
int smeg_q2_quantize(const float *w, int layout, size_t n, size_t k, size_t block,
                     const int8_t codebook[4], smeg_lowbit **out);
/* Q1Weights::new (src/kernels/lowbit/q1.rs:47-106): one sign bit per weight (1 =
 * +scale), idx = j*k + d (OutIn) or d*n + j (InOut), low bit first. */
int smeg_q1_create(const uint8_t *signs, const uint16_t *scales, int layout, size_t n, size_t k,
                   size_t block, smeg_lowbit **out);
/* Q1Weights::quantize (src/kernels/lowbit/q1.rs:116-144). */
int smeg_q1_quantize(const float *w, int layout, size_t n, size_t k, size_t block, smeg_lowbit **out);
/* From the reference's band-major arrays (src/kernels/lowbit/q2.rs:146-161,
 * q1.rs:188-201; scale order q2.rs:17-20). */
int smeg_q2_from_band(const uint8_t *codes, const uint16_t *scales, size_t n, size_t k, size_t block,
                      const int8_t codebook[4], smeg_lowbit **out);
int smeg_q1_from_band(const uint8_t *signs, const uint16_t *scales, size_t n, size_t k, size_t block,
                      smeg_lowbit **out);
void smeg_lowbit_destroy(smeg_lowbit *w);
size_t smeg_lowbit_n(const smeg_lowbit *w);
size_t smeg_lowbit_k(const smeg_lowbit *w);
size_t smeg_lowbit_block(const smeg_lowbit *w);
int smeg_lowbit_bits(const smeg_lowbit *w);   /* 2 or 1 */
/* Inverse of create: 2-bit codes in the input order of smeg_q2_create, or sign
 * bits in OutIn order (pack round-trips: q2.rs:197-223, q1.rs:245-274). */
int smeg_lowbit_unpack(const smeg_lowbit *w, uint8_t *bits_out, uint16_t *scales);
size_t smeg_lowbit_device_bytes(const smeg_lowbit *w);

/* ---- host-side preparation, no device needed ---------------------------------- */
/* The quantisers and the prepack that the create / quantize functions above run,
 * on caller-provided host buffers.  bits: 4, 2 or 1.  `wbits` is the logical
 * array of the matching create function (nibbles / 2-bit codes / sign bits; for
 * 1-bit, `layout` gives the bit order on pack, unpack returns OutIn order). */
size_t smeg_packed_code_bytes(int bits, size_t n, size_t k);
size_t smeg_packed_scale_elems(int bits, size_t n, size_t k, size_t block);
int smeg_host_pack(int bits, const uint8_t *wbits, int layout, const uint16_t *scales, size_t n, size_t k,
                   size_t block, uint8_t *codes_out, uint16_t *scales_out);
int smeg_host_unpack(int bits, const uint8_t *codes, const uint16_t *packed_scales, size_t n, size_t k,
                     size_t block, uint8_t *wbits_out, uint16_t *scales_out);
/* Q4Weights::quantize / Q2Weights::quantize / Q1Weights::quantize into logical arrays. */
int smeg_host_q4_quantize(const float *w, int layout, size_t n, size_t k, size_t block, uint8_t *quants,
                          uint16_t *scales);
int smeg_host_q2_quantize(const float *w, int layout, size_t n, size_t k, size_t block,
                          const int8_t codebook[4], uint8_t *codes, uint16_t *scales);
int smeg_host_q1_quantize(const float *w, int layout, size_t n, size_t k, size_t block, uint8_t *signs,
                          uint16_t *scales);

/* ---- compute, device pointers (the timed paths) ------------------------------ */

/* matmul_q4_ep / matmul_q4_bf16_ep (src/kernels/q4/matmul.rs:21-103, 178-271):
 * C[m][n] = ep(A[m][k] @ dequant(W)).  ep may be NULL. */
int smeg_matmul_q4_f16_dev(const smeg_q4 *w, const uint16_t *a, uint16_t *c, size_t m,
                           const ep_desc16 *ep, void *stream);
int smeg_matmul_q4_bf16_dev(const smeg_q4 *w, const uint16_t *a, uint16_t *c, size_t m,
                            const ep_desc16 *ep, void *stream);
/* matmul_q2_ep / matmul_q1_ep (src/kernels/lowbit/matmul.rs:38-84, 326-337): int8
 * activation path, f16 in / out.  Integer block sums and the activation
 * quantisation are bit-exact with quantize_row / reference (:354-398). */
int smeg_matmul_lowbit_dev(const smeg_lowbit *w, const uint16_t *a, uint16_t *c, size_t m,
                           const ep_desc16 *ep, void *stream);
/* matmul_q2_mopa_ep / matmul_q1_mopa_ep (src/kernels/lowbit/matmul.rs:100-139, mopa_impl
 * :339-350): the same weights on the f16 path -- f16 activations, no int8 quantisation,
 * weights f16(scale * value) as Codes::dequant (:178-197) rounds them, f32 accumulation on
 * the tensor cores.  The first such call on a handle builds a 4-bit twin of the weights on
 * the device (synchronously; smeg_lowbit_prepare_f16 does it ahead of time, e.g. before a
 * stream capture).  A 2-bit codebook with a value outside [-8, 7] does not fit 4-bit codes: its twin is a dense f16
 * matrix of the same rounded weights (2 bytes per weight). */
int smeg_lowbit_prepare_f16(const smeg_lowbit *w);
int smeg_matmul_lowbit_f16_dev(const smeg_lowbit *w, const uint16_t *a, uint16_t *c, size_t m,
                               const ep_desc16 *ep, void *stream);
/* Same, also writing the intermediate integers for parity checks: q (m*k int8),
 * sa (m*ceil(k/block) f32), sums (m*n*ceil(k/block) int32); any may be NULL. */
int smeg_matmul_lowbit_debug_dev(const smeg_lowbit *w, const uint16_t *a, uint16_t *c, size_t m,
                                 int8_t *q_out, float *sa_out, int32_t *sums_out, void *stream);
/* No counterpart in the reference.  smeg_matmul_lowbit_dev for callers that cannot allocate
 * device memory (a serving loop with a frozen memory map, a process that handed all of HBM
 * to weights and caches, a sandbox without cudaMalloc): the int8-activation scratch lives in
 * a fixed array inside the library image instead of coming from the allocator.  Holds on
 * every GPU that loads the library, until exit, about 200 KB.  Limits: m <= 8, depth (padded
 * to the weight unit) <= 16384, <= 1024 K-blocks per row, <= 16 epilogue nodes; rc = -4 beyond
 * them.  All calls on a device share the array: calls that overlap on the GPU race, so keep
 * them on one stream.  The first call on a device resolves the array's address and must come
 * before any stream capture.  Results are bit-identical to smeg_matmul_lowbit_dev. */
int smeg_matmul_lowbit_static_dev(const smeg_lowbit *w, const uint16_t *a, uint16_t *c, size_t m,
                                  const ep_desc16 *ep, void *stream);
/* neon_glu_f16 / neon_add_f16_to_f32 / neon_act_f16 / converts
 * (csrc/sme_gemm_api.h:216-220; glu: src/linear.rs:804-835; add: src/convert.rs:37-48). */
int smeg_glu_f16_dev(uint16_t *out, const uint16_t *both, size_t m, size_t n, uint32_t act, void *stream);
int smeg_add_f16_to_f32_dev(float *dst, const uint16_t *src, size_t len, void *stream);
int smeg_act_f16_dev(uint16_t *dst, const uint16_t *src, size_t len, uint32_t act, void *stream);
int smeg_f32_to_f16_dev(uint16_t *dst, const float *src, size_t len, void *stream);
int smeg_f16_to_f32_dev(float *dst, const uint16_t *src, size_t len, void *stream);

/* Norm::forward on f32 rows into f16 (y16) and / or f32 (y32) rows: layer_norm (rms == 0) or rms_norm
 * (src/nn.rs:73-161, norm_row :126-153; replaces neon_norm_row_f16 / _f32, csrc/sme_gemm_api.h:221-224).
 * weight: dim f32; bias: dim f32 or NULL.  The step before the MLP in Block::accumulate (src/block.rs:96-105). */
int smeg_norm_rows_dev(uint16_t *y16, float *y32, const float *x, const float *weight, const float *bias,
                       size_t rows, size_t dim, float eps, int rms, void *stream);
/* rms_scales (src/nn.rs:234-248): out[i] = f16(1 / sqrt(mean(x_i^2) + eps)) per k-wide f16 row -- the leading
 * MulRow operand of a Linear whose RMS-norm weight was folded into it (src/linear.rs:305-308, 452-457). */
int smeg_rms_scales_dev(uint16_t *out, const uint16_t *x, size_t rows, size_t k, float eps, void *stream);

/* ---- compute, host pointers, handle based ------------------------------------ */

int smeg_matmul_q4_f16(const smeg_q4 *w, const uint16_t *a, uint16_t *c, size_t m, const ep_desc16 *ep);
int smeg_matmul_q4_bf16(const smeg_q4 *w, const uint16_t *a, uint16_t *c, size_t m, const ep_desc16 *ep);
int smeg_matmul_lowbit(const smeg_lowbit *w, const uint16_t *a, uint16_t *c, size_t m, const ep_desc16 *ep);
int smeg_matmul_lowbit_f16(const smeg_lowbit *w, const uint16_t *a, uint16_t *c, size_t m, const ep_desc16 *ep);

/* ---- dense 16-bit weights: the Gemm builder --------------------------------------- */

/* prepack_f16 / prepack_bf16 (src/kernels/f16.rs:212, src/kernels/bf16.rs): b is k x n row-major
 * T bits; the handle keeps it K-major on the device. */
int smeg_dense_create(const uint16_t *b, size_t n, size_t k, int bf16, smeg_dense **out);
void smeg_dense_destroy(smeg_dense *w);
size_t smeg_dense_n(const smeg_dense *w);
size_t smeg_dense_k(const smeg_dense *w);
/* Gemm::run (src/exec/builder.rs:803-813 -> packed_ep_impl, src/exec/macros.rs:98-200):
 * C = ep( T(beta * (A @ B)) ), C row-major m x n or, with col_major, c[i + j * m].  Replaces
 * gemm_sme_f16f16_run_packed / gemm_sme_b16b16_run_packed (csrc/sme_gemm_api.h) for this use.
 * Any k: a depth that is not a multiple of 8, or an A whose rows do not start on 16-byte boundaries, is staged through a
 * zero-padded copy of A in stream-ordered scratch (k == 0 is refused: rc = -3). */
int smeg_gemm_dense_dev(const smeg_dense *w, const uint16_t *a, uint16_t *c, size_t m, uint16_t beta_bits,
                        int col_major, const ep_desc16 *ep, void *stream);
int smeg_gemm_dense(const smeg_dense *w, const uint16_t *a, uint16_t *c, size_t m, uint16_t beta_bits,
                    int col_major, const ep_desc16 *ep);

/* ---- MLP block ---------------------------------------------------------------- */

/* The attention step of SelfAttention::accumulate (src/self_attention.rs:189-231) on the device.
 * smeg_kv_append_dev -- KvCache::extend (src/kernels/kv_attention.rs:499-520): `rows` rows of row_len = kv_heads *
 * head_dim f16 values each for keys and values, taken from rows of `src` (src_stride elements apart, the keys at
 * element k_off and the values at v_off of a row: the [q | k | v] rows a fused projection produced), copied to cache
 * rows pos .. pos + rows.
 * smeg_attn_kv_causal_dev -- attention_kv_causal_f16 (src/kernels/kv_attention.rs:155-242; rows = 1, start = len - 1 is
 * attention_kv_f16, :29-139): query row i attends to keys 0..=start+i of caches that already hold start + rows rows;
 * q is f16 bits (q_f32 = 0) or f32 rows of heads * head_dim values q_stride elements apart, out f32 [rows][heads *
 * head_dim].  Per head softmax(f16(q * scale) . k) @ v with f32 sums in key / depth order.  head_dim a multiple of 8 in
 * 8..=256 and heads a positive multiple of kv_heads (-4 otherwise, where the reference panics); -3 beyond ~50 k keys. */
int smeg_kv_append_dev(uint16_t *k_cache, uint16_t *v_cache, const uint16_t *src, size_t src_stride, size_t k_off,
                       size_t v_off, size_t row_len, size_t pos, size_t rows, void *stream);
int smeg_attn_kv_causal_dev(float *out, const void *q, int q_f32, size_t q_stride, const uint16_t *k, const uint16_t *v,
                            size_t start, size_t rows, size_t heads, size_t kv_heads, size_t head_dim, float scale,
                            void *stream);

/* Mlp::gated (src/mlp.rs:80-92): gate_up is the 2*hidden-column interleaved
 * matrix GatedLinear::quantize builds (32 gate columns then 32 up columns,
 * src/linear.rs:603-656), down is hidden -> d.  The handles are borrowed and
 * must outlive the block.  gate_act: SMEG_ACT_SILU or SMEG_ACT_GELU. */
int smeg_mlp_create(const smeg_q4 *gate_up, const smeg_q4 *down, uint32_t gate_act, smeg_mlp **out);
void smeg_mlp_destroy(smeg_mlp *mlp);
/* Mlp::accumulate (src/mlp.rs:113-146): y (m x d, f32) += down(glu(x @ gate_up)),
 * x is m x k f16. */
int smeg_mlp_accumulate_dev(smeg_mlp *mlp, const uint16_t *x, float *y, size_t m, void *stream);
int smeg_mlp_accumulate(smeg_mlp *mlp, const uint16_t *x, float *y, size_t m);
/* Tensor-parallel halves of the same step: `partial` (m x d, f32) receives this
 * rank's un-rounded down-projection partial sums (its rows of W_down); after the
 * ranks' partials are summed, finish applies the f16 store rounding and the
 * residual add, y += f32(f16(sum)). */
int smeg_mlp_partial_dev(smeg_mlp *mlp, const uint16_t *x, float *partial, size_t m, void *stream);
/* The same for one projection whose input width is split over the ranks (the out projection of a self-attention
 * block sharded by heads; no counterpart in the reference, which runs on one device): partial (m x n, f32) receives
 * the un-rounded f32 sums A @ dequant(W) of this rank's rows of W.  Q4_0 weights, f16 activations (rc -3: affine). */
int smeg_matmul_q4_partial_dev(const smeg_q4 *w, const uint16_t *a, float *partial, size_t m, void *stream);
int smeg_mlp_finish_dev(float *y, const float *sum, size_t len, void *stream);
/* The sum over ranks and finish in one kernel over peer memory (no counterpart in the
 * reference, whose Mlp::accumulate, src/mlp.rs:124-146, runs on one device): every rank
 * has left its partial in a buffer all ranks can address (buf_ptrs[s] = rank s's buffer as
 * mapped into this process: len floats of partial sums followed by room for len f16 results,
 * i.e. 6 * len bytes; len % 4 == 0) and owns a zero-initialised array of SMEG_TP_FLAG_WORDS
 * uint32 flags (flag_ptrs[s], likewise mapped).  Each rank calls this once per step with
 * the same seq (1, 2, 3, ... per step); on return of the kernel y += f32(f16(sum over ranks,
 * added in rank order)) on every rank and the buffers may be overwritten.  world <= 8.
 * oneshot != 0 (short vectors): every rank adds all partials itself and no second flag
 * round runs; the caller must then alternate between two buffers from step to step.
 * A peer that never arrives ends the wait after a second: rc -7 at the next status read;
 * y is untouched when that happens in the first flag round. */
#define SMEG_TP_FLAG_WORDS 1288
int smeg_mlp_reduce_finish_dev(float *y, const uint64_t *buf_ptrs, const uint64_t *flag_ptrs, int rank, int world,
                               size_t len, uint32_t seq, int oneshot, void *stream);

/* The same exchange with the partial sums PUSHED: smeg_mlp_partial_push_dev runs the rank's two GEMMs and its down
 * projection's last stage stores every f32 result row straight into the receive area of the rank that owns it (plain
 * stores to peer-mapped memory; row i belongs to rank i / rows, rows = ceil(m / world)), so that the owner later sums
 * from its own memory.  A buffer is then world slots of rows * d floats (slot s = rank s's partial of this rank's rows)
 * followed by m * d result words of 4 bytes: (world * rows * d + m * d) * 4 bytes.  smeg_mlp_reduce_finish_pushed_dev is
 * the matching finish: one "ready" flag round as above, then every owner sums its rows from its own memory and sends the
 * f16 results to the peers as 8-byte words that carry the call's sequence number beside two values, which the receivers
 * poll -- no fence and no second flag round; same guarantees as above (bounded waits, rc -7), no one-shot form.  rc -3: the step is too small for
 * this form (m <= 64) -- use smeg_mlp_partial_dev + smeg_mlp_reduce_finish_dev. */
int smeg_mlp_partial_push_dev(smeg_mlp *mlp, const uint16_t *x, const uint64_t *buf_ptrs, int rank, int world, size_t m,
                              void *stream);
int smeg_mlp_reduce_finish_pushed_dev(float *y, const uint64_t *buf_ptrs, const uint64_t *flag_ptrs, int rank, int world,
                                      size_t m, size_t d, uint32_t seq, void *stream);

/* ---- drop-in entry points: the reference's own signatures --------------------- */
/* These take what src/kernels/{q4,lowbit}/matmul.rs pass today: host pointers and
 * the reference's band-major packed arrays.  The first call on a weight set
 * converts it to the GPU layout and keeps it resident on the device, keyed by the
 * packed array's address and shape; later calls find it.  A weight set that is
 * freed must be dropped with smeg_forget so a new allocation at the same address
 * is not mistaken for it. */

/* csrc/sme_gemm_api.h:97-99 */
int gemm_sme_f16f16_q4(size_t m, size_t n, size_t k, uint16_t *dst, const uint16_t *lhs,
                       const uint8_t *nibbles, const uint16_t *scales, const uint16_t *mins,
                       size_t block, const ep_desc16 *ep);
/* csrc/sme_gemm_api.h:66-69 (scales_bf16 / mins_bf16 are derived copies and unused here) */
int gemm_sme_b16b16_q4(size_t m, size_t n, size_t k, uint16_t *dst, const uint16_t *lhs,
                       const uint8_t *nibbles, const uint16_t *scales, const uint16_t *mins,
                       const uint16_t *scales_bf16, const uint16_t *mins_bf16, size_t block,
                       const ep_desc16 *ep);
/* csrc/sme_gemm_api.h:208-213 */
int gemm_sme_f16_q1(size_t m, size_t n, size_t k, uint16_t *dst, const uint16_t *lhs,
                    const uint8_t *signs, const uint16_t *scales, size_t block, const ep_desc16 *ep);
int gemm_sme_f16_q2(size_t m, size_t n, size_t k, uint16_t *dst, const uint16_t *lhs,
                    const uint8_t *codes, const uint16_t *scales, const int8_t *codebook, size_t block,
                    const ep_desc16 *ep);
/* csrc/sme_gemm_api.h:110-115: the same weights on the f16 path */
int gemm_sme_f16f16_q1(size_t m, size_t n, size_t k, uint16_t *dst, const uint16_t *lhs,
                       const uint8_t *signs, const uint16_t *scales, size_t block, const ep_desc16 *ep);
int gemm_sme_f16f16_q2(size_t m, size_t n, size_t k, uint16_t *dst, const uint16_t *lhs,
                       const uint8_t *codes, const uint16_t *scales, const int8_t *codebook, size_t block,
                       const ep_desc16 *ep);
/* csrc/sme_gemm_api.h:216-220 (host pointers) */
void neon_glu_f16(uint16_t *out, const uint16_t *in, size_t m, size_t n, uint32_t act);
void neon_add_f16_to_f32(float *dst, const uint16_t *src, size_t n);
void neon_act_f16(uint16_t *dst, const uint16_t *src, size_t n, uint32_t act);
void neon_f32_to_f16(uint16_t *dst, const float *src, size_t n);
void neon_f16_to_f32(float *dst, const uint16_t *src, size_t n);
/* Drops the device copy cached for a packed array (call from the weights' Drop). */
void smeg_forget(const void *packed);

#ifdef __cplusplus
}
#endif
#endif /* SMEG_API_H */
