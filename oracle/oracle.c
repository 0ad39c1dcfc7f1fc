/*
 * CPU oracle: a plain-C restatement of the portable scalar path of
 * electricapp/sme-gemm for the weight-quantized matmul hot path.
 *
 * THIS IS TEST INFRASTRUCTURE, NOT PRODUCT CODE.  Only the test-suite, the
 * smoke check and the benchmark's CPU-baseline legs may load it; the CUDA
 * library never calls into it and has no CPU fallback.
 *
 * Parity status: the reference is a Rust crate and no Rust toolchain exists in
 * the build environment, so this restatement cannot be compared with outputs
 * of the reference executed here.  It is pinned instead by (1) every
 * closed-form known-answer test the reference's own unit tests contain for this
 * path (pack round trips, grid-weight recovery, half-step quantisation error,
 * k == 0, the analytic q2 error bound), restated in tests/, and (2) bit
 * equality with an independent numpy restatement written from the same
 * reference lines (oracle/np_oracle.py).  The reference holds no golden-vector
 * files for this path.
 *
 * Third-party arithmetic restated here: crate `half` 2.7.1 (Cargo.lock) --
 * f16::from_f32 / from_f64 / to_f32 and bf16::from_f32 are IEEE round-to-
 * nearest-even conversions (f64 -> f16 is a single direct rounding).
 *
 * Build: gcc -O3 -ffp-contract=off -fno-fast-math -pthread -shared -fPIC
 * (see Makefile).  -ffp-contract=off matters: the reference keeps every f32
 * multiply and add separately rounded except where it calls mul_add.
 *
 * Every function cites the reference file:line it follows (paths are relative
 * to the reference project root).
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <pthread.h>
#include <stdatomic.h>
#include <unistd.h>

/* ------------------------------------------------------------------ */
/* half / bfloat16 conversions (crate `half` 2.7.1 semantics)          */
/* ------------------------------------------------------------------ */

static inline uint32_t f32_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float bits_f32(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static inline uint64_t f64_bits(double f) { uint64_t u; memcpy(&u, &f, 8); return u; }

/* f16 bits -> f32 (exact). */
float orc_f16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1f;
    uint32_t man = h & 0x3ffu;
    if (exp == 0) {
        if (man == 0) return bits_f32(sign);
        /* subnormal: value = man * 2^-24 */
        float v = (float)man * 5.9604644775390625e-08f;
        return sign ? -v : v;
    }
    if (exp == 31) return bits_f32(sign | 0x7f800000u | (man << 13));
    return bits_f32(sign | ((exp + 112) << 23) | (man << 13));
}

/* f64 -> f16 bits, one direct rounding to nearest even (half::f16::from_f64). */
uint16_t orc_f64_to_f16(double d) {
    uint64_t x = f64_bits(d);
    uint16_t sign = (uint16_t)((x >> 48) & 0x8000u);
    int64_t exp = (int64_t)((x >> 52) & 0x7ff);
    uint64_t man = x & 0xfffffffffffffull;
    if (exp == 0x7ff) {
        if (man == 0) return sign | 0x7c00u;
        return sign | 0x7e00u | (uint16_t)(man >> 42); /* quiet NaN, payload top bits */
    }
    int64_t e = exp - 1023; /* unbiased */
    if (exp == 0) return sign; /* f64 subnormals are far below f16 range */
    if (e > 15) return sign | 0x7c00u;
    uint64_t sig = man | (1ull << 52); /* 53-bit significand */
    int shift;                         /* bits to drop from sig to reach the f16 grid */
    int64_t he;                        /* biased half exponent of the result before carry */
    if (e >= -14) {
        shift = 42; /* keep 11 bits (1 hidden + 10) */
        he = e + 15;
    } else {
        /* subnormal half: grid is 2^-24 */
        shift = (int)(42 + (-14 - e));
        he = 0;
        if (shift > 63) return sign;
    }
    uint64_t kept = sig >> shift;
    uint64_t rem = sig & ((1ull << shift) - 1);
    uint64_t half = 1ull << (shift - 1);
    if (rem > half || (rem == half && (kept & 1))) kept++;
    uint32_t out;
    if (he == 0) {
        out = (uint32_t)kept; /* may carry into exponent 1 naturally */
    } else {
        out = (uint32_t)(((uint64_t)he << 10) + (kept - (1ull << 10)));
        /* carry out of the significand bumps the exponent through the add */
    }
    if (out >= 0x7c00u) out = 0x7c00u;
    return sign | (uint16_t)out;
}

/* f32 -> f16 bits (half::f16::from_f32): f32 -> f64 is exact, so one rounding. */
uint16_t orc_f32_to_f16(float f) { return orc_f64_to_f16((double)f); }

/* f32 -> bf16 bits, round to nearest even (half::bf16::from_f32). */
uint16_t orc_f32_to_bf16(float f) {
    uint32_t x = f32_bits(f);
    if ((x & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((x >> 16) | 0x0040u);
    uint32_t round_bit = 0x00008000u;
    if ((x & round_bit) != 0 && (x & (3 * round_bit - 1)) != 0) return (uint16_t)((x >> 16) + 1);
    return (uint16_t)(x >> 16);
}
float orc_bf16_to_f32(uint16_t h) { return bits_f32((uint32_t)h << 16); }

void orc_f32_to_f16_slice(const float *src, uint16_t *dst, size_t n) {
    for (size_t i = 0; i < n; i++) dst[i] = orc_f32_to_f16(src[i]);
}
void orc_f32_to_bf16_slice(const float *src, uint16_t *dst, size_t n) {
    for (size_t i = 0; i < n; i++) dst[i] = orc_f32_to_bf16(src[i]);
}
void orc_f16_to_f32_slice(const uint16_t *src, float *dst, size_t n) {
    for (size_t i = 0; i < n; i++) dst[i] = orc_f16_to_f32(src[i]);
}

static inline float t_to_f32(uint16_t v, int bf16) { return bf16 ? orc_bf16_to_f32(v) : orc_f16_to_f32(v); }
static inline uint16_t f32_to_t(float v, int bf16) { return bf16 ? orc_f32_to_bf16(v) : orc_f32_to_f16(v); }

static int g_threads = 1;
/* Threads used by the GEMM-shaped loops (rows or columns are independent, so
 * results do not depend on the count).  The reference's scalar path is single
 * threaded; more threads are for the timed all-core baseline only. */
void orc_set_threads(int t) { g_threads = t < 1 ? 1 : t; }
int orc_get_threads(void) { return g_threads; }
int orc_max_threads(void) {
    long c = sysconf(_SC_NPROCESSORS_ONLN);
    return c < 1 ? 1 : (int)c;
}

/* Minimal parallel-for over independent items (pthreads; items are claimed
 * from a shared counter, so the split never changes any result). */
typedef void (*par_body)(size_t item, void *ctx, void *scratch);
typedef struct {
    par_body body;
    void *ctx;
    size_t first, end, scratch_bytes;
    atomic_size_t next;
} par_job;
static void *par_worker(void *p) {
    par_job *job = (par_job *)p;
    void *scratch = job->scratch_bytes ? malloc(job->scratch_bytes) : NULL;
    for (;;) {
        size_t i = atomic_fetch_add(&job->next, 1);
        if (i >= job->end) break;
        job->body(i, job->ctx, scratch);
    }
    free(scratch);
    return NULL;
}
static void par_for(size_t first, size_t end, par_body body, void *ctx, size_t scratch_bytes) {
    par_job job;
    job.body = body; job.ctx = ctx; job.first = first; job.end = end;
    job.scratch_bytes = scratch_bytes;
    atomic_init(&job.next, first);
    size_t items = end > first ? end - first : 0;
    int nt = g_threads;
    if ((size_t)nt > items) nt = (int)items;
    if (nt <= 1) { par_worker(&job); return; }
    pthread_t *th = (pthread_t *)malloc(sizeof(pthread_t) * (size_t)nt);
    for (int t = 1; t < nt; t++) pthread_create(&th[t], NULL, par_worker, &job);
    par_worker(&job);
    for (int t = 1; t < nt; t++) pthread_join(th[t], NULL);
    free(th);
}

/* ------------------------------------------------------------------ */
/* Q4: quantise, dequantise                                            */
/* ------------------------------------------------------------------ */

/* Q4Weights::quantize, src/kernels/q4/quantize.rs:29-81.
 * layout 0 = OutIn (w[j*k+d]), 1 = InOut (w[d*n+j]).
 * quants: ceil(k*n/2) bytes, weight idx = d*n+j in nibble idx%2 (low first),
 * two's-complement 4-bit codes.  scales/mins: [j*nbk + b] f16 bits
 * (mins only when affine). */
void orc_q4_quantize(const float *w, int layout, size_t n, size_t k, size_t block, int affine,
                     uint8_t *quants, uint16_t *scales, uint16_t *mins) {
    size_t nbk = (k + block - 1) / block;
    memset(quants, 0, (k * n + 1) / 2);
    for (size_t j = 0; j < n; j++) {
        for (size_t b = 0; b < nbk; b++) {
            size_t d0 = b * block, d1 = (b + 1) * block < k ? (b + 1) * block : k;
            uint16_t scale, min = 0;
#define AT(J, D) (layout == 0 ? w[(J) * k + (D)] : w[(D) * n + (J)])
            if (affine) {
                float lo = INFINITY, hi = -INFINITY;
                for (size_t d = d0; d < d1; d++) {
                    float x = AT(j, d);
                    lo = fminf(lo, x);
                    hi = fmaxf(hi, x);
                }
                scale = orc_f32_to_f16((hi - lo) / 15.0f);
                min = orc_f32_to_f16(lo + 8.0f * orc_f16_to_f32(scale));
            } else {
                float m = 0.0f;
                for (size_t d = d0; d < d1; d++) {
                    float x = AT(j, d);
                    if (fabsf(x) > fabsf(m)) m = x;
                }
                scale = orc_f32_to_f16(m / -8.0f);
            }
            scales[j * nbk + b] = scale;
            if (affine) mins[j * nbk + b] = min;
            float s = orc_f16_to_f32(scale), mn = orc_f16_to_f32(min);
            float inv = s == 0.0f ? 0.0f : 1.0f / s;
            for (size_t d = d0; d < d1; d++) {
                float r = roundf((AT(j, d) - mn) * inv); /* f32::round: half away from zero */
                if (r < -8.0f) r = -8.0f;
                if (r > 7.0f) r = 7.0f;
                int code = isnan(r) ? 0 : (int)r; /* `as i8`: NaN -> 0 */
                size_t idx = d * n + j;
                quants[idx / 2] |= (uint8_t)((code & 0x0f) << (4 * (idx % 2)));
            }
#undef AT
        }
    }
}

static inline int q4_code(const uint8_t *quants, size_t idx) {
    int nib = (idx % 2 == 0) ? (quants[idx / 2] & 0x0f) : (quants[idx / 2] >> 4);
    return nib < 8 ? nib : nib - 16;
}

/* Q4Weights::dequant_rows, src/kernels/q4/weights.rs:232-259 (+ :190-203):
 * w[d][j] = round_T( f64(scale) * code (+ f64(min)) ), T = f16 directly from
 * f64, or bf16 through f32.  Output row-major k x n. */
typedef struct {
    const uint8_t *quants; const uint16_t *scales, *mins;
    size_t n, k, block; int bf16; uint16_t *out;
} dq_ctx;
static void dq_row(size_t d, void *p, void *scratch) {
    (void)scratch;
    dq_ctx *c = (dq_ctx *)p;
    size_t n = c->n, nbk = (c->k + c->block - 1) / c->block;
    for (size_t j = 0; j < n; j++) {
        int code = q4_code(c->quants, d * n + j);
        size_t si = j * nbk + d / c->block;
        double v = (double)orc_f16_to_f32(c->scales[si]) * (double)code;
        if (c->mins) v += (double)orc_f16_to_f32(c->mins[si]);
        c->out[d * n + j] = c->bf16 ? orc_f32_to_bf16((float)v) : orc_f64_to_f16(v);
    }
}
void orc_q4_dequant(const uint8_t *quants, const uint16_t *scales, const uint16_t *mins, size_t n,
                    size_t k, size_t block, int bf16, uint16_t *out) {
    dq_ctx c = {quants, scales, mins, n, k, block, bf16, out};
    par_for(0, k, dq_row, &c, 0);
}

/* ------------------------------------------------------------------ */
/* dense 16-bit GEMM, f32 accumulate                                   */
/* ------------------------------------------------------------------ */

/* reference::gemm_f16 / gemm_bf16, src/reference.rs:308-387, as the packed
 * fallback calls them (alpha = 0, beta = 1, src/exec/macros.rs:186-203):
 * ikj, acc[j] (f32) += f32(a[i][l]) * f32(b[l][j]) for l ascending, separate
 * multiply and add; c = T(0 + 1*acc).  a: m x k, b: k x n, c: m x n row-major.
 * Rows first..first+rows-1 only (for sub-sampled timing). */
typedef struct {
    size_t n, k; uint16_t *c; const uint16_t *a; const float *bf; int bf16;
} gm_ctx;
static void gm_row(size_t i, void *p, void *scratch) {
    gm_ctx *g = (gm_ctx *)p;
    float *acc = (float *)scratch;
    size_t n = g->n, k = g->k;
    for (size_t j = 0; j < n; j++) acc[j] = 0.0f;
    for (size_t l = 0; l < k; l++) {
        float av = t_to_f32(g->a[i * k + l], g->bf16);
        const float *br = g->bf + l * n;
        for (size_t j = 0; j < n; j++) acc[j] += av * br[j];
    }
    for (size_t j = 0; j < n; j++) g->c[i * n + j] = f32_to_t(0.0f + 1.0f * acc[j], g->bf16);
}
typedef struct { float *bf; const uint16_t *b; size_t n; int bf16; } wd_ctx;
static void wd_row(size_t l, void *p, void *scratch) {
    (void)scratch;
    wd_ctx *w = (wd_ctx *)p;
    for (size_t j = 0; j < w->n; j++) w->bf[l * w->n + j] = t_to_f32(w->b[l * w->n + j], w->bf16);
}
void orc_gemm16_rows(size_t m, size_t n, size_t k, uint16_t *c, const uint16_t *a,
                     const uint16_t *b, int bf16, size_t first, size_t rows) {
    (void)m;
    float *bf = (float *)malloc(sizeof(float) * (k * n ? k * n : 1));
    wd_ctx w = {bf, b, n, bf16};
    par_for(0, k, wd_row, &w, 0);
    gm_ctx g = {n, k, c, a, bf, bf16};
    par_for(first, first + rows, gm_row, &g, sizeof(float) * (n ? n : 1));
    free(bf);
}
/* The same product left in f32 (no store rounding): the un-rounded partial sums a
 * tensor-parallel rank contributes.  Not a reference function. */
void orc_gemm16_f32(size_t m, size_t n, size_t k, float *c, const uint16_t *a, const uint16_t *b, int bf16) {
    for (size_t i = 0; i < m; i++) {
        for (size_t j = 0; j < n; j++) c[i * n + j] = 0.0f;
        for (size_t l = 0; l < k; l++) {
            float av = t_to_f32(a[i * k + l], bf16);
            for (size_t j = 0; j < n; j++) c[i * n + j] += av * t_to_f32(b[l * n + j], bf16);
        }
    }
}
void orc_gemm16(size_t m, size_t n, size_t k, uint16_t *c, const uint16_t *a, const uint16_t *b,
                int bf16) {
    orc_gemm16_rows(m, n, k, c, a, b, bf16, 0, m);
}

/* ------------------------------------------------------------------ */
/* epilogue op-graph                                                   */
/* ------------------------------------------------------------------ */

/* Byte-identical to EpNode in csrc/epilogue.h:214-229. */
typedef struct {
    uint32_t op;
    uint32_t aux;
    float scalar;
    const void *ptr;
    size_t ld;
} OrcEpNode;

static double clampd(double x, double lo, double hi) { /* f64::clamp: NaN stays NaN */
    if (x < lo) return lo;
    if (x > hi) return hi;
    return x;
}

/* erf_approx, src/epilogue/mod.rs:92-103 (Abramowitz-Stegun 7.1.26). */
static double erf_as(double x) {
    double ax = fabs(x);
    double t = 1.0 / (1.0 + 0.3275911 * ax);
    double poly =
        ((((1.061405429 * t - 1.453152027) * t + 1.421413741) * t - 0.284496736) * t + 0.254829592) * t;
    double e = 1.0 - poly * exp(-ax * ax);
    return x < 0.0 ? -e : e;
}

/* act_apply_f64_a, src/epilogue/mod.rs:40-86. */
double orc_act_f64(uint32_t kind, double x, double alpha) {
    switch (kind) {
    case 1: return fmax(x, 0.0);
    case 2: return 0.5 * x * (1.0 + tanh(0.7978845608028654 * (x + 0.044715 * x * x * x)));
    case 3: return x / (1.0 + exp(-x));
    case 4: return tanh(x);
    case 5: return 1.0 / (1.0 + exp(-x));
    case 6: return x >= 0.0 ? x : alpha * x;
    case 7: return clampd(x, 0.0, 6.0);
    case 8: return clampd(x / 6.0 + 0.5, 0.0, 1.0);
    case 9: return x * clampd(x / 6.0 + 0.5, 0.0, 1.0);
    case 10: return fabs(x);
    case 11: return -x;
    case 12: return x * x;
    case 13: return x > 0.0 ? 1.0 : (x < 0.0 ? -1.0 : 0.0);
    case 14: return sqrt(x);
    case 15: return x / (1.0 + fabs(x));
    case 16: return 1.0 / x;
    case 17: return 1.0 / sqrt(x);
    case 18: return exp(x);
    case 19: return log(x);
    case 20: return x >= 0.0 ? x : alpha * expm1(x);
    case 21: return 1.0507009873554805 * (x >= 0.0 ? x : 1.6732632423543772 * expm1(x));
    case 22: return fmax(x, 0.0) + log1p(exp(-fabs(x)));
    case 23: return x * tanh(fmax(x, 0.0) + log1p(exp(-fabs(x))));
    case 24: return 0.5 * x * (1.0 + erf_as(x * 0.70710678118654752440));
    default: return x;
    }
}

/* ep_apply_cell, src/exec/scalar.rs:58-120, over an already resolved node
 * list (trailing activation appended as a final Act node with scalar 0, as
 * resolve_nodes does, src/exec/scalar.rs:28-53).  Every node is one rounded
 * f32 operation; activations widen to f64 and narrow. */
static float ep_cell(const OrcEpNode *nodes, uint32_t nn, float x, size_t i, size_t j, size_t n,
                     int bf16) {
    for (uint32_t q = 0; q < nn; q++) {
        const OrcEpNode *nd = &nodes[q];
        const uint16_t *p = (const uint16_t *)nd->ptr;
        size_t ld = nd->ld == 0 ? n : nd->ld;
#define RD(IDX) t_to_f32(p[(IDX)], bf16)
        switch (nd->op) {
        case 0: x += nd->scalar; break;
        case 1: x *= nd->scalar; break;
        case 2: x += RD(i); break;
        case 3: x *= RD(i); break;
        case 4: x += RD(j); break;
        case 5: x *= RD(j); break;
        case 6: x += RD(i * ld + j); break;
        case 7: x *= RD(i * ld + j); break;
        case 8: x = (float)orc_act_f64(nd->aux, (double)x, (double)nd->scalar); break;
        case 9: x = fmaxf(x, nd->scalar); break;
        case 10: x = fminf(x, nd->scalar); break;
        case 11: x -= nd->scalar; break;
        case 12: x -= RD(i); break;
        case 13: x -= RD(j); break;
        case 14: x -= RD(i * ld + j); break;
        case 15: x /= nd->scalar; break;
        case 16: x /= RD(i); break;
        case 17: x /= RD(j); break;
        case 18: x /= RD(i * ld + j); break;
        case 19: x = fmaxf(x, RD(i)); break;
        case 20: x = fmaxf(x, RD(j)); break;
        case 21: x = fmaxf(x, RD(i * ld + j)); break;
        case 22: x = fminf(x, RD(i)); break;
        case 23: x = fminf(x, RD(j)); break;
        case 24: x = fminf(x, RD(i * ld + j)); break;
        default: break;
        }
#undef RD
    }
    return x;
}

/* apply_ep_scalar, src/exec/scalar.rs:125-140: read the stored T value, run
 * the graph in f32, round back to T.  c row-major m x n, rows first.. only. */
void orc_apply_ep_rows(uint16_t *c, size_t m, size_t n, const OrcEpNode *nodes, uint32_t nn,
                       int bf16, size_t first, size_t rows) {
    (void)m;
    if (nn == 0) return;
    for (size_t i = first; i < first + rows; i++)
        for (size_t j = 0; j < n; j++)
            c[i * n + j] = f32_to_t(ep_cell(nodes, nn, t_to_f32(c[i * n + j], bf16), i, j, n, bf16), bf16);
}
void orc_apply_ep(uint16_t *c, size_t m, size_t n, const OrcEpNode *nodes, uint32_t nn, int bf16) {
    orc_apply_ep_rows(c, m, n, nodes, nn, bf16, 0, m);
}

/* matmul_q4_ep / matmul_q4_bf16_ep off Apple hardware,
 * src/kernels/q4/matmul.rs:93-102 and :257-270: dequantise to row-major T,
 * dense reference GEMM, scalar epilogue.  `wdeq` (k*n T) may be passed in to
 * skip the per-call dequant (the timed "dequant excluded" variant); NULL
 * dequantises here. */
void orc_matmul_q4(const uint16_t *a, const uint8_t *quants, const uint16_t *scales,
                   const uint16_t *mins, size_t n, size_t k, size_t block, uint16_t *c, size_t m,
                   const OrcEpNode *nodes, uint32_t nn, int bf16, const uint16_t *wdeq,
                   size_t first, size_t rows) {
    uint16_t *tmp = NULL;
    if (m == 0 || n == 0) return;
    if (!wdeq) {
        tmp = (uint16_t *)malloc(sizeof(uint16_t) * (k * n ? k * n : 1));
        orc_q4_dequant(quants, scales, mins, n, k, block, bf16, tmp);
        wdeq = tmp;
    }
    orc_gemm16_rows(m, n, k, c, a, wdeq, bf16, first, rows);
    orc_apply_ep_rows(c, m, n, nodes, nn, bf16, first, rows);
    free(tmp);
}

/* ------------------------------------------------------------------ */
/* 2-bit / 1-bit: quantise, int8 activation path, mopa weights         */
/* ------------------------------------------------------------------ */

/* Logical (unpacked) weight formats used by the oracle:
 *   q2: codes four to a byte, weight idx = d*n+j at bits 2*(idx%4) of byte
 *       idx/4 (the input format of Q2Weights::new, src/kernels/lowbit/q2.rs:43-47)
 *   q1: signs one bit per weight, idx = j*k+d (OutIn, layout 0) or d*n+j
 *       (InOut, layout 1), low bit first, 1 = +scale
 *       (Q1Weights::new, src/kernels/lowbit/q1.rs:35-41)
 *   scales: [j*nbk + blk] f16 bits. */

static inline int q2_code(const uint8_t *codes, size_t n, size_t d, size_t j) {
    size_t idx = d * n + j;
    return (codes[idx / 4] >> (2 * (idx % 4))) & 3;
}
static inline int q1_sign(const uint8_t *signs, int layout, size_t n, size_t k, size_t d, size_t j) {
    size_t idx = layout == 0 ? j * k + d : d * n + j;
    return (signs[idx / 8] >> (idx % 8)) & 1;
}

/* Q2Weights::quantize, src/kernels/lowbit/q2.rs:110-144.  Returns -1 for an
 * all-zero codebook (the reference panics). */
int orc_q2_quantize(const float *w, int layout, size_t n, size_t k, size_t block,
                    const int8_t codebook[4], uint8_t *codes, uint16_t *scales) {
    float cb[4], cmax = 0.0f;
    for (int i = 0; i < 4; i++) {
        cb[i] = (float)codebook[i];
        cmax = fmaxf(cmax, fabsf(cb[i]));
    }
    if (!(cmax > 0.0f)) return -1;
    size_t nbk = (k + block - 1) / block;
    memset(codes, 0, (k * n + 3) / 4);
    for (size_t j = 0; j < n; j++)
        for (size_t b = 0; b < nbk; b++) {
            size_t d0 = b * block, d1 = (b + 1) * block < k ? (b + 1) * block : k;
#define AT(J, D) (layout == 0 ? w[(J) * k + (D)] : w[(D) * n + (J)])
            float amax = 0.0f;
            for (size_t d = d0; d < d1; d++) amax = fmaxf(amax, fabsf(AT(j, d)));
            scales[j * nbk + b] = orc_f32_to_f16(amax / cmax);
            float s = orc_f16_to_f32(scales[j * nbk + b]);
            for (size_t d = d0; d < d1; d++) {
                float x = AT(j, d);
                int best = 0;
                float bd = fabsf(x - s * cb[0]);
                for (int c = 1; c < 4; c++) { /* nearest value, ties to the lower code */
                    float dd = fabsf(x - s * cb[c]);
                    if (dd < bd) { bd = dd; best = c; }
                }
                size_t idx = d * n + j;
                codes[idx / 4] |= (uint8_t)(best << (2 * (idx % 4)));
            }
#undef AT
        }
    return 0;
}

/* Q1Weights::quantize, src/kernels/lowbit/q1.rs:116-144.  Signs come out in
 * OutIn bit order (idx = j*k+d). */
void orc_q1_quantize(const float *w, int layout, size_t n, size_t k, size_t block, uint8_t *signs,
                     uint16_t *scales) {
    size_t nbk = (k + block - 1) / block;
    memset(signs, 0, (k * n + 7) / 8);
    for (size_t j = 0; j < n; j++)
        for (size_t b = 0; b < nbk; b++) {
            size_t d0 = b * block, d1 = (b + 1) * block < k ? (b + 1) * block : k;
#define AT(J, D) (layout == 0 ? w[(J) * k + (D)] : w[(D) * n + (J)])
            float sum = 0.0f;
            for (size_t d = d0; d < d1; d++) sum += fabsf(AT(j, d));
            scales[j * nbk + b] = orc_f32_to_f16(sum / (float)(d1 - d0));
            for (size_t d = d0; d < d1; d++)
                if (AT(j, d) >= 0.0f) {
                    size_t idx = j * k + d;
                    signs[idx / 8] |= (uint8_t)(1u << (idx % 8));
                }
#undef AT
        }
}

/* quantize_row, src/kernels/lowbit/matmul.rs:354-371: per K-block amax (NaN
 * sticky), inv = amax > 0 ? 127/amax : 0, s = amax/127,
 * q = saturating_i8(round_ties_even(f32(a) * inv)), NaN -> 0. */
void orc_quantize_row(const uint16_t *a, size_t k, size_t block, int8_t *q, float *s) {
    size_t nbk = (k + block - 1) / block;
    for (size_t b = 0; b < nbk; b++) {
        size_t d0 = b * block, d1 = (b + 1) * block < k ? (b + 1) * block : k;
        float amax = 0.0f;
        for (size_t d = d0; d < d1; d++) {
            float x = fabsf(orc_f16_to_f32(a[d]));
            if (isnan(x) || isnan(amax)) amax = NAN;
            else amax = fmaxf(amax, x);
        }
        float inv = amax > 0.0f ? 127.0f / amax : 0.0f;
        s[b] = amax / 127.0f;
        for (size_t d = d0; d < d1; d++) {
            float r = rintf(orc_f16_to_f32(a[d]) * inv); /* default mode: ties to even */
            int v;
            if (isnan(r)) v = 0;
            else if (r <= -128.0f) v = -128;
            else if (r >= 127.0f) v = 127;
            else v = (int)r;
            q[d] = (int8_t)v;
        }
    }
}

/* reference(), src/kernels/lowbit/matmul.rs:376-398: exact i32 block sums,
 * total = fmaf((float)sum, scale(blk,j) * sa[blk], total) in K order, f16
 * store; k == 0 gives zeros.  kind 2 = 2-bit (wbits = codes, codebook used),
 * kind 1 = 1-bit (wbits = signs in `layout`).  Optional debug outputs (NULL to
 * skip): q_out m*k int8, sa_out m*nbk f32, sums_out m*n*nbk i32. */
typedef struct {
    const uint16_t *a, *scales; size_t n, k, block, nbk; uint16_t *c;
    int8_t *q_out; float *sa_out; int32_t *sums_out; const int8_t *val;
} lb_ctx;
static void lb_row(size_t i, void *p, void *scratch) {
    lb_ctx *L = (lb_ctx *)p;
    size_t n = L->n, k = L->k, nbk = L->nbk, block = L->block;
    /* carve the scratch: s | sum | total | q (4-byte aligned parts first) */
    float *s = (float *)scratch;
    int32_t *sum = (int32_t *)(s + nbk + 1);
    float *total = (float *)(sum + n);
    int8_t *q = (int8_t *)(total + n);
    orc_quantize_row(L->a + i * k, k, block, q, s);
    if (L->q_out) memcpy(L->q_out + i * k, q, k);
    if (L->sa_out) memcpy(L->sa_out + i * nbk, s, sizeof(float) * nbk);
    for (size_t j = 0; j < n; j++) total[j] = 0.0f;
    for (size_t b = 0; b < nbk; b++) {
        size_t d0 = b * block, d1 = (b + 1) * block < k ? (b + 1) * block : k;
        for (size_t j = 0; j < n; j++) sum[j] = 0;
        for (size_t d = d0; d < d1; d++) {
            int32_t qv = q[d];
            const int8_t *vr = L->val + d * n;
            for (size_t j = 0; j < n; j++) sum[j] += qv * (int32_t)vr[j];
        }
        for (size_t j = 0; j < n; j++) {
            if (L->sums_out) L->sums_out[(i * n + j) * nbk + b] = sum[j];
            float sc = orc_f16_to_f32(L->scales[j * nbk + b]);
            total[j] = fmaf((float)sum[j], sc * s[b], total[j]);
        }
    }
    for (size_t j = 0; j < n; j++) L->c[i * n + j] = orc_f32_to_f16(total[j]);
}
void orc_lowbit_matmul(const uint16_t *a, int kind, const uint8_t *wbits, int layout,
                       const uint16_t *scales, const int8_t *codebook, size_t n, size_t k,
                       size_t block, uint16_t *c, size_t m, int8_t *q_out, float *sa_out,
                       int32_t *sums_out) {
    size_t nbk = (k + block - 1) / block;
    if (m == 0 || n == 0) return;
    /* the weights' int8 values, expanded once: val[d*n+j] */
    int8_t *val = (int8_t *)malloc(k * n ? k * n : 1);
    for (size_t d = 0; d < k; d++)
        for (size_t j = 0; j < n; j++)
            val[d * n + j] = kind == 2 ? codebook[q2_code(wbits, n, d, j)]
                                       : (q1_sign(wbits, layout, n, k, d, j) ? 1 : -1);
    lb_ctx L = {a, scales, n, k, block, nbk, c, q_out, sa_out, sums_out, val};
    par_for(0, m, lb_row, &L, k + 16 + (sizeof(float) + 0) * (nbk + 1) + (sizeof(int32_t) + sizeof(float)) * n + 64);
    free(val);
}

/* Codes::dequant, src/kernels/lowbit/matmul.rs:178-197: the f16 weights the
 * mopa path multiplies: f16(s * codebook[code]) or +-s; row-major k x n. */
void orc_lowbit_dequant(int kind, const uint8_t *wbits, int layout, const uint16_t *scales,
                        const int8_t *codebook, size_t n, size_t k, size_t block, uint16_t *out) {
    size_t nbk = (k + block - 1) / block;
    for (size_t d = 0; d < k; d++)
        for (size_t j = 0; j < n; j++) {
            float s = orc_f16_to_f32(scales[j * nbk + d / block]);
            float v = kind == 2 ? s * (float)codebook[q2_code(wbits, n, d, j)]
                                : (q1_sign(wbits, layout, n, k, d, j) ? s : -s);
            out[d * n + j] = orc_f32_to_f16(v);
        }
}

/* ------------------------------------------------------------------ */
/* MLP block pieces                                                    */
/* ------------------------------------------------------------------ */

/* glu(), src/linear.rs:804-835 (portable arm): 32-column interleave, f32 math
 * with f32 libm, f16 store.  gate_kind 3 = silu, 2 = gelu (tanh form). */
void orc_glu(uint16_t *y, const uint16_t *both, size_t m, size_t n, int gate_kind) {
    for (size_t i = 0; i < m; i++) {
        const uint16_t *br = both + i * 2 * n;
        uint16_t *yr = y + i * n;
        for (size_t c0 = 0; c0 < n; c0 += 32) {
            size_t w = n - c0 < 32 ? n - c0 : 32;
            for (size_t j = 0; j < w; j++) {
                float g = orc_f16_to_f32(br[2 * c0 + j]), u = orc_f16_to_f32(br[2 * c0 + w + j]);
                float a;
                if (gate_kind == 3) a = g / (1.0f + expf(-g));
                else a = 0.5f * g * (1.0f + tanhf(0.7978846f * (g + 0.044715f * g * g * g)));
                yr[c0 + j] = orc_f32_to_f16(a * u);
            }
        }
    }
}

/* convert::add_f16, src/convert.rs:37-48: dst (f32) += f32(src f16). */
void orc_add_f16(const uint16_t *src, float *dst, size_t len) {
    for (size_t i = 0; i < len; i++) dst[i] += orc_f16_to_f32(src[i]);
}

/* lane_sum, src/nn.rs:20-32: eight running sums over whole groups of eight, their sum
 * (in index order) plus the tail's sum.  sq: sum of (x - mean)^2, else of x. */
static float orc_lane_sum(const float *x, size_t n, float mean, int sq) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    size_t whole = n / 8 * 8;
    for (size_t i = 0; i < whole; i += 8)
        for (int l = 0; l < 8; l++) {
            float v = x[i + l];
            acc[l] += sq ? (v - mean) * (v - mean) : v;
        }
    float tail = 0.0f;
    for (size_t i = whole; i < n; i++) {
        float v = x[i];
        tail += sq ? (v - mean) * (v - mean) : v;
    }
    float sum = 0.0f;
    for (int l = 0; l < 8; l++) sum += acc[l];
    return sum + tail;
}

/* layer_norm / rms_norm rows, portable arm of norm_row (src/nn.rs:126-153), f32 in, rounded to
 * f16 (y16) and / or kept as f32 (y32): (v - mean) * r * w + b with r = 1 / sqrt(ss / dim + eps). */
void orc_norm_rows(const float *x, const float *weight, const float *bias, float eps, int rms, size_t rows,
                   size_t dim, uint16_t *y16, float *y32) {
    for (size_t i = 0; i < rows; i++) {
        const float *xr = x + i * dim;
        float fdim = (float)dim;
        float mean = rms ? 0.0f : orc_lane_sum(xr, dim, 0.0f, 0) / fdim;
        float r = 1.0f / sqrtf(orc_lane_sum(xr, dim, mean, 1) / fdim + eps);
        for (size_t j = 0; j < dim; j++) {
            float o = (xr[j] - mean) * r * weight[j] + (bias ? bias[j] : 0.0f);
            if (y16) y16[i * dim + j] = orc_f32_to_f16(o);
            if (y32) y32[i * dim + j] = o;
        }
    }
}

/* rms_scales, src/nn.rs:234-248: out[i] = f16(1 / sqrt(mean(x_i^2) + eps)) per k-wide f16 row. */
void orc_rms_scales(const uint16_t *x, size_t rows, size_t k, float eps, uint16_t *out) {
    for (size_t i = 0; i < rows; i++) {
        const uint16_t *xr = x + i * k;
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        size_t whole = k / 8 * 8;
        for (size_t d = 0; d < whole; d += 8)
            for (int l = 0; l < 8; l++) {
                float v = orc_f16_to_f32(xr[d + l]);
                acc[l] += v * v;
            }
        float tail = 0.0f;
        for (size_t d = whole; d < k; d++) {
            float v = orc_f16_to_f32(xr[d]);
            tail += v * v;
        }
        float sum = 0.0f;
        for (int l = 0; l < 8; l++) sum += acc[l];
        float ms = (sum + tail) / (float)k;
        out[i] = orc_f32_to_f16(1.0f / sqrtf(ms + eps));
    }
}

/* interleave(), src/linear.rs:603-617: [gate | up] as k x 2n row-major,
 * 32 gate columns then 32 up columns per chunk.  g, u: k x n row-major
 * (InOut).  Generic over element size `es` bytes. */
void orc_interleave(const void *g, const void *u, size_t n, size_t k, size_t es, void *out) {
    const uint8_t *gp = (const uint8_t *)g, *up = (const uint8_t *)u;
    uint8_t *op = (uint8_t *)out;
    for (size_t d = 0; d < k; d++)
        for (size_t c0 = 0; c0 < n; c0 += 32) {
            size_t c1 = c0 + 32 < n ? c0 + 32 : n;
            size_t len = (c1 - c0) * es;
            memcpy(op, gp + (d * n + c0) * es, len); op += len;
            memcpy(op, up + (d * n + c0) * es, len); op += len;
        }
}

/* Mlp::accumulate, gated arm, src/mlp.rs:113-146 with GatedLinear::forward
 * (src/linear.rs:779-788): both = x @ dequant(W_gateup) (m x 2h, f16),
 * hid = glu(both), out = hid @ dequant(W_down) (f16), y (f32) += f32(out).
 * Weights come as logical Q4 arrays (quants/scales as orc_q4_quantize writes
 * them); gate/up already interleaved into one 2h-column matrix.  Rows
 * first..first+rows-1 of the m rows are computed. */
void orc_mlp_accumulate(const uint16_t *x, float *y, size_t m, size_t d_model, size_t hidden,
                        const uint8_t *gu_quants, const uint16_t *gu_scales,
                        const uint8_t *dn_quants, const uint16_t *dn_scales, size_t block,
                        int gate_kind, size_t first, size_t rows) {
    size_t n2 = 2 * hidden;
    uint16_t *both = (uint16_t *)calloc(m * n2 ? m * n2 : 1, 2);
    uint16_t *hid = (uint16_t *)calloc(m * hidden ? m * hidden : 1, 2);
    uint16_t *out = (uint16_t *)calloc(m * d_model ? m * d_model : 1, 2);
    orc_matmul_q4(x, gu_quants, gu_scales, NULL, n2, d_model, block, both, m, NULL, 0, 0, NULL, first, rows);
    orc_glu(hid + first * hidden, both + first * n2, rows, hidden, gate_kind);
    orc_matmul_q4(hid, dn_quants, dn_scales, NULL, d_model, hidden, block, out, m, NULL, 0, 0, NULL, first, rows);
    orc_add_f16(out + first * d_model, y + first * d_model, rows * d_model);
    free(both); free(hid); free(out);
}

/* ------------------------------------------------------------------ */
/* the reference's packed (band-major) layouts, for the drop-in tests   */
/* ------------------------------------------------------------------ */

/* Q4Weights::with_params, src/kernels/q4/weights.rs:63-123: 128-column bands,
 * byte b*k*64 + d*64 + c/2, nibble c%2; scales [band][blk][128]. */
size_t orc_q4_band_nibble_bytes(size_t n, size_t k) { return ((n + 127) / 128) * k * 64; }
size_t orc_q4_band_scale_elems(size_t n, size_t k, size_t block) {
    return ((n + 127) / 128) * ((k + block - 1) / block) * 128;
}
void orc_q4_pack_band(const uint8_t *quants, const uint16_t *scales, const uint16_t *mins, size_t n,
                      size_t k, size_t block, uint8_t *nibbles, uint16_t *sc, uint16_t *mn) {
    size_t nbk = (k + block - 1) / block;
    memset(nibbles, 0, orc_q4_band_nibble_bytes(n, k));
    memset(sc, 0, 2 * orc_q4_band_scale_elems(n, k, block));
    if (mn) memset(mn, 0, 2 * orc_q4_band_scale_elems(n, k, block));
    for (size_t d = 0; d < k; d++)
        for (size_t j = 0; j < n; j++) {
            size_t idx = d * n + j;
            uint8_t nib = (idx % 2 == 0) ? (quants[idx / 2] & 0x0f) : (quants[idx / 2] >> 4);
            size_t b = j / 128, c = j % 128;
            nibbles[b * k * 64 + d * 64 + c / 2] |= (uint8_t)(nib << (4 * (c % 2)));
        }
    for (size_t j = 0; j < n; j++)
        for (size_t blk = 0; blk < nbk; blk++) {
            size_t dst = (j / 128) * nbk * 128 + blk * 128 + j % 128;
            sc[dst] = scales[j * nbk + blk];
            if (mn && mins) mn[dst] = mins[j * nbk + blk];
        }
}

/* scale_index, src/kernels/lowbit/q2.rs:17-20. */
static size_t lb_scale_index(size_t sc_per_band, size_t blk, size_t j) {
    size_t c = j % 64;
    return (j / 64) * sc_per_band + blk * 64 + (c / 32) * 32 + 2 * (c % 16) + (c % 32) / 16;
}
size_t orc_q2_band_code_bytes(size_t n, size_t k) { return ((n + 63) / 64) * ((k + 15) / 16 * 16) * 16; }
size_t orc_q1_band_sign_bytes(size_t n, size_t k) { return ((n + 63) / 64) * ((k + 15) / 16 * 16) * 8; }
size_t orc_lowbit_band_scale_elems(size_t n, size_t k, size_t block) {
    return ((n + 63) / 64) * ((k + block - 1) / block) * 64;
}
/* Q2Weights::new, src/kernels/lowbit/q2.rs:48-84. */
void orc_q2_pack_band(const uint8_t *codes, const uint16_t *scales, size_t n, size_t k, size_t block,
                      uint8_t *packed, uint16_t *sc) {
    size_t nbk = (k + block - 1) / block;
    size_t band_bytes = ((k + 15) / 16 * 16) * 16, spb = nbk * 64;
    memset(packed, 0, orc_q2_band_code_bytes(n, k));
    memset(sc, 0, 2 * orc_lowbit_band_scale_elems(n, k, block));
    for (size_t d = 0; d < k; d++)
        for (size_t j = 0; j < n; j++) {
            int code = q2_code(codes, n, d, j);
            packed[(j / 64) * band_bytes + (d / 4) * 64 + j % 64] |= (uint8_t)(code << (2 * (d % 4)));
        }
    for (size_t j = 0; j < n; j++)
        for (size_t blk = 0; blk < nbk; blk++) sc[lb_scale_index(spb, blk, j)] = scales[j * nbk + blk];
}
/* Q1Weights::new, src/kernels/lowbit/q1.rs:47-106 (bit(): :195-201). */
void orc_q1_pack_band(const uint8_t *signs, int layout, const uint16_t *scales, size_t n, size_t k,
                      size_t block, uint8_t *packed, uint16_t *sc) {
    size_t nbk = (k + block - 1) / block;
    size_t band_bytes = ((k + 15) / 16 * 16) * 8, spb = nbk * 64;
    memset(packed, 0, orc_q1_band_sign_bytes(n, k));
    memset(sc, 0, 2 * orc_lowbit_band_scale_elems(n, k, block));
    for (size_t j = 0; j < n; j++) {
        for (size_t d = 0; d < k; d++)
            if (q1_sign(signs, layout, n, k, d, j)) {
                size_t c = j % 64;
                packed[(j / 64) * band_bytes + (d / 4) * 32 + c / 2] |= (uint8_t)(1u << (4 * (c % 2) + d % 4));
            }
        for (size_t blk = 0; blk < nbk; blk++) sc[lb_scale_index(spb, blk, j)] = scales[j * nbk + blk];
    }
}

/* attention_kv_causal_f16, portable arm (src/kernels/kv_attention.rs:155-242 with one_row :281-331): query row i of
 * `rows` attends to keys 0..=start+i of an f16 cache whose rows hold kv_heads * head_dim values; per head
 * softmax(f16(q * scale) . k) @ v with f32 sums in key / depth order, probabilities exp(s - max) in f32, the division
 * by their sum last.  q and out are [rows][heads][head_dim] f32.  (attention_kv_f16, :29-139, is rows = 1 with
 * start = len - 1.) */
void orc_attention_kv_causal(const float *q, const uint16_t *k, const uint16_t *v, size_t start, size_t rows,
                             size_t heads, size_t kv_heads, size_t head_dim, float scale, float *out) {
    size_t ld = kv_heads * head_dim, qr = heads * head_dim, group = heads / kv_heads;
    float *scores = (float *)malloc((start + rows) * sizeof(float));
    float *qh = (float *)malloc(head_dim * sizeof(float));
    for (size_t i = 0; i < rows; i++) {
        size_t len = start + i + 1;
        for (size_t h = 0; h < heads; h++) {
            size_t off = (h / group) * head_dim;
            for (size_t d = 0; d < head_dim; d++) qh[d] = orc_f16_to_f32(orc_f32_to_f16(q[i * qr + h * head_dim + d] * scale));
            float mx = -INFINITY;
            for (size_t t = 0; t < len; t++) {
                float s = 0.0f;
                for (size_t d = 0; d < head_dim; d++) s += qh[d] * orc_f16_to_f32(k[t * ld + off + d]);
                scores[t] = s;
                mx = s > mx ? s : mx;          /* f32::max */
            }
            float sum = 0.0f;
            for (size_t t = 0; t < len; t++) {
                scores[t] = expf(scores[t] - mx);
                sum += scores[t];
            }
            float *oh = out + i * qr + h * head_dim;
            for (size_t d = 0; d < head_dim; d++) oh[d] = 0.0f;
            for (size_t t = 0; t < len; t++)
                for (size_t d = 0; d < head_dim; d++) oh[d] += scores[t] * orc_f16_to_f32(v[t * ld + off + d]);
            for (size_t d = 0; d < head_dim; d++) oh[d] /= sum;
        }
    }
    free(scores);
    free(qh);
}
