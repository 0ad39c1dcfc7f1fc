// The fused epilogue op-graph, evaluated per output cell at the C store.
//
// Semantics follow the reference's scalar evaluator exactly (ep_apply_cell,
// src/exec/scalar.rs:58-120, reached through apply_ep_scalar :125-140): the
// product is first rounded to the output type T, widened to f32, every node is
// one separately rounded f32 operation (no fused multiply-add), MAX/MIN are
// maxNum/minNum, and the result is rounded to T once more.  Named trailing
// activations arrive here already appended as a final ACT node
// (resolve_nodes, src/exec/scalar.rs:28-53).
//
// The opcodes and activation kinds are the values of enum ep_op / enum ep_act in
// csrc/epilogue.h:136-200 of the reference.
#pragma once
#include "common.cuh"

namespace smeg {

constexpr int kMaxInlineNodes = 16;

struct EpNodeDev {
    uint32_t op;       // low 8 bits: opcode; bits 8..15: activation kind
    float scalar;      // *_SCALAR operand, or alpha of leaky_relu / elu
    const uint16_t* ptr;  // ROW / COL / TENSOR operand (T bit patterns), device memory
    size_t ld;         // TENSOR row stride in elements (already resolved, never 0)
};

struct EpParams {
    int n_nodes;                       // 0 = identity
    const EpNodeDev* ext;              // device array when n_nodes > kMaxInlineNodes
    EpNodeDev nodes[kMaxInlineNodes];  // inline copy otherwise
};

// Activations whose reference definition is cheap and exact in f64, or rare:
// evaluated in double like the reference (act_apply_f64_a,
// src/epilogue/mod.rs:40-86) and narrowed once.
static __device__ __noinline__ float act_rare(uint32_t kind, float xf, float alphaf) {
    double x = (double)xf, alpha = (double)alphaf, r = x;
    switch (kind) {
    case 6: r = x >= 0.0 ? x : alpha * x; break;
    case 7: r = x < 0.0 ? 0.0 : (x > 6.0 ? 6.0 : x); break;
    case 8: { double t = x / 6.0 + 0.5; r = t < 0.0 ? 0.0 : (t > 1.0 ? 1.0 : t); } break;
    case 9: { double t = x / 6.0 + 0.5; r = x * (t < 0.0 ? 0.0 : (t > 1.0 ? 1.0 : t)); } break;
    case 10: r = fabs(x); break;
    case 11: r = -x; break;
    case 12: r = x * x; break;
    case 13: r = x > 0.0 ? 1.0 : (x < 0.0 ? -1.0 : 0.0); break;
    case 14: r = sqrt(x); break;
    case 15: r = x / (1.0 + fabs(x)); break;
    case 16: r = 1.0 / x; break;
    case 17: r = 1.0 / sqrt(x); break;
    case 18: r = exp(x); break;
    case 19: r = log(x); break;
    case 20: r = x >= 0.0 ? x : alpha * expm1(x); break;
    case 21: r = 1.0507009873554805 * (x >= 0.0 ? x : 1.6732632423543772 * expm1(x)); break;
    case 22: r = fmax(x, 0.0) + log1p(exp(-fabs(x))); break;
    case 23: r = x * tanh(fmax(x, 0.0) + log1p(exp(-fabs(x)))); break;
    case 24: {  // Abramowitz-Stegun 7.1.26 erf, as src/epilogue/mod.rs:92-103
        double z = x * 0.70710678118654752440, az = fabs(z);
        double t = 1.0 / (1.0 + 0.3275911 * az);
        double poly = ((((1.061405429 * t - 1.453152027) * t + 1.421413741) * t - 0.284496736) * t + 0.254829592) * t;
        double e = 1.0 - poly * exp(-az * az);
        r = 0.5 * x * (1.0 + (z < 0.0 ? -e : e));
    } break;
    default: break;
    }
    return (float)r;
}

// The five named activations (relu, gelu, silu, tanh, sigmoid) run in f32 with
// the accurate libdevice functions: within a couple of f32 ulps of the f64
// reference value, far inside the output type's rounding.
__device__ __forceinline__ float act_apply(uint32_t kind, float x, float alpha) {
    switch (kind) {
    case 0: return x;
    case 1: return fmaxf(x, 0.0f);
    case 2: return 0.5f * x * (1.0f + tanhf(0.7978845608f * (x + 0.044715f * x * x * x)));
    case 3: return __fdiv_rn(x, 1.0f + expf(-x));
    case 4: return tanhf(x);
    case 5: return __fdiv_rn(1.0f, 1.0f + expf(-x));
    default: return act_rare(kind, x, alpha);
    }
}

template <int BF16>
__device__ __forceinline__ float ep_node(const EpNodeDev& nd, float x, size_t i, size_t j) {
    const uint32_t op = nd.op & 0xffu;
    float o = nd.scalar;
    switch (op) {
    case 2: case 3: case 12: case 16: case 19: case 22: o = t_to_f32<BF16>(nd.ptr[i]); break;
    case 4: case 5: case 13: case 17: case 20: case 23: o = t_to_f32<BF16>(nd.ptr[j]); break;
    case 6: case 7: case 14: case 18: case 21: case 24: o = t_to_f32<BF16>(nd.ptr[i * nd.ld + j]); break;
    default: break;
    }
    switch (op) {
    case 0: case 2: case 4: case 6: return __fadd_rn(x, o);
    case 1: case 3: case 5: case 7: return __fmul_rn(x, o);
    case 11: case 12: case 13: case 14: return __fsub_rn(x, o);
    case 15: case 16: case 17: case 18: return __fdiv_rn(x, o);
    case 9: case 19: case 20: case 21: return fmaxf(x, o);
    case 10: case 22: case 23: case 24: return fminf(x, o);
    case 8: return act_apply((nd.op >> 8) & 0xffu, x, nd.scalar);
    default: return x;
    }
}

// Same, over an explicit node array (shared or global memory).  Out of line: the interpreter
// with every activation inlined is large, and the callers sit in unrolled loops.
template <int BF16>
__device__ __noinline__ uint16_t ep_store_nodes(const EpNodeDev* nodes, int nn, float acc, size_t i, size_t j) {
    uint16_t c = f32_to_t<BF16>(acc);
    if (nn == 0) return c;
    float x = t_to_f32<BF16>(c);
#pragma unroll 1
    for (int q = 0; q < nn; ++q) x = ep_node<BF16>(nodes[q], x, i, j);
    return f32_to_t<BF16>(x);
}

// acc (f32 accumulator) -> stored T bits at output cell (i, j).  `ep` must be addressable
// (a __grid_constant__ kernel parameter, or a copy in shared memory): the interpreter is one
// out-of-line function, so that kernels which store from unrolled loops do not carry a copy of
// every activation per store.
template <int BF16>
__device__ __forceinline__ uint16_t ep_store_value(const EpParams& ep, float acc, size_t i, size_t j) {
    const int nn = ep.n_nodes;
    if (nn == 0) return f32_to_t<BF16>(acc);
    return ep_store_nodes<BF16>(nn <= kMaxInlineNodes ? ep.nodes : ep.ext, nn, acc, i, j);
}

// A graph of at most four nodes whose operands are scalars or per-column vectors and
// whose activations are the five named kinds, resolved once per thread for the
// thread's output column: the per-cell work is then four predictable steps on
// registers.  Arithmetic is the interpreter's (separately rounded f32 ops on the
// T-rounded product); silu and sigmoid use the fast exponential and division, whose
// error (about 1e-6 relative) is three orders below the 16-bit output's rounding.
struct FastEp {
    int n;
    int cls[4];     // 1 add, 2 mul, 3 sub, 4 div, 5 max, 6 min, 8 + kind for an activation
    float v[4];
};

// Host-side test: can this resolved graph run as a FastEp?
inline bool fast_ep_eligible(const EpParams& ep) {
    if (ep.n_nodes < 1 || ep.n_nodes > 4) return false;
    for (int q = 0; q < ep.n_nodes; ++q) {
        const uint32_t op = ep.nodes[q].op & 0xffu, kind = (ep.nodes[q].op >> 8) & 0xffu;
        const bool scalar = op == 0 || op == 1 || op == 9 || op == 10 || op == 11 || op == 15;
        const bool col = op == 4 || op == 5 || op == 13 || op == 17 || op == 20 || op == 23;
        if (!(scalar || col || (op == 8 && kind >= 1 && kind <= 5))) return false;
    }
    return true;
}

template <int BF16>
__device__ __forceinline__ void fast_ep_build(const EpNodeDev* nodes, int nn, int col, bool col_ok, FastEp& f) {
    f.n = nn;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        f.cls[q] = 0;
        f.v[q] = 0.0f;
        if (q < nn) {
            const uint32_t op = nodes[q].op & 0xffu;
            int cls = 0;
            switch (op) {
            case 0: case 4: cls = 1; break;
            case 1: case 5: cls = 2; break;
            case 11: case 13: cls = 3; break;
            case 15: case 17: cls = 4; break;
            case 9: case 20: cls = 5; break;
            case 10: case 23: cls = 6; break;
            case 8: cls = 8 + (int)((nodes[q].op >> 8) & 0xffu); break;
            default: break;
            }
            const bool is_col = op == 4 || op == 5 || op == 13 || op == 17 || op == 20 || op == 23;
            f.cls[q] = cls;
            f.v[q] = is_col ? (col_ok ? t_to_f32<BF16>(nodes[q].ptr[col]) : 0.0f) : nodes[q].scalar;
        }
    }
}

// The long cases (IEEE division, gelu, tanh) as one out-of-line routine over a 16-value array in
// local memory: inlined and unrolled they cost the calling kernel registers in its main loop
// and a few thousand instructions of code, for graphs that few callers build.
static __device__ __noinline__ void fast_ep_rare16(int cls, float o, float* t) {
#pragma unroll 1
    for (int j = 0; j < 16; ++j) {
        const float v = t[j];
        t[j] = cls == 4 ? __fdiv_rn(v, o) : act_apply(cls == 8 + 2 ? 2u : 4u, v, 0.0f);
    }
}

// Applies the graph to 16 accumulators of one output column at once.  The walk over the
// slots is outside the walk over the values: one uniform branch per slot and a straight run
// of 16 operations under it, so the code stays a few hundred instructions however it is
// unrolled (a per-value walk of every case, unrolled 16 times, overflowed the instruction
// cache and made the drain fetch-bound).
template <int BF16>
__device__ __forceinline__ void fast_ep_apply16(const FastEp& f, const uint32_t (&acc)[16], uint16_t (&out)[16]) {
    float x[16];
#pragma unroll
    for (int j = 0; j < 16; j += 2) {
        const float2 v = round2_t<BF16>(__uint_as_float(acc[j]), __uint_as_float(acc[j + 1]));
        x[j] = v.x;
        x[j + 1] = v.y;
    }
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const int cls = f.cls[q];
        const float o = f.v[q];
        if (cls == 0) continue;
        switch (cls) {
        case 1:
#pragma unroll
            for (int j = 0; j < 16; ++j) x[j] = __fadd_rn(x[j], o);
            break;
        case 2:
#pragma unroll
            for (int j = 0; j < 16; ++j) x[j] = __fmul_rn(x[j], o);
            break;
        case 3:
#pragma unroll
            for (int j = 0; j < 16; ++j) x[j] = __fsub_rn(x[j], o);
            break;
        case 4: case 8 + 2: case 8 + 4: {
            float t[16];   // a copy: x[] itself must never be indexed or have its address taken, or it leaves the registers
#pragma unroll
            for (int j = 0; j < 16; ++j) t[j] = x[j];
            fast_ep_rare16(cls, o, t);
#pragma unroll
            for (int j = 0; j < 16; ++j) x[j] = t[j];
            break;
        }
        case 5:
#pragma unroll
            for (int j = 0; j < 16; ++j) x[j] = fmaxf(x[j], o);
            break;
        case 6:
#pragma unroll
            for (int j = 0; j < 16; ++j) x[j] = fminf(x[j], o);
            break;
        case 8 + 1:
#pragma unroll
            for (int j = 0; j < 16; ++j) x[j] = fmaxf(x[j], 0.0f);
            break;
        case 8 + 3:
#pragma unroll
            for (int j = 0; j < 16; ++j) x[j] = __fdividef(x[j], 1.0f + __expf(-x[j]));
            break;
        case 8 + 5:
#pragma unroll
            for (int j = 0; j < 16; ++j) x[j] = __fdividef(1.0f, 1.0f + __expf(-x[j]));
            break;
        default: break;
        }
    }
#pragma unroll
    for (int j = 0; j < 16; j += 2) {
        const uint32_t v = pack2_t<BF16>(x[j], x[j + 1]);
        out[j] = (uint16_t)(v & 0xffffu);
        out[j + 1] = (uint16_t)(v >> 16);
    }
}

// The gate activation of the gated MLP product (act 3 = SiLU, else the tanh form of GELU), the same expression at every
// site that forms act(gate) * up so that the fused drain, the depth-split reduce and the element-wise pass agree bit
// for bit.  Both are x * sigmoid(y) -- 0.5 x (1 + tanh z) = x / (1 + exp(-2 z)) -- on the hardware's approximate
// exp2 and reciprocal: relative error of a few 2^-22, far below the f16 / bf16 rounding of the store that follows, and a
// dozen instructions less per element than the exact division and expf (the drain of a 256 x 256 tile is bound by them).
__device__ __forceinline__ float glu_gate(uint32_t act, float g) {
    float y = g;
    if (act != 3u) y = __fmul_rn(1.5957691f, __fadd_rn(g, __fmul_rn(__fmul_rn(__fmul_rn(0.044715f, g), g), g)));
    return __fdividef(g, __fadd_rn(1.0f, __expf(-y)));
}

template <int BF16>
__device__ __forceinline__ uint16_t fast_ep_store(const FastEp& f, float acc) {
    float x = t_to_f32<BF16>(f32_to_t<BF16>(acc));
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const int cls = f.cls[q];
        const float o = f.v[q];
        switch (cls) {
        case 1: x = __fadd_rn(x, o); break;
        case 2: x = __fmul_rn(x, o); break;
        case 3: x = __fsub_rn(x, o); break;
        case 4: x = __fdiv_rn(x, o); break;
        case 5: x = fmaxf(x, o); break;
        case 6: x = fminf(x, o); break;
        case 8 + 1: x = fmaxf(x, 0.0f); break;
        case 8 + 2: x = act_apply(2u, x, 0.0f); break;
        case 8 + 4: x = act_apply(4u, x, 0.0f); break;
        case 8 + 3: x = __fdividef(x, 1.0f + __expf(-x)); break;
        case 8 + 5: x = __fdividef(1.0f, 1.0f + __expf(-x)); break;
        default: break;
        }
    }
    return f32_to_t<BF16>(x);
}

}  // namespace smeg
