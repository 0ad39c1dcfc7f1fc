// smeg.hpp -- C++17 host mirror of the reference's Rust API for the weight-quantised matmul path, header-only, over the
// C ABI of smeg_api.h.  It stands where the reference's safe layer stands above src/ffi.rs: the same type and method
// names, argument meaning and error behaviour (where the reference panics this throws std::invalid_argument with the
// reference's message; a non-zero return of the library throws smeg::Error -- there is no CPU fallback behind it).
//
//   Q4Params / Q4Weights           src/kernels/q4/mod.rs:55-103, weights.rs:26-271, quantize.rs:29-81
//   Q2Params / Q2Weights, Q1Weights src/kernels/lowbit/mod.rs:38-94, q2.rs:31-186, q1.rs:23-233
//   Epilogue<T>                    src/epilogue/graph.rs:33-432 (trailing activation rule :38-42, 185-223),
//                                  resolve_nodes src/exec/scalar.rs:28-53, validate_ep src/exec/guard.rs:112-150
//   matmul_q4{,_ep}{,_bf16}        src/kernels/q4/matmul.rs:21-271
//   matmul_q2 / q1 {,_ep}{,_mopa}  src/kernels/lowbit/matmul.rs:38-139
//   Packed<T>, Gemm<T>             src/exec/builder.rs:220-227, 428-813
//   Linear, GatedLinear, Mlp       src/linear.rs:133-835, src/mlp.rs:56-146
//   Norm, KvCache                  src/nn.rs:163-230, src/kernels/kv_attention.rs:354-581 (device memory only)
//
// Every compute call exists twice: on host slices (the library copies in and out, as the drop-in symbols do) and, with
// the suffix _dev, on device pointers plus a CUDA stream (what a GPU-resident caller and every timed path use; epilogue
// operands are then device pointers too).  16-bit floats travel as uint16_t bit patterns, as in the C ABI.
#ifndef SMEG_HPP
#define SMEG_HPP

#include <cmath>
#include <cstdint>
#include <cstring>
#include <memory>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "smeg_api.h"

namespace smeg {

// A non-zero return code of the library (outputs untouched).
struct Error : std::runtime_error {
    int rc;
    Error(const char* what, int code) : std::runtime_error(std::string(what) + " failed with rc " + std::to_string(code)), rc(code) {}
};
inline void check(const char* what, int rc) {
    if (rc != 0) throw Error(what, rc);
}
inline void require(bool ok, const std::string& msg) {
    if (!ok) throw std::invalid_argument(msg);
}

// A borrowed run of elements with its length (a Rust slice).
template <class E>
struct Slice {
    E* ptr = nullptr;
    size_t len = 0;
    Slice() = default;
    Slice(E* p, size_t n) : ptr(p), len(n) {}
    template <class V, class = decltype(std::declval<V&>().data())>
    Slice(V& v) : ptr(v.data()), len(v.size()) {}
};
using Bits = Slice<const uint16_t>;      // f16 or bf16 bit patterns, read
using BitsMut = Slice<uint16_t>;         // ... written

enum class WeightLayout : int { OutIn = SMEG_LAYOUT_OUT_IN, InOut = SMEG_LAYOUT_IN_OUT };
enum class Gate : uint32_t { Gelu = SMEG_ACT_GELU, Silu = SMEG_ACT_SILU };

// Element tags of the two 16-bit types.
struct f16 {
    static constexpr bool is_bf16 = false;
};
struct bf16 {
    static constexpr bool is_bf16 = true;
};

// ---- IEEE conversions (crate `half`: round to nearest even) ------------------------------------------------------
inline uint32_t f32_bits(float x) {
    uint32_t u;
    std::memcpy(&u, &x, 4);
    return u;
}
inline float f32_from_bits(uint32_t u) {
    float x;
    std::memcpy(&x, &u, 4);
    return x;
}
inline uint16_t f32_to_bf16_bits(float x) {
    const uint32_t u = f32_bits(x);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u);      // NaN stays a NaN
    return (uint16_t)((u + 0x7fffu + ((u >> 16) & 1u)) >> 16);
}
inline float bf16_bits_to_f32(uint16_t h) { return f32_from_bits((uint32_t)h << 16); }
inline uint16_t f32_to_f16_bits(float x) {
    const uint32_t u = f32_bits(x), sign = (u >> 16) & 0x8000u, mag = u & 0x7fffffffu;
    if (mag > 0x7f800000u) return (uint16_t)(sign | 0x7e00u);                           // NaN
    if (mag >= 0x47800000u) return (uint16_t)(sign | 0x7c00u);                          // >= 65536 (and infinity)
    if (mag < 0x33000000u) return (uint16_t)sign;                                       // below half the smallest subnormal
    int e = (int)(mag >> 23) - 127;
    uint32_t man = (mag & 0x7fffffu) | 0x800000u;                                       // 24 significant bits
    int shift = e >= -14 ? 13 : 13 + (-14 - e);                                         // bits dropped
    uint32_t kept = man >> shift, rest = man & ((1u << shift) - 1u), half = 1u << (shift - 1);
    if (rest > half || (rest == half && (kept & 1u))) ++kept;
    uint32_t out = e >= -14 ? ((uint32_t)(e + 15) << 10) + (kept - 0x400u) : kept;      // a carry moves into the exponent
    if (out >= 0x7c00u) out = 0x7c00u;
    return (uint16_t)(sign | out);
}
inline float f16_bits_to_f32(uint16_t h) {
    const uint32_t sign = ((uint32_t)h & 0x8000u) << 16, e = (h >> 10) & 31u, man = h & 0x3ffu;
    if (e == 31) return f32_from_bits(sign | 0x7f800000u | (man << 13));
    if (e == 0) {
        if (man == 0) return f32_from_bits(sign);
        float v = (float)man * 5.9604644775390625e-8f;                                  // man * 2^-24, exact
        return sign ? -v : v;
    }
    return f32_from_bits(sign | ((e + 112u) << 23) | (man << 13));
}
template <class T>
inline float round_to(float v) {
    return T::is_bf16 ? bf16_bits_to_f32(f32_to_bf16_bits(v)) : f16_bits_to_f32(f32_to_f16_bits(v));
}

inline bool is_pow2(size_t v) { return v != 0 && (v & (v - 1)) == 0; }
inline size_t ceil_div(size_t a, size_t b) { return (a + b - 1) / b; }

// ---- weight parameters and handles -------------------------------------------------------------------------------

constexpr size_t Q4_BLOCK = 32;      // src/kernels/q4/mod.rs:29
constexpr size_t Q2_BLOCK = 256;     // src/kernels/lowbit/mod.rs:26

// Q4Params, src/kernels/q4/mod.rs:55-103.
class Q4Params {
    size_t block_;
    bool affine_ = false;

public:
    explicit Q4Params(size_t block = Q4_BLOCK) : block_(block) {
        require(is_pow2(block), "q4 block size must be a power of two, got " + std::to_string(block));
    }
    Q4Params affine() const {
        Q4Params p(block_);
        p.affine_ = true;
        return p;
    }
    size_t block() const { return block_; }
    bool is_affine() const { return affine_; }
};

// Q2Params, src/kernels/lowbit/mod.rs:38-94: block size and the four int8 values the codes stand for.
class Q2Params {
    size_t block_;
    int8_t codebook_[4] = {-1, 0, 1, 0};

public:
    explicit Q2Params(size_t block = Q2_BLOCK) : block_(block) {
        require(is_pow2(block) && block >= 16 && block <= 65536,
                "q2 block size must be a power of two in 16..=65536, got " + std::to_string(block));
    }
    Q2Params with_codebook(const int8_t (&values)[4]) const {
        Q2Params p(block_);
        std::memcpy(p.codebook_, values, 4);
        return p;
    }
    size_t block() const { return block_; }
    const int8_t* codebook() const { return codebook_; }
};

// Q4Weights, src/kernels/q4/weights.rs:26-271: prepacked on the device at construction, immutable, shareable.
class Q4Weights {
    smeg_q4* h_ = nullptr;
    Q4Params p_;
    Q4Weights(smeg_q4* h, Q4Params p) : h_(h), p_(p) {}

public:
    Q4Weights(Q4Weights&& o) noexcept : h_(o.h_), p_(o.p_) { o.h_ = nullptr; }
    Q4Weights& operator=(Q4Weights&& o) noexcept {
        if (this != &o) {
            if (h_) smeg_q4_destroy(h_);
            h_ = o.h_;
            p_ = o.p_;
            o.h_ = nullptr;
        }
        return *this;
    }
    Q4Weights(const Q4Weights&) = delete;
    Q4Weights& operator=(const Q4Weights&) = delete;
    ~Q4Weights() {
        if (h_) smeg_q4_destroy(h_);
    }

    // Q4Weights::with_params (weights.rs:63-123): nibbles idx = d*n + j, low first; scales / mins [j*nbk + blk].
    static Q4Weights with_params(Slice<const uint8_t> quants, Bits scales, Bits mins, size_t n, size_t k, Q4Params p) {
        const size_t nbk = ceil_div(k, p.block());
        require(quants.len == (n * k + 1) / 2, "quants is ceil(n*k/2) bytes");
        require(scales.len == n * nbk, "scales is n*ceil(k/block)");
        if (p.is_affine()) {
            require(mins.ptr != nullptr, "Q4Form::Affine requires a mins array");
            require(mins.len == n * nbk, "mins is n*ceil(k/block)");
        } else {
            require(mins.ptr == nullptr, "Q4Form::Scale takes no mins array");
        }
        smeg_q4* h = nullptr;
        check("smeg_q4_create", smeg_q4_create(quants.ptr, scales.ptr, mins.ptr, n, k, p.block(), &h));
        return Q4Weights(h, p);
    }
    // Q4Weights::new: Q4_0, block 32.
    static Q4Weights new_(Slice<const uint8_t> quants, Bits scales, size_t n, size_t k) {
        return with_params(quants, scales, Bits(), n, k, Q4Params());
    }
    // Q4Weights::quantize (quantize.rs:29-81).
    static Q4Weights quantize(Slice<const float> w, WeightLayout layout, size_t n, size_t k, Q4Params p = Q4Params()) {
        require(w.len == n * k, "w is n*k");
        smeg_q4* h = nullptr;
        check("smeg_q4_quantize", smeg_q4_quantize(w.ptr, (int)layout, n, k, p.block(), p.is_affine() ? 1 : 0, &h));
        return Q4Weights(h, p);
    }
    // From the band-major arrays a reference-side Q4Weights holds (weights.rs:92-113).
    static Q4Weights from_band(Slice<const uint8_t> nibbles, Bits scales, Bits mins, size_t n, size_t k, Q4Params p = Q4Params()) {
        smeg_q4* h = nullptr;
        check("smeg_q4_from_band", smeg_q4_from_band(nibbles.ptr, scales.ptr, mins.ptr, n, k, p.block(), &h));
        return Q4Weights(h, p);
    }
    size_t n() const { return smeg_q4_n(h_); }
    size_t k() const { return smeg_q4_k(h_); }
    const Q4Params& params() const { return p_; }
    size_t device_bytes() const { return smeg_q4_device_bytes(h_); }
    const smeg_q4* handle() const { return h_; }
    // The logical arrays back (pack then unpack is the identity, weights.rs:425-463).
    void unpack(std::vector<uint8_t>& quants, std::vector<uint16_t>& scales) const {
        quants.assign((n() * k() + 1) / 2, 0);
        scales.assign(n() * ceil_div(k(), p_.block()), 0);
        check("smeg_q4_unpack", smeg_q4_unpack(h_, quants.data(), scales.data()));
    }
};

// Q2Weights / Q1Weights, src/kernels/lowbit/q2.rs:31-186, q1.rs:23-233.
class LowbitWeights {
protected:
    smeg_lowbit* h_ = nullptr;
    explicit LowbitWeights(smeg_lowbit* h) : h_(h) {}

public:
    LowbitWeights(LowbitWeights&& o) noexcept : h_(o.h_) { o.h_ = nullptr; }
    LowbitWeights& operator=(LowbitWeights&& o) noexcept {
        if (this != &o) {
            if (h_) smeg_lowbit_destroy(h_);
            h_ = o.h_;
            o.h_ = nullptr;
        }
        return *this;
    }
    LowbitWeights(const LowbitWeights&) = delete;
    LowbitWeights& operator=(const LowbitWeights&) = delete;
    ~LowbitWeights() {
        if (h_) smeg_lowbit_destroy(h_);
    }
    size_t n() const { return smeg_lowbit_n(h_); }
    size_t k() const { return smeg_lowbit_k(h_); }
    size_t block() const { return smeg_lowbit_block(h_); }
    int bits() const { return smeg_lowbit_bits(h_); }
    size_t device_bytes() const { return smeg_lowbit_device_bytes(h_); }
    const smeg_lowbit* handle() const { return h_; }
};

class Q2Weights : public LowbitWeights {
    Q2Params p_;
    Q2Weights(smeg_lowbit* h, Q2Params p) : LowbitWeights(h), p_(p) {}

public:
    // Q2Weights::new (q2.rs:48-84): codes four to a byte, idx = d*n + j at bits 2*(idx%4); scales [j*nbk + blk].
    static Q2Weights new_(Slice<const uint8_t> codes, Bits scales, size_t n, size_t k, Q2Params p = Q2Params()) {
        require(codes.len == (n * k + 3) / 4, "codes is ceil(n*k/4) bytes");
        require(scales.len == n * ceil_div(k, p.block()), "scales is n*ceil(k/block)");
        smeg_lowbit* h = nullptr;
        check("smeg_q2_create", smeg_q2_create(codes.ptr, scales.ptr, n, k, p.block(), p.codebook(), &h));
        return Q2Weights(h, p);
    }
    // Q2Weights::quantize (q2.rs:110-144).
    static Q2Weights quantize(Slice<const float> w, WeightLayout layout, size_t n, size_t k, Q2Params p = Q2Params()) {
        require(w.len == n * k, "w is n*k");
        smeg_lowbit* h = nullptr;
        check("smeg_q2_quantize", smeg_q2_quantize(w.ptr, (int)layout, n, k, p.block(), p.codebook(), &h));
        return Q2Weights(h, p);
    }
    const Q2Params& params() const { return p_; }
};

class Q1Weights : public LowbitWeights {
    explicit Q1Weights(smeg_lowbit* h) : LowbitWeights(h) {}

public:
    // Q1Weights::new (q1.rs:47-106): one sign bit per weight (1 = +scale), idx = j*k + d (OutIn) or d*n + j (InOut).
    static Q1Weights new_(Slice<const uint8_t> signs, Bits scales, WeightLayout layout, size_t n, size_t k, size_t block) {
        require(is_pow2(block) && block >= 16 && block <= 65536,
                "q1 block size must be a power of two in 16..=65536, got " + std::to_string(block));
        require(signs.len == (n * k + 7) / 8, "signs is ceil(n*k/8) bytes");
        require(scales.len == n * ceil_div(k, block), "scales is n*ceil(k/block)");
        smeg_lowbit* h = nullptr;
        check("smeg_q1_create", smeg_q1_create(signs.ptr, scales.ptr, (int)layout, n, k, block, &h));
        return Q1Weights(h);
    }
    // Q1Weights::quantize (q1.rs:116-144).
    static Q1Weights quantize(Slice<const float> w, WeightLayout layout, size_t n, size_t k, size_t block) {
        require(w.len == n * k, "w is n*k");
        smeg_lowbit* h = nullptr;
        check("smeg_q1_quantize", smeg_q1_quantize(w.ptr, (int)layout, n, k, block, &h));
        return Q1Weights(h);
    }
};

// ---- the fused epilogue as an ordered op-graph --------------------------------------------------------------------

// Epilogue<'a, T>, src/epilogue/graph.rs:33-432.  Methods push nodes in call order, except relu / gelu / silu / tanh /
// sigmoid, which set a TRAILING activation applied last whatever the call order (graph.rs:38-42, 185-223): the builder
// call .add_col(bias).silu().clamp(-6, 6) evaluates bias -> clamp -> silu.  Scalars are given in the element type T and
// carried as f32 (push_scalar, graph.rs:84-95).  Operands are borrowed: they must outlive the call that uses the graph.
template <class T>
class Epilogue {
    std::vector<EpNode> nodes_;
    std::vector<size_t> lens_;           // operand lengths, for validate
    uint32_t act_ = SMEG_ACT_NONE;
    mutable std::vector<EpNode> resolved_;

    Epilogue& push(uint32_t op, uint32_t aux, float scalar, const uint16_t* ptr, size_t len, size_t ld) {
        EpNode nd;
        nd.op = op; nd.aux = aux; nd.scalar = scalar; nd.ptr = ptr; nd.ld = ld;
        nodes_.push_back(nd);
        lens_.push_back(len);
        return *this;
    }
    Epilogue& scalar(uint32_t op, float v) { return push(op, 0, round_to<T>(v), nullptr, 0, 0); }
    Epilogue& operand(uint32_t op, Bits v, size_t ld = 0) { return push(op, 0, 0.0f, v.ptr, v.len, ld); }
    Epilogue& named(uint32_t kind, float alpha = 0.0f) { return push(SMEG_OP_ACT, kind, alpha, nullptr, 0, 0); }

public:
    Epilogue() = default;
    static Epilogue new_() { return Epilogue(); }

    Epilogue& add_scalar(float v) { return scalar(SMEG_OP_ADD_SCALAR, v); }
    Epilogue& mul_scalar(float v) { return scalar(SMEG_OP_MUL_SCALAR, v); }
    Epilogue& sub_scalar(float v) { return scalar(SMEG_OP_SUB_SCALAR, v); }
    Epilogue& div_scalar(float v) { return scalar(SMEG_OP_DIV_SCALAR, v); }
    Epilogue& max(float lo) { return scalar(SMEG_OP_MAX_SCALAR, lo); }
    Epilogue& min(float hi) { return scalar(SMEG_OP_MIN_SCALAR, hi); }
    Epilogue& clamp(float lo, float hi) { return max(lo).min(hi); }

    Epilogue& add_row(Bits v) { return operand(SMEG_OP_ADD_ROW, v); }
    Epilogue& mul_row(Bits v) { return operand(SMEG_OP_MUL_ROW, v); }
    Epilogue& sub_row(Bits v) { return operand(SMEG_OP_SUB_ROW, v); }
    Epilogue& div_row(Bits v) { return operand(SMEG_OP_DIV_ROW, v); }
    Epilogue& max_row(Bits v) { return operand(SMEG_OP_MAX_ROW, v); }
    Epilogue& min_row(Bits v) { return operand(SMEG_OP_MIN_ROW, v); }
    Epilogue& add_col(Bits v) { return operand(SMEG_OP_ADD_COL, v); }
    Epilogue& mul_col(Bits v) { return operand(SMEG_OP_MUL_COL, v); }
    Epilogue& sub_col(Bits v) { return operand(SMEG_OP_SUB_COL, v); }
    Epilogue& div_col(Bits v) { return operand(SMEG_OP_DIV_COL, v); }
    Epilogue& max_col(Bits v) { return operand(SMEG_OP_MAX_COL, v); }
    Epilogue& min_col(Bits v) { return operand(SMEG_OP_MIN_COL, v); }
    Epilogue& add_tensor(Bits v) { return operand(SMEG_OP_ADD_TENSOR, v); }
    Epilogue& mul_tensor(Bits v) { return operand(SMEG_OP_MUL_TENSOR, v); }
    Epilogue& sub_tensor(Bits v) { return operand(SMEG_OP_SUB_TENSOR, v); }
    Epilogue& div_tensor(Bits v) { return operand(SMEG_OP_DIV_TENSOR, v); }
    Epilogue& max_tensor(Bits v) { return operand(SMEG_OP_MAX_TENSOR, v); }
    Epilogue& min_tensor(Bits v) { return operand(SMEG_OP_MIN_TENSOR, v); }
    Epilogue& add_tensor_strided(Bits v, size_t ld) { return operand(SMEG_OP_ADD_TENSOR, v, ld); }
    Epilogue& mul_tensor_strided(Bits v, size_t ld) { return operand(SMEG_OP_MUL_TENSOR, v, ld); }
    Epilogue& sub_tensor_strided(Bits v, size_t ld) { return operand(SMEG_OP_SUB_TENSOR, v, ld); }
    Epilogue& div_tensor_strided(Bits v, size_t ld) { return operand(SMEG_OP_DIV_TENSOR, v, ld); }
    Epilogue& max_tensor_strided(Bits v, size_t ld) { return operand(SMEG_OP_MAX_TENSOR, v, ld); }
    Epilogue& min_tensor_strided(Bits v, size_t ld) { return operand(SMEG_OP_MIN_TENSOR, v, ld); }

    // the trailing activation
    Epilogue& relu() { act_ = SMEG_ACT_RELU; return *this; }
    Epilogue& gelu() { act_ = SMEG_ACT_GELU; return *this; }
    Epilogue& silu() { act_ = SMEG_ACT_SILU; return *this; }
    Epilogue& tanh() { act_ = SMEG_ACT_TANH; return *this; }
    Epilogue& sigmoid() { act_ = SMEG_ACT_SIGMOID; return *this; }
    // activations that are ordinary nodes, in call order
    Epilogue& leaky_relu(float alpha) { return named(SMEG_ACT_LEAKY_RELU, alpha); }
    Epilogue& relu6() { return named(SMEG_ACT_RELU6); }
    Epilogue& hardsigmoid() { return named(SMEG_ACT_HARDSIGMOID); }
    Epilogue& hardswish() { return named(SMEG_ACT_HARDSWISH); }
    Epilogue& abs() { return named(SMEG_ACT_ABS); }
    Epilogue& neg() { return named(SMEG_ACT_NEG); }
    Epilogue& square() { return named(SMEG_ACT_SQUARE); }
    Epilogue& sign() { return named(SMEG_ACT_SIGN); }
    Epilogue& sqrt() { return named(SMEG_ACT_SQRT); }
    Epilogue& softsign() { return named(SMEG_ACT_SOFTSIGN); }
    Epilogue& recip() { return named(SMEG_ACT_RECIP); }
    Epilogue& rsqrt() { return named(SMEG_ACT_RSQRT); }
    Epilogue& exp() { return named(SMEG_ACT_EXP); }
    Epilogue& log() { return named(SMEG_ACT_LOG); }
    Epilogue& elu(float alpha) { return named(SMEG_ACT_ELU, alpha); }
    Epilogue& selu() { return named(SMEG_ACT_SELU); }
    Epilogue& softplus() { return named(SMEG_ACT_SOFTPLUS); }
    Epilogue& mish() { return named(SMEG_ACT_MISH); }
    Epilogue& gelu_exact() { return named(SMEG_ACT_GELU_EXACT); }

    // lead's nodes ahead of this graph's, this graph's activation kept (with_leading, graph.rs:149-157)
    Epilogue with_leading(const Epilogue& lead) const {
        Epilogue out;
        out.nodes_ = lead.nodes_;
        out.lens_ = lead.lens_;
        out.nodes_.insert(out.nodes_.end(), nodes_.begin(), nodes_.end());
        out.lens_.insert(out.lens_.end(), lens_.begin(), lens_.end());
        out.act_ = act_;
        return out;
    }
    bool is_empty() const { return nodes_.empty() && act_ == SMEG_ACT_NONE; }
    uint32_t trailing_act() const { return act_; }
    const std::vector<EpNode>& nodes() const { return nodes_; }

    // The node array as the FFI sees it (resolve_nodes, src/exec/scalar.rs:28-53): a TENSOR stride of 0 becomes n and
    // the trailing activation arrives as a final ACT node.
    std::vector<EpNode> resolved(size_t n) const {
        std::vector<EpNode> out = nodes_;
        for (EpNode& nd : out)
            if (is_tensor(nd.op) && nd.ld == 0) nd.ld = n;
        if (act_ != SMEG_ACT_NONE) {
            EpNode nd;
            nd.op = SMEG_OP_ACT; nd.aux = act_; nd.scalar = 0.0f; nd.ptr = nullptr; nd.ld = 0;
            out.push_back(nd);
        }
        return out;
    }
    // validate_ep, src/exec/guard.rs:112-150.
    void validate(size_t m, size_t n) const {
        for (size_t i = 0; i < nodes_.size(); ++i) {
            const uint32_t op = nodes_[i].op;
            if (is_row(op)) require(lens_[i] == m, "row operand is per-M (length m)");
            else if (is_col(op)) require(lens_[i] == n, "col operand is per-N (length n)");
            else if (is_tensor(op)) {
                const size_t ld = nodes_[i].ld ? nodes_[i].ld : n;
                require(ld >= n, "tensor row stride must be >= n");
                require(m == 0 || lens_[i] >= (m - 1) * ld + n, "tensor must hold m*n elements (stride ld)");
            }
        }
    }
    // The descriptor of a call on an m x n output (kept alive by this object until the next desc()).
    ep_desc16 desc(size_t n) const {
        resolved_ = resolved(n);
        ep_desc16 d;
        d.n_nodes = (uint32_t)resolved_.size();
        d.nodes = resolved_.empty() ? nullptr : resolved_.data();
        return d;
    }

    static bool is_row(uint32_t op) {
        return op == SMEG_OP_ADD_ROW || op == SMEG_OP_MUL_ROW || op == SMEG_OP_SUB_ROW || op == SMEG_OP_DIV_ROW ||
               op == SMEG_OP_MAX_ROW || op == SMEG_OP_MIN_ROW;
    }
    static bool is_col(uint32_t op) {
        return op == SMEG_OP_ADD_COL || op == SMEG_OP_MUL_COL || op == SMEG_OP_SUB_COL || op == SMEG_OP_DIV_COL ||
               op == SMEG_OP_MAX_COL || op == SMEG_OP_MIN_COL;
    }
    static bool is_tensor(uint32_t op) {
        return op == SMEG_OP_ADD_TENSOR || op == SMEG_OP_MUL_TENSOR || op == SMEG_OP_SUB_TENSOR || op == SMEG_OP_DIV_TENSOR ||
               op == SMEG_OP_MAX_TENSOR || op == SMEG_OP_MIN_TENSOR;
    }
};

// ---- matmuls on quantised weights ----------------------------------------------------------------------------------

namespace detail {
inline void check_io(size_t a_len, size_t c_len, size_t m, size_t n, size_t k) {
    require(a_len == m * k, "a is m*k");
    require(c_len == m * n, "c is m*n");
}
template <class T>
inline void run_q4(Bits a, const Q4Weights& w, BitsMut c, size_t m, const Epilogue<T>* ep, void* stream, bool dev) {
    const size_t n = w.n(), k = w.k();
    check_io(a.len, c.len, m, n, k);
    if (ep) ep->validate(m, n);
    if (m == 0 || n == 0) return;
    ep_desc16 d;
    if (ep) d = ep->desc(n);
    const ep_desc16* dp = ep && d.n_nodes ? &d : nullptr;
    if (dev) {
        if (T::is_bf16) check("smeg_matmul_q4_bf16_dev", smeg_matmul_q4_bf16_dev(w.handle(), a.ptr, c.ptr, m, dp, stream));
        else check("smeg_matmul_q4_f16_dev", smeg_matmul_q4_f16_dev(w.handle(), a.ptr, c.ptr, m, dp, stream));
    } else {
        if (T::is_bf16) check("smeg_matmul_q4_bf16", smeg_matmul_q4_bf16(w.handle(), a.ptr, c.ptr, m, dp));
        else check("smeg_matmul_q4_f16", smeg_matmul_q4_f16(w.handle(), a.ptr, c.ptr, m, dp));
    }
}
inline void run_lowbit(Bits a, const LowbitWeights& w, BitsMut c, size_t m, const Epilogue<f16>* ep, bool mopa, void* stream,
                       bool dev) {
    const size_t n = w.n(), k = w.k();
    check_io(a.len, c.len, m, n, k);
    if (ep) ep->validate(m, n);
    if (m == 0 || n == 0) return;
    ep_desc16 d;
    if (ep) d = ep->desc(n);
    const ep_desc16* dp = ep && d.n_nodes ? &d : nullptr;
    if (dev) {
        if (mopa) check("smeg_matmul_lowbit_f16_dev", smeg_matmul_lowbit_f16_dev(w.handle(), a.ptr, c.ptr, m, dp, stream));
        else check("smeg_matmul_lowbit_dev", smeg_matmul_lowbit_dev(w.handle(), a.ptr, c.ptr, m, dp, stream));
    } else {
        if (mopa) check("smeg_matmul_lowbit_f16", smeg_matmul_lowbit_f16(w.handle(), a.ptr, c.ptr, m, dp));
        else check("smeg_matmul_lowbit", smeg_matmul_lowbit(w.handle(), a.ptr, c.ptr, m, dp));
    }
}
}  // namespace detail

// C[m][n] = ep(A[m][k] @ dequant(W)) -- matmul_q4 / matmul_q4_ep (src/kernels/q4/matmul.rs:21-35), f16.
inline void matmul_q4(Bits a, const Q4Weights& w, BitsMut c, size_t m) { detail::run_q4<f16>(a, w, c, m, nullptr, nullptr, false); }
inline void matmul_q4_ep(Bits a, const Q4Weights& w, BitsMut c, size_t m, const Epilogue<f16>& ep) { detail::run_q4<f16>(a, w, c, m, &ep, nullptr, false); }
// matmul_q4_bf16 / matmul_q4_bf16_ep (:178-196).
inline void matmul_q4_bf16(Bits a, const Q4Weights& w, BitsMut c, size_t m) { detail::run_q4<bf16>(a, w, c, m, nullptr, nullptr, false); }
inline void matmul_q4_bf16_ep(Bits a, const Q4Weights& w, BitsMut c, size_t m, const Epilogue<bf16>& ep) { detail::run_q4<bf16>(a, w, c, m, &ep, nullptr, false); }
// ... on device pointers and a stream
inline void matmul_q4_dev(Bits a, const Q4Weights& w, BitsMut c, size_t m, void* stream) { detail::run_q4<f16>(a, w, c, m, nullptr, stream, true); }
inline void matmul_q4_ep_dev(Bits a, const Q4Weights& w, BitsMut c, size_t m, const Epilogue<f16>& ep, void* stream) { detail::run_q4<f16>(a, w, c, m, &ep, stream, true); }
inline void matmul_q4_bf16_dev(Bits a, const Q4Weights& w, BitsMut c, size_t m, void* stream) { detail::run_q4<bf16>(a, w, c, m, nullptr, stream, true); }
inline void matmul_q4_bf16_ep_dev(Bits a, const Q4Weights& w, BitsMut c, size_t m, const Epilogue<bf16>& ep, void* stream) { detail::run_q4<bf16>(a, w, c, m, &ep, stream, true); }

// matmul_q2 / matmul_q1 {,_ep} (src/kernels/lowbit/matmul.rs:38-84): int8 activations, exact integer block sums.
inline void matmul_q2(Bits a, const Q2Weights& w, BitsMut c, size_t m) { detail::run_lowbit(a, w, c, m, nullptr, false, nullptr, false); }
inline void matmul_q2_ep(Bits a, const Q2Weights& w, BitsMut c, size_t m, const Epilogue<f16>& ep) { detail::run_lowbit(a, w, c, m, &ep, false, nullptr, false); }
inline void matmul_q1(Bits a, const Q1Weights& w, BitsMut c, size_t m) { detail::run_lowbit(a, w, c, m, nullptr, false, nullptr, false); }
inline void matmul_q1_ep(Bits a, const Q1Weights& w, BitsMut c, size_t m, const Epilogue<f16>& ep) { detail::run_lowbit(a, w, c, m, &ep, false, nullptr, false); }
// matmul_q2_mopa / matmul_q1_mopa {,_ep} (:100-139): f16 activations, no int8 step.
inline void matmul_q2_mopa(Bits a, const Q2Weights& w, BitsMut c, size_t m) { detail::run_lowbit(a, w, c, m, nullptr, true, nullptr, false); }
inline void matmul_q2_mopa_ep(Bits a, const Q2Weights& w, BitsMut c, size_t m, const Epilogue<f16>& ep) { detail::run_lowbit(a, w, c, m, &ep, true, nullptr, false); }
inline void matmul_q1_mopa(Bits a, const Q1Weights& w, BitsMut c, size_t m) { detail::run_lowbit(a, w, c, m, nullptr, true, nullptr, false); }
inline void matmul_q1_mopa_ep(Bits a, const Q1Weights& w, BitsMut c, size_t m, const Epilogue<f16>& ep) { detail::run_lowbit(a, w, c, m, &ep, true, nullptr, false); }
// ... on device pointers and a stream (ep may be null)
inline void matmul_lowbit_dev(Bits a, const LowbitWeights& w, BitsMut c, size_t m, const Epilogue<f16>* ep, void* stream) { detail::run_lowbit(a, w, c, m, ep, false, stream, true); }
inline void matmul_lowbit_mopa_dev(Bits a, const LowbitWeights& w, BitsMut c, size_t m, const Epilogue<f16>* ep, void* stream) { detail::run_lowbit(a, w, c, m, ep, true, stream, true); }

// ---- dense 16-bit weights: Packed<T> and the Gemm builder ----------------------------------------------------------

// Packed<f16> / Packed<bf16> (prepack_f16 / prepack_bf16, src/kernels/f16.rs:212): b is k x n row-major T bits.
template <class T>
class Packed {
    smeg_dense* h_ = nullptr;

public:
    Packed(Bits b, size_t n, size_t k) {
        require(b.len == n * k, "b is k*n");
        check("smeg_dense_create", smeg_dense_create(b.ptr, n, k, T::is_bf16 ? 1 : 0, &h_));
    }
    Packed(Packed&& o) noexcept : h_(o.h_) { o.h_ = nullptr; }
    Packed(const Packed&) = delete;
    Packed& operator=(const Packed&) = delete;
    ~Packed() {
        if (h_) smeg_dense_destroy(h_);
    }
    size_t n() const { return smeg_dense_n(h_); }
    size_t k() const { return smeg_dense_k(h_); }
    const smeg_dense* handle() const { return h_; }
};
inline Packed<f16> prepack_f16(Bits b, size_t n, size_t k) { return Packed<f16>(b, n, k); }
inline Packed<bf16> prepack_bf16(Bits b, size_t n, size_t k) { return Packed<bf16>(b, n, k); }

// Gemm::new(a, &packed, m).add_col(bias).gelu().run(&mut c) (src/exec/builder.rs:220-227, 428-813):
// C = ep( T(beta * (A @ B)) ).  `ep()` gives the graph to build on (every Epilogue method, same trailing-activation rule).
template <class T>
class Gemm {
    Bits a_;
    const Packed<T>& p_;
    size_t m_;
    float beta_ = 1.0f;
    bool col_major_ = false;
    Epilogue<T> ep_;

public:
    Gemm(Bits a, const Packed<T>& packed, size_t m) : a_(a), p_(packed), m_(m) {}
    static Gemm new_(Bits a, const Packed<T>& packed, size_t m) { return Gemm(a, packed, m); }
    Epilogue<T>& ep() { return ep_; }
    Gemm& beta(float b) {
        beta_ = round_to<T>(b);
        return *this;
    }
    Gemm& col_major_output() {
        col_major_ = true;
        return *this;
    }
    void run(BitsMut c, void* stream = nullptr, bool dev = false) const {
        const size_t n = p_.n(), k = p_.k();
        detail::check_io(a_.len, c.len, m_, n, k);
        ep_.validate(m_, n);
        if (m_ == 0 || n == 0) return;
        const uint16_t beta_bits = T::is_bf16 ? f32_to_bf16_bits(beta_) : f32_to_f16_bits(beta_);
        ep_desc16 d = ep_.desc(n);
        const ep_desc16* dp = d.n_nodes ? &d : nullptr;
        if (dev) check("smeg_gemm_dense_dev", smeg_gemm_dense_dev(p_.handle(), a_.ptr, c.ptr, m_, beta_bits, col_major_ ? 1 : 0, dp, stream));
        else check("smeg_gemm_dense", smeg_gemm_dense(p_.handle(), a_.ptr, c.ptr, m_, beta_bits, col_major_ ? 1 : 0, dp));
    }
};

// ---- layers: Linear, GatedLinear, Mlp -----------------------------------------------------------------------------

// [gate | up] as one k x 2n row-major (InOut) matrix, 32 gate columns then 32 up columns at a time
// (interleave, src/linear.rs:603-617).  g, u: n x k (OutIn) or k x n (InOut) f32.
inline std::vector<float> interleave_gate_up(Slice<const float> g, Slice<const float> u, WeightLayout layout, size_t n, size_t k) {
    require(g.len == n * k && u.len == n * k, "gate and up are n*k");
    std::vector<float> out(2 * n * k);
    auto at = [&](const float* w, size_t d, size_t j) { return layout == WeightLayout::OutIn ? w[j * k + d] : w[d * n + j]; };
    for (size_t d = 0; d < k; ++d) {
        size_t col = 0;
        for (size_t c0 = 0; c0 < n; c0 += 32) {
            const size_t c1 = c0 + 32 < n ? c0 + 32 : n;
            for (size_t j = c0; j < c1; ++j) out[d * 2 * n + col++] = at(g.ptr, d, j);
            for (size_t j = c0; j < c1; ++j) out[d * 2 * n + col++] = at(u.ptr, d, j);
        }
    }
    return out;
}

// Linear (src/linear.rs:133-155): Q4, 2-bit or 1-bit weights with an optional bias, which rides as a leading AddCol
// (with_lead, :440-463).  2-bit / 1-bit layers run on the int8-activation kernels, or -- opted in with lowbit_mopa() --
// on the f16 tensor-core path from LOWBIT_MOPA_ROWS rows (:168, 535-552).  The bias (n f16 bits) is borrowed; for the _dev
// calls it is a device pointer.
class Linear {
    std::unique_ptr<Q4Weights> q4_;
    std::unique_ptr<Q2Weights> q2_;
    std::unique_ptr<Q1Weights> q1_;
    Bits bias_;
    bool mopa_ = false;

    void check_bias() const { require(bias_.ptr == nullptr || bias_.len == n(), "bias holds n values"); }

public:
    static constexpr size_t LOWBIT_MOPA_ROWS = 64;

    explicit Linear(Q4Weights w, Bits bias = Bits()) : q4_(new Q4Weights(std::move(w))), bias_(bias) { check_bias(); }
    static Linear quantize(Slice<const float> w, WeightLayout layout, size_t n, size_t k, Q4Params p = Q4Params(), Bits bias = Bits()) {
        return Linear(Q4Weights::quantize(w, layout, n, k, p), bias);
    }
    static Linear from_q4(Q4Weights w, Bits bias = Bits()) { return Linear(std::move(w), bias); }
    // Linear::from_q2, src/linear.rs:214
    static Linear from_q2(Q2Weights w, Bits bias = Bits()) {
        Linear l;
        l.q2_.reset(new Q2Weights(std::move(w)));
        l.bias_ = bias;
        l.check_bias();
        return l;
    }
    // Linear::from_q1, src/linear.rs:234
    static Linear from_q1(Q1Weights w, Bits bias = Bits()) {
        Linear l;
        l.q1_.reset(new Q1Weights(std::move(w)));
        l.bias_ = bias;
        l.check_bias();
        return l;
    }
    // Linear::lowbit_mopa: 2-bit / 1-bit weights on the f16 tensor-core path from LOWBIT_MOPA_ROWS rows
    Linear& lowbit_mopa(bool on = true) {
        mopa_ = on;
        return *this;
    }
    size_t n() const { return q4_ ? q4_->n() : (q2_ ? q2_->n() : q1_->n()); }
    size_t k() const { return q4_ ? q4_->k() : (q2_ ? q2_->k() : q1_->k()); }
    bool is_q4() const { return (bool)q4_; }
    const Q4Weights& weights() const {
        require(is_q4(), "this layer holds no Q4 weights");
        return *q4_;
    }
    bool has_bias() const { return bias_.ptr != nullptr; }
    // y = ep(x @ W + bias): the bias ahead of the caller's graph
    void forward_ep(Bits x, BitsMut y, size_t m, const Epilogue<f16>& ep, void* stream = nullptr, bool dev = false) const {
        Epilogue<f16> full = ep;
        if (has_bias()) {
            Epilogue<f16> lead;
            lead.add_col(bias_);
            full = ep.with_leading(lead);
        }
        if (q4_) detail::run_q4<f16>(x, *q4_, y, m, &full, stream, dev);
        else detail::run_lowbit(x, q2_ ? static_cast<const LowbitWeights&>(*q2_) : static_cast<const LowbitWeights&>(*q1_), y, m, &full,
                                mopa_ && m >= LOWBIT_MOPA_ROWS, stream, dev);
    }
    void forward(Bits x, BitsMut y, size_t m, void* stream = nullptr, bool dev = false) const { forward_ep(x, y, m, Epilogue<f16>(), stream, dev); }

private:
    Linear() = default;
};

// act(x @ W_gate) * (x @ W_up) from one interleaved 2n-column Q4 matrix (GatedLinear, src/linear.rs:603-656, 779-835).
class GatedLinear {
    Linear inner_;
    Gate gate_;

public:
    GatedLinear(Linear inner, Gate gate) : inner_(std::move(inner)), gate_(gate) { require(inner_.n() % 2 == 0, "the interleaved layer has 2n columns"); }
    static GatedLinear quantize(Slice<const float> w_gate, Slice<const float> w_up, WeightLayout layout, size_t n, size_t k, Gate gate,
                                Q4Params p = Q4Params()) {
        const std::vector<float> both = interleave_gate_up(w_gate, w_up, layout, n, k);
        return GatedLinear(Linear::quantize(Slice<const float>(both.data(), both.size()), WeightLayout::InOut, 2 * n, k, p), gate);
    }
    size_t n() const { return inner_.n() / 2; }
    size_t k() const { return inner_.k(); }
    Gate gate() const { return gate_; }
    const Linear& inner() const { return inner_; }
};

// y += down(act(x @ W_gate) * (x @ W_up)) -- Mlp::gated and Mlp::accumulate, src/mlp.rs:80-146, as one library call
// (fused kernels above 64 rows, the one-wave decode kernels at a few rows).  x: m x k f16 bits, y: m x d f32.
class Mlp {
    GatedLinear up_;
    Linear down_;
    smeg_mlp* h_ = nullptr;

public:
    Mlp(GatedLinear up, Linear down) : up_(std::move(up)), down_(std::move(down)) {
        require(down_.k() == up_.n(), "down takes up's outputs");
        require(!up_.inner().has_bias() && !down_.has_bias(), "the fused block takes layers without bias");
        check("smeg_mlp_create", smeg_mlp_create(up_.inner().weights().handle(), down_.weights().handle(), (uint32_t)up_.gate(), &h_));
    }
    static Mlp gated(GatedLinear up, Linear down) { return Mlp(std::move(up), std::move(down)); }
    Mlp(Mlp&& o) noexcept : up_(std::move(o.up_)), down_(std::move(o.down_)), h_(o.h_) { o.h_ = nullptr; }
    Mlp(const Mlp&) = delete;
    Mlp& operator=(const Mlp&) = delete;
    ~Mlp() {
        if (h_) smeg_mlp_destroy(h_);
    }
    size_t k() const { return up_.k(); }
    size_t n() const { return down_.n(); }
    size_t hidden() const { return down_.k(); }
    void accumulate(Bits x, Slice<float> y, size_t m) {
        require(x.len == m * k(), "x is m*k");
        require(y.len == m * n(), "y is m*n");
        check("smeg_mlp_accumulate", smeg_mlp_accumulate(h_, x.ptr, y.ptr, m));
    }
    void accumulate_dev(Bits x, Slice<float> y, size_t m, void* stream) {
        require(x.len == m * k(), "x is m*k");
        require(y.len == m * n(), "y is m*n");
        check("smeg_mlp_accumulate_dev", smeg_mlp_accumulate_dev(h_, x.ptr, y.ptr, m, stream));
    }
};

// ---- the steps either side of the MLP in a layer, on device memory --------------------------------------------------

// Norm::layer / Norm::rms (src/nn.rs:163-230): f32 rows in, f16 (or f32) rows out.  weight and bias (dim f32 each, bias
// may be null) are DEVICE pointers, borrowed.
class Norm {
    const float* weight_;
    const float* bias_;
    size_t dim_;
    float eps_;
    bool rms_;
    Norm(const float* w, const float* b, size_t dim, float eps, bool rms) : weight_(w), bias_(b), dim_(dim), eps_(eps), rms_(rms) {
        require(dim > 0, "a norm needs at least one feature");
    }

public:
    static Norm layer(const float* weight_dev, const float* bias_dev, size_t dim, float eps) { return Norm(weight_dev, bias_dev, dim, eps, false); }
    static Norm rms(const float* weight_dev, size_t dim, float eps) { return Norm(weight_dev, nullptr, dim, eps, true); }
    size_t width() const { return dim_; }
    // x: rows * dim f32 on the device; y16 / y32: either may be null
    void forward_dev(Slice<const float> x, uint16_t* y16, float* y32, void* stream) const {
        require(x.len % dim_ == 0, "x holds whole rows of weight.len()");
        check("smeg_norm_rows_dev", smeg_norm_rows_dev(y16, y32, x.ptr, weight_, bias_, x.len / dim_, dim_, eps_, rms_ ? 1 : 0, stream));
    }
};

// KvCache (src/kernels/kv_attention.rs:354-581) over caller-provided DEVICE buffers of capacity * kv_heads * head_dim f16
// values each: rows appended in order, queries of `heads` heads (a multiple of kv_heads) attending causally.
class KvCache {
    uint16_t* k_;
    uint16_t* v_;
    size_t heads_, kv_heads_, head_dim_, capacity_, len_ = 0;
    float scale_;

public:
    KvCache(uint16_t* k_dev, uint16_t* v_dev, size_t heads, size_t kv_heads, size_t head_dim, size_t capacity)
        : k_(k_dev), v_(v_dev), heads_(heads), kv_heads_(kv_heads), head_dim_(head_dim), capacity_(capacity) {
        require(head_dim % 8 == 0 && head_dim >= 8 && head_dim <= 256, "head_dim must be a multiple of 8 in 8..=256");
        require(kv_heads > 0 && heads > 0 && heads % kv_heads == 0, "heads must be a positive multiple of kv_heads");
        scale_ = 1.0f / std::sqrt((float)head_dim);             // in f32, as the reference computes it
    }
    KvCache& with_scale(float scale) {
        scale_ = scale;
        return *this;
    }
    size_t len() const { return len_; }
    bool is_empty() const { return len_ == 0; }
    size_t capacity() const { return capacity_; }
    size_t row_len() const { return kv_heads_ * head_dim_; }
    size_t query_len() const { return heads_ * head_dim_; }
    float scale() const { return scale_; }
    void clear() { len_ = 0; }
    void truncate(size_t n) { len_ = len_ < n ? len_ : n; }
    // `rows` key and value rows out of rows of src (stride elements apart; keys at k_off, values at v_off of a row)
    void extend_from_dev(const uint16_t* src, size_t stride, size_t k_off, size_t v_off, size_t rows, void* stream) {
        require(len_ + rows <= capacity_, "KvCache full: " + std::to_string(len_) + " + " + std::to_string(rows) + " rows over capacity " + std::to_string(capacity_));
        check("smeg_kv_append_dev", smeg_kv_append_dev(k_, v_, src, stride, k_off, v_off, row_len(), len_, rows, stream));
        len_ += rows;
    }
    // `rows` f16 query rows (q_stride elements apart), row i attending to positions 0..=len - rows + i; out: rows * query_len f32
    void attend_causal_dev(const uint16_t* q, size_t q_stride, size_t rows, float* out, void* stream) const {
        require(rows <= len_, "attend_causal: " + std::to_string(rows) + " rows but " + std::to_string(len_) + " cached");
        check("smeg_attn_kv_causal_dev", smeg_attn_kv_causal_dev(out, q, 0, q_stride, k_, v_, len_ - rows, rows, heads_, kv_heads_, head_dim_, scale_, stream));
    }
};

}  // namespace smeg

#endif  // SMEG_HPP
