// Exercises include/smeg.hpp, the C++ host mirror of the reference's API.
//
//   host_mirror_check cpu IN_F32 OUT_DIR   the parts that need no GPU: conversions (written to files for a comparison with
//                                          numpy), parameter checks, the epilogue builder, interleave, the error path
//   host_mirror_check gpu                  a Q4 matmul, a dense Gemm and an MLP block against closed-form answers (constant
//                                          rows times constant weights: every partial sum is an exact binary fraction)
//
// Prints one line per check and exits non-zero on the first failure.
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <string>
#include <vector>

#include "smeg.hpp"

using namespace smeg;

static int g_failed = 0;
#define EXPECT(cond)                                                        \
    do {                                                                    \
        if (!(cond)) {                                                      \
            std::printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond);   \
            g_failed = 1;                                                   \
        }                                                                   \
    } while (0)

template <class F>
static std::string thrown(F f) {
    try {
        f();
    } catch (const std::invalid_argument& e) {
        return e.what();
    } catch (const Error& e) {
        return std::string("rc ") + std::to_string(e.rc);
    }
    return "";
}

static void write_file(const std::string& path, const void* p, size_t bytes) {
    FILE* f = std::fopen(path.c_str(), "wb");
    if (!f || std::fwrite(p, 1, bytes, f) != bytes) {
        std::printf("FAILED to write %s\n", path.c_str());
        g_failed = 1;
    }
    if (f) std::fclose(f);
}

static int run_cpu(const char* in_f32, const std::string& out) {
    // ---- conversions: every f16 pattern widened, and the given floats narrowed to f16 and bf16 ----
    std::vector<float> widened(65536);
    for (uint32_t h = 0; h < 65536; ++h) widened[h] = f16_bits_to_f32((uint16_t)h);
    write_file(out + "/f16_to_f32.bin", widened.data(), widened.size() * 4);
    std::vector<float> xs;
    if (FILE* f = std::fopen(in_f32, "rb")) {
        float v;
        while (std::fread(&v, 4, 1, f) == 1) xs.push_back(v);
        std::fclose(f);
    }
    EXPECT(!xs.empty());
    std::vector<uint16_t> h16(xs.size()), b16(xs.size());
    for (size_t i = 0; i < xs.size(); ++i) {
        h16[i] = f32_to_f16_bits(xs[i]);
        b16[i] = f32_to_bf16_bits(xs[i]);
    }
    write_file(out + "/f32_to_f16.bin", h16.data(), h16.size() * 2);
    write_file(out + "/f32_to_bf16.bin", b16.data(), b16.size() * 2);

    // ---- parameters ----
    EXPECT(Q4Params().block() == 32 && !Q4Params().is_affine() && Q4Params(64).affine().is_affine() && Q4Params(64).affine().block() == 64);
    EXPECT(thrown([] { Q4Params(24); }) == "q4 block size must be a power of two, got 24");
    EXPECT(thrown([] { Q2Params(8); }) == "q2 block size must be a power of two in 16..=65536, got 8");
    const int8_t book[4] = {-2, -1, 1, 2};
    const Q2Params q2p = Q2Params(128).with_codebook(book);
    EXPECT(q2p.block() == 128 && q2p.codebook()[0] == -2 && q2p.codebook()[3] == 2 && Q2Params().codebook()[2] == 1);

    // ---- epilogue: call order, the trailing activation, scalars rounded to T, resolve, validate ----
    std::vector<uint16_t> bias(7, 0x3c00), rowv(3, 0x3c00), tens(3 * 9, 0);
    Epilogue<bf16> e4;
    e4.add_col(bias).silu().clamp(-6.0f, 6.0f);            // the builder order of BASELINE's config 4
    const std::vector<EpNode> r4 = e4.resolved(7);
    EXPECT(r4.size() == 4);
    EXPECT(r4[0].op == SMEG_OP_ADD_COL && r4[0].ptr == bias.data());
    EXPECT(r4[1].op == SMEG_OP_MAX_SCALAR && r4[1].scalar == -6.0f && r4[2].op == SMEG_OP_MIN_SCALAR && r4[2].scalar == 6.0f);
    EXPECT(r4[3].op == SMEG_OP_ACT && r4[3].aux == SMEG_ACT_SILU);          // bias -> clamp -> silu
    EXPECT(Epilogue<f16>().add_scalar(0.1f).nodes()[0].scalar == 0.0999755859375f);
    EXPECT(Epilogue<bf16>().add_scalar(0.1f).nodes()[0].scalar == 0.10009765625f);
    Epilogue<f16> e;
    e.mul_row(rowv).leaky_relu(0.25f).add_tensor(tens).sub_tensor_strided(tens, 9).gelu().neg();
    const std::vector<EpNode> r = e.resolved(7);
    EXPECT(r.size() == 6 && r[1].op == SMEG_OP_ACT && r[1].aux == SMEG_ACT_LEAKY_RELU && r[1].scalar == 0.25f);
    EXPECT(r[2].op == SMEG_OP_ADD_TENSOR && r[2].ld == 7 && r[3].op == SMEG_OP_SUB_TENSOR && r[3].ld == 9);
    EXPECT(r[4].aux == SMEG_ACT_NEG && r[5].op == SMEG_OP_ACT && r[5].aux == SMEG_ACT_GELU);
    EXPECT(e.desc(7).n_nodes == 6 && Epilogue<f16>().desc(7).n_nodes == 0 && Epilogue<f16>().is_empty() && !e.is_empty());
    e.validate(3, 7);
    EXPECT(thrown([&] { e.validate(4, 7); }) == "row operand is per-M (length m)");
    EXPECT(thrown([&] { Epilogue<f16>().add_col(bias).validate(3, 8); }) == "col operand is per-N (length n)");
    EXPECT(thrown([&] { Epilogue<f16>().add_tensor_strided(tens, 5).validate(3, 7); }) == "tensor row stride must be >= n");
    EXPECT(thrown([&] { Epilogue<f16>().add_tensor(tens).validate(5, 7); }) == "tensor must hold m*n elements (stride ld)");
    Epilogue<f16> lead;
    lead.add_col(bias);
    const Epilogue<f16> both = Epilogue<f16>().mul_scalar(2.0f).relu().with_leading(lead);
    const std::vector<EpNode> rb = both.resolved(7);
    EXPECT(rb.size() == 3 && rb[0].op == SMEG_OP_ADD_COL && rb[1].op == SMEG_OP_MUL_SCALAR && rb[2].aux == SMEG_ACT_RELU);
    EXPECT(sizeof(EpNode) == 32 && sizeof(ep_desc16) == 16);

    // ---- interleave: 32 gate columns then 32 up columns; written out for a comparison with the Python mirror ----
    const size_t n = 70, k = 5;
    std::vector<float> g(n * k), u(n * k);
    for (size_t i = 0; i < n * k; ++i) {
        g[i] = (float)i;
        u[i] = -(float)i - 1.0f;
    }
    const std::vector<float> oi = interleave_gate_up(g, u, WeightLayout::OutIn, n, k);
    const std::vector<float> io = interleave_gate_up(g, u, WeightLayout::InOut, n, k);
    EXPECT(oi.size() == 2 * n * k && oi[0] == g[0] && oi[32] == u[0] && oi[64] == g[32 * k]);
    write_file(out + "/interleave_outin.bin", oi.data(), oi.size() * 4);
    write_file(out + "/interleave_inout.bin", io.data(), io.size() * 4);

    // ---- slices are checked before the library is asked; a failing library call throws with its code ----
    std::vector<uint8_t> quants(8, 0x33);
    std::vector<uint16_t> scales(4, 0x3400);
    EXPECT(thrown([&] { Q4Weights::new_(quants, scales, 4, 5); }) == "quants is ceil(n*k/2) bytes");
    EXPECT(thrown([&] { Q4Weights::with_params(quants, scales, Bits(), 4, 4, Q4Params().affine()); }) == "Q4Form::Affine requires a mins array");
    EXPECT(thrown([&] { Q4Weights::with_params(quants, scales, scales, 4, 4, Q4Params()); }) == "Q4Form::Scale takes no mins array");
    std::vector<float> w(16, 0.5f);
    EXPECT(thrown([&] { Q4Weights::quantize(w, WeightLayout::OutIn, 4, 5); }) == "w is n*k");

    // ---- the cache's bookkeeping and refusals (no device memory is touched before a launch) ----
    KvCache cache(nullptr, nullptr, 8, 2, 80, 16);
    EXPECT(cache.scale() == 0.11180339753627777f && cache.row_len() == 160 && cache.query_len() == 640 && cache.is_empty());
    EXPECT(thrown([] { KvCache(nullptr, nullptr, 8, 2, 20, 4); }) == "head_dim must be a multiple of 8 in 8..=256");
    EXPECT(thrown([] { KvCache(nullptr, nullptr, 6, 4, 64, 4); }) == "heads must be a positive multiple of kv_heads");
    EXPECT(thrown([&] { cache.extend_from_dev(nullptr, 960, 640, 800, 17, nullptr); }) == "KvCache full: 0 + 17 rows over capacity 16");
    EXPECT(thrown([&] { cache.attend_causal_dev(nullptr, 960, 1, nullptr, nullptr); }) == "attend_causal: 1 rows but 0 cached");
    EXPECT(thrown([] { Norm::rms(nullptr, 0, 1e-5f); }) == "a norm needs at least one feature");
    EXPECT(Norm::layer(nullptr, nullptr, 96, 1e-5f).width() == 96);
    std::printf(g_failed ? "CPU CHECKS FAILED\n" : "CPU CHECKS OK\n");
    return g_failed;
}

static bool all_equal(const std::vector<uint16_t>& c, size_t m, size_t n, const float* per_row) {
    for (size_t i = 0; i < m; ++i)
        for (size_t j = 0; j < n; ++j)
            if (f16_bits_to_f32(c[i * n + j]) != per_row[i]) return false;
    return true;
}

static int run_gpu() {
    const size_t m = 3, n = 256, k = 128;
    const float rows[3] = {0.5f, 1.0f, 2.0f};
    std::vector<uint16_t> a(m * k), c(m * n, 0);
    for (size_t i = 0; i < m; ++i)
        for (size_t d = 0; d < k; ++d) a[i * k + d] = f32_to_f16_bits(rows[i]);
    // Q4: every code 3, every scale 0.25 -> weights of 0.75; C = 96 * a(i)
    std::vector<uint8_t> quants(n * k / 2, 0x33);
    std::vector<uint16_t> scales(n * (k / 32), f32_to_f16_bits(0.25f));
    const Q4Weights w = Q4Weights::new_(quants, scales, n, k);
    matmul_q4(a, w, c, m);
    const float want[3] = {48.0f, 96.0f, 192.0f};
    EXPECT(all_equal(c, m, n, want));
    // ... + bias 1, then relu: C + 1
    std::vector<uint16_t> bias(n, f32_to_f16_bits(1.0f));
    Epilogue<f16> ep;
    ep.add_col(bias).relu();
    matmul_q4_ep(a, w, c, m, ep);
    const float want1[3] = {49.0f, 97.0f, 193.0f};
    EXPECT(all_equal(c, m, n, want1));
    // dense Gemm on the same weights as f16, beta 0.5
    std::vector<uint16_t> b(k * n, f32_to_f16_bits(0.75f));
    const Packed<f16> packed = prepack_f16(b, n, k);
    Gemm<f16> gm(a, packed, m);
    gm.beta(0.5f).run(c);
    const float want2[3] = {24.0f, 48.0f, 96.0f};
    EXPECT(all_equal(c, m, n, want2));
    // MLP block: gate = up = 0.75 * sum(x) = 96 x; silu(g) * u is not a binary fraction, so only check y against the same
    // block run twice from a zero stream (y2 = 2 * y1 exactly) and the sign of the result
    const size_t d = 128, f = 64;
    std::vector<float> wg(f * d, 0.01f), wu(f * d, 0.02f), wd(d * f, 0.03f);
    Mlp mlp = Mlp::gated(GatedLinear::quantize(wg, wu, WeightLayout::OutIn, f, d, Gate::Silu), Linear::quantize(wd, WeightLayout::OutIn, d, f));
    std::vector<uint16_t> x(2 * d, f32_to_f16_bits(1.0f));
    std::vector<float> y(2 * d, 0.0f);
    mlp.accumulate(x, y, 2);
    const std::vector<float> y1 = y;
    mlp.accumulate(x, y, 2);
    bool ok = true;
    for (size_t i = 0; i < y.size(); ++i) ok = ok && y1[i] > 0.0f && y[i] == 2.0f * y1[i];
    EXPECT(ok);
    EXPECT(smeg_last_status() == 0);
    // a 1-bit layer (every sign +, scale 0.5) with a bias, through Linear's routing: rows of constant x quantise to q = 127,
    // sa = x / 127; the cell is the fold of k / 32 blocks of sum 127 * 32, then + 1
    std::vector<uint8_t> signs(n * k / 8, 0xFF);
    std::vector<uint16_t> sc1(n * (k / 32), f32_to_f16_bits(0.5f));
    Linear l1 = Linear::from_q1(Q1Weights::new_(signs, sc1, WeightLayout::OutIn, n, k, 32), bias);
    l1.forward(a, c, m);
    float want3[3];
    for (size_t i = 0; i < m; ++i) {
        const float wgt = 0.5f * (rows[i] / 127.0f);
        float tot = 0.0f;
        for (size_t blk = 0; blk < k / 32; ++blk) tot = std::fma(4064.0f, wgt, tot);
        want3[i] = f16_bits_to_f32(f32_to_f16_bits(f16_bits_to_f32(f32_to_f16_bits(tot)) + 1.0f));
    }
    EXPECT(all_equal(c, m, n, want3));
    std::printf(g_failed ? "GPU CHECKS FAILED\n" : "GPU CHECKS OK\n");
    return g_failed;
}

int main(int argc, char** argv) {
    try {
        if (argc >= 4 && std::string(argv[1]) == "cpu") return run_cpu(argv[2], argv[3]);
        if (argc >= 2 && std::string(argv[1]) == "gpu") return run_gpu();
    } catch (const std::exception& e) {
        std::printf("error: %s\n", e.what());
        return 3;
    }
    std::printf("usage: host_mirror_check cpu IN_F32 OUT_DIR | gpu\n");
    return 2;
}
