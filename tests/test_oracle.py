"""Pins the CPU oracle (oracle/oracle.c) before anything is checked against it.

Two anchors, because the reference (Rust) cannot be executed in this
environment and ships no golden-vector files for this path:
  1. bit equality with an independent numpy restatement (oracle/np_oracle.py);
  2. the closed-form known-answer tests of the reference's own unit tests,
     restated with the reference's seeds and shapes.
"""
import numpy as np
import pytest

import oracle as orc
from oracle import np_oracle as npo
from refgen import Lcg, data


def rng(seed):
    return np.random.default_rng(seed)


# ---------------------------------------------------------------- conversions

def test_f16_bf16_conversions_match_numpy():
    r = rng(1)
    x = np.concatenate([
        r.standard_normal(20000).astype(np.float32),
        (r.standard_normal(5000) * 1e-6).astype(np.float32),     # f16 subnormals
        (r.standard_normal(5000) * 1e5).astype(np.float32),      # overflow to inf
        np.array([0.0, -0.0, np.inf, -np.inf, 65504.0, 65520.0, 65519.99, 2.0 ** -24, 2.0 ** -25,
                  1.5 * 2.0 ** -25, 2.0 ** -14, 1.0009765625, 1.00048828125], np.float32),
    ])
    assert np.array_equal(orc.f32_to_f16_bits(x), npo.f16_bits(x))
    assert np.array_equal(orc.f32_to_bf16_bits(x), npo.bf16_bits(x))
    bits = np.arange(65536, dtype=np.uint16)
    a, b = orc.f16_bits_to_f32(bits), npo.f16_val(bits)
    ok = (a == b) | (np.isnan(a) & np.isnan(b))
    assert ok.all()
    # direct f64 -> f16 (single rounding), where f64 -> f32 -> f16 would double round
    L = orc.lib()
    d = 1.0 + 2.0 ** -11 + 2.0 ** -30            # just above an f16 tie
    assert L.orc_f64_to_f16(d) == np.float64(d).astype(np.float16).view(np.uint16)
    assert L.orc_f64_to_f16(d) != np.float32(1.0 + 2.0 ** -11).astype(np.float16).view(np.uint16)
    for v in r.standard_normal(2000) * 3.0:
        assert L.orc_f64_to_f16(float(v)) == np.float64(v).astype(np.float16).view(np.uint16)


# ------------------------------------------------------- C == numpy, Q4 path

@pytest.mark.parametrize("n,k,block,affine,layout", [
    (33, 64, 32, False, 0), (40, 100, 32, True, 1), (8, 96, 64, False, 1), (17, 130, 16, True, 0),
    (64, 256, 32, False, 0), (5, 7, 1, False, 0), (5, 9, 2, True, 1),
])
def test_q4_quantize_dequant_c_equals_numpy(n, k, block, affine, layout):
    w = (rng(n * 1000 + k).standard_normal(n * k) * 0.02).astype(np.float32)
    w[::17] = 0.0
    qc, sc, mc = orc.q4_quantize(w, layout, n, k, block, affine)
    qn, sn, mn = npo.q4_quantize(w, layout, n, k, block, affine)
    assert np.array_equal(qc, qn) and np.array_equal(sc, sn)
    if affine:
        assert np.array_equal(mc, mn)
    for bf16 in (False, True):
        assert np.array_equal(orc.q4_dequant(qc, sc, mc, n, k, block, bf16).reshape(-1),
                              npo.q4_dequant(qn, sn, mn, n, k, block, bf16).reshape(-1))


@pytest.mark.parametrize("m,n,k,bf16", [(1, 33, 256, False), (3, 70, 129, True), (7, 5, 3, False), (2, 96, 64, True)])
def test_gemm16_c_equals_numpy(m, n, k, bf16):
    r = rng(m + n + k)
    to = orc.f32_to_bf16_bits if bf16 else orc.f32_to_f16_bits
    a = to(r.standard_normal((m, k)).astype(np.float32))
    b = to((r.standard_normal((k, n)) * 0.05).astype(np.float32))
    assert np.array_equal(orc.gemm16(a, b, m, n, k, bf16), npo.gemm16(a, b, m, n, k, bf16))


def _node_items(m, n, bf16, seed):
    r = rng(seed)
    to = orc.f32_to_bf16_bits if bf16 else orc.f32_to_f16_bits
    row = to(r.standard_normal(m).astype(np.float32))
    col = to((r.standard_normal(n) + 2.0).astype(np.float32))
    ten = to(r.standard_normal(m * (n + 3)).astype(np.float32))
    items = [(5, 0, 0.0, col, 0), (4, 0, 0.0, col, 0), (2, 0, 0.0, row, 0), (6, 0, 0.0, ten, n + 3),
             (1, 0, 0.75, None, 0), (11, 0, 0.1, None, 0), (17, 0, 0.0, col, 0), (9, 0, -2.0, None, 0),
             (10, 0, 2.5, None, 0), (22, 0, 0.0, row, 0), (21, 0, 0.0, ten, n + 3), (15, 0, 3.0, None, 0)]
    return items


@pytest.mark.parametrize("bf16", [False, True])
def test_epilogue_binary_nodes_c_equals_numpy(bf16):
    m, n = 5, 37
    to = orc.f32_to_bf16_bits if bf16 else orc.f32_to_f16_bits
    c = to(rng(3).standard_normal((m, n)).astype(np.float32) * 3)
    items = _node_items(m, n, bf16, 11)
    got = orc.apply_ep(c, m, n, orc.Nodes(items), bf16)
    want = npo.apply_ep(c, m, n, items, bf16)
    assert np.array_equal(got, want)


@pytest.mark.parametrize("kind", list(range(1, 25)))
def test_epilogue_activations_c_equals_numpy(kind):
    m, n = 3, 64
    x = np.linspace(-9, 9, m * n).astype(np.float32)
    x[5] = 0.0
    c = orc.f32_to_f16_bits(x).reshape(m, n)
    alpha = 0.2 if kind in (6, 20) else 0.0
    items = [(8, kind, alpha, None, 0)]
    got = orc.f16_bits_to_f32(orc.apply_ep(c, m, n, orc.Nodes(items)))
    want = orc.f16_bits_to_f32(npo.apply_ep(c, m, n, items))
    same = (got == want) | (np.isnan(got) & np.isnan(want))
    assert same.all(), (kind, got[~same][:4], want[~same][:4])


def test_trailing_activation_order_cfg4_graph():
    """add_col(bias).silu().clamp(-6,6) resolves to bias -> max(-6) -> min(6) -> silu
    (src/epilogue/graph.rs:185-238, src/exec/scalar.rs:28-53)."""
    m, n = 2, 8
    c = orc.f32_to_f16_bits(np.array([[-9, -7, -1, 0, 1, 5, 7, 9]] * 2, np.float32))
    bias = orc.f32_to_f16_bits(np.full(n, 0.5, np.float32))
    items = [(4, 0, 0.0, bias, 0), (9, 0, -6.0, None, 0), (10, 0, 6.0, None, 0), (8, 3, 0.0, None, 0)]
    got = orc.f16_bits_to_f32(orc.apply_ep(c, m, n, orc.Nodes(items)))
    x = np.clip(np.array([-9, -7, -1, 0, 1, 5, 7, 9], np.float64) + 0.5, -6, 6)
    want = (x / (1 + np.exp(-x))).astype(np.float32).astype(np.float16).astype(np.float32)
    assert np.array_equal(got[0], want)


def test_nan_rules_of_min_max_and_clamp_activations():
    """MAX/MIN/ReLU are maxNum (drop NaN), clamp-style activations propagate it
    (tests/correctness/nan.rs of the reference)."""
    c = np.array([[0x7e00, 0x3c00]], np.uint16)  # NaN, 1.0
    out = orc.f16_bits_to_f32(orc.apply_ep(c, 1, 2, orc.Nodes([(9, 0, 0.5, None, 0)])))
    assert out[0, 0] == 0.5 and out[0, 1] == 1.0
    out = orc.f16_bits_to_f32(orc.apply_ep(c, 1, 2, orc.Nodes([(8, 1, 0.0, None, 0)])))
    assert out[0, 0] == 0.0
    out = orc.f16_bits_to_f32(orc.apply_ep(c, 1, 2, orc.Nodes([(8, 7, 0.0, None, 0)])))
    assert np.isnan(out[0, 0]) and out[0, 1] == 1.0


# ------------------------------------------------------ C == numpy, low-bit

@pytest.mark.parametrize("k,block", [(256, 64), (37, 16), (300, 128), (1, 16), (513, 4096)])
def test_quantize_row_c_equals_numpy(k, block):
    a = orc.f32_to_f16_bits(rng(k).standard_normal(k).astype(np.float32) * 2)
    if k > 20:
        a[3] = 0x7e00  # NaN poisons its block's scale and quantises to 0
        a[k - 1] = 0x7c00  # +inf
    qc, sc = orc.quantize_row(a, block)
    qn, sn = npo.quantize_row(a, block)
    assert np.array_equal(qc, qn)
    assert np.array_equal(sc.view(np.uint32), sn.view(np.uint32))


def test_quantize_row_ties_to_even_and_saturation():
    # amax = 127 -> inv = 1: 0.5 -> 0, 1.5 -> 2, 2.5 -> 2, -0.5 -> -0 (0), -1.5 -> -2
    a = np.array([127.0, 0.5, 1.5, 2.5, -0.5, -1.5, -127.0, 0.0] + [0.0] * 8, np.float16).view(np.uint16)
    q, s = orc.quantize_row(a, 16)
    assert list(q[:8]) == [127, 0, 2, 2, 0, -2, -127, 0]
    assert s[0] == np.float32(1.0)


SHAPES = [(1, 64, 256), (1, 65, 37), (1, 1, 1), (2, 200, 300), (3, 64, 16), (5, 130, 513)]
BOOKS = [[-1, 0, 1, 0], [-2, -1, 1, 2], [-128, 127, 3, -7]]


@pytest.mark.parametrize("si", range(len(SHAPES)))
def test_lowbit_matmul_c_equals_numpy_on_reference_shapes(si):
    """Inputs regenerated as src/kernels/lowbit/matmul.rs:457-494 builds them."""
    m, n, k = SHAPES[si]
    for bi, block in enumerate([16, 64, 128, 4096]):
        nbk = -(-k // block)
        scales = orc.f32_to_f16_bits(data(si + 7, n * nbk).astype(np.float32) * np.float32(1e-3) - np.float32(0.1))
        a = orc.f32_to_f16_bits((data(si + 99, m * k).astype(np.float32) - np.float32(128.0)) / np.float32(37.0))
        book = BOOKS[(si + bi) % 3]
        codes = data(si * 31 + bi, (k * n + 3) // 4)
        c, q, sa, sums = orc.lowbit_matmul(a, 2, codes, 1, scales, book, n, k, block, m, debug=True)
        cn, sums_n = npo.lowbit_matmul(a, npo.q2_values(codes, n, k, book), scales, n, k, block, m)
        assert np.array_equal(sums, sums_n)
        assert np.array_equal(c, cn), f"q2 {m}x{n}x{k} block {block}"
        signs = data(si * 17 + bi, (k * n + 7) // 8)
        for layout in (0, 1):
            c = orc.lowbit_matmul(a, 1, signs, layout, scales, None, n, k, block, m)
            cn, _ = npo.lowbit_matmul(a, npo.q1_values(signs, layout, n, k), scales, n, k, block, m)
            assert np.array_equal(c, cn), f"q1 {m}x{n}x{k} block {block} layout {layout}"


def test_lowbit_k_zero_gives_zeros():
    """src/kernels/lowbit/matmul.rs:395-397."""
    c = orc.lowbit_matmul(np.zeros(0, np.uint16), 2, np.zeros(0, np.uint8), 1, np.zeros(0, np.uint16),
                          BOOKS[0], 4, 0, 16, 2)
    assert (c == 0).all()


def test_lowbit_dequant_c_equals_numpy():
    n, k, block = 70, 130, 64
    scales = orc.f32_to_f16_bits(rng(5).uniform(0.01, 0.05, n * 3).astype(np.float32))
    codes = data(5, (k * n + 3) // 4)
    for book in BOOKS:
        assert np.array_equal(orc.lowbit_dequant(2, codes, 1, scales, book, n, k, block).reshape(-1),
                              npo.lowbit_dequant(npo.q2_values(codes, n, k, book), scales, n, k, block, False).reshape(-1))
    signs = data(6, (k * n + 7) // 8)
    for layout in (0, 1):
        assert np.array_equal(orc.lowbit_dequant(1, signs, layout, scales, None, n, k, block).reshape(-1),
                              npo.lowbit_dequant(npo.q1_values(signs, layout, n, k), scales, n, k, block, True).reshape(-1))


# ------------------------------------- the reference's closed-form unit tests

def _weights_pattern(n, k):
    i = np.arange(n * k, dtype=np.uint64)
    return (((i * np.uint64(2654435761)) % np.uint64(1000)).astype(np.float32) / np.float32(500.0) - np.float32(1.0))


@pytest.mark.parametrize("n,k,block", [(33, 64, 32), (40, 100, 32), (8, 96, 64)])
def test_q4_quantize_round_trips_within_half_a_step(n, k, block):
    """src/kernels/q4/quantize.rs:100-134."""
    w = _weights_pattern(n, k)
    t = w.reshape(n, k).T.copy().reshape(-1)
    for affine in (False, True):
        qa = orc.q4_quantize(w, 0, n, k, block, affine)
        qb = orc.q4_quantize(t, 1, n, k, block, affine)
        da = orc.f16_bits_to_f32(orc.q4_dequant(*qa, n, k, block))
        db = orc.f16_bits_to_f32(orc.q4_dequant(*qb, n, k, block))
        assert np.array_equal(da, db)
        W = w.reshape(n, k)
        for d in range(k):
            blk = W[:, (d // block) * block:min((d // block + 1) * block, k)]
            lo, hi = blk.min(axis=1), blk.max(axis=1)
            step, bound = ((hi - lo) / 15.0, 0.5) if affine else (np.maximum(np.abs(lo), np.abs(hi)) / 8.0, 1.0)
            assert (np.abs(da[d] - W[:, d]) <= step * bound + 0.01).all()


def test_q4_scale_equals_affine_with_zero_mins_and_min_shifts_by_one():
    """src/kernels/q4/weights.rs:358-397."""
    n, k, block = 48, 64, 32
    nbk = k // block
    quants = (np.arange((k * n + 1) // 2) % 251).astype(np.uint8)
    scales = orc.f32_to_f16_bits(np.float32(0.02) + np.float32(0.001) * (np.arange(n * nbk) % 3).astype(np.float32))
    plain = orc.q4_dequant(quants, scales, None, n, k, block)
    aff = orc.q4_dequant(quants, scales, np.zeros(n * nbk, np.uint16), n, k, block)
    assert np.array_equal(plain, aff)
    ones = orc.f32_to_f16_bits(np.ones(n * nbk, np.float32))
    shifted = orc.q4_dequant(quants, scales, ones, n, k, block)
    assert (np.abs(orc.f16_bits_to_f32(shifted) - orc.f16_bits_to_f32(plain) - 1.0) < 1e-2).all()


@pytest.mark.parametrize("n,k", [(1, 1), (3, 5), (32, 32), (33, 31), (48, 1), (17, 64), (64, 65), (31, 96)])
def test_q4_dequant_equals_canonical_f32_product(n, k):
    """src/kernels/q4/weights.rs:399-463: f16(f32(scale) * code) is the same
    value as the f64-exact product rounded once."""
    s = Lcg(0xa4a45151dead0001 ^ (n * 131 + k * 17))
    quants = s.bytes((k * n + 1) // 2)
    nbk = -(-k // 32)
    scales = orc.f32_to_f16_bits(np.float32(0.01) + np.float32(0.001) * (np.arange(n * nbk) % 7).astype(np.float32))
    got = orc.q4_dequant(quants, scales, None, n, k, 32)
    codes = npo.q4_codes_from_quants(quants, n, k).astype(np.float32)
    sc = orc.f16_bits_to_f32(scales).reshape(n, nbk)[:, np.arange(k) // 32].T
    want = orc.f32_to_f16_bits((sc * codes).astype(np.float32))
    assert np.array_equal(got, want)


def _band_q4_code(nib, n, k, d, j):
    byte = nib[(j // 128) * k * 64 + d * 64 + (j % 128) // 2]
    return (byte >> (4 * (j % 2))) & 0x0F   # c % 2 == j % 2 because 128 is even


@pytest.mark.parametrize("n,k,block", [(33, 96, 16), (130, 70, 32), (17, 130, 64), (1, 1, 32)])
def test_reference_band_pack_q4_round_trips(n, k, block):
    """Q4Weights::with_params layout (src/kernels/q4/weights.rs:92-113) read back
    the way dequant_rows reads it (:240-249)."""
    quants = data(n * 7 + k, (k * n + 1) // 2)
    nbk = -(-k // block)
    scales = np.arange(n * nbk, dtype=np.uint16) + 1
    nib, sc, _ = orc.q4_pack_band(quants, scales, None, n, k, block)
    for d in range(0, k, max(1, k // 7)):
        for j in range(n):
            idx = d * n + j
            want = (quants[idx // 2] >> (4 * (idx % 2))) & 0x0F
            assert _band_q4_code(nib, n, k, d, j) == want
            assert sc[(j // 128) * nbk * 128 + (d // block) * 128 + j % 128] == scales[j * nbk + d // block]


def _scale_index(spb, blk, j):
    c = j % 64
    return (j // 64) * spb + blk * 64 + (c // 32) * 32 + 2 * (c % 16) + (c % 32) // 16


@pytest.mark.parametrize("n,k,block", [(1, 1, 16), (65, 37, 16), (130, 300, 256)])
def test_reference_band_pack_q2_round_trips(n, k, block):
    """src/kernels/lowbit/q2.rs:197-223."""
    nbk = -(-k // block)
    codes = ((np.arange((k * n + 3) // 4) * 37) % 251).astype(np.uint8)
    scales = orc.f32_to_f16_bits(np.arange(n * nbk, dtype=np.float32) * np.float32(0.5))
    packed, sc = orc.q2_pack_band(codes, scales, n, k, block)
    band_bytes = (-(-k // 16) * 16) * 16
    for d in range(k):
        for j in range(n):
            idx = d * n + j
            want = (codes[idx // 4] >> (2 * (idx % 4))) & 3
            got = (packed[(j // 64) * band_bytes + (d // 4) * 64 + j % 64] >> (2 * (d % 4))) & 3
            assert got == want
    for j in range(n):
        for b in range(nbk):
            assert sc[_scale_index(nbk * 64, b, j)] == scales[j * nbk + b]


@pytest.mark.parametrize("n,k,block", [(1, 1, 16), (65, 37, 16), (130, 300, 128)])
def test_reference_band_pack_q1_round_trips(n, k, block):
    """src/kernels/lowbit/q1.rs:245-274."""
    nbk = -(-k // block)
    signs = ((np.arange((k * n + 7) // 8) * 37) % 251).astype(np.uint8)
    scales = orc.f32_to_f16_bits(np.arange(n * nbk, dtype=np.float32) * np.float32(0.5))
    band_bytes = (-(-k // 16) * 16) * 8
    for layout in (0, 1):
        packed, sc = orc.q1_pack_band(signs, layout, scales, n, k, block)
        for j in range(n):
            for d in range(k):
                idx = j * k + d if layout == 0 else d * n + j
                want = (signs[idx // 8] >> (idx % 8)) & 1
                c = j % 64
                got = (packed[(j // 64) * band_bytes + (d // 4) * 32 + c // 2] >> (4 * (c % 2) + d % 4)) & 1
                assert got == want


def test_q2_quantize_recovers_grid_weights():
    """src/kernels/lowbit/q2.rs:225-261."""
    n, k = 70, 300
    for cb, levels in (([-1, 0, 1, 0], [-1.0, 0.0, 1.0]), ([-2, -1, 1, 2], [-2.0, -1.0, 1.0, 2.0])):
        i = np.arange(n * k)
        lv = np.asarray(levels, np.float32)[(i * 7 + i // 5) % len(levels)]
        w = (lv * np.float32(0.03125) * (1 + i // k % 3).astype(np.float32)).astype(np.float32)
        t = w.reshape(n, k).T.copy().reshape(-1)
        for arr, layout in ((w, 0), (t, 1)):
            codes, scales = orc.q2_quantize(arr, layout, n, k, 64, cb)
            vals = npo.q2_values(codes, n, k, cb).astype(np.float32)
            sc = orc.f16_bits_to_f32(scales).reshape(n, -1)[:, np.arange(k) // 64].T
            got = (sc * vals).astype(np.float32)
            assert np.array_equal(got.T.reshape(-1).view(np.uint32), w.view(np.uint32))


def test_q1_quantize_recovers_sign_weights():
    """src/kernels/lowbit/q1.rs:278-296."""
    n, k, block = 70, 300, 64
    i = np.arange(n * k)
    w = (np.where((i * 7 + i // 5) % 3 == 0, -1.0, 1.0) * 0.25 * (1 + i // k % 3)).astype(np.float32)
    signs, scales = orc.q1_quantize(w, 0, n, k, block)
    vals = npo.q1_values(signs, 0, n, k).astype(np.float32)
    sc = orc.f16_bits_to_f32(scales).reshape(n, -1)[:, np.arange(k) // block].T
    assert np.array_equal((sc * vals).T.reshape(-1), w)


def test_q2_matches_f64_product_within_activation_rounding():
    """The analytic bound of tests/correctness/q2.rs:43-78:
    |got - want| <= sum|w|*amax/254*1.001 + |want|/1024 + 1e-6."""
    for (m, n, k), block, cb in (((7, 50, 200), 256, [-1, 0, 1, 0]), ((33, 17, 9), 32, [-2, -1, 1, 2]),
                                 ((7, 400, 800), 256, [-1, 0, 1, 0])):
        r = rng(k)
        nbk = -(-k // block)
        codes = r.integers(0, 256, (k * n + 3) // 4).astype(np.uint8)
        scales = orc.f32_to_f16_bits(r.uniform(0.01, 0.05, n * nbk).astype(np.float32))
        a = Lcg(0x02029401dead0001 ^ (m * 131 + n * 17 + k + block)).fill(m * k)
        c = orc.f16_bits_to_f32(orc.lowbit_matmul(a, 2, codes, 1, scales, cb, n, k, block, m)).astype(np.float64)
        wf = (orc.f16_bits_to_f32(scales).reshape(n, nbk)[:, np.arange(k) // block].T.astype(np.float64)
              * npo.q2_values(codes, n, k, cb))
        af = a.astype(np.float64).reshape(m, k)
        want = af @ wf
        amax = np.stack([np.abs(af[:, b * block:(b + 1) * block]).max(axis=1) for b in range(nbk)], axis=1)
        bound = (amax[:, np.arange(k) // block] / 254.0) @ np.abs(wf)
        assert (np.abs(c - want) <= bound * 1.001 + np.abs(want) / 1024.0 + 1e-6).all()


def test_glu_and_interleave_follow_the_32_column_chunks():
    """src/linear.rs:603-617 and :804-835; n = 70 has a ragged last chunk."""
    m, n, k = 3, 70, 5
    g = np.arange(k * n, dtype=np.float32).reshape(k, n)
    u = -g
    both = orc.interleave(g, u, n, k)
    assert np.array_equal(both[:, 0:32], g[:, 0:32]) and np.array_equal(both[:, 32:64], u[:, 0:32])
    assert np.array_equal(both[:, 128:134], g[:, 64:70]) and np.array_equal(both[:, 134:140], u[:, 64:70])
    r = rng(9)
    bb = orc.f32_to_f16_bits(r.standard_normal((m, 2 * n)).astype(np.float32) * 3)
    y = orc.f16_bits_to_f32(orc.glu(bb, m, n))
    yn = orc.f16_bits_to_f32(npo.glu(bb, m, n))
    # numpy's f32 exp is not glibc's expf: allow the last f16 place
    assert (np.abs(y - yn) <= np.abs(yn) * 2.0 ** -10 + 1e-7).all()
    dst = np.ones(6, np.float32)
    orc.add_f16(np.array([1, 2, 3, 4, 5, 6], np.float16), dst)
    assert np.array_equal(dst, np.array([2, 3, 4, 5, 6, 7], np.float32))


def test_threads_do_not_change_results():
    m, n, k = 6, 70, 96
    r = rng(4)
    w = (r.standard_normal(n * k) * 0.02).astype(np.float32)
    q, s, _ = orc.q4_quantize(w, 0, n, k)
    a = orc.f32_to_f16_bits(r.standard_normal((m, k)).astype(np.float32))
    orc.set_threads(1)
    c1 = orc.matmul_q4(a, q, s, None, n, k, 32, m)
    orc.set_threads(4)
    c4 = orc.matmul_q4(a, q, s, None, n, k, 32, m)
    orc.set_threads(1)
    assert np.array_equal(c1, c4)
    assert np.array_equal(c1, orc.gemm16(a, orc.q4_dequant(q, s, None, n, k), m, n, k))


@pytest.mark.parametrize("heads,kv_heads,hd,start,rows", [(4, 4, 16, 0, 1), (6, 2, 32, 7, 5), (2, 1, 64, 30, 3)])
def test_attention_oracle_against_an_f64_statement(heads, kv_heads, hd, start, rows):
    """orc_attention_kv_causal (src/kernels/kv_attention.rs:155-331) against the same formula in f64: q * scale rounded
    to f16 once, grouped-query head mapping, causal prefix, softmax, value average."""
    rng = np.random.default_rng(heads + start)
    n = start + rows
    q = rng.standard_normal((rows, heads * hd)).astype(np.float32)
    k = orc.f32_to_f16_bits(rng.standard_normal((n, kv_heads * hd)).astype(np.float32))
    v = orc.f32_to_f16_bits(rng.standard_normal((n, kv_heads * hd)).astype(np.float32))
    scale = 1.0 / np.sqrt(hd)
    got = orc.attention_kv_causal(q, k, v, start, rows, heads, kv_heads, hd, scale).reshape(rows, heads, hd)
    kf = orc.f16_bits_to_f32(k).reshape(n, kv_heads, hd).astype(np.float64)
    vf = orc.f16_bits_to_f32(v).reshape(n, kv_heads, hd).astype(np.float64)
    qh = orc.f16_bits_to_f32(orc.f32_to_f16_bits(q * np.float32(scale))).reshape(rows, heads, hd).astype(np.float64)
    group = heads // kv_heads
    for i in range(rows):
        length = start + i + 1
        for h in range(heads):
            s = kf[:length, h // group] @ qh[i, h]
            p = np.exp(s - s.max())
            want = (p[:, None] * vf[:length, h // group]).sum(0) / p.sum()
            assert np.max(np.abs(got[i, h] - want)) <= 2e-6 * (1.0 + np.max(np.abs(want)))
    # one row with start = len - 1 is attention_kv_f16; a row of a block equals the one-row call over its prefix exactly
    one = orc.attention_kv_causal(q[rows - 1:], k, v, n - 1, 1, heads, kv_heads, hd, scale)
    assert np.array_equal(one.reshape(-1), got[rows - 1].reshape(-1))


def test_closed_form_products_with_exactly_representable_inputs():
    """Known answers that need no second implementation (in the spirit of the reference's closed form C = k * a(i) * b(j),
    tests/concurrency.rs:31-39): constant rows against constant weights whose every partial sum is an exact binary
    fraction, so the result is known without any rounding."""
    m, n, k, block = 3, 5, 64, 32
    # Q4: every code 3, every scale 0.25 -> every weight 0.75; row i of A is the constant 2^(i-1)
    quants = np.full((k * n + 1) // 2, 0x33, np.uint8)
    scales = orc.f32_to_f16_bits(np.full(n * (k // block), 0.25, np.float32))
    a = np.repeat(np.array([0.5, 1.0, 2.0], np.float32), k).reshape(m, k)
    c = orc.f16_bits_to_f32(orc.matmul_q4(orc.f32_to_f16_bits(a), quants, scales, None, n, k, block, m)).reshape(m, n)
    assert np.array_equal(c, np.repeat(np.array([24.0, 48.0, 96.0], np.float32), n).reshape(m, n))
    # the affine form adds the block's minimum to every weight: + 0.25 -> weights of 1.0
    mins = orc.f32_to_f16_bits(np.full(n * (k // block), 0.25, np.float32))
    c = orc.f16_bits_to_f32(orc.matmul_q4(orc.f32_to_f16_bits(a), quants, scales, mins, n, k, block, m)).reshape(m, n)
    assert np.array_equal(c, np.repeat(np.array([32.0, 64.0, 128.0], np.float32), n).reshape(m, n))
    # 2-bit, codebook [-2, -1, 1, 2], every code 3 (value 2), scale 0.5; a row of constant x quantises to q = 127 with
    # sa = x / 127, so a block's sum is 2 * 127 * 32 = 8128 and the cell is 2 blocks * 8128 * (0.5 * sa)
    codes = np.full((k * n + 3) // 4, 0xFF, np.uint8)
    sc2 = orc.f32_to_f16_bits(np.full(n * (k // block), 0.5, np.float32))
    c, q, sa, sums = orc.lowbit_matmul(orc.f32_to_f16_bits(a), 2, codes, 1, sc2, [-2, -1, 1, 2], n, k, block, m, debug=True)
    assert (q == 127).all() and (sums == 8128).all()
    for i, x in enumerate((0.5, 1.0, 2.0)):
        s = np.float32(x) / np.float32(127.0)
        assert (sa[i] == s).all()
        w = np.float32(0.5) * s
        tot = np.float32(np.float64(8128.0) * np.float64(w))                               # fmaf(8128, w, 0): one rounding
        tot = np.float32(np.float64(8128.0) * np.float64(w) + np.float64(tot))             # fmaf(8128, w, tot)
        assert (orc.f16_bits_to_f32(c[i]) == orc.f16_bits_to_f32(orc.f32_to_f16_bits(np.array([tot], np.float32)))[0]).all()
    # 1-bit, every sign +: the block's sum is 127 * 32
    signs = np.full((k * n + 7) // 8, 0xFF, np.uint8)
    c, q, sa, sums = orc.lowbit_matmul(orc.f32_to_f16_bits(a), 1, signs, 0, sc2, None, n, k, block, m, debug=True)
    assert (sums == 127 * 32).all()
