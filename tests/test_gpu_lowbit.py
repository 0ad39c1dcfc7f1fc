"""2-bit / 1-bit int8-activation kernels on the GPU: BIT-EXACT against the CPU
oracle (quantize_row + reference, src/kernels/lowbit/matmul.rs:354-398) --
int8 activation codes, per-block activation scales, int32 block sums and the f16
output, for the reference's own shape / block / codebook / layout grid
(src/kernels/lowbit/matmul.rs:419-494), through the C ABI."""
import numpy as np
import pytest
import torch

import oracle as orc
import sme_gemm_b200 as sg
from gpu_util import bits_of, f16_bits_dev
from refgen import Lcg, data

pytestmark = pytest.mark.gpu

SHAPES = [(1, 64, 256), (1, 65, 37), (1, 1, 1), (2, 200, 300), (3, 64, 16), (5, 130, 513), (6, 192, 256),
          (7, 100, 64), (12, 70, 200), (1, 2048, 1024), (4, 1536, 512), (9, 1024, 384)]
BOOKS = [[-1, 0, 1, 0], [-2, -1, 1, 2], [-128, 127, 3, -7]]


def _canon16(bits):
    """f16 bit patterns with every NaN mapped to one pattern (NaN payloads are not part of the contract)."""
    b = np.array(bits, np.uint16, copy=True)
    b[(b & 0x7fff) > 0x7c00] = 0x7e00
    return b


def _canon32(x):
    b = np.array(x, np.float32, copy=True).view(np.uint32)
    b[(b & 0x7fffffff) > 0x7f800000] = 0x7fc00000
    return b


def check_bits(w, kind, wbits, layout, scales, book, n, k, block, m, a_bits, what):
    c, q, sa, sums = sg.matmul_lowbit_debug(f16_bits_dev(a_bits).reshape(m, k), w, m)
    torch.cuda.synchronize()
    assert sg.last_status() == 0
    wc, wq, wsa, wsums = orc.lowbit_matmul(a_bits, kind, wbits, layout, scales, book, n, k, block, m, debug=True)
    assert np.array_equal(q.cpu().numpy(), wq), f"{what}: int8 activation codes differ"
    assert np.array_equal(_canon32(sa.cpu().numpy()), _canon32(wsa)), f"{what}: activation scales differ"
    assert np.array_equal(sums.cpu().numpy(), wsums), f"{what}: int32 block sums differ"
    got, wc = _canon16(bits_of(c)), _canon16(wc)
    bad = np.nonzero(got != wc)
    assert bad[0].size == 0, f"{what}: {bad[0].size} of {got.size} f16 outputs differ, first at {bad[0][0]},{bad[1][0]}"
    # the plain entry point gives the same bits
    c2 = torch.full((m, n), 9.0, dtype=torch.float16, device="cuda")
    (sg.matmul_q2 if kind == 2 else sg.matmul_q1)(f16_bits_dev(a_bits), w, c2, m)
    assert np.array_equal(_canon16(bits_of(c2)), wc), f"{what}: plain call differs"


@pytest.mark.parametrize("si", range(len(SHAPES)))
def test_kernels_match_reference_bits(si):
    m, n, k = SHAPES[si]
    for bi, block in enumerate([16, 64, 128, 4096]):
        nbk = -(-k // block)
        scales = orc.f32_to_f16_bits(data(si + 7, n * nbk).astype(np.float32) * np.float32(1e-3) - np.float32(0.1))
        a_bits = orc.f32_to_f16_bits((data(si + 99, m * k).astype(np.float32) - np.float32(128.0)) / np.float32(37.0))
        book = BOOKS[(si + bi) % 3]
        codes = data(si * 31 + bi, (k * n + 3) // 4)
        w2 = sg.Q2Weights.new(codes, scales, n, k, sg.Q2Params(block).with_codebook(book))
        check_bits(w2, 2, codes, 1, scales, book, n, k, block, m, a_bits, f"q2 {m}x{n}x{k} block {block} {book}")
        signs = data(si * 17 + bi, (k * n + 7) // 8)
        for layout in (0, 1):
            w1 = sg.Q1Weights.new(signs, scales, sg.WeightLayout(layout), n, k, block)
            check_bits(w1, 1, signs, layout, scales, None, n, k, block, m, a_bits, f"q1 {m}x{n}x{k} block {block} layout {layout}")


def test_results_do_not_depend_on_m():
    """"Results do not depend on m" (src/kernels/lowbit/matmul.rs:24-25): row i of an
    m-row call equals the one-row call on that row, bit for bit."""
    n, k, block = 200, 1024, 128
    rng = np.random.default_rng(2)
    codes = rng.integers(0, 256, (k * n + 3) // 4).astype(np.uint8)
    scales = orc.f32_to_f16_bits(rng.uniform(0.01, 0.05, n * (k // block)).astype(np.float32))
    w = sg.Q2Weights.new(codes, scales, n, k, sg.Q2Params(block))
    a = torch.from_numpy(rng.standard_normal((19, k)).astype(np.float16)).cuda()
    c = torch.zeros((19, n), dtype=torch.float16, device="cuda")
    sg.matmul_q2(a, w, c, 19)
    for i in (0, 7, 8, 18):
        ci = torch.zeros((1, n), dtype=torch.float16, device="cuda")
        sg.matmul_q2(a[i:i + 1].contiguous(), w, ci, 1)
        assert torch.equal(ci.view(torch.int16)[0], c.view(torch.int16)[i])


def test_nan_and_inf_activations_follow_quantize_row():
    n, k, block = 64, 256, 64
    rng = np.random.default_rng(3)
    signs = rng.integers(0, 256, (k * n + 7) // 8).astype(np.uint8)
    scales = orc.f32_to_f16_bits(rng.uniform(0.005, 0.03, n * (k // block)).astype(np.float32))
    a = rng.standard_normal((2, k)).astype(np.float16)
    a[0, 5] = np.nan
    a[1, 70] = np.inf
    w = sg.Q1Weights.new(signs, scales, sg.WeightLayout.OutIn, n, k, block)
    check_bits(w, 1, signs, 0, scales, None, n, k, block, 2, a.view(np.uint16), "nan/inf rows")


def test_epilogue_on_the_f16_rounded_product_is_bit_exact():
    """config 3's graph: mul_col(s).add_col(b), evaluated as apply_ep_scalar does
    (src/kernels/lowbit/matmul.rs:335-336, src/exec/scalar.rs:125-140); plus a bias /
    row scale / trailing gelu graph within 1e-2 (tests/correctness/q2.rs:83-106)."""
    m, n, k, block = 8, 300, 512, 128
    rng = np.random.default_rng(4)
    signs = rng.integers(0, 256, (k * n + 7) // 8).astype(np.uint8)
    scales = orc.f32_to_f16_bits(rng.uniform(0.005, 0.03, n * (k // block)).astype(np.float32))
    a_bits = orc.f32_to_f16_bits(rng.standard_normal((m, k)).astype(np.float32))
    s_bits = orc.f32_to_f16_bits(rng.uniform(0.5, 1.5, n).astype(np.float32))
    b_bits = orc.f32_to_f16_bits((rng.standard_normal(n) * 0.1).astype(np.float32))
    w = sg.Q1Weights.new(signs, scales, sg.WeightLayout.InOut, n, k, block)
    c = torch.zeros((m, n), dtype=torch.float16, device="cuda")
    sg.matmul_q1_ep(f16_bits_dev(a_bits), w, c, m, sg.Epilogue().mul_col(f16_bits_dev(s_bits)).add_col(f16_bits_dev(b_bits)))
    want = orc.lowbit_matmul(a_bits, 1, signs, 1, scales, None, n, k, block, m)
    want = orc.apply_ep(want, m, n, orc.Nodes([(5, 0, 0.0, s_bits, 0), (4, 0, 0.0, b_bits, 0)]))
    assert np.array_equal(bits_of(c), want)
    row = orc.f32_to_f16_bits(rng.uniform(0.5, 1.5, m).astype(np.float32))
    sg.matmul_q1_ep(f16_bits_dev(a_bits), w, c, m,
                    sg.Epilogue().add_col(f16_bits_dev(b_bits)).mul_row(f16_bits_dev(row)).gelu())
    want = orc.lowbit_matmul(a_bits, 1, signs, 1, scales, None, n, k, block, m)
    want = orc.apply_ep(want, m, n, orc.Nodes([(4, 0, 0.0, b_bits, 0), (3, 0, 0.0, row, 0), (8, 2, 0.0, None, 0)]))
    assert np.max(np.abs(c.float().cpu().numpy() - orc.f16_bits_to_f32(want))) <= 1e-2


def test_config2_ternary_gemv_full_size():
    """M=1, K=4096, N=11008, codes i.i.d. in {-1,0,+1}, block 256, scales U(0.01,0.05)."""
    m, n, k, block = 1, 11008, 4096, 256
    rng = np.random.default_rng(12)
    two = rng.integers(0, 3, k * n).astype(np.uint8)
    codes = (two[0::4] | (two[1::4] << 2) | (two[2::4] << 4) | (two[3::4] << 6)).astype(np.uint8)
    scales = orc.f32_to_f16_bits(rng.uniform(0.01, 0.05, n * (k // block)).astype(np.float32))
    a_bits = orc.f32_to_f16_bits(rng.standard_normal((m, k)).astype(np.float32))
    w = sg.Q2Weights.new(codes, scales, n, k)
    check_bits(w, 2, codes, 1, scales, BOOKS[0], n, k, block, m, a_bits, "config 2")


def test_config3_one_bit_batch_full_size():
    """M=8, K=4096, N=14336, Bernoulli(0.5) signs, block 128, mul_col(s).add_col(b)."""
    m, n, k, block = 8, 14336, 4096, 128
    rng = np.random.default_rng(13)
    signs = rng.integers(0, 256, (k * n) // 8).astype(np.uint8)
    scales = orc.f32_to_f16_bits(rng.uniform(0.005, 0.03, n * (k // block)).astype(np.float32))
    a_bits = orc.f32_to_f16_bits(rng.standard_normal((m, k)).astype(np.float32))
    w = sg.Q1Weights.new(signs, scales, sg.WeightLayout.OutIn, n, k, block)
    check_bits(w, 1, signs, 0, scales, None, n, k, block, m, a_bits, "config 3")
    s_bits = orc.f32_to_f16_bits(rng.uniform(0.5, 1.5, n).astype(np.float32))
    b_bits = orc.f32_to_f16_bits((rng.standard_normal(n) * 0.1).astype(np.float32))
    c = torch.zeros((m, n), dtype=torch.float16, device="cuda")
    sg.matmul_q1_ep(f16_bits_dev(a_bits), w, c, m, sg.Epilogue().mul_col(f16_bits_dev(s_bits)).add_col(f16_bits_dev(b_bits)))
    want = orc.apply_ep(orc.lowbit_matmul(a_bits, 1, signs, 0, scales, None, n, k, block, m), m, n,
                        orc.Nodes([(5, 0, 0.0, s_bits, 0), (4, 0, 0.0, b_bits, 0)]))
    assert np.array_equal(bits_of(c), want)


def test_host_and_drop_in_entries_and_pack_roundtrip():
    m, n, k, block = 4, 130, 300, 64
    rng = np.random.default_rng(6)
    codes = rng.integers(0, 256, (k * n + 3) // 4).astype(np.uint8)
    codes[-1] &= (1 << (2 * ((k * n) % 4 or 4))) - 1
    nbk = -(-k // block)
    scales = orc.f32_to_f16_bits(rng.uniform(0.01, 0.05, n * nbk).astype(np.float32))
    a = rng.standard_normal((m, k)).astype(np.float16)
    book = BOOKS[1]
    want = orc.lowbit_matmul(a, 2, codes, 1, scales, book, n, k, block, m)
    w = sg.Q2Weights.new(codes, scales, n, k, sg.Q2Params(block).with_codebook(book))
    c = np.zeros((m, n), np.float16)
    sg.matmul_q2(a, w, c, m)
    assert np.array_equal(c.view(np.uint16), want)
    back, sback = w.unpack()
    assert np.array_equal(back, codes) and np.array_equal(sback, scales)
    # the reference's band-major arrays through the reference's own symbols
    packed, sc = orc.q2_pack_band(codes, scales, n, k, block)
    L = sg.lib()
    cb = np.asarray(book, np.int8)
    c2 = np.zeros((m, n), np.uint16)
    assert L.gemm_sme_f16_q2(m, n, k, c2.ctypes.data, a.ctypes.data, packed.ctypes.data, sc.ctypes.data, cb.ctypes.data, block, None) == 0
    assert np.array_equal(c2, want)
    L.smeg_forget(packed.ctypes.data)
    signs = rng.integers(0, 256, (k * n + 7) // 8).astype(np.uint8)
    want1 = orc.lowbit_matmul(a, 1, signs, 0, scales, None, n, k, block, m)
    packed1, sc1 = orc.q1_pack_band(signs, 0, scales, n, k, block)
    c3 = np.zeros((m, n), np.uint16)
    assert L.gemm_sme_f16_q1(m, n, k, c3.ctypes.data, a.ctypes.data, packed1.ctypes.data, sc1.ctypes.data, block, None) == 0
    assert np.array_equal(c3, want1)
    L.smeg_forget(packed1.ctypes.data)


def test_q1_interleave_keeps_every_column():
    """src/kernels/lowbit/q1.rs:298-319."""
    n, k, block = 70, 300, 64
    rng = np.random.default_rng(8)
    wg = rng.standard_normal(n * k).astype(np.float32)
    wu = rng.standard_normal(n * k).astype(np.float32)
    g = sg.Q1Weights.quantize(wg, sg.WeightLayout.OutIn, n, k, block)
    u = sg.Q1Weights.quantize(wu, sg.WeightLayout.OutIn, n, k, block)
    both = sg.Q1Weights.interleave(g, u)
    a = torch.from_numpy(rng.standard_normal((2, k)).astype(np.float16)).cuda()
    cg, cu = (torch.zeros((2, n), dtype=torch.float16, device="cuda") for _ in range(2))
    cb = torch.zeros((2, 2 * n), dtype=torch.float16, device="cuda")
    sg.matmul_q1(a, g, cg, 2); sg.matmul_q1(a, u, cu, 2); sg.matmul_q1(a, both, cb, 2)
    col = 0
    for c0 in range(0, n, 32):
        w = min(32, n - c0)
        assert torch.equal(cb[:, col:col + w], cg[:, c0:c0 + w]); col += w
        assert torch.equal(cb[:, col:col + w], cu[:, c0:c0 + w]); col += w


@pytest.mark.parametrize("m,n,k", [(65, 70, 512), (200, 300, 1024), (130, 1000, 320)])
def test_many_rows_on_the_tensor_cores_are_the_reference_bits(m, n, k):
    """Seventeen rows and up run on tcgen05 (64-row tiles, or 128-row tiles with the totals in tensor memory where a
    K-block is 64 to 256 deep): the plain entry points against the scalar statement, ragged column tiles included."""
    rng = np.random.default_rng(m + n)
    a_bits = orc.f32_to_f16_bits(rng.standard_normal((m, k)).astype(np.float32))
    for block in (16, 64, 128, 256, 1024):
        nbk = -(-k // block)
        scales = orc.f32_to_f16_bits(rng.uniform(0.01, 0.05, n * nbk).astype(np.float32))
        codes = rng.integers(0, 256, (k * n + 3) // 4).astype(np.uint8)
        book = BOOKS[(block // 16) % 3]
        w2 = sg.Q2Weights.new(codes, scales, n, k, sg.Q2Params(block).with_codebook(book))
        c = torch.full((m, n), 9.0, dtype=torch.float16, device="cuda")
        sg.matmul_q2(f16_bits_dev(a_bits), w2, c, m)
        want = orc.lowbit_matmul(a_bits, 2, codes, 1, scales, book, n, k, block, m)
        assert np.array_equal(_canon16(bits_of(c)), _canon16(want)), f"q2 {m}x{n}x{k} block {block}"
        signs = rng.integers(0, 256, (k * n + 7) // 8).astype(np.uint8)
        w1 = sg.Q1Weights.new(signs, scales, sg.WeightLayout.OutIn, n, k, block)
        sg.matmul_q1(f16_bits_dev(a_bits), w1, c, m)
        want = orc.lowbit_matmul(a_bits, 1, signs, 0, scales, None, n, k, block, m)
        assert np.array_equal(_canon16(bits_of(c)), _canon16(want)), f"q1 {m}x{n}x{k} block {block}"
    assert sg.last_status() == 0
