"""matmul_q2_mopa / matmul_q1_mopa on the GPU: the 2-bit / 1-bit weights on the f16 path
(f16 activations, weights f16(scale * value), f32 accumulation), against the CPU oracle's
statement of mopa_impl's portable arm -- Codes::dequant then the dense f16 reference GEMM
and the scalar epilogue (src/kernels/lowbit/matmul.rs:178-197, 339-350) -- on the shape /
block / codebook grid of the reference's mopa_matches_eager_dequant (:527-566).
Tolerance: max |got - want| / (1 + |want|) <= 1e-2 (f32 accumulation in a different order,
one f16 rounding)."""
import numpy as np
import pytest
import torch

import oracle as orc
import sme_gemm_b200 as sg
from gpu_util import bits_of, f16_bits_dev, max_rel
from refgen import data

pytestmark = pytest.mark.gpu

TOL = 1e-2
BOOKS = [[-1, 0, 1, 0], [-2, -1, 1, 2], [-128, 127, 3, -7]]
SHAPES = [(8, 64, 256), (1, 65, 37), (3, 200, 301), (33, 130, 514), (40, 4200, 1030), (200, 1000, 2048)]


def _want(a_bits, kind, wbits, layout, scales, book, n, k, block, m, nodes):
    wd = orc.lowbit_dequant(kind, wbits, layout, scales, book, n, k, block)
    c = orc.gemm16(a_bits, wd, m, n, k)
    return orc.apply_ep(c, m, n, nodes) if nodes is not None else c


def _check(fn, w, a_bits, m, n, k, ep, want, what):
    c = torch.full((m, n), 9.0, dtype=torch.float16, device="cuda")
    a = f16_bits_dev(a_bits).reshape(m, k)
    if ep is None:
        fn[0](a, w, c, m)
    else:
        fn[1](a, w, c, m, ep)
    torch.cuda.synchronize()
    assert sg.last_status() == 0
    got = orc.f16_bits_to_f32(bits_of(c)).reshape(m, n)
    err = max_rel(got, orc.f16_bits_to_f32(want).reshape(m, n))
    assert err <= TOL, f"{what}: max_rel {err:.3e} > {TOL}"


@pytest.mark.parametrize("si", range(len(SHAPES)))
def test_mopa_matches_eager_dequant(si):
    m, n, k = SHAPES[si]
    bias_f = (np.arange(n, dtype=np.float32) * np.float32(0.01) - np.float32(1.0)).astype(np.float16)
    bias = torch.from_numpy(bias_f).cuda()
    for bi, block in enumerate([16, 128, 4096]):
        nbk = -(-k // block)
        scales = orc.f32_to_f16_bits(data(si + 3, n * nbk).astype(np.float32) * np.float32(1e-3) - np.float32(0.1))
        a_bits = orc.f32_to_f16_bits((data(si + 77, m * k).astype(np.float32) - np.float32(128.0)) / np.float32(61.0))
        book = BOOKS[(si + bi) % 3]
        codes = data(si * 13 + bi, (k * n + 3) // 4)
        signs = data(si * 19 + bi, (k * n + 7) // 8)
        q2 = sg.Q2Weights.new(codes, scales, n, k, sg.Q2Params(block).with_codebook(book))
        q1 = sg.Q1Weights.new(signs, scales, sg.WeightLayout.OutIn, n, k, block)
        for ei in (0, 1):
            ep = None if ei == 0 else sg.Epilogue("f16").add_col(bias).silu()
            nodes = None if ei == 0 else orc.Nodes([(4, 0, 0.0, bias_f.view(np.uint16), 0), (8, 3, 0.0, None, 0)])
            what = f"{m}x{n}x{k} block {block} ep {ei}"
            # values inside [-8, 7] run on the 4-bit twin, any other codebook (the reference's own third test
            # codebook among them) on a dense f16 twin
            want = _want(a_bits, 2, codes, 1, scales, book, n, k, block, m, nodes)
            _check((sg.matmul_q2_mopa, sg.matmul_q2_mopa_ep), q2, a_bits, m, n, k, ep, want, f"q2 {book} {what}")
            want = _want(a_bits, 1, signs, 0, scales, None, n, k, block, m, nodes)
            _check((sg.matmul_q1_mopa, sg.matmul_q1_mopa_ep), q1, a_bits, m, n, k, ep, want, f"q1 {what}")


def test_mopa_twin_is_bit_identical_to_dequant():
    """The 4-bit twin dequantises to exactly Codes::dequant's weights: run the twin path with
    one-hot activations (each output is then a single weight, no summation)."""
    n, k, block = 48, 64, 16
    rng = np.random.default_rng(5)
    codes = rng.integers(0, 256, (k * n + 3) // 4).astype(np.uint8)
    scales = orc.f32_to_f16_bits(rng.uniform(-0.2, 0.2, n * (k // block)).astype(np.float32))
    book = [-8, 7, 3, -5]
    w = sg.Q2Weights.new(codes, scales, n, k, sg.Q2Params(block).with_codebook(book))
    eye = torch.eye(k, dtype=torch.float16, device="cuda")
    c = torch.zeros((k, n), dtype=torch.float16, device="cuda")
    sg.matmul_q2_mopa(eye, w, c, k)
    torch.cuda.synchronize()
    want = orc.lowbit_dequant(2, codes, 1, scales, book, n, k, block)
    got, want = bits_of(c).reshape(k, n).copy(), want.reshape(k, n).copy()
    # +0 and -0 are the same weight
    got[got == 0x8000] = 0
    want[want == 0x8000] = 0
    assert np.array_equal(got, want)


def test_wide_codebook_twin_is_bit_identical_to_dequant():
    """A codebook with values outside [-8, 7]: the dense f16 twin holds exactly Codes::dequant's weights
    (one-hot activations: each output is a single weight), for a depth that is not a multiple of 8 as well."""
    for (n, k, block) in ((48, 64, 16), (33, 52, 32)):
        rng = np.random.default_rng(6)
        codes = rng.integers(0, 256, (k * n + 3) // 4).astype(np.uint8)
        nbk = -(-k // block)
        scales = orc.f32_to_f16_bits(rng.uniform(-0.2, 0.2, n * nbk).astype(np.float32))
        book = [-128, 127, 3, -7]
        w = sg.Q2Weights.new(codes, scales, n, k, sg.Q2Params(block).with_codebook(book))
        eye = torch.eye(k, dtype=torch.float16, device="cuda")
        c = torch.zeros((k, n), dtype=torch.float16, device="cuda")
        sg.matmul_q2_mopa(eye, w, c, k)
        torch.cuda.synchronize()
        assert sg.last_status() == 0
        want = orc.lowbit_dequant(2, codes, 1, scales, book, n, k, block).reshape(k, n).copy()
        got = bits_of(c).reshape(k, n).copy()
        got[got == 0x8000] = 0
        want[want == 0x8000] = 0
        assert np.array_equal(got, want)
