"""Known answers that involve no oracle: constant activation rows against constant weights whose every partial sum is an
exact binary fraction (in the spirit of the reference's closed form C = k * a(i) * b(j), tests/concurrency.rs:31-39), through
every kernel family -- one-wave decode kernels (3 rows), the staged / warp-level forms (9 rows) and the tcgen05 kernels
(70 rows).  `expected_*` are also checked against the oracle on the CPU (test_expected_values_are_the_oracles)."""
import numpy as np
import pytest

import oracle as orc

N, K, BLOCK = 256, 128, 32
ROW_VALUES = (0.5, 1.0, 2.0)


def rows_of(m):
    return np.array([ROW_VALUES[i % 3] for i in range(m)], np.float32)


def activations(m):
    return np.repeat(rows_of(m), K).reshape(m, K).astype(np.float16)


def expected_q4(m, weight):
    """Every weight `weight`: C[i][j] = K * weight * a(i), exact."""
    return np.repeat(rows_of(m) * np.float32(K * weight), N).reshape(m, N)


def expected_lowbit(m, block_sum):
    """Every block's integer sum is `block_sum` (q = 127 everywhere), scale 0.5, sa = x / 127: the reference's fold
    total = fmaf(sum, scale * sa, total) over K / BLOCK blocks, then f16."""
    out = np.zeros((m, N), np.float32)
    for i, x in enumerate(rows_of(m)):
        w = np.float32(0.5) * (np.float32(x) / np.float32(127.0))
        tot = np.float32(0.0)
        for _ in range(K // BLOCK):
            tot = np.float32(np.float64(block_sum) * np.float64(w) + np.float64(tot))     # exact in f64, one rounding: fmaf
        out[i, :] = np.float32(np.float16(tot))
    return out


def q4_arrays():
    quants = np.full(K * N // 2, 0x33, np.uint8)                      # every code 3
    scales = orc.f32_to_f16_bits(np.full(N * (K // BLOCK), 0.25, np.float32))
    return quants, scales


@pytest.mark.parametrize("m", [3, 9, 70])
def test_expected_values_are_the_oracles(m):
    a = activations(m).view(np.uint16)
    quants, scales = q4_arrays()
    got = orc.f16_bits_to_f32(orc.matmul_q4(a, quants, scales, None, N, K, BLOCK, m)).reshape(m, N)
    assert np.array_equal(got, expected_q4(m, 0.75))
    got = orc.f16_bits_to_f32(orc.matmul_q4(a, quants, scales, scales, N, K, BLOCK, m)).reshape(m, N)
    assert np.array_equal(got, expected_q4(m, 1.0))
    sc = orc.f32_to_f16_bits(np.full(N * (K // BLOCK), 0.5, np.float32))
    c = orc.lowbit_matmul(a, 2, np.full(K * N // 4, 0xFF, np.uint8), 1, sc, [-2, -1, 1, 2], N, K, BLOCK, m)
    assert np.array_equal(orc.f16_bits_to_f32(c).reshape(m, N), expected_lowbit(m, 2 * 127 * BLOCK))
    c = orc.lowbit_matmul(a, 1, np.full(K * N // 8, 0xFF, np.uint8), 0, sc, None, N, K, BLOCK, m)
    assert np.array_equal(orc.f16_bits_to_f32(c).reshape(m, N), expected_lowbit(m, 127 * BLOCK))


@pytest.mark.gpu
@pytest.mark.parametrize("m", [3, 9, 70])
def test_cuda_kernels_give_the_closed_form_answers(m):
    import torch
    import sme_gemm_b200 as sg
    a = torch.from_numpy(activations(m)).cuda()
    quants, scales = q4_arrays()
    # Q4_0, f16 and bf16 entries: every partial sum is exact in any order
    w = sg.Q4Weights.new(quants, scales, N, K)
    c = torch.zeros((m, N), dtype=torch.float16, device="cuda")
    sg.matmul_q4(a, w, c, m)
    assert np.array_equal(c.float().cpu().numpy(), expected_q4(m, 0.75))
    cb = torch.zeros((m, N), dtype=torch.bfloat16, device="cuda")
    sg.matmul_q4_bf16(a.to(torch.bfloat16), w, cb, m)
    assert np.array_equal(cb.float().cpu().numpy(), expected_q4(m, 0.75))
    # Q4_1: scale * code + min = 1.0
    wa = sg.Q4Weights.with_params(quants, scales, scales, N, K, sg.Q4Params(BLOCK).affine())
    sg.matmul_q4(a, wa, c, m)
    assert np.array_equal(c.float().cpu().numpy(), expected_q4(m, 1.0))
    # 2-bit (every code the codebook's 2) and 1-bit (every sign +): integer block sums and f16 outputs
    sc = orc.f32_to_f16_bits(np.full(N * (K // BLOCK), 0.5, np.float32))
    w2 = sg.Q2Weights.new(np.full(K * N // 4, 0xFF, np.uint8), sc, N, K, sg.Q2Params(BLOCK).with_codebook([-2, -1, 1, 2]))
    w1 = sg.Q1Weights.new(np.full(K * N // 8, 0xFF, np.uint8), sc, sg.WeightLayout.OutIn, N, K, BLOCK)
    for wl, fn, block_sum in ((w2, sg.matmul_q2, 2 * 127 * BLOCK), (w1, sg.matmul_q1, 127 * BLOCK)):
        cd, q, sa, sums = sg.matmul_lowbit_debug(a, wl, m)
        assert (q.cpu().numpy() == 127).all() and (sums.cpu().numpy() == block_sum).all()
        assert np.array_equal(cd.float().cpu().numpy(), expected_lowbit(m, block_sum))
        fn(a, wl, c, m)
        assert np.array_equal(c.float().cpu().numpy(), expected_lowbit(m, block_sum))
    torch.cuda.synchronize()
    assert sg.last_status() == 0
