"""The committed golden vectors (tests/golden/vectors.npz, made by tests/golden/make_golden.py).
CPU: both restatements of the reference's algorithm reproduce them (guards the checker itself).
GPU: the CUDA path, through the C ABI, against the same vectors -- bit-exact for the int8
activation codes, int32 block sums and low-bit outputs, within 1e-2 (the reference's
max |got - want| / (1 + |want|)) for the Q4 f16 / bf16 outputs and the MLP block."""
import os

import numpy as np
import pytest

import oracle as orc
import sme_gemm_b200 as sg

G = np.load(os.path.join(os.path.dirname(__file__), "golden", "vectors.npz"))
TOL = 1e-2


def _rel(got, want):
    g, w = np.asarray(got, np.float64), np.asarray(want, np.float64)
    return float(np.max(np.abs(g - w) / (1.0 + np.abs(w))))


def _nodes(bias):
    return [(4, 0, 0.0, bias, 0), (9, 0, -6.0, None, 0), (10, 0, 6.0, None, 0), (8, 3, 0.0, None, 0)]


@pytest.mark.parametrize("ci", range(3))
def test_oracle_reproduces_q4_vectors(ci):
    m, n, k, block = (int(v) for v in G[f"q4_{ci}_dims"])
    q, s, _ = orc.q4_quantize(G[f"q4_{ci}_w"], 0, n, k, block)
    assert np.array_equal(q, G[f"q4_{ci}_quants"]) and np.array_equal(s, G[f"q4_{ci}_scales"])
    for bf16 in (False, True):
        tag = f"q4_{ci}_{'bf16' if bf16 else 'f16'}"
        c0 = orc.matmul_q4(G[tag + "_a"], q, s, None, n, k, block, m, None, bf16)
        c1 = orc.matmul_q4(G[tag + "_a"], q, s, None, n, k, block, m, orc.Nodes(_nodes(G[tag + "_bias"])), bf16)
        assert np.array_equal(c0, G[tag + "_c"]) and np.array_equal(c1, G[tag + "_c_ep"])


@pytest.mark.parametrize("ci", range(3))
def test_oracle_reproduces_lowbit_vectors(ci):
    d = [int(v) for v in G[f"lb_{ci}_dims"]]
    m, n, k, block, book = d[0], d[1], d[2], d[3], d[4:]
    a, sc = G[f"lb_{ci}_a"], G[f"lb_{ci}_scales"]
    c2, q8, sa, s2 = orc.lowbit_matmul(a, 2, G[f"lb_{ci}_codes"], 1, sc, book, n, k, block, m, debug=True)
    c1, _, _, s1 = orc.lowbit_matmul(a, 1, G[f"lb_{ci}_signs"], 0, sc, None, n, k, block, m, debug=True)
    assert np.array_equal(q8, G[f"lb_{ci}_q"]) and np.array_equal(sa.view(np.uint32), G[f"lb_{ci}_sa"].view(np.uint32))
    assert np.array_equal(s2, G[f"lb_{ci}_q2_sums"]) and np.array_equal(c2, G[f"lb_{ci}_q2_c"])
    assert np.array_equal(s1, G[f"lb_{ci}_q1_sums"]) and np.array_equal(c1, G[f"lb_{ci}_q1_c"])


def test_oracle_reproduces_mlp_vector():
    m, d, f = (int(v) for v in G["mlp_dims"])
    both = sg.interleave_gate_up(G["mlp_wg"], G["mlp_wu"], sg.WeightLayout.OutIn, f, d)
    guq, gus, _ = orc.q4_quantize(both, 1, 2 * f, d)
    dq, ds, _ = orc.q4_quantize(G["mlp_wd"], 0, d, f)
    y = np.zeros((m, d), np.float32)
    orc.mlp_accumulate(G["mlp_x"].view(np.float16).reshape(m, d), y, m, d, f, guq, gus, dq, ds)
    assert np.array_equal(y.view(np.uint32), G["mlp_y"].view(np.uint32))


# ------------------------------------------------------------------------------------ GPU

@pytest.mark.gpu
@pytest.mark.parametrize("ci", range(3))
def test_cuda_q4_against_golden(ci):
    import torch
    from gpu_util import bf16_bits_dev, bits_of, f16_bits_dev
    m, n, k, block = (int(v) for v in G[f"q4_{ci}_dims"])
    w = sg.Q4Weights.quantize(G[f"q4_{ci}_w"], sg.WeightLayout.OutIn, n, k, sg.Q4Params(block))
    uq, us = w.unpack()
    assert np.array_equal(uq, G[f"q4_{ci}_quants"]) and np.array_equal(us, G[f"q4_{ci}_scales"])   # the library's own quantiser
    for bf16 in (False, True):
        tag = f"q4_{ci}_{'bf16' if bf16 else 'f16'}"
        todev = bf16_bits_dev if bf16 else f16_bits_dev
        tof = orc.bf16_bits_to_f32 if bf16 else orc.f16_bits_to_f32
        a = todev(G[tag + "_a"]).reshape(m, k)
        bias = todev(G[tag + "_bias"])
        c = torch.zeros((m, n), dtype=torch.bfloat16 if bf16 else torch.float16, device="cuda")
        (sg.matmul_q4_bf16 if bf16 else sg.matmul_q4)(a, w, c, m)
        assert _rel(tof(bits_of(c)), tof(G[tag + "_c"])) <= TOL
        ep = sg.Epilogue("bf16" if bf16 else "f16").add_col(bias).silu().clamp(-6.0, 6.0)
        (sg.matmul_q4_bf16_ep if bf16 else sg.matmul_q4_ep)(a, w, c, m, ep)
        torch.cuda.synchronize()
        assert _rel(tof(bits_of(c)), tof(G[tag + "_c_ep"])) <= (2e-2 if bf16 else TOL)   # one bf16 ulp through the epilogue
    assert sg.last_status() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("ci", range(3))
def test_cuda_lowbit_against_golden_bit_exact(ci):
    import torch
    from gpu_util import bits_of, f16_bits_dev
    d = [int(v) for v in G[f"lb_{ci}_dims"]]
    m, n, k, block, book = d[0], d[1], d[2], d[3], d[4:]
    a = f16_bits_dev(G[f"lb_{ci}_a"]).reshape(m, k)
    sc = G[f"lb_{ci}_scales"]
    w2 = sg.Q2Weights.new(G[f"lb_{ci}_codes"], sc, n, k, sg.Q2Params(block).with_codebook(book))
    w1 = sg.Q1Weights.new(G[f"lb_{ci}_signs"], sc, sg.WeightLayout.OutIn, n, k, block)
    for w, kind in ((w2, "q2"), (w1, "q1")):
        c, q, sa, sums = sg.matmul_lowbit_debug(a, w, m)
        torch.cuda.synchronize()
        assert np.array_equal(q.cpu().numpy(), G[f"lb_{ci}_q"])
        assert np.array_equal(sa.cpu().numpy().view(np.uint32), G[f"lb_{ci}_sa"].view(np.uint32))
        assert np.array_equal(sums.cpu().numpy(), G[f"lb_{ci}_{kind}_sums"])
        assert np.array_equal(bits_of(c), G[f"lb_{ci}_{kind}_c"])
    assert sg.last_status() == 0


@pytest.mark.gpu
def test_cuda_mlp_against_golden():
    import torch
    m, d, f = (int(v) for v in G["mlp_dims"])
    up = sg.GatedLinear.quantize(G["mlp_wg"], G["mlp_wu"], sg.WeightLayout.OutIn, f, d, sg.Gate.Silu)
    down = sg.Linear.quantize(G["mlp_wd"], sg.WeightLayout.OutIn, d, f)
    mlp = sg.Mlp.gated(up, down)
    x = torch.from_numpy(G["mlp_x"].view(np.float16).reshape(m, d)).cuda()
    y = torch.zeros((m, d), dtype=torch.float32, device="cuda")
    mlp.accumulate(x, y, m)
    torch.cuda.synchronize()
    assert _rel(y.cpu().numpy(), G["mlp_y"]) <= TOL
