"""The model-block surface above the kernels -- Linear on every weight kind, the folded RMS norm, GatedLinear on
1-bit weights, the plain Mlp, Norm and the MLP half of Block -- against their parts and the oracle
(restating tests/correctness/model.rs:19-76, 209-322 and tests/correctness/q2.rs:111-166)."""
import numpy as np
import pytest
import torch

import oracle as orc
import sme_gemm_b200 as sg
from gpu_util import bits_of, f16_bits_dev, max_rel, q4_logical

pytestmark = pytest.mark.gpu


def _lowbit(rng, bits, n, k, block):
    nbk = -(-k // block)
    scales = orc.f32_to_f16_bits(rng.uniform(0.01, 0.05, n * nbk).astype(np.float32))
    if bits == 2:
        codes = rng.integers(0, 256, (k * n + 3) // 4).astype(np.uint8)
        return sg.Q2Weights.new(codes, scales, n, k, sg.Q2Params(block))
    signs = rng.integers(0, 256, (k * n + 7) // 8).astype(np.uint8)
    return sg.Q1Weights.new(signs, scales, sg.WeightLayout.OutIn, n, k, block)


@pytest.mark.parametrize("bits", [2, 1])
@pytest.mark.parametrize("m", [1, 3, 9, 64])
def test_linear_on_lowbit_weights_is_the_matmul_with_a_leading_bias(bits, m):
    rng = np.random.default_rng(100 + m)
    n, k = 200, 512
    w = _lowbit(rng, bits, n, k, 128)
    bias = f16_bits_dev(orc.f32_to_f16_bits(rng.standard_normal(n).astype(np.float32) * 0.1))
    lin = (sg.Linear.from_q2 if bits == 2 else sg.Linear.from_q1)(w, bias)
    x = f16_bits_dev(orc.f32_to_f16_bits(rng.standard_normal((m, k)).astype(np.float32)))
    y = torch.zeros((m, n), dtype=torch.float16, device="cuda")
    lin.forward(x, y, m)
    want = torch.zeros_like(y)
    (sg.matmul_q2_ep if bits == 2 else sg.matmul_q1_ep)(x, w, want, m, sg.Epilogue().add_col(bias))
    assert np.array_equal(bits_of(y), bits_of(want))
    # opted into the f16 path: the tensor-core form from LOWBIT_MOPA_ROWS rows, the int8 form below
    lin.lowbit_mopa()
    lin.forward(x, y, m)
    if m >= sg.Linear.LOWBIT_MOPA_ROWS:
        (sg.matmul_q2_mopa_ep if bits == 2 else sg.matmul_q1_mopa_ep)(x, w, want, m, sg.Epilogue().add_col(bias))
    assert np.array_equal(bits_of(y), bits_of(want))
    assert sg.last_status() == 0


@pytest.mark.parametrize("m", [1, 5, 40])
def test_rms_norm_folded_into_a_linear(m):
    """Linear::rms_norm_input (src/linear.rs:295-308): rms_norm(x, gamma) @ W as a leading MulRow of 1 / rms over
    weights whose inputs carry gamma."""
    rng = np.random.default_rng(7 + m)
    n, k, eps = 96, 256, 1e-6
    q, s = q4_logical(rng, n, k, 32)
    lin = sg.Linear.from_q4(sg.Q4Weights.new(q, s, n, k)).rms_norm_input(eps)
    xb = orc.f32_to_f16_bits((rng.standard_normal((m, k)) * 2.0).astype(np.float32))
    y = torch.zeros((m, n), dtype=torch.float16, device="cuda")
    lin.forward(f16_bits_dev(xb), y, m)
    r = orc.rms_scales(xb, k, eps)
    want = orc.matmul_q4(xb, q, s, None, n, k, 32, m, orc.Nodes([(3, 0, 0.0, r, 0)]))
    # the row scale is an f32 sum taken in another order: at most one f16 step on the scale
    assert max_rel(orc.f16_bits_to_f32(bits_of(y)), orc.f16_bits_to_f32(want)) <= 3e-3
    # the scales themselves
    rd = torch.zeros(m, dtype=torch.float16, device="cuda")
    assert sg.lib().smeg_rms_scales_dev(rd.data_ptr(), f16_bits_dev(xb).data_ptr(), m, k, eps, torch.cuda.current_stream().cuda_stream) == 0
    assert np.max(np.abs(bits_of(rd).astype(np.int32) - r.astype(np.int32))) <= 1


@pytest.mark.parametrize("rms", [False, True])
@pytest.mark.parametrize("rows,dim", [(1, 8), (3, 70), (5, 4096), (2, 1027)])
def test_norm_rows_match_the_scalar_statement(rms, rows, dim):
    rng = np.random.default_rng(dim + rows)
    x = (rng.standard_normal((rows, dim)) * 1.5 + 0.3).astype(np.float32)
    w = rng.uniform(0.5, 1.5, dim).astype(np.float32)
    b = None if rms else (rng.standard_normal(dim) * 0.1).astype(np.float32)
    norm = sg.Norm.rms(w, 1e-5) if rms else sg.Norm.layer(w, b, 1e-5)
    xd = torch.from_numpy(x).cuda()
    y16 = torch.zeros((rows, dim), dtype=torch.float16, device="cuda")
    y32 = torch.zeros((rows, dim), dtype=torch.float32, device="cuda")
    norm.forward(xd, y16)
    norm.forward(xd, y32)
    w16, w32 = orc.norm_rows(x, w, b, 1e-5, rms)
    assert np.max(np.abs(y32.cpu().numpy() - w32)) <= 1e-5 * (1.0 + np.max(np.abs(w32)))
    assert max_rel(orc.f16_bits_to_f32(bits_of(y16)), orc.f16_bits_to_f32(w16)) <= 1e-3


@pytest.mark.parametrize("m", [1, 3, 9])
def test_gated_linear_from_1bit_weights_equals_two_linears(m):
    """tests/correctness/model.rs:276-322 on GatedLinear::from_q1: gate and up as one interleaved layer against the
    two layers run apart and the f32 act(g) * u."""
    rng = np.random.default_rng(31 + m)
    n, k = 100, 256
    gate, up = _lowbit(rng, 1, n, k, 128), _lowbit(rng, 1, n, k, 128)
    gl = sg.GatedLinear.from_q1(gate, up, sg.Gate.Silu)
    x = f16_bits_dev(orc.f32_to_f16_bits(rng.standard_normal((m, k)).astype(np.float32)))
    y = torch.zeros((m, n), dtype=torch.float16, device="cuda")
    gl.forward(x, y, m)
    g = torch.zeros((m, n), dtype=torch.float16, device="cuda")
    u = torch.zeros_like(g)
    sg.matmul_q1(x, gate, g, m)
    sg.matmul_q1(x, up, u, m)
    gf, uf = g.float(), u.float()
    want = (gf / (1.0 + torch.exp(-gf)) * uf).half()
    assert max_rel(y.float().cpu().numpy(), want.float().cpu().numpy()) <= 2e-3


@pytest.mark.parametrize("m", [1, 3, 70])
@pytest.mark.parametrize("act", [sg.Gate.Gelu, sg.Gate.Silu])
def test_plain_mlp_and_block_equal_their_parts(m, act):
    """Mlp::new == its calls, bit for bit (tests/correctness/model.rs:447-510); Block's MLP half == norm2 then the MLP
    (model.rs:209-270), and close to the oracle's statement of the same chain."""
    rng = np.random.default_rng(5 + m)
    d, f = 160, 1100
    wu = (rng.standard_normal((f, d)) * 0.05).astype(np.float32)
    wd = (rng.standard_normal((d, f)) * 0.05).astype(np.float32)
    up, down = sg.Linear.quantize(wu, sg.WeightLayout.OutIn, f, d), sg.Linear.quantize(wd, sg.WeightLayout.OutIn, d, f)
    mlp = sg.Mlp.new(up, act, down)
    gamma = rng.uniform(0.5, 1.5, d).astype(np.float32)
    block = sg.Block(sg.Norm.rms(gamma, 1e-5), mlp)
    x0 = rng.standard_normal((m, d)).astype(np.float32)
    x = torch.from_numpy(x0).cuda()
    block.accumulate(x, m)
    # the parts
    h = torch.zeros((m, d), dtype=torch.float16, device="cuda")
    block.norm2.forward(torch.from_numpy(x0).cuda(), h)
    hid = torch.zeros((m, f), dtype=torch.float16, device="cuda")
    sg.matmul_q4_ep(h, up.q4, hid, m, sg.Epilogue().gelu() if act == sg.Gate.Gelu else sg.Epilogue().silu())
    out = torch.zeros((m, d), dtype=torch.float16, device="cuda")
    sg.matmul_q4(hid, down.q4, out, m)
    want = torch.from_numpy(x0).cuda() + out.float()
    assert torch.equal(x, want)
    # the oracle's chain from the GPU's own normed rows
    uq, us, _ = orc.q4_quantize(wu, 0, f, d)
    dq, ds, _ = orc.q4_quantize(wd, 0, d, f)
    hid_o = orc.matmul_q4(bits_of(h), uq, us, None, f, d, 32, m, orc.Nodes([(8, int(act), 0.0, None, 0)]))
    out_o = orc.matmul_q4(hid_o, dq, ds, None, d, f, 32, m)
    want_o = x0 + orc.f16_bits_to_f32(out_o).reshape(m, d)
    assert max_rel(x.cpu().numpy(), want_o) <= 1e-2
    assert sg.last_status() == 0
