"""Epilogue op-graph semantics and the MLP block on the GPU against the oracle."""
import numpy as np
import pytest
import torch

import oracle as orc
import sme_gemm_b200 as sg
from gpu_util import bf16_bits_dev, bits_of, f16_bits_dev, max_rel, q4_logical

pytestmark = pytest.mark.gpu


def _setup(m, n, k, bf16, seed):
    rng = np.random.default_rng(seed)
    q, s = q4_logical(rng, n, k, 32)
    w = sg.Q4Weights.new(q, s, n, k)
    a32 = rng.standard_normal((m, k)).astype(np.float32)
    a_bits = orc.f32_to_bf16_bits(a32) if bf16 else orc.f32_to_f16_bits(a32)
    to_dev = bf16_bits_dev if bf16 else f16_bits_dev
    return rng, q, s, w, a_bits, to_dev


@pytest.mark.parametrize("bf16", [False, True])
def test_every_binary_op_with_every_operand_kind(bf16):
    """tests/correctness/exhaustive.rs: each op x {scalar, row, col, tensor}."""
    m, n, k = 5, 70, 96
    rng, q, s, w, a_bits, to_dev = _setup(m, n, k, bf16, 21)
    to_bits = orc.f32_to_bf16_bits if bf16 else orc.f32_to_f16_bits
    row = to_bits(rng.uniform(0.5, 1.5, m).astype(np.float32))
    col = to_bits(rng.uniform(0.5, 1.5, n).astype(np.float32))
    ld = n + 5
    ten = to_bits(rng.uniform(0.5, 1.5, m * ld).astype(np.float32))
    dt = "bf16" if bf16 else "f16"
    base = orc.matmul_q4(a_bits, q, s, None, n, k, 32, m, None, bf16)
    names = {"add": (0, 2, 4, 6), "mul": (1, 3, 5, 7), "sub": (11, 12, 13, 14), "div": (15, 16, 17, 18),
             "max": (9, 19, 20, 21), "min": (10, 22, 23, 24)}
    for name, (os_, or_, oc, ot) in names.items():
        for kind, op in (("scalar", os_), ("row", or_), ("col", oc), ("tensor", ot)):
            ep = sg.Epilogue(dt)
            if kind == "scalar":
                meth = {"add": "add_scalar", "mul": "mul_scalar", "sub": "sub_scalar", "div": "div_scalar",
                        "max": "max", "min": "min"}[name]
                ep = getattr(ep, meth)(0.75)
                sc = 0.75
                items = [(op, 0, sc, None, 0)]
            elif kind == "tensor":
                ep = getattr(ep, f"{name}_tensor_strided")(to_dev(ten), ld)
                items = [(op, 0, 0.0, ten, ld)]
            else:
                operand = row if kind == "row" else col
                ep = getattr(ep, f"{name}_{kind}")(to_dev(operand))
                items = [(op, 0, 0.0, operand, 0)]
            c = torch.zeros((m, n), dtype=torch.bfloat16 if bf16 else torch.float16, device="cuda")
            (sg.matmul_q4_bf16_ep if bf16 else sg.matmul_q4_ep)(to_dev(a_bits), w, c, m, ep)
            # apply the oracle graph to the GPU's own rounded product: isolates the epilogue, bit-exact
            c0 = torch.zeros_like(c)
            (sg.matmul_q4_bf16 if bf16 else sg.matmul_q4)(to_dev(a_bits), w, c0, m)
            want = orc.apply_ep(bits_of(c0), m, n, orc.Nodes(items), bf16)
            assert np.array_equal(bits_of(c), want), f"{name} {kind}"
            assert max_rel(orc.t_bits_to_f32(bits_of(c0), bf16), orc.t_bits_to_f32(base, bf16)) <= 1e-2


@pytest.mark.parametrize("kind", list(range(1, 25)))
def test_every_activation(kind):
    """tests/correctness/exhaustive.rs: every activation against the f64 definition
    (src/epilogue/mod.rs:40-86), applied to the GPU's own rounded product."""
    m, n, k = 3, 130, 64
    rng, q, s, w, a_bits, to_dev = _setup(m, n, k, False, 22)
    names = {1: "relu", 2: "gelu", 3: "silu", 4: "tanh", 5: "sigmoid", 6: "leaky_relu", 7: "relu6", 8: "hardsigmoid",
             9: "hardswish", 10: "abs", 11: "neg", 12: "square", 13: "sign", 14: "sqrt", 15: "softsign", 16: "recip",
             17: "rsqrt", 18: "exp", 19: "log", 20: "elu", 21: "selu", 22: "softplus", 23: "mish", 24: "gelu_exact"}
    alpha = 0.2 if kind in (6, 20) else 0.0
    ep = sg.Epilogue().mul_scalar(4.0)
    ep = getattr(ep, names[kind])(alpha) if kind in (6, 20) else getattr(ep, names[kind])()
    c = torch.zeros((m, n), dtype=torch.float16, device="cuda")
    sg.matmul_q4_ep(to_dev(a_bits), w, c, m, ep)
    c0 = torch.zeros_like(c)
    sg.matmul_q4(to_dev(a_bits), w, c0, m)
    want = orc.apply_ep(bits_of(c0), m, n, orc.Nodes([(1, 0, 4.0, None, 0), (8, kind, alpha, None, 0)]))
    got32, want32 = orc.f16_bits_to_f32(bits_of(c)), orc.f16_bits_to_f32(want)
    both_nan = np.isnan(got32) & np.isnan(want32)
    with np.errstate(invalid="ignore"):
        # one f16 ulp: the f32 transcendental may land on the other side of a rounding boundary
        ok = both_nan | (got32 == want32) | (np.abs(got32 - want32) <= np.abs(want32) * 2.0 ** -10 + 1e-7)
    assert ok.all(), (names[kind], got32[~ok][:4], want32[~ok][:4])
    if kind in (1, 6, 7, 10, 11, 13):   # exact kinds must be bit-identical
        assert np.array_equal(bits_of(c)[~both_nan], want[~both_nan])


def test_trailing_activation_runs_last_whatever_the_call_order():
    """config 4's builder order add_col(bias).silu().clamp(-6, 6) evaluates bias -> clamp -> silu
    (src/epilogue/graph.rs:38-42,185-238)."""
    m, n, k = 4, 96, 128
    rng, q, s, w, a_bits, to_dev = _setup(m, n, k, True, 23)
    bias = orc.f32_to_bf16_bits((rng.standard_normal(n) * 3).astype(np.float32))
    ep = sg.Epilogue("bf16").add_col(to_dev(bias)).silu().clamp(-6.0, 6.0)
    assert [it[0] for it in ep.resolved()] == [4, 9, 10, 8] and ep.resolved()[-1][1] == 3
    c = torch.zeros((m, n), dtype=torch.bfloat16, device="cuda")
    sg.matmul_q4_bf16_ep(to_dev(a_bits), w, c, m, ep)
    want = orc.matmul_q4(a_bits, q, s, None, n, k, 32, m,
                         orc.Nodes([(4, 0, 0.0, bias, 0), (9, 0, -6.0, None, 0), (10, 0, 6.0, None, 0), (8, 3, 0.0, None, 0)]), True)
    assert max_rel(c.float().cpu().numpy(), orc.bf16_bits_to_f32(want)) <= 1e-2


def test_more_nodes_than_the_inline_capacity():
    m, n, k = 2, 64, 64
    rng, q, s, w, a_bits, to_dev = _setup(m, n, k, False, 24)
    ep, items = sg.Epilogue(), []
    for i in range(20):
        v = float(np.float16(0.01 * (i + 1)))
        ep = ep.add_scalar(v) if i % 2 == 0 else ep.mul_scalar(1.0 + v)
        items.append((0 if i % 2 == 0 else 1, 0, v if i % 2 == 0 else float(np.float32(np.float16(1.0 + v))), None, 0))
    c = torch.zeros((m, n), dtype=torch.float16, device="cuda")
    c0 = torch.zeros_like(c)
    sg.matmul_q4_ep(to_dev(a_bits), w, c, m, ep)
    sg.matmul_q4(to_dev(a_bits), w, c0, m)
    assert np.array_equal(bits_of(c), orc.apply_ep(bits_of(c0), m, n, orc.Nodes(items)))


def test_glu_and_residual_add_match_the_scalar_statements():
    m, n = 5, 70
    rng = np.random.default_rng(25)
    both = orc.f32_to_f16_bits((rng.standard_normal((m, 2 * n)) * 3).astype(np.float32))
    y = torch.zeros((m, n), dtype=torch.float16, device="cuda")
    L = sg.lib()
    for act in (3, 2):
        assert L.smeg_glu_f16_dev(y.data_ptr(), f16_bits_dev(both).data_ptr(), m, n, act, 0) == 0
        torch.cuda.synchronize()
        want = orc.f16_bits_to_f32(orc.glu(both, m, n, act))
        got = y.float().cpu().numpy()
        # the device's approximate exp2 / reciprocal against glibc's expf / tanhf and an exact division: at most the last f16 place
        # (0.5 g (1 + tanh z) cancels for very negative g: there the f32 statement itself is only good to about |g u| 2^-22,
        # and the inputs here stay below 16)
        assert (np.abs(got - want) <= np.abs(want) * 2.0 ** -10 + 2.0 ** -16).all()
        assert (got == want).mean() > (0.97 if act == 3 else 0.85), (act, (got == want).mean())
    dst = torch.from_numpy(rng.standard_normal(m * n).astype(np.float32)).cuda()
    want = dst.cpu().numpy().copy()
    src = orc.f32_to_f16_bits(rng.standard_normal(m * n).astype(np.float32))
    orc.add_f16(src, want)
    assert L.smeg_add_f16_to_f32_dev(dst.data_ptr(), f16_bits_dev(src).data_ptr(), m * n, 0) == 0
    assert np.array_equal(dst.cpu().numpy(), want)


@pytest.mark.parametrize("m", [1, 3, 9])
def test_mlp_equals_its_three_calls_and_the_oracle(m):
    """tests/correctness/model.rs:447-510 (d = 160, f = 1100): Mlp::accumulate is bit-identical
    to GatedLinear::forward + Linear::forward + add_f16, and matches the oracle block."""
    d, f = 160, 1100
    rng = np.random.default_rng(30 + m)
    wg = (rng.standard_normal(f * d) * 0.05).astype(np.float32)
    wu = (rng.standard_normal(f * d) * 0.05).astype(np.float32)
    wd = (rng.standard_normal(d * f) * 0.05).astype(np.float32)
    up = sg.GatedLinear.quantize(wg, wu, sg.WeightLayout.OutIn, f, d, sg.Gate.Silu)
    down = sg.Linear.quantize(wd, sg.WeightLayout.OutIn, d, f)
    mlp = sg.Mlp.gated(up, down)
    x = torch.from_numpy(rng.standard_normal((m, d)).astype(np.float16)).cuda()
    y0 = rng.standard_normal((m, d)).astype(np.float32)
    y = torch.from_numpy(y0.copy()).cuda()
    mlp.accumulate(x, y, m)
    # the three calls
    hid = torch.zeros((m, f), dtype=torch.float16, device="cuda")
    out = torch.zeros((m, d), dtype=torch.float16, device="cuda")
    up.forward(x, hid, m)
    down.forward(hid, out, m)
    y3 = torch.from_numpy(y0.copy()).cuda()
    assert sg.lib().smeg_add_f16_to_f32_dev(y3.data_ptr(), out.data_ptr(), m * d, 0) == 0
    torch.cuda.synchronize()
    assert torch.equal(y, y3)
    # the oracle block
    both_w = sg.interleave_gate_up(wg, wu, sg.WeightLayout.OutIn, f, d)
    guq, gus, _ = orc.q4_quantize(both_w, 1, 2 * f, d)
    dq, ds, _ = orc.q4_quantize(wd, 0, d, f)
    want = y0.copy()
    orc.mlp_accumulate(x.cpu().numpy(), want, m, d, f, guq, gus, dq, ds)
    assert max_rel(y.cpu().numpy() - y0, want - y0) <= 1e-2
    # host-pointer entry gives the device path's bits
    yh = y0.copy()
    mlp.accumulate(x.cpu().numpy(), yh, m)
    assert np.array_equal(yh, y.cpu().numpy())
    # tensor-parallel halves on one rank: partial + finish == accumulate up to the f16 store of one f32 sum
    part = torch.zeros((m, d), dtype=torch.float32, device="cuda")
    mlp.partial(x, part, m)
    y4 = torch.from_numpy(y0.copy()).cuda()
    sg.Mlp.finish(y4, part)
    torch.cuda.synchronize()
    assert torch.equal(y4, y)


@pytest.mark.parametrize("m,d,f", [(65, 256, 1152), (130, 192, 2048), (300, 512, 1024)])
def test_prefill_mlp_with_fused_gate_and_residual_equals_its_three_calls(m, d, f):
    """Above 64 rows the block runs as two tensor-core GEMMs -- the gated product formed in the
    gate/up GEMM's store, the residual add in the down GEMM's -- and must give the bits of the
    three separate calls plus add_f16 (tests/correctness/model.rs:447-510), also through the
    tensor-parallel partial / finish pair."""
    rng = np.random.default_rng(m)
    wg = (rng.standard_normal(f * d) * 0.05).astype(np.float32)
    wu = (rng.standard_normal(f * d) * 0.05).astype(np.float32)
    wd = (rng.standard_normal(d * f) * 0.05).astype(np.float32)
    up = sg.GatedLinear.quantize(wg, wu, sg.WeightLayout.OutIn, f, d, sg.Gate.Silu)
    down = sg.Linear.quantize(wd, sg.WeightLayout.OutIn, d, f)
    mlp = sg.Mlp.gated(up, down)
    x = torch.from_numpy(rng.standard_normal((m, d)).astype(np.float16)).cuda()
    y0 = rng.standard_normal((m, d)).astype(np.float32)
    y = torch.from_numpy(y0.copy()).cuda()
    mlp.accumulate(x, y, m)
    hid = torch.zeros((m, f), dtype=torch.float16, device="cuda")
    out = torch.zeros((m, d), dtype=torch.float16, device="cuda")
    up.forward(x, hid, m)
    down.forward(hid, out, m)
    y3 = torch.from_numpy(y0.copy()).cuda()
    assert sg.lib().smeg_add_f16_to_f32_dev(y3.data_ptr(), out.data_ptr(), m * d, 0) == 0
    torch.cuda.synchronize()
    assert sg.last_status() == 0
    assert torch.equal(y, y3)
    part = torch.zeros((m, d), dtype=torch.float32, device="cuda")
    mlp.partial(x, part, m)
    y4 = torch.from_numpy(y0.copy()).cuda()
    sg.Mlp.finish(y4, part)
    torch.cuda.synchronize()
    assert torch.equal(y4, y)
    # sampled rows against the oracle block
    both_w = sg.interleave_gate_up(wg, wu, sg.WeightLayout.OutIn, f, d)
    guq, gus, _ = orc.q4_quantize(both_w, 1, 2 * f, d)
    dq, ds, _ = orc.q4_quantize(wd, 0, d, f)
    xs = x.cpu().numpy()
    for r0 in (0, m // 2, m - 1):
        want = y0[r0:r0 + 1].copy()
        orc.mlp_accumulate(xs[r0:r0 + 1], want, 1, d, f, guq, gus, dq, ds)
        assert max_rel(y.cpu().numpy()[r0:r0 + 1] - y0[r0:r0 + 1], want - y0[r0:r0 + 1]) <= 1e-2


def test_concurrent_host_threads_share_weights_bit_identically():
    """tests/concurrency.rs:130-180: 4 threads x 4 repetitions on shared weights."""
    import threading
    m, n, k = 3, 500, 700
    rng = np.random.default_rng(40)
    q, s = q4_logical(rng, n, k, 32)
    w = sg.Q4Weights.new(q, s, n, k)
    a = rng.standard_normal((m, k)).astype(np.float16)
    base = np.zeros((m, n), np.float16)
    sg.matmul_q4(a, w, base, m)
    results, errs = [], []

    def work():
        try:
            for _ in range(4):
                c = np.zeros((m, n), np.float16)
                sg.matmul_q4(a, w, c, m)
                results.append(c)
        except Exception as e:  # pragma: no cover
            errs.append(e)

    th = [threading.Thread(target=work) for _ in range(4)]
    [t.start() for t in th]
    [t.join() for t in th]
    assert not errs and len(results) == 16
    assert all(np.array_equal(r.view(np.uint16), base.view(np.uint16)) for r in results)


def test_converts_and_activation_passes_device_and_host_entries():
    """neon_f32_to_f16 / neon_f16_to_f32 / neon_act_f16 (csrc/sme_gemm_api.h:216-220; convert::to_f16,
    src/convert.rs:12-35): the device entries and the host-pointer drop-ins against the oracle's conversions and
    its scalar activation (the epilogue's ACT node on an identity product)."""
    import ctypes as C
    L = sg.lib()
    rng = np.random.default_rng(41)
    n = 5003
    x = (rng.standard_normal(n) * 3.0).astype(np.float32)
    x[:4] = [0.0, -0.0, 65520.0, 1e-8]
    want16 = orc.f32_to_f16_bits(x)
    # device entries
    xd = torch.from_numpy(x).cuda()
    h = torch.zeros(n, dtype=torch.float16, device="cuda")
    s = torch.cuda.current_stream().cuda_stream
    assert L.smeg_f32_to_f16_dev(h.data_ptr(), xd.data_ptr(), n, s) == 0
    assert np.array_equal(bits_of(h), want16)
    back = torch.zeros(n, dtype=torch.float32, device="cuda")
    assert L.smeg_f16_to_f32_dev(back.data_ptr(), h.data_ptr(), n, s) == 0
    assert np.array_equal(back.cpu().numpy().view(np.uint32), orc.f16_bits_to_f32(want16).view(np.uint32))
    # host drop-ins
    out16 = np.zeros(n, np.uint16)
    L.neon_f32_to_f16(out16.ctypes.data, x.ctypes.data, n)
    assert np.array_equal(out16, want16)
    out32 = np.zeros(n, np.float32)
    L.neon_f16_to_f32(out32.ctypes.data, want16.ctypes.data, n)
    assert np.array_equal(out32.view(np.uint32), orc.f16_bits_to_f32(want16).view(np.uint32))
    for kind in (1, 2, 3, 4, 5):
        small = orc.f32_to_f16_bits((rng.standard_normal(n) * 2.0).astype(np.float32))
        want = orc.apply_ep(small.reshape(1, n), 1, n, orc.Nodes([(8, kind, 0.0, None, 0)])).reshape(-1)
        got_h = np.zeros(n, np.uint16)
        L.neon_act_f16(got_h.ctypes.data, small.ctypes.data, n, kind)
        got_d = torch.zeros(n, dtype=torch.float16, device="cuda")
        assert L.smeg_act_f16_dev(got_d.data_ptr(), f16_bits_dev(small).data_ptr(), n, kind, s) == 0
        assert np.array_equal(bits_of(got_d), got_h)
        g32, w32 = orc.f16_bits_to_f32(got_h), orc.f16_bits_to_f32(want)
        err = np.abs(g32 - w32) - (np.abs(w32) * 2.0 ** -9 + 1e-6)
        assert (err <= 0).all(), (kind, float(err.max()), g32[err > 0][:4], w32[err > 0][:4])


def test_concurrent_host_threads_on_shapes_that_grow_the_scratch():
    """Host threads calling shapes with different scratch needs on one stream (the streaming decode kernel's shares and
    counters, the depth-split GEMM's partial tiles): a block that is outgrown stays valid for the launch that read its
    address, and every result equals the quiet run's bits (tests/concurrency.rs:130-180)."""
    import threading
    rng = np.random.default_rng(77)
    cases = []
    for (m, n, k) in ((1, 4096, 2048), (5, 9216, 4096), (40, 256, 8192), (1, 12288, 4096), (33, 512, 4096)):
        q, s = q4_logical(rng, n, k, 32, from_f32=False)
        w = sg.Q4Weights.new(q, s, n, k)
        a = f16_bits_dev(orc.f32_to_f16_bits(rng.standard_normal((m, k)).astype(np.float32)))
        c = torch.zeros((m, n), dtype=torch.float16, device="cuda")
        sg.matmul_q4(a, w, c, m)
        torch.cuda.synchronize()
        cases.append((m, w, a, bits_of(c).copy()))
    errors = []

    def worker(order):
        try:
            torch.cuda.set_device(0)
            for rep in range(3):
                for ci in order:
                    m, w, a, want = cases[ci]
                    c = torch.zeros((m, w.n()), dtype=torch.float16, device="cuda")
                    sg.matmul_q4(a, w, c, m)
                    torch.cuda.synchronize()
                    if not np.array_equal(bits_of(c), want):
                        errors.append((ci, rep))
        except Exception as e:      # pragma: no cover
            errors.append(repr(e))

    threads = [threading.Thread(target=worker, args=(o,)) for o in ([0, 1, 2, 3, 4], [4, 3, 2, 1, 0], [2, 0, 4, 1, 3], [1, 3, 0, 2, 4])]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors[:5]
    assert sg.last_status() == 0
