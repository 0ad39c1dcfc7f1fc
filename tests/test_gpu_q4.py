"""Q4 GEMV / small-M GEMM on the GPU against the CPU oracle (the restated
portable path of the reference), through the C ABI.

Tolerances (float outputs): against the oracle, which also accumulates in f32
over the same weights, max |g-w|/(1+|w|) <= 1e-2 flat; against an f64 product of
the same dequantised weights, the reference's sqrt(k)-scaled bound
max(1e-2, 1e-2*sqrt(k)/4) (tests/correctness/q4.rs:56 uses 3e-2 for its
f16-accumulating kernels)."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle as orc
import sme_gemm_b200 as sg
from gpu_util import bf16_bits_dev, bits_of, f16_bits_dev, half_tol, max_rel, q4_logical
from refgen import Lcg

pytestmark = pytest.mark.gpu
TOL = 1e-2

# tests/correctness/gemv.rs:234-243
GEMV_SHAPES = [(1, 33, 256), (1, 389, 1027), (1, 1100, 2051), (2, 100, 70), (3, 129, 1027), (4, 4109, 4099),
               (5, 70, 513), (7, 1030, 2050)]


def run_q4(m, n, k, block, bf16=False, ep_builder=None, seed=0, from_f32=True, host=False):
    rng = np.random.default_rng(seed + m * 131 + n * 17 + k)
    q, s = q4_logical(rng, n, k, block, from_f32)
    w = sg.Q4Weights.with_params(q, s, None, n, k, sg.Q4Params(block))
    a32 = rng.standard_normal((m, k)).astype(np.float32)
    a_bits = orc.f32_to_bf16_bits(a32) if bf16 else orc.f32_to_f16_bits(a32)
    nodes, ep = None, None
    if ep_builder is not None:
        ep_np, ep_dev, items = ep_builder(rng, m, n, bf16)
        ep = ep_np if host else ep_dev
        nodes = orc.Nodes(items)
    want = orc.matmul_q4(a_bits, q, s, None, n, k, block, m, nodes, bf16)
    if host:
        c = np.full((m, n), 0x4880, np.uint16)
        a_host = a_bits if bf16 else a_bits.view(np.float16)
        fn = (sg.matmul_q4_bf16_ep if bf16 else sg.matmul_q4_ep) if ep is not None else (sg.matmul_q4_bf16 if bf16 else sg.matmul_q4)
        fn(*((a_host, w, c, m, ep) if ep is not None else (a_host, w, c, m)))
        got = c
    else:
        a_dev = bf16_bits_dev(a_bits) if bf16 else f16_bits_dev(a_bits)
        c = torch.full((m, n), 9.0, dtype=a_dev.dtype, device="cuda")
        fn = (sg.matmul_q4_bf16_ep if bf16 else sg.matmul_q4_ep) if ep is not None else (sg.matmul_q4_bf16 if bf16 else sg.matmul_q4)
        fn(*((a_dev, w, c, m, ep) if ep is not None else (a_dev, w, c, m)))
        torch.cuda.synchronize()
        got = bits_of(c)
    assert sg.last_status() == 0
    g32, w32 = orc.t_bits_to_f32(got, bf16), orc.t_bits_to_f32(want, bf16)
    return g32, w32, (q, s, a_bits)


def bias_relu(rng, m, n, bf16):
    """add_col(bias).relu() (tests/correctness/gemv.rs Q4 epilogue case)."""
    b32 = (rng.standard_normal(n) * 0.1).astype(np.float32)
    bits = orc.f32_to_bf16_bits(b32) if bf16 else orc.f32_to_f16_bits(b32)
    dt = "bf16" if bf16 else "f16"
    ep_np = sg.Epilogue(dt).add_col(bits if bf16 else bits.view(np.float16)).relu()
    ep_dev = sg.Epilogue(dt).add_col(bf16_bits_dev(bits) if bf16 else f16_bits_dev(bits)).relu()
    return ep_np, ep_dev, [(4, 0, 0.0, bits, 0), (8, 1, 0.0, None, 0)]


@pytest.mark.parametrize("m,n,k", GEMV_SHAPES)
@pytest.mark.parametrize("block", [16, 32, 64])
def test_q4_gemv_f16_matches_oracle(m, n, k, block):
    g, w, (q, s, a_bits) = run_q4(m, n, k, block)
    mr = max_rel(g, w)
    assert mr <= TOL, f"{m}x{n}x{k} block {block}: max_rel {mr}"
    # and against an f64 product over the same dequantised weights
    wd = orc.f16_bits_to_f32(orc.q4_dequant(q, s, None, n, k, block)).astype(np.float64)
    want64 = orc.f16_bits_to_f32(a_bits).astype(np.float64).reshape(m, k) @ wd
    assert max_rel(g, want64) <= half_tol(1e-2, k)


@pytest.mark.parametrize("m,n,k", [(1, 33, 256), (3, 129, 1027), (7, 1030, 2050)])
@pytest.mark.parametrize("block", [16, 32, 64])
def test_q4_gemv_bias_relu_epilogue(m, n, k, block):
    g, w, _ = run_q4(m, n, k, block, ep_builder=bias_relu)
    assert max_rel(g, w) <= TOL


@pytest.mark.parametrize("m,n,k", [(1, 33, 256), (2, 100, 70), (5, 70, 513), (4, 1030, 1027)])
@pytest.mark.parametrize("block", [16, 32, 128])
def test_q4_gemv_bf16_matches_oracle(m, n, k, block):
    g, w, _ = run_q4(m, n, k, block, bf16=True)
    assert max_rel(g, w) <= TOL
    g, w, _ = run_q4(m, n, k, block, bf16=True, ep_builder=bias_relu)
    assert max_rel(g, w) <= TOL


@pytest.mark.parametrize("block", [1, 2, 8])
def test_q4_tiny_blocks(block):
    """tests/correctness/q4.rs:199-203 runs blocks 1 and 2."""
    g, w, _ = run_q4(3, 70, 130, block, from_f32=False)
    assert max_rel(g, w) <= TOL


@pytest.mark.parametrize("m", [1, 2, 7, 8, 9, 12, 17, 33, 64])
def test_q4_row_counts_either_side_of_the_row_group(m):
    """tests/correctness/model.rs:19-76 checks m in {1,3,7,8,9,64} across the kernel switch."""
    g, w, _ = run_q4(m, 160, 320, 32)
    assert max_rel(g, w) <= TOL


def test_q4_random_byte_codes_reference_generator():
    """q4_resident (tests/correctness/q4.rs:60-123): random code bytes, scales 0.01 + 0.001*(i%5)."""
    for (m, n, k) in [(1, 1, 1), (7, 5, 3), (31, 31, 31), (32, 32, 32), (33, 17, 9), (64, 96, 48), (7, 50, 200)]:
        s = Lcg(0x44449999dead0001 ^ (m * 131 + n * 17 + k))
        a = s.fill(m * k)
        nbk = -(-k // 32)
        quants = s.bytes((k * n + 1) // 2)
        scales = orc.f32_to_f16_bits((0.01 + 0.001 * (np.arange(n * nbk) % 5)).astype(np.float32))
        w = sg.Q4Weights.new(quants, scales, n, k)
        c = torch.zeros((m, n), dtype=torch.float16, device="cuda")
        sg.matmul_q4(torch.from_numpy(a).cuda(), w, c, m)
        want = orc.matmul_q4(a, quants, scales, None, n, k, 32, m)
        assert max_rel(c.float().cpu().numpy(), orc.f16_bits_to_f32(want)) <= TOL


def test_empty_graph_equals_plain_call_bit_for_bit():
    """tests/correctness/q4.rs:509-513."""
    m, n, k = 3, 129, 1027
    rng = np.random.default_rng(3)
    q, s = q4_logical(rng, n, k, 32)
    w = sg.Q4Weights.new(q, s, n, k)
    a = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float16)).cuda()
    c1 = torch.zeros((m, n), dtype=torch.float16, device="cuda")
    c2 = torch.zeros_like(c1)
    sg.matmul_q4(a, w, c1, m)
    sg.matmul_q4_ep(a, w, c2, m, sg.Epilogue())
    assert torch.equal(c1.view(torch.int16), c2.view(torch.int16))


@pytest.fixture
def stream_every_size(monkeypatch):
    """The streaming decode kernel normally takes only matrices of a few hundred KB per SM; the tuning
    knob (read per call by the library) sends every call that fits it there."""
    monkeypatch.setenv("SMEG_Q4_STREAM", "2")


# k % 8 == 0 (rows of A travel by bulk copy); n and k chosen so that column groups are cut by the
# per-CTA ranges, stages end short, and the last column group is partly outside the matrix
STREAM_SHAPES = [(1, 33, 256), (1, 4109, 4096), (3, 1030, 2056), (4, 100, 72), (7, 2000, 1032), (8, 160, 11008),
                 (9, 389, 1024), (16, 1100, 2048), (2, 16, 14336)]


@pytest.mark.parametrize("m,n,k", STREAM_SHAPES)
@pytest.mark.parametrize("block", [16, 32, 128])
def test_q4_streaming_decode_kernel_matches_oracle(stream_every_size, m, n, k, block):
    g, w, _ = run_q4(m, n, k, block)
    assert max_rel(g, w) <= TOL, f"{m}x{n}x{k} block {block}"
    g, w, _ = run_q4(m, n, k, block, ep_builder=bias_relu)
    assert max_rel(g, w) <= TOL
    if block != 16:
        g, w, _ = run_q4(m, n, k, block, bf16=True)
        assert max_rel(g, w) <= TOL


@pytest.mark.parametrize("block", [8, 4096])
def test_q4_streaming_decode_kernel_block_extremes(stream_every_size, block):
    g, w, _ = run_q4(3, 200, 8192 if block == 4096 else 264, block, from_f32=False)
    assert max_rel(g, w) <= TOL


def test_q4_streaming_decode_kernel_is_repeatable_and_leaves_its_counters_clear(stream_every_size):
    """Column groups cut between CTAs are summed in range order by whichever CTA arrives last: the result
    does not depend on which one that is, and the arrival counters are zero again for the next call."""
    m, n, k = 2, 1200, 4096
    rng = np.random.default_rng(11)
    q, s = q4_logical(rng, n, k, 32)
    w = sg.Q4Weights.new(q, s, n, k)
    a = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float16)).cuda()
    outs = []
    for _ in range(5):
        c = torch.zeros((m, n), dtype=torch.float16, device="cuda")
        sg.matmul_q4(a, w, c, m)
        outs.append(c)
    torch.cuda.synchronize()
    assert sg.last_status() == 0
    for c in outs[1:]:
        assert torch.equal(c.view(torch.int16), outs[0].view(torch.int16))


def test_q4_streaming_decode_kernel_at_the_size_that_selects_it():
    """Down projection of the MLP block at two rows: large enough to stream without the knob."""
    g, w, _ = run_q4(2, 4096, 14336, 32, seed=2)
    assert max_rel(g, w) <= TOL


def test_config1_decode_gemv_full_size():
    """M=1, K=4096, N=4096, A ~ N(0,1) f16, W ~ N(0,0.02) -> Q4_0 block 32."""
    g, w, _ = run_q4(1, 4096, 4096, 32, seed=1)
    mr = max_rel(g, w)
    assert mr <= TOL, mr


def test_host_pointer_entry_and_pack_roundtrip_through_the_device():
    g, w, (q, s, _) = run_q4(2, 100, 70, 32, host=True)
    assert max_rel(g, w) <= TOL
    g, w, _ = run_q4(3, 129, 1027, 32, host=True, ep_builder=bias_relu)
    assert max_rel(g, w) <= TOL
    wt = sg.Q4Weights.new(q, s, 100, 70)
    q2, s2 = wt.unpack()
    assert np.array_equal(q2, q) and np.array_equal(s2, s)


def test_drop_in_entry_takes_the_reference_band_major_arrays():
    """gemm_sme_f16f16_q4 / gemm_sme_b16b16_q4 with the arrays a reference-side
    Q4Weights holds (src/kernels/q4/weights.rs:92-113)."""
    m, n, k, block = 3, 200, 300, 32
    rng = np.random.default_rng(5)
    q, s = q4_logical(rng, n, k, block)
    nib, sc, _ = orc.q4_pack_band(q, s, None, n, k, block)
    a32 = rng.standard_normal((m, k)).astype(np.float32)
    L = sg.lib()
    for bf16 in (False, True):
        a_bits = orc.f32_to_bf16_bits(a32) if bf16 else orc.f32_to_f16_bits(a32)
        c = np.zeros((m, n), np.uint16)
        if bf16:
            rc = L.gemm_sme_b16b16_q4(m, n, k, c.ctypes.data, a_bits.ctypes.data, nib.ctypes.data, sc.ctypes.data, None,
                                      None, None, block, None)
        else:
            rc = L.gemm_sme_f16f16_q4(m, n, k, c.ctypes.data, a_bits.ctypes.data, nib.ctypes.data, sc.ctypes.data, None,
                                      block, None)
        assert rc == 0
        want = orc.matmul_q4(a_bits, q, s, None, n, k, block, m, None, bf16)
        assert max_rel(orc.t_bits_to_f32(c, bf16), orc.t_bits_to_f32(want, bf16)) <= TOL
    L.smeg_forget(nib.ctypes.data)
    # rc contract: bad block size -> -1 and dst untouched (csrc/gemm_f16f16_q4.h:474)
    c = np.full((m, n), 7, np.uint16)
    assert L.gemm_sme_f16f16_q4(m, n, k, c.ctypes.data, a_bits.ctypes.data, nib.ctypes.data, sc.ctypes.data, None, 24, None) == -1
    assert (c == 7).all()


def test_length_contracts_raise_like_the_reference_panics():
    q, s = q4_logical(np.random.default_rng(0), 16, 32, 32)
    w = sg.Q4Weights.new(q, s, 16, 32)
    a = torch.zeros(31, dtype=torch.float16, device="cuda")
    c = torch.zeros(16, dtype=torch.float16, device="cuda")
    with pytest.raises(AssertionError, match="a is m\\*k"):
        sg.matmul_q4(a, w, c, 1)
    with pytest.raises(AssertionError, match="col operand"):
        sg.matmul_q4_ep(torch.zeros(32, dtype=torch.float16, device="cuda"), w, c, 1,
                        sg.Epilogue().add_col(torch.zeros(15, dtype=torch.float16, device="cuda")))
    # m == 0: nothing touched
    sg.matmul_q4(torch.zeros(0, dtype=torch.float16, device="cuda"), w, torch.zeros(0, dtype=torch.float16, device="cuda"), 0)


# ---- Q4_1: the affine form (weight = scale * code + min) ----

@pytest.mark.parametrize("bf16", [False, True])
@pytest.mark.parametrize("m,n,k,block", [(1, 33, 256, 32), (3, 129, 1027, 32), (7, 200, 513, 64), (64, 300, 1024, 32), (130, 257, 2050, 128)])
def test_affine_weights_match_the_scalar_statement(m, n, k, block, bf16):
    """tests/correctness/q4.rs:272-328 on the GPU: quantised with per-block minima, the product runs on the weights
    round_T(f64(scale) * code + f64(min)) (dequant_rows, src/kernels/q4/weights.rs:250-256) with f32 accumulation."""
    rng = np.random.default_rng(900 + m + n + k)
    w32 = (rng.standard_normal((n, k)) * 0.05 + 0.02).astype(np.float32)
    q, s, mins = orc.q4_quantize(w32, 0, n, k, block, True)
    w = sg.Q4Weights.with_params(q, s, mins, n, k, sg.Q4Params(block).affine())
    a32 = rng.standard_normal((m, k)).astype(np.float32)
    a_bits = orc.f32_to_bf16_bits(a32) if bf16 else orc.f32_to_f16_bits(a32)
    bias = (rng.standard_normal(n) * 0.1).astype(np.float32)
    b_bits = orc.f32_to_bf16_bits(bias) if bf16 else orc.f32_to_f16_bits(bias)
    b_dev = bf16_bits_dev(b_bits) if bf16 else f16_bits_dev(b_bits)
    ep = sg.Epilogue("bf16" if bf16 else "f16").add_col(b_dev).relu()
    want = orc.matmul_q4(a_bits, q, s, mins, n, k, block, m, orc.Nodes([(4, 0, 0.0, b_bits, 0), (8, 1, 0.0, None, 0)]), bf16)
    a_dev = bf16_bits_dev(a_bits) if bf16 else f16_bits_dev(a_bits)
    c = torch.full((m, n), 9.0, dtype=a_dev.dtype, device="cuda")
    (sg.matmul_q4_bf16_ep if bf16 else sg.matmul_q4_ep)(a_dev, w, c, m, ep)
    torch.cuda.synchronize()
    assert sg.last_status() == 0
    g32, w32o = orc.t_bits_to_f32(bits_of(c), bf16), orc.t_bits_to_f32(want, bf16)
    assert max_rel(g32, w32o) <= (2e-2 if bf16 else TOL)


def test_affine_with_zero_minima_equals_the_scale_form_and_the_library_quantiser_agrees():
    """Scale == Affine(zero mins) (tests/correctness/q4.rs:300-328), and Q4Weights.quantize with the affine parameter
    produces the oracle's codes, scales and minima."""
    rng = np.random.default_rng(77)
    m, n, k, block = 5, 96, 512, 32
    q, s = q4_logical(rng, n, k, block)
    a = f16_bits_dev(orc.f32_to_f16_bits(rng.standard_normal((m, k)).astype(np.float32)))
    scale_form = sg.Q4Weights.with_params(q, s, None, n, k, sg.Q4Params(block))
    affine = sg.Q4Weights.with_params(q, s, np.zeros(n * (k // block), np.uint16), n, k, sg.Q4Params(block).affine())
    c0 = torch.zeros((m, n), dtype=torch.float16, device="cuda")
    c1 = torch.zeros_like(c0)
    sg.matmul_q4(a, scale_form, c0, m)
    sg.matmul_q4(a, affine, c1, m)
    assert max_rel(c1.float().cpu().numpy(), c0.float().cpu().numpy()) <= 3e-3      # f16 block sums against f32 accumulation
    w32 = (rng.standard_normal((n, k)) * 0.05 + 0.01).astype(np.float32)
    wq = sg.Q4Weights.quantize(w32, sg.WeightLayout.OutIn, n, k, sg.Q4Params(block).affine())
    qo, so, mo = orc.q4_quantize(w32, 0, n, k, block, True)
    want = orc.matmul_q4(bits_of(a), qo, so, mo, n, k, block, m)
    sg.matmul_q4(a, wq, c1, m)
    assert max_rel(c1.float().cpu().numpy(), orc.f16_bits_to_f32(want).reshape(m, n)) <= TOL
