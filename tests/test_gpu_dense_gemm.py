"""The Gemm builder on pre-packed dense f16 / bf16 weights (src/exec/builder.rs:220-227, 428-813;
packed_ep_impl, src/exec/macros.rs:98-200): C = ep( T(beta * (A @ B)) ), row- or column-major,
against the CPU oracle's dense reference GEMM (f32 accumulate in K order, src/reference.rs:308-387)
and scalar epilogue.  Tolerance: max |got - want| / (1 + |want|) <= 1e-2 (2e-2 through a bf16
epilogue: one bf16 ulp of the rounded product can flip)."""
import numpy as np
import pytest
import torch

import oracle as orc
import sme_gemm_b200 as sg
from gpu_util import bf16_bits_dev, bits_of, f16_bits_dev, max_rel

pytestmark = pytest.mark.gpu


def _case(m, n, k, bf16, seed):
    rng = np.random.default_rng(seed)
    tb = orc.f32_to_bf16_bits if bf16 else orc.f32_to_f16_bits
    a = tb(rng.standard_normal(m * k).astype(np.float32))
    b = tb((rng.standard_normal(k * n) * 0.05).astype(np.float32))
    bias = tb((rng.standard_normal(n) * 0.1).astype(np.float32))
    return a, b, bias


@pytest.mark.parametrize("m,n,k", [(1, 64, 64), (7, 100, 72), (33, 130, 512), (200, 1000, 256), (300, 384, 1024)])
@pytest.mark.parametrize("bf16", [False, True])
def test_gemm_builder_matches_dense_reference(m, n, k, bf16):
    a, b, bias = _case(m, n, k, bf16, m + n)
    tof = orc.bf16_bits_to_f32 if bf16 else orc.f16_bits_to_f32
    todev = bf16_bits_dev if bf16 else f16_bits_dev
    dt = torch.bfloat16 if bf16 else torch.float16
    w = (sg.prepack_bf16 if bf16 else sg.prepack_f16)(b, n, k)
    ad, biasd = todev(a).reshape(m, k), todev(bias)
    want0 = orc.gemm16(a, b, m, n, k, bf16)
    # plain
    c = torch.full((m, n), 9.0, dtype=dt, device="cuda")
    sg.Gemm.new(ad, w, m).run(c)
    assert max_rel(tof(bits_of(c)), tof(want0)) <= 1e-2
    # the documented example: bias then gelu (trailing), and an in-order chain with a clamp
    sg.Gemm.new(ad, w, m).add_col(biasd).gelu().run(c)
    want = orc.apply_ep(want0, m, n, orc.Nodes([(4, 0, 0.0, bias, 0), (8, 2, 0.0, None, 0)]), bf16)
    assert max_rel(tof(bits_of(c)), tof(want)) <= (2e-2 if bf16 else 1e-2)
    sg.Gemm.new(ad, w, m).mul_col(biasd).add_col(biasd).silu().clamp(-6.0, 6.0).run(c)
    want = orc.apply_ep(want0, m, n, orc.Nodes([(5, 0, 0.0, bias, 0), (4, 0, 0.0, bias, 0), (9, 0, -6.0, None, 0),
                                                (10, 0, 6.0, None, 0), (8, 3, 0.0, None, 0)]), bf16)
    assert max_rel(tof(bits_of(c)), tof(want)) <= (2e-2 if bf16 else 1e-2)
    torch.cuda.synchronize()
    assert sg.last_status() == 0


def test_beta_and_column_major_output():
    m, n, k = 37, 96, 128
    a, b, bias = _case(m, n, k, False, 3)
    w = sg.prepack_f16(b, n, k)
    ad = f16_bits_dev(a).reshape(m, k)
    # beta scales the f32 product before the store rounding: reference::gemm_f16 stores f16(beta * acc)
    acc = orc.gemm16_f32(a, b, m, n, k)
    want = orc.f32_to_f16_bits((np.float32(0.5) * acc).astype(np.float32)).reshape(m, n)
    c = torch.zeros((m, n), dtype=torch.float16, device="cuda")
    sg.Gemm.new(ad, w, m).beta(0.5).run(c)
    assert max_rel(orc.f16_bits_to_f32(bits_of(c)), orc.f16_bits_to_f32(want)) <= 1e-2
    ccm = torch.zeros((n, m), dtype=torch.float16, device="cuda")      # c[i + j * m]
    sg.Gemm.new(ad, w, m).beta(0.5).col_major_output().add_col(f16_bits_dev(bias)).run(ccm.view(m, n))
    want_cm = orc.apply_ep(want, m, n, orc.Nodes([(4, 0, 0.0, bias, 0)]))
    got = orc.f16_bits_to_f32(bits_of(ccm)).reshape(n, m).T
    assert max_rel(got, orc.f16_bits_to_f32(want_cm).reshape(m, n)) <= 1e-2


def test_host_pointer_entry_and_unsupported_depth():
    m, n, k = 5, 48, 64
    a, b, _ = _case(m, n, k, False, 9)
    w = sg.prepack_f16(b, n, k)
    c = np.zeros((m, n), np.float16)
    sg.Gemm.new(a.view(np.float16).reshape(m, k), w, m).relu().run(c)
    want = orc.apply_ep(orc.gemm16(a, b, m, n, k), m, n, orc.Nodes([(8, 1, 0.0, None, 0)]))
    assert max_rel(c.astype(np.float32), orc.f16_bits_to_f32(want).reshape(m, n)) <= 1e-2


@pytest.mark.parametrize("m,n,k", [(5, 48, 60), (3, 130, 37), (70, 200, 513)])
def test_ragged_depth_runs_through_a_padded_copy(m, n, k):
    """Gemm::run takes any k (src/exec/builder.rs:803-813): a depth that is not a multiple of 8, or an A that is not
    16-byte aligned, is staged through a zero-padded copy on the device."""
    a, b, _ = _case(m, n, k, False, 9)
    w = sg.prepack_f16(b, n, k)
    ad = torch.from_numpy(a.view(np.float16).reshape(m, k).copy()).cuda()
    c = torch.zeros((m, n), dtype=torch.float16, device="cuda")
    sg.Gemm.new(ad, w, m).relu().run(c)
    torch.cuda.synchronize()
    want = orc.apply_ep(orc.gemm16(a, b, m, n, k), m, n, orc.Nodes([(8, 1, 0.0, None, 0)]))
    assert max_rel(c.float().cpu().numpy(), orc.f16_bits_to_f32(want).reshape(m, n)) <= 1e-2
    assert sg.last_status() == 0
