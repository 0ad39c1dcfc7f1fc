"""Prefill GEMM (tcgen05 / TMEM) on the GPU against the CPU oracle, through the C ABI.

Rows above the decode kernel's row cap run the tensor-core kernel.  Tolerance as
for the decode path: max |g-w|/(1+|w|) <= 1e-2 against the oracle (same f32
accumulation over the same rounded weights; only the summation order differs)."""
import numpy as np
import pytest
import torch

import oracle as orc
import sme_gemm_b200 as sg
from gpu_util import bf16_bits_dev, bits_of, f16_bits_dev, max_rel, q4_logical

pytestmark = pytest.mark.gpu
TOL = 1e-2
# bf16 through an epilogue: the product is rounded to bf16 before the graph (as the reference does), a different
# summation order can flip that rounding by one ulp (2^-8 relative), and the activation carries it to at most two ulps
# of the result: 2e-2 on the 1/(1+|w|) metric.  Still far inside the reference's own sqrt(k)-scaled bound
# (max(1e-2, 1e-2*sqrt(k)/4) = 0.16 at k = 4096).
TOL_BF16_EP = 2e-2


def run(m, n, k, block, bf16, seed=0, ep=None, sample_rows=None):
    rng = np.random.default_rng(seed + m * 131 + n * 17 + k)
    q, s = q4_logical(rng, n, k, block)
    w = sg.Q4Weights.with_params(q, s, None, n, k, sg.Q4Params(block))
    a32 = rng.standard_normal((m, k)).astype(np.float32)
    a_bits = orc.f32_to_bf16_bits(a32) if bf16 else orc.f32_to_f16_bits(a32)
    to_dev = bf16_bits_dev if bf16 else f16_bits_dev
    dt = "bf16" if bf16 else "f16"
    epi, nodes = None, None
    if ep == "cfg4":   # add_col(bias).silu().clamp(-6, 6)
        bias = orc.f32_to_bf16_bits((rng.standard_normal(n) * 0.1).astype(np.float32)) if bf16 else \
            orc.f32_to_f16_bits((rng.standard_normal(n) * 0.1).astype(np.float32))
        epi = sg.Epilogue(dt).add_col(to_dev(bias)).silu().clamp(-6.0, 6.0)
        nodes = orc.Nodes([(4, 0, 0.0, bias, 0), (9, 0, -6.0, None, 0), (10, 0, 6.0, None, 0), (8, 3, 0.0, None, 0)])
    c = torch.full((m, n), 9.0, dtype=torch.bfloat16 if bf16 else torch.float16, device="cuda")
    fn = (sg.matmul_q4_bf16_ep if bf16 else sg.matmul_q4_ep) if epi is not None else (sg.matmul_q4_bf16 if bf16 else sg.matmul_q4)
    fn(*((to_dev(a_bits), w, c, m, epi) if epi is not None else (to_dev(a_bits), w, c, m)))
    torch.cuda.synchronize()
    assert sg.last_status() == 0
    got = orc.t_bits_to_f32(bits_of(c), bf16)
    if sample_rows is None:
        want = orc.t_bits_to_f32(orc.matmul_q4(a_bits, q, s, None, n, k, block, m, nodes, bf16), bf16)
        return max_rel(got, want)
    wdeq = orc.q4_dequant(q, s, None, n, k, block, bf16)
    worst = 0.0
    for r0 in sample_rows:
        want = orc.matmul_q4(a_bits, q, s, None, n, k, block, m, nodes, bf16, wdeq=wdeq, first=r0, rows=1)
        worst = max(worst, max_rel(got[r0], orc.t_bits_to_f32(want[r0], bf16)))
    return worst


# tests/correctness/q4.rs:132,199-203,422 and src/kernels/lowbit/matmul.rs:534-541 shapes
@pytest.mark.parametrize("m,n,k,block", [(64, 96, 128, 32), (65, 33, 256, 32), (800, 520, 512, 32), (40, 4200, 2048, 32),
                                         (200, 4100, 2048, 32), (33, 130, 512, 16), (96, 4130, 1024, 8), (300, 200, 4096, 128),
                                         (513, 256, 576, 64)])
@pytest.mark.parametrize("bf16", [False, True])
def test_q4_gemm_matches_oracle(m, n, k, block, bf16):
    mr = run(m, n, k, block, bf16)
    assert mr <= TOL, f"{m}x{n}x{k} block {block} bf16={bf16}: max_rel {mr}"


@pytest.mark.parametrize("bf16", [False, True])
def test_q4_gemm_epilogue_graph(bf16):
    assert run(100, 300, 512, 32, bf16, ep="cfg4") <= (TOL_BF16_EP if bf16 else TOL)


def test_ragged_depth_falls_back_to_the_decode_kernel_rows():
    """k % 8 != 0 cannot use a tensor map; the call still runs and matches."""
    assert run(40, 200, 1030, 32, False) <= TOL
    assert run(96, 130, 1027, 1, False) <= TOL


def test_config4_prefill_full_size_sampled_rows():
    """M=512, K=4096, N=14336 bf16, add_col(bias).silu().clamp(-6,6); 12 sampled rows against the oracle."""
    rows = [0, 1, 127, 128, 255, 256, 300, 383, 384, 500, 510, 511]
    mr = run(512, 14336, 4096, 32, True, seed=4, ep="cfg4", sample_rows=rows)
    assert mr <= TOL_BF16_EP, mr


def test_mlp_block_m256_sampled_rows():
    """config 5 at M=256 (hidden 4096, intermediate 14336): sampled rows against the oracle block."""
    d, f, m = 4096, 14336, 256
    rng = np.random.default_rng(55)
    wg = (rng.standard_normal((f, d)) * 0.02).astype(np.float32)
    wu = (rng.standard_normal((f, d)) * 0.02).astype(np.float32)
    wd = (rng.standard_normal((d, f)) * 0.02).astype(np.float32)
    up = sg.GatedLinear.quantize(wg, wu, sg.WeightLayout.OutIn, f, d, sg.Gate.Silu)
    down = sg.Linear.quantize(wd, sg.WeightLayout.OutIn, d, f)
    mlp = sg.Mlp.gated(up, down)
    x = torch.from_numpy(rng.standard_normal((m, d)).astype(np.float16)).cuda()
    y = torch.zeros((m, d), dtype=torch.float32, device="cuda")
    mlp.accumulate(x, y, m)
    torch.cuda.synchronize()
    assert sg.last_status() == 0
    both_w = sg.interleave_gate_up(wg, wu, sg.WeightLayout.OutIn, f, d)
    guq, gus, _ = orc.q4_quantize(both_w, 1, 2 * f, d)
    dq, ds, _ = orc.q4_quantize(wd, 0, d, f)
    orc.set_threads(orc.max_threads())
    xs = x.cpu().numpy()
    got = y.cpu().numpy()
    for r0 in (0, 100, 255):
        want = np.zeros((1, d), np.float32)
        orc.mlp_accumulate(xs[r0:r0 + 1], want, 1, d, f, guq, gus, dq, ds)
        assert max_rel(got[r0], want[0]) <= TOL
    orc.set_threads(1)
