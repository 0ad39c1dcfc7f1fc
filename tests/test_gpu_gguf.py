"""GGUF files through to the kernels: Q1_0 (the Bonsai model's format, examples/bonsai/model.rs:134-160), Q4_0, Q4_1 and TQ2_0
tensors written to a file, loaded as weight sets and multiplied against the oracle on the arrays the loader made."""
import numpy as np
import pytest
import torch

import oracle as orc
import sme_gemm_b200 as sg
from gpu_util import bits_of, f16_bits_dev, max_rel
from sme_gemm_b200 import gguf
from test_gguf import q1_blocks, q4_1_blocks, q4_blocks, tq2_blocks, write_gguf

pytestmark = pytest.mark.gpu


def test_gguf_weight_sets_multiply_like_their_arrays(tmp_path):
    rng = np.random.default_rng(11)
    k = 512
    path = tmp_path / "synthetic.gguf"
    path.write_bytes(write_gguf(
        [("general.architecture", 8, "synthetic"), ("synthetic.block_count", 4, 1)],
        [("blk.0.attn_q.weight", [k, 48], gguf.Q1_0, q1_blocks(rng, 48, k)[0]),
         ("blk.0.attn_k.weight", [k, 16], gguf.Q1_0, q1_blocks(rng, 16, k)[0]),
         ("blk.0.ffn_up.weight", [k, 72], gguf.Q4_0, q4_blocks(rng, 72, k)),
         ("blk.0.ffn_gate.weight", [k, 56], gguf.Q4_1, q4_1_blocks(rng, 56, k)),
         ("blk.0.ffn_down.weight", [k, 40], gguf.TQ2_0, tq2_blocks(rng, 40, k))]))
    g = gguf.Gguf.load(path)
    assert g.int("synthetic.block_count") == 1 and g.str("general.architecture") == "synthetic"
    for m in (1, 9, 70):
        a32 = rng.standard_normal((m, k)).astype(np.float32)
        a16 = a32.astype(np.float16)
        a = torch.from_numpy(a16).cuda()
        # Q1_0: q and k projections stacked into one weight set, bit-exact on the int8-activation path
        w1 = gguf.q1(g, ["blk.0.attn_q.weight", "blk.0.attn_k.weight"])
        signs, scales, n, _ = gguf.q1_arrays(g, ["blk.0.attn_q.weight", "blk.0.attn_k.weight"])
        c = torch.zeros((m, n), dtype=torch.float16, device="cuda")
        sg.matmul_q1(a, w1, c, m)
        assert np.array_equal(bits_of(c), orc.lowbit_matmul(a16, 1, signs, 0, scales, None, n, k, 128, m))
        # TQ2_0: ternary codes, block 256
        w2 = gguf.tq2_0(g, ["blk.0.ffn_down.weight"])
        codes, scales2, n2, _ = gguf.tq2_0_arrays(g, ["blk.0.ffn_down.weight"])
        c2 = torch.zeros((m, n2), dtype=torch.float16, device="cuda")
        sg.matmul_q2(a, w2, c2, m)
        assert np.array_equal(bits_of(c2), orc.lowbit_matmul(a16, 2, codes, 1, scales2, gguf.TQ2_CODEBOOK, n2, k, 256, m))
        # Q4_0
        w4 = gguf.q4_0(g, ["blk.0.ffn_up.weight"])
        quants, scales4, n4, _ = gguf.q4_0_arrays(g, ["blk.0.ffn_up.weight"])
        c4 = torch.zeros((m, n4), dtype=torch.float16, device="cuda")
        sg.matmul_q4(a, w4, c4, m)
        want = orc.f16_bits_to_f32(orc.matmul_q4(orc.f32_to_f16_bits(a16.astype(np.float32)), quants, scales4, None, n4, k, 32, m))
        assert max_rel(c4.float().cpu().numpy(), want.reshape(m, n4)) <= 1e-2
        # and against the format's own dequantised weights in f64
        ref = a16.astype(np.float64) @ gguf.dequant(g, "blk.0.ffn_up.weight").astype(np.float64).T
        assert max_rel(c4.float().cpu().numpy(), ref.astype(np.float32)) <= 2e-2
        # Q4_1: the affine form (offset m + 8 d rounded to f16 once)
        w41 = gguf.q4_1(g, ["blk.0.ffn_gate.weight"])
        quants1, scales1, mins1, n1, _ = gguf.q4_1_arrays(g, ["blk.0.ffn_gate.weight"])
        c41 = torch.zeros((m, n1), dtype=torch.float16, device="cuda")
        sg.matmul_q4(a, w41, c41, m)
        want = orc.f16_bits_to_f32(orc.matmul_q4(orc.f32_to_f16_bits(a16.astype(np.float32)), quants1, scales1, mins1, n1, k, 32, m))
        assert max_rel(c41.float().cpu().numpy(), want.reshape(m, n1)) <= 1e-2
        ref = a16.astype(np.float64) @ gguf.dequant(g, "blk.0.ffn_gate.weight").astype(np.float64).T
        assert max_rel(c41.float().cpu().numpy(), ref.astype(np.float32)) <= 2e-2
    assert sg.last_status() == 0
