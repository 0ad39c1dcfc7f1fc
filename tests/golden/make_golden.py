"""Generates tests/golden/vectors.npz: input / output vectors of the hot path for a few small,
seeded cases, produced by the C oracle (oracle/oracle.c) and accepted only where the independent
numpy restatement (oracle/np_oracle.py) gives the same bits.

The reference itself is a Rust crate and cannot run where this was built (no cargo / rustc), so
these vectors pin the two restatements and the CUDA path to each other, not to an execution of the
reference: parity stays "unpinned" in that sense.  The inputs come from the reference's own test
generators (tests/refgen.py restates `fill` and `data`), so a maintainer with the Rust crate can
regenerate the same inputs there and compare outputs.

Run from the repository root:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import oracle as orc                      # noqa: E402
import sme_gemm_b200 as sg                # noqa: E402  (host-side layout helper only; no device needed)
from oracle import np_oracle as npo       # noqa: E402
from refgen import Lcg, data              # noqa: E402


def main():
    out = {}
    # ---- Q4: quantise, dequantise, f16 / bf16 matmul, with and without an epilogue ----
    for ci, (m, n, k, block) in enumerate([(1, 48, 96, 32), (5, 33, 130, 16), (9, 128, 256, 64)]):
        w = (Lcg(100 + ci).fill(n * k).astype(np.float32) * np.float32(0.08))
        q, s, _ = orc.q4_quantize(w, 0, n, k, block)
        q2, s2, _ = npo.q4_quantize(w, 0, n, k, block)
        assert np.array_equal(q, q2) and np.array_equal(s, s2)
        a = Lcg(200 + ci).fill(m * k).view(np.uint16)
        bias = Lcg(300 + ci).fill(n).view(np.uint16)
        nodes = [(4, 0, 0.0, bias, 0), (9, 0, -6.0, None, 0), (10, 0, 6.0, None, 0), (8, 3, 0.0, None, 0)]
        for bf16 in (False, True):
            ab = orc.f32_to_bf16_bits(orc.f16_bits_to_f32(a)) if bf16 else a
            bb = orc.f32_to_bf16_bits(orc.f16_bits_to_f32(bias)) if bf16 else bias
            nd = [(4, 0, 0.0, bb, 0)] + nodes[1:]
            c0 = orc.matmul_q4(ab, q, s, None, n, k, block, m, None, bf16)
            c1 = orc.matmul_q4(ab, q, s, None, n, k, block, m, orc.Nodes(nd), bf16)
            wd = npo.q4_dequant(q, s, None, n, k, block, bf16)
            assert np.array_equal(c0.reshape(-1), npo.gemm16(ab, wd, m, n, k, bf16).reshape(-1))
            assert np.array_equal(c1.reshape(-1), npo.apply_ep(c0, m, n, nd, bf16).reshape(-1))
            tag = f"q4_{ci}_{'bf16' if bf16 else 'f16'}"
            out[tag + "_a"], out[tag + "_bias"], out[tag + "_c"], out[tag + "_c_ep"] = ab, bb, c0, c1
        out[f"q4_{ci}_dims"] = np.array([m, n, k, block])
        out[f"q4_{ci}_w"], out[f"q4_{ci}_quants"], out[f"q4_{ci}_scales"] = w, q, s
    # ---- 2-bit / 1-bit: int8 activations, block sums, outputs ----
    for ci, (m, n, k, block, book) in enumerate([(1, 64, 256, 128, [-1, 0, 1, 0]), (3, 37, 200, 16, [-2, -1, 1, 2]),
                                                  (8, 80, 512, 256, [-128, 127, 3, -7])]):
        nbk = -(-k // block)
        scales = orc.f32_to_f16_bits(data(ci + 7, n * nbk).astype(np.float32) * np.float32(1e-3) - np.float32(0.1))
        a = orc.f32_to_f16_bits((data(ci + 99, m * k).astype(np.float32) - np.float32(128.0)) / np.float32(37.0))
        codes = data(ci * 31 + 1, (k * n + 3) // 4)
        signs = data(ci * 17 + 2, (k * n + 7) // 8)
        c2, q8, sa, sums2 = orc.lowbit_matmul(a, 2, codes, 1, scales, book, n, k, block, m, debug=True)
        c1, _, _, sums1 = orc.lowbit_matmul(a, 1, signs, 0, scales, None, n, k, block, m, debug=True)
        n2c, n2s = npo.lowbit_matmul(a, npo.q2_values(codes, n, k, book), scales, n, k, block, m)
        assert np.array_equal(c2.reshape(-1), n2c.reshape(-1)) and np.array_equal(sums2.reshape(-1), n2s.reshape(-1))
        n1c, n1s = npo.lowbit_matmul(a, npo.q1_values(signs, 0, n, k), scales, n, k, block, m)
        assert np.array_equal(c1.reshape(-1), n1c.reshape(-1)) and np.array_equal(sums1.reshape(-1), n1s.reshape(-1))
        out[f"lb_{ci}_dims"] = np.array([m, n, k, block] + list(book))
        out[f"lb_{ci}_a"], out[f"lb_{ci}_scales"], out[f"lb_{ci}_codes"], out[f"lb_{ci}_signs"] = a, scales, codes, signs
        out[f"lb_{ci}_q"], out[f"lb_{ci}_sa"] = q8, sa
        out[f"lb_{ci}_q2_sums"], out[f"lb_{ci}_q2_c"] = sums2, c2
        out[f"lb_{ci}_q1_sums"], out[f"lb_{ci}_q1_c"] = sums1, c1
    # ---- the gated MLP block ----
    m, d, f = 3, 64, 96
    wg = Lcg(41).fill(f * d).astype(np.float32) * np.float32(0.2)
    wu = Lcg(42).fill(f * d).astype(np.float32) * np.float32(0.2)
    wd = Lcg(43).fill(d * f).astype(np.float32) * np.float32(0.2)
    x = Lcg(44).fill(m * d).view(np.uint16)
    both = sg.interleave_gate_up(wg, wu, sg.WeightLayout.OutIn, f, d)   # [gate | up] as d x 2f, 32 columns at a time
    guq, gus, _ = orc.q4_quantize(both, 1, 2 * f, d)
    dq, ds, _ = orc.q4_quantize(wd, 0, d, f)
    y = np.zeros((m, d), np.float32)
    orc.mlp_accumulate(x.view(np.float16).reshape(m, d), y, m, d, f, guq, gus, dq, ds)
    out["mlp_dims"] = np.array([m, d, f])
    out["mlp_wg"], out["mlp_wu"], out["mlp_wd"], out["mlp_x"], out["mlp_y"] = wg, wu, wd, x, y
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "vectors.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes,", len(out), "arrays")


if __name__ == "__main__":
    main()
