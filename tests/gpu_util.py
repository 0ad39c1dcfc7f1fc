"""Helpers shared by the GPU parity tests."""
import numpy as np
import torch

import oracle as orc


def dev(x_np, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(x_np)).cuda()
    return t if dtype is None else t.view(dtype)


def f16_bits_dev(bits):
    return dev(np.ascontiguousarray(bits, dtype=np.uint16).view(np.float16))


def bf16_bits_dev(bits):
    return dev(np.ascontiguousarray(bits, dtype=np.uint16).view(np.int16)).view(torch.bfloat16)


def bits_of(t):
    """torch f16 / bf16 CUDA tensor -> numpy uint16 bit patterns."""
    return t.detach().contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def max_rel(got_f32, want_f32):
    """The reference's metric (tests/correctness/main.rs:63-68): max |g - w| / (1 + |w|)."""
    g, w = np.asarray(got_f32, np.float64), np.asarray(want_f32, np.float64)
    return float(np.max(np.abs(g - w) / (1.0 + np.abs(w)))) if g.size else 0.0


def half_tol(base, k):
    """tests/proptest.rs:83-85: max(base, base * sqrt(k) / 4)."""
    return max(base, base * (k ** 0.5) / 4.0)


def q4_logical(rng, n, k, block, from_f32=True):
    """Seeded Q4 weights in the logical layout: (quants, scales)."""
    if from_f32:
        w = (rng.standard_normal(n * k) * 0.02).astype(np.float32)
        q, s, _ = orc.q4_quantize(w, 0, n, k, block)
        return q, s
    q = rng.integers(0, 256, (k * n + 1) // 2).astype(np.uint8)
    if (k * n) % 2:
        q[-1] &= 0x0F
    nbk = -(-k // block)
    s = orc.f32_to_f16_bits((0.01 + 0.001 * (np.arange(n * nbk) % 5)).astype(np.float32))
    return q, s
