"""Independent numpy restatement of the reference's portable scalar path.

TEST INFRASTRUCTURE ONLY.  Written from the same reference lines as
oracle/oracle.c but sharing no code with it; tests require the two to agree bit
for bit before either is trusted (the reference cannot be executed here: it is
Rust and no Rust toolchain exists in the build environment).

numpy float32 arithmetic is IEEE and never fused, numpy's float64 -> float16
cast is a single round-to-nearest-even, which is what crate `half` 2.7.1 does.
16-bit values are carried as uint16 bit patterns.
"""
from __future__ import annotations

import math

import numpy as np

F32 = np.float32


# ---- conversions -----------------------------------------------------------

def f16_bits(x) -> np.ndarray:
    """f32/f64 array -> f16 bit patterns (one rounding, ties to even)."""
    with np.errstate(over="ignore"):
        return np.asarray(x).astype(np.float16).view(np.uint16)


def f16_val(bits) -> np.ndarray:
    return np.asarray(bits, np.uint16).view(np.float16).astype(np.float32)


def bf16_bits(x) -> np.ndarray:
    """f32 -> bf16 bits, ties to even; NaN keeps a quiet payload (half::bf16::from_f32)."""
    u = np.asarray(x, np.float32).view(np.uint32).astype(np.uint64)
    nan = (u & 0x7FFFFFFF) > 0x7F800000
    rounded = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    out = np.where(nan, (u >> 16) | 0x40, rounded)
    return out.astype(np.uint16)


def bf16_val(bits) -> np.ndarray:
    return (np.asarray(bits, np.uint16).astype(np.uint32) << 16).view(np.float32)


def t_val(bits, bf16):
    return bf16_val(bits) if bf16 else f16_val(bits)


def t_bits(x, bf16):
    return bf16_bits(x) if bf16 else f16_bits(x)


# ---- Q4 ---------------------------------------------------------------------

def q4_codes_from_quants(quants, n, k) -> np.ndarray:
    """Row-major k x n signed codes from the packed nibbles (idx = d*n+j, low nibble first)."""
    q = np.asarray(quants, np.uint8)
    nib = np.empty(q.size * 2, np.uint8)
    nib[0::2] = q & 0x0F
    nib[1::2] = q >> 4
    nib = nib[: k * n].astype(np.int32)
    return np.where(nib < 8, nib, nib - 16).reshape(k, n)


def q4_quantize(w, layout, n, k, block=32, affine=False):
    """src/kernels/q4/quantize.rs:29-81."""
    w = np.asarray(w, np.float32)
    wj = w.reshape(n, k) if layout == 0 else w.reshape(k, n).T  # [j][d]
    nbk = -(-k // block)
    codes = np.zeros((k, n), np.int32)
    scales = np.zeros((n, nbk), np.uint16)
    mins = np.zeros((n, nbk), np.uint16)
    for b in range(nbk):
        blk = wj[:, b * block:(b + 1) * block]  # n x len
        if affine:
            lo, hi = blk.min(axis=1), blk.max(axis=1)
            sc = f16_bits((hi - lo) / F32(15.0))
            mn = f16_bits(lo + F32(8.0) * f16_val(sc))
        else:
            idx = np.argmax(np.abs(blk), axis=1)  # first of the largest magnitudes
            m = blk[np.arange(n), idx]
            m = np.where(np.abs(m) > 0, m, F32(0.0))
            sc = f16_bits(m / F32(-8.0))
            mn = np.zeros(n, np.uint16)
        scales[:, b], mins[:, b] = sc, mn
        s, mv = f16_val(sc), f16_val(mn)
        with np.errstate(divide="ignore"):
            inv = np.where(s == 0, F32(0.0), F32(1.0) / s).astype(np.float32)
        t = ((blk - mv[:, None]).astype(np.float32) * inv[:, None]).astype(np.float32)
        r = np.sign(t) * np.floor(np.abs(t) + F32(0.5))  # round half away from zero
        codes[b * block:b * block + blk.shape[1], :] = np.clip(r, -8, 7).astype(np.int32).T
    flat = (codes.reshape(-1) & 0x0F).astype(np.uint8)
    if flat.size % 2:
        flat = np.append(flat, np.uint8(0))
    quants = (flat[0::2] | (flat[1::2] << 4)).astype(np.uint8)
    return quants, scales.reshape(-1), (mins.reshape(-1) if affine else None)


def q4_dequant(quants, scales, mins, n, k, block=32, bf16=False) -> np.ndarray:
    """src/kernels/q4/weights.rs:232-259: exact f64 product, one rounding."""
    codes = q4_codes_from_quants(quants, n, k).astype(np.float64)
    nbk = -(-k // block)
    sc = f16_val(scales).astype(np.float64).reshape(n, nbk)
    blk = np.arange(k) // block
    v = sc[:, blk].T * codes
    if mins is not None:
        v = v + f16_val(mins).astype(np.float64).reshape(n, nbk)[:, blk].T
    return bf16_bits(v.astype(np.float32)) if bf16 else f16_bits(v)


def gemm16(a_bits, b_bits, m, n, k, bf16=False) -> np.ndarray:
    """src/reference.rs:308-387 with alpha = 0, beta = 1."""
    a = t_val(a_bits, bf16).reshape(m, k)
    b = t_val(b_bits, bf16).reshape(k, n)
    acc = np.zeros((m, n), np.float32)
    for l in range(k):
        acc += (a[:, l:l + 1] * b[l:l + 1, :]).astype(np.float32)
    return t_bits(F32(0.0) + F32(1.0) * acc, bf16)


# ---- epilogue -----------------------------------------------------------------

_SELU_A, _SELU_L = 1.6732632423543772, 1.0507009873554805


def _erf_as(x):
    ax = abs(x)
    t = 1.0 / (1.0 + 0.3275911 * ax)
    poly = ((((1.061405429 * t - 1.453152027) * t + 1.421413741) * t - 0.284496736) * t + 0.254829592) * t
    e = 1.0 - poly * math.exp(-ax * ax)
    return -e if x < 0 else e


def _clamp(x, lo, hi):
    if x < lo:
        return lo
    if x > hi:
        return hi
    return x


def act_f64(kind, x, alpha=0.0):
    """src/epilogue/mod.rs:40-86 (scalar, python floats are f64)."""
    try:
        if kind == 1:
            return 0.0 if math.isnan(x) else max(x, 0.0)
        if kind == 2:
            return 0.5 * x * (1.0 + math.tanh(0.7978845608028654 * (x + 0.044715 * x * x * x)))
        if kind == 3:
            return x / (1.0 + _exp(-x))
        if kind == 4:
            return math.tanh(x)
        if kind == 5:
            return 1.0 / (1.0 + _exp(-x))
        if kind == 6:
            return x if x >= 0 else alpha * x
        if kind == 7:
            return _clamp(x, 0.0, 6.0)
        if kind == 8:
            return _clamp(x / 6.0 + 0.5, 0.0, 1.0)
        if kind == 9:
            return x * _clamp(x / 6.0 + 0.5, 0.0, 1.0)
        if kind == 10:
            return abs(x)
        if kind == 11:
            return -x
        if kind == 12:
            return x * x
        if kind == 13:
            return 1.0 if x > 0 else (-1.0 if x < 0 else 0.0)
        if kind == 14:
            return math.sqrt(x) if x >= 0 else float("nan")
        if kind == 15:
            return x / (1.0 + abs(x))
        if kind == 16:
            return float(np.float64(1.0) / np.float64(x))
        if kind == 17:
            return float(np.float64(1.0) / np.sqrt(np.float64(x)))
        if kind == 18:
            return _exp(x)
        if kind == 19:
            return float(np.log(np.float64(x)))
        if kind == 20:
            return x if x >= 0 else alpha * math.expm1(x)
        if kind == 21:
            return _SELU_L * (x if x >= 0 else _SELU_A * math.expm1(x))
        if kind == 22:
            return max(x, 0.0) + math.log1p(_exp(-abs(x)))
        if kind == 23:
            return x * math.tanh(max(x, 0.0) + math.log1p(_exp(-abs(x))))
        if kind == 24:
            return 0.5 * x * (1.0 + _erf_as(x * 0.7071067811865476))
    except (OverflowError, ValueError):
        return float("nan")
    return x


def _exp(x):
    try:
        return math.exp(x)
    except OverflowError:
        return float("inf")


def apply_ep(c_bits, m, n, nodes, bf16=False) -> np.ndarray:
    """src/exec/scalar.rs:58-140.  nodes: list of (op, aux, scalar, operand_bits or None, ld)."""
    c = t_val(c_bits, bf16).reshape(m, n).copy()
    i_idx, j_idx = np.meshgrid(np.arange(m), np.arange(n), indexing="ij")
    with np.errstate(all="ignore"):
        for op, aux, scalar, operand, ld in nodes:
            s = F32(scalar)
            if operand is not None:
                ov = t_val(operand, bf16).reshape(-1)
                ld = ld or n
                if op in (2, 3, 12, 16, 19, 22):
                    o = ov[i_idx]
                elif op in (4, 5, 13, 17, 20, 23):
                    o = ov[j_idx]
                else:
                    o = ov[i_idx * ld + j_idx]
            else:
                o = s
            if op in (0, 2, 4, 6):
                c = (c + o).astype(np.float32)
            elif op in (1, 3, 5, 7):
                c = (c * o).astype(np.float32)
            elif op in (11, 12, 13, 14):
                c = (c - o).astype(np.float32)
            elif op in (15, 16, 17, 18):
                c = (c / o).astype(np.float32)
            elif op in (9, 19, 20, 21):
                c = np.fmax(c, o).astype(np.float32)
            elif op in (10, 22, 23, 24):
                c = np.fmin(c, o).astype(np.float32)
            elif op == 8:
                flat = c.reshape(-1)
                out = np.array([act_f64(aux, float(v), float(F32(scalar))) for v in flat], np.float64)
                c = out.astype(np.float32).reshape(m, n)
    return t_bits(c, bf16)


# ---- low-bit ------------------------------------------------------------------

def quantize_row(a_bits, block):
    """src/kernels/lowbit/matmul.rs:354-371."""
    a = f16_val(a_bits).reshape(-1)
    k = a.size
    nbk = -(-k // block)
    q = np.zeros(k, np.int8)
    s = np.zeros(nbk, np.float32)
    with np.errstate(all="ignore"):
        for b in range(nbk):
            ab = a[b * block:(b + 1) * block]
            amax = np.abs(ab).max() if not np.isnan(ab).any() else F32(np.nan)
            amax = F32(amax)
            inv = F32(127.0) / amax if amax > 0 else F32(0.0)
            s[b] = amax / F32(127.0)
            r = np.rint((ab * inv).astype(np.float32))  # ties to even
            r = np.where(np.isnan(r), 0, np.clip(r, -128, 127))
            q[b * block:b * block + ab.size] = r.astype(np.int8)
    return q, s


def q2_values(codes, n, k, codebook) -> np.ndarray:
    c = np.asarray(codes, np.uint8)
    two = np.empty(c.size * 4, np.uint8)
    for i in range(4):
        two[i::4] = (c >> (2 * i)) & 3
    return np.asarray(codebook, np.int32)[two[: k * n]].reshape(k, n)


def q1_values(signs, layout, n, k) -> np.ndarray:
    bits = np.unpackbits(np.asarray(signs, np.uint8), bitorder="little")[: k * n]
    v = np.where(bits == 1, 1, -1).astype(np.int32)
    return v.reshape(n, k).T.copy() if layout == 0 else v.reshape(k, n)


def lowbit_matmul(a_bits, values, scales, n, k, block, m):
    """src/kernels/lowbit/matmul.rs:376-398.  values: k x n int32."""
    a = np.asarray(a_bits, np.uint16).reshape(m, k) if k else np.zeros((m, 0), np.uint16)
    nbk = -(-k // block)
    sc = f16_val(scales).reshape(n, nbk) if nbk else np.zeros((n, 0), np.float32)
    c = np.zeros((m, n), np.uint16)
    sums_all = np.zeros((m, n, nbk), np.int32)
    with np.errstate(all="ignore"):
        for i in range(m):
            q, s = quantize_row(a[i], block)
            total = np.zeros(n, np.float64)  # holds an f32 value exactly
            for b in range(nbk):
                sl = slice(b * block, min((b + 1) * block, k))
                sums = q[sl].astype(np.int32) @ values[sl]
                sums_all[i, :, b] = sums
                f = sums.astype(np.float32).astype(np.float64)
                p = (sc[:, b] * s[b]).astype(np.float32).astype(np.float64)
                # fused multiply-add rounded once to f32: f*p is exact in f64
                # (24+24 bits); the f64 sum can round, so use exact rational fallback
                total = _fma32(f, p, total)
            c[i] = f16_bits(total.astype(np.float32))
    return c, sums_all


def _fma32(f, p, t):
    """Correctly rounded f32 fma of f32-valued f64 arrays (exact via fractions when needed)."""
    from fractions import Fraction
    prod = f * p  # exact: two 24-bit significands
    s = prod + t
    out = s.astype(np.float32).astype(np.float64)
    # the f64 add may have rounded; re-do inexact lanes exactly
    err = (s - prod) - t
    bad = np.nonzero((err != 0) | ~np.isfinite(s))[0]
    for idx in bad:
        if not (np.isfinite(prod[idx]) and np.isfinite(t[idx])):
            continue
        exact = Fraction(float(prod[idx])) + Fraction(float(t[idx]))
        out[idx] = _round_fraction_f32(exact)
    return out


def _round_fraction_f32(x):
    from fractions import Fraction
    if x == 0:
        return 0.0
    lo = float(np.nextafter(np.float32(float(x)), np.float32(-np.inf)))
    cands = [lo, float(np.float32(float(x))), float(np.nextafter(np.float32(float(x)), np.float32(np.inf)))]
    best = min(cands, key=lambda c: (abs(Fraction(c) - x), int(np.float32(c).view(np.uint32)) & 1))
    return best


def lowbit_dequant(values, scales, n, k, block, is_q1) -> np.ndarray:
    """src/kernels/lowbit/matmul.rs:178-197."""
    nbk = -(-k // block)
    sc = f16_val(scales).reshape(n, nbk)
    s = sc[:, np.arange(k) // block].T  # k x n
    v = np.where(values > 0, s, -s) if is_q1 else (s * values.astype(np.float32)).astype(np.float32)
    return f16_bits(v)


def glu(both_bits, m, n, gate_kind=3) -> np.ndarray:
    """src/linear.rs:804-835, silu arm (f32 math)."""
    both = f16_val(both_bits).reshape(m, 2 * n)
    y = np.zeros((m, n), np.uint16)
    for c0 in range(0, n, 32):
        w = min(32, n - c0)
        g = both[:, 2 * c0:2 * c0 + w]
        u = both[:, 2 * c0 + w:2 * c0 + 2 * w]
        assert gate_kind == 3
        a = (g / (F32(1.0) + np.exp(-g, dtype=np.float32))).astype(np.float32)
        y[:, c0:c0 + w] = f16_bits((a * u).astype(np.float32))
    return y
