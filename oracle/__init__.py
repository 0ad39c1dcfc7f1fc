"""ctypes loader for the CPU oracle (oracle/oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, the smoke check and the CPU
baseline legs of bench.py.  The CUDA library never imports or links this.

All matrices are numpy arrays; 16-bit floats travel as uint16 bit patterns.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")


def build(force: bool = False) -> str:
    """Compile oracle.c with the committed Makefile (gcc, a second or two)."""
    src = os.path.join(_HERE, "oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "liboracle.so"], stdout=subprocess.DEVNULL)
    return _LIB_PATH


class EpNode(C.Structure):
    """Byte-identical to EpNode in csrc/epilogue.h:214-229 of the reference."""

    _fields_ = [("op", C.c_uint32), ("aux", C.c_uint32), ("scalar", C.c_float),
                ("ptr", C.c_void_p), ("ld", C.c_size_t)]


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        _lib = C.CDLL(build())
        _lib.orc_f16_to_f32.restype = C.c_float
        _lib.orc_f16_to_f32.argtypes = [C.c_uint16]
        _lib.orc_bf16_to_f32.restype = C.c_float
        _lib.orc_bf16_to_f32.argtypes = [C.c_uint16]
        _lib.orc_f64_to_f16.restype = C.c_uint16
        _lib.orc_f64_to_f16.argtypes = [C.c_double]
        _lib.orc_f32_to_f16.restype = C.c_uint16
        _lib.orc_f32_to_f16.argtypes = [C.c_float]
        _lib.orc_f32_to_bf16.restype = C.c_uint16
        _lib.orc_f32_to_bf16.argtypes = [C.c_float]
        _lib.orc_act_f64.restype = C.c_double
        _lib.orc_act_f64.argtypes = [C.c_uint32, C.c_double, C.c_double]
        for name in ("orc_q4_band_nibble_bytes", "orc_q2_band_code_bytes", "orc_q1_band_sign_bytes"):
            getattr(_lib, name).restype = C.c_size_t
            getattr(_lib, name).argtypes = [C.c_size_t, C.c_size_t]
        for name in ("orc_q4_band_scale_elems", "orc_lowbit_band_scale_elems"):
            getattr(_lib, name).restype = C.c_size_t
            getattr(_lib, name).argtypes = [C.c_size_t, C.c_size_t, C.c_size_t]
        _lib.orc_max_threads.restype = C.c_int
        _lib.orc_get_threads.restype = C.c_int
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _u16(a):
    a = np.ascontiguousarray(a)
    if a.dtype == np.float16:
        a = a.view(np.uint16)
    assert a.dtype == np.uint16, a.dtype
    return a


def set_threads(t: int) -> None:
    lib().orc_set_threads(C.c_int(int(t)))


def max_threads() -> int:
    return int(lib().orc_max_threads())


# ---- conversions -----------------------------------------------------------

def f32_to_f16_bits(x) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, np.uint16)
    lib().orc_f32_to_f16_slice(_p(x), _p(out), C.c_size_t(x.size))
    return out


def f32_to_bf16_bits(x) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, np.uint16)
    lib().orc_f32_to_bf16_slice(_p(x), _p(out), C.c_size_t(x.size))
    return out


def f16_bits_to_f32(x) -> np.ndarray:
    x = _u16(x)
    out = np.empty(x.shape, np.float32)
    lib().orc_f16_to_f32_slice(_p(x), _p(out), C.c_size_t(x.size))
    return out


def bf16_bits_to_f32(x) -> np.ndarray:
    return (np.ascontiguousarray(x, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def t_bits_to_f32(x, bf16: bool) -> np.ndarray:
    return bf16_bits_to_f32(x) if bf16 else f16_bits_to_f32(x)


# ---- epilogue node lists -----------------------------------------------------

class Nodes:
    """A resolved node array plus the numpy operands it points at (kept alive)."""

    def __init__(self, items):
        # items: list of (op, aux, scalar, operand ndarray(uint16) or None, ld)
        self.keep = []
        self.arr = (EpNode * max(1, len(items)))()
        self.n = len(items)
        for i, (op, aux, scalar, operand, ld) in enumerate(items):
            ptr = None
            if operand is not None:
                operand = _u16(operand)
                self.keep.append(operand)
                ptr = operand.ctypes.data
            self.arr[i] = EpNode(op, aux, float(scalar), ptr, ld)


# ---- Q4 ---------------------------------------------------------------------

def q4_quantize(w, layout: int, n: int, k: int, block: int = 32, affine: bool = False):
    w = np.ascontiguousarray(w, dtype=np.float32).reshape(-1)
    assert w.size == n * k
    nbk = -(-k // block)
    quants = np.zeros((k * n + 1) // 2, np.uint8)
    scales = np.zeros(n * nbk, np.uint16)
    mins = np.zeros(n * nbk, np.uint16) if affine else None
    lib().orc_q4_quantize(_p(w), C.c_int(layout), C.c_size_t(n), C.c_size_t(k), C.c_size_t(block),
                          C.c_int(int(affine)), _p(quants), _p(scales), _p(mins))
    return quants, scales, mins


def q4_dequant(quants, scales, mins, n, k, block=32, bf16=False) -> np.ndarray:
    out = np.zeros((k, n), np.uint16)
    lib().orc_q4_dequant(_p(quants), _p(scales), _p(mins), C.c_size_t(n), C.c_size_t(k),
                         C.c_size_t(block), C.c_int(int(bf16)), _p(out))
    return out


def gemm16(a, b, m, n, k, bf16=False) -> np.ndarray:
    a, b = _u16(a), _u16(b)
    c = np.zeros((m, n), np.uint16)
    lib().orc_gemm16(C.c_size_t(m), C.c_size_t(n), C.c_size_t(k), _p(c), _p(a), _p(b), C.c_int(int(bf16)))
    return c


def gemm16_f32(a, b, m, n, k, bf16=False) -> np.ndarray:
    """The dense product left in f32 (a tensor-parallel rank's partial sums)."""
    a, b = _u16(a), _u16(b)
    c = np.zeros((m, n), np.float32)
    lib().orc_gemm16_f32(C.c_size_t(m), C.c_size_t(n), C.c_size_t(k), _p(c), _p(a), _p(b), C.c_int(int(bf16)))
    return c


def apply_ep(c, m, n, nodes: Nodes, bf16=False) -> np.ndarray:
    c = _u16(c).copy()
    lib().orc_apply_ep(_p(c), C.c_size_t(m), C.c_size_t(n), nodes.arr, C.c_uint32(nodes.n), C.c_int(int(bf16)))
    return c


def matmul_q4(a, quants, scales, mins, n, k, block, m, nodes: Nodes | None = None, bf16=False,
              wdeq=None, first=0, rows=None) -> np.ndarray:
    a = _u16(a)
    c = np.zeros((m, n), np.uint16)
    rows = m - first if rows is None else rows
    lib().orc_matmul_q4(_p(a), _p(quants), _p(scales), _p(mins), C.c_size_t(n), C.c_size_t(k),
                        C.c_size_t(block), _p(c), C.c_size_t(m),
                        nodes.arr if nodes else None, C.c_uint32(nodes.n if nodes else 0),
                        C.c_int(int(bf16)), _p(wdeq), C.c_size_t(first), C.c_size_t(rows))
    return c


# ---- low-bit ----------------------------------------------------------------

def q2_quantize(w, layout, n, k, block=256, codebook=(-1, 0, 1, 0)):
    w = np.ascontiguousarray(w, dtype=np.float32).reshape(-1)
    nbk = -(-k // block)
    codes = np.zeros((k * n + 3) // 4, np.uint8)
    scales = np.zeros(n * nbk, np.uint16)
    cb = np.asarray(codebook, np.int8)
    rc = lib().orc_q2_quantize(_p(w), C.c_int(layout), C.c_size_t(n), C.c_size_t(k), C.c_size_t(block),
                               _p(cb), _p(codes), _p(scales))
    if rc != 0:
        raise ValueError("q2 codebook is all zeros")
    return codes, scales


def q1_quantize(w, layout, n, k, block=128):
    w = np.ascontiguousarray(w, dtype=np.float32).reshape(-1)
    nbk = -(-k // block)
    signs = np.zeros((k * n + 7) // 8, np.uint8)
    scales = np.zeros(n * nbk, np.uint16)
    lib().orc_q1_quantize(_p(w), C.c_int(layout), C.c_size_t(n), C.c_size_t(k), C.c_size_t(block),
                          _p(signs), _p(scales))
    return signs, scales


def quantize_row(a, block):
    a = _u16(a).reshape(-1)
    k = a.size
    nbk = -(-k // block)
    q = np.zeros(k, np.int8)
    s = np.zeros(nbk, np.float32)
    lib().orc_quantize_row(_p(a), C.c_size_t(k), C.c_size_t(block), _p(q), _p(s))
    return q, s


def lowbit_matmul(a, kind, wbits, layout, scales, codebook, n, k, block, m, debug=False):
    """kind 2 = 2-bit codes (+codebook), kind 1 = sign bits in `layout`.
    Returns c (m x n f16 bits) and, with debug, (q int8 m x k, sa f32 m x nbk,
    sums i32 m x n x nbk)."""
    a = _u16(a)
    nbk = -(-k // block)
    c = np.zeros((m, n), np.uint16)
    cb = np.asarray(codebook if codebook is not None else (0, 0, 0, 0), np.int8)
    q = np.zeros((m, k), np.int8) if debug else None
    sa = np.zeros((m, nbk), np.float32) if debug else None
    sums = np.zeros((m, n, nbk), np.int32) if debug else None
    lib().orc_lowbit_matmul(_p(a), C.c_int(kind), _p(wbits), C.c_int(layout), _p(_u16(scales)), _p(cb),
                            C.c_size_t(n), C.c_size_t(k), C.c_size_t(block), _p(c), C.c_size_t(m),
                            _p(q), _p(sa), _p(sums))
    return (c, q, sa, sums) if debug else c


def lowbit_dequant(kind, wbits, layout, scales, codebook, n, k, block) -> np.ndarray:
    out = np.zeros((k, n), np.uint16)
    cb = np.asarray(codebook if codebook is not None else (0, 0, 0, 0), np.int8)
    lib().orc_lowbit_dequant(C.c_int(kind), _p(wbits), C.c_int(layout), _p(_u16(scales)), _p(cb),
                             C.c_size_t(n), C.c_size_t(k), C.c_size_t(block), _p(out))
    return out


# ---- MLP pieces ---------------------------------------------------------------

def glu(both, m, n, gate_kind=3) -> np.ndarray:
    both = _u16(both)
    y = np.zeros((m, n), np.uint16)
    lib().orc_glu(_p(y), _p(both), C.c_size_t(m), C.c_size_t(n), C.c_int(gate_kind))
    return y


def add_f16(src, dst) -> None:
    src = _u16(src)
    assert dst.dtype == np.float32 and dst.flags.c_contiguous
    lib().orc_add_f16(_p(src), _p(dst), C.c_size_t(src.size))


def norm_rows(x, weight, bias, eps: float, rms: bool):
    """layer_norm / rms_norm (src/nn.rs:73-161) over every row: (f16 bits, f32) outputs."""
    x = np.ascontiguousarray(x, np.float32)
    weight = np.ascontiguousarray(weight, np.float32)
    dim = weight.size
    rows = x.size // dim
    b = None if bias is None else np.ascontiguousarray(bias, np.float32)
    y16 = np.zeros((rows, dim), np.uint16)
    y32 = np.zeros((rows, dim), np.float32)
    lib().orc_norm_rows(_p(x), _p(weight), _p(b) if b is not None else None, C.c_float(eps), C.c_int(1 if rms else 0),
                        C.c_size_t(rows), C.c_size_t(dim), _p(y16), _p(y32))
    return y16, y32


def rms_scales(x, k: int, eps: float) -> np.ndarray:
    """rms_scales (src/nn.rs:234-248): f16 bits of 1 / sqrt(mean(x_i^2) + eps) per k-wide row of f16 x."""
    x = _u16(x)
    rows = x.size // k
    out = np.zeros(rows, np.uint16)
    lib().orc_rms_scales(_p(x), C.c_size_t(rows), C.c_size_t(k), C.c_float(eps), _p(out))
    return out


def interleave(g, u, n, k) -> np.ndarray:
    """g, u: k x n row-major (InOut) arrays of one dtype -> k x 2n."""
    g, u = np.ascontiguousarray(g), np.ascontiguousarray(u)
    out = np.zeros((k, 2 * n), g.dtype)
    lib().orc_interleave(_p(g), _p(u), C.c_size_t(n), C.c_size_t(k), C.c_size_t(g.itemsize), _p(out))
    return out


def mlp_accumulate(x, y, m, d_model, hidden, gu_quants, gu_scales, dn_quants, dn_scales, block=32,
                   gate_kind=3, first=0, rows=None) -> None:
    x = _u16(x)
    rows = m - first if rows is None else rows
    lib().orc_mlp_accumulate(_p(x), _p(y), C.c_size_t(m), C.c_size_t(d_model), C.c_size_t(hidden),
                             _p(gu_quants), _p(gu_scales), _p(dn_quants), _p(dn_scales),
                             C.c_size_t(block), C.c_int(gate_kind), C.c_size_t(first), C.c_size_t(rows))


# ---- the reference's own packed layouts (drop-in entry point tests) ----------

def q4_pack_band(quants, scales, mins, n, k, block):
    L = lib()
    nib = np.zeros(L.orc_q4_band_nibble_bytes(n, k), np.uint8)
    ne = L.orc_q4_band_scale_elems(n, k, block)
    sc = np.zeros(ne, np.uint16)
    mn = np.zeros(ne, np.uint16) if mins is not None else None
    L.orc_q4_pack_band(_p(quants), _p(scales), _p(mins), C.c_size_t(n), C.c_size_t(k), C.c_size_t(block),
                       _p(nib), _p(sc), _p(mn))
    return nib, sc, mn


def q2_pack_band(codes, scales, n, k, block):
    L = lib()
    packed = np.zeros(L.orc_q2_band_code_bytes(n, k), np.uint8)
    sc = np.zeros(L.orc_lowbit_band_scale_elems(n, k, block), np.uint16)
    L.orc_q2_pack_band(_p(codes), _p(_u16(scales)), C.c_size_t(n), C.c_size_t(k), C.c_size_t(block),
                       _p(packed), _p(sc))
    return packed, sc


def q1_pack_band(signs, layout, scales, n, k, block):
    L = lib()
    packed = np.zeros(L.orc_q1_band_sign_bytes(n, k), np.uint8)
    sc = np.zeros(L.orc_lowbit_band_scale_elems(n, k, block), np.uint16)
    L.orc_q1_pack_band(_p(signs), C.c_int(layout), _p(_u16(scales)), C.c_size_t(n), C.c_size_t(k),
                       C.c_size_t(block), _p(packed), _p(sc))
    return packed, sc


def attention_kv_causal(q, k, v, start: int, rows: int, heads: int, kv_heads: int, head_dim: int, scale: float) -> np.ndarray:
    """attention_kv_causal_f16, portable arm (src/kernels/kv_attention.rs:155-331): q f32 [rows][heads][head_dim], k / v
    f16 bits [start + rows][kv_heads * head_dim]; returns out f32 like q."""
    q = np.ascontiguousarray(q, np.float32)
    k, v = _u16(k), _u16(v)
    out = np.zeros(rows * heads * head_dim, np.float32)
    lib().orc_attention_kv_causal(_p(q), _p(k), _p(v), C.c_size_t(start), C.c_size_t(rows), C.c_size_t(heads),
                                  C.c_size_t(kv_heads), C.c_size_t(head_dim), C.c_float(scale), _p(out))
    return out.reshape(rows, heads * head_dim)
