"""Host-side mirror of the reference's Rust API for the weight-quantised path.

Same names, argument meaning and error behaviour as the reference
(src/kernels/q4, src/kernels/lowbit, src/epilogue/graph.rs, src/linear.rs,
src/mlp.rs), over the C ABI of include/smeg_api.h.  Where the reference panics
on inconsistent lengths, these raise AssertionError with the same message.

Two kinds of buffers are accepted everywhere:
  * numpy arrays (host memory): the call copies in, runs on the GPU, copies out;
  * torch CUDA tensors: the call only enqueues work on torch's current stream
    (device-resident path -- the one the benchmarks time).
f16 values are numpy float16 / torch.float16; bf16 values are numpy uint16 bit
patterns / torch.bfloat16.
"""
from __future__ import annotations

import ctypes as C
from enum import IntEnum

import numpy as np

from ._lib import EpDesc16, EpNode, SmegError, check, lib

try:  # torch is plumbing for device memory and streams only
    import torch
except Exception:  # pragma: no cover
    torch = None


class WeightLayout(IntEnum):
    """src/layout.rs: OutIn = w[j*k + d] (one row per output), InOut = w[d*n + j]."""

    OutIn = 0
    InOut = 1


class Gate(IntEnum):
    """src/linear.rs Gate: the activation on the gate half."""

    Gelu = 2
    Silu = 3


Q4_BLOCK = 32
Q2_BLOCK = 256
Q2_TERNARY = (-1, 0, 1, 0)


class Q4Params:
    """src/kernels/q4/mod.rs:55-103."""

    def __init__(self, block: int = Q4_BLOCK):
        assert block != 0 and block & (block - 1) == 0, f"q4 block size must be a power of two, got {block}"
        self._block, self._affine = block, False

    def affine(self) -> "Q4Params":
        p = Q4Params(self._block)
        p._affine = True
        return p

    def block(self) -> int:
        return self._block

    def is_affine(self) -> bool:
        return self._affine


class Q2Params:
    """src/kernels/lowbit/mod.rs:38-94."""

    def __init__(self, block: int = Q2_BLOCK):
        assert block & (block - 1) == 0 and 16 <= block <= 1 << 16, \
            f"q2 block size must be a power of two from 16 to 65536, got {block}"
        self._block, self._codebook = block, Q2_TERNARY

    def with_codebook(self, values) -> "Q2Params":
        p = Q2Params(self._block)
        p._codebook = tuple(int(v) for v in values)
        assert len(p._codebook) == 4
        return p

    def block(self) -> int:
        return self._block

    def codebook(self):
        return self._codebook


# --------------------------------------------------------------------------- buffers

def _is_torch(x) -> bool:
    return torch is not None and isinstance(x, torch.Tensor)


def _np_bits(x, what: str) -> np.ndarray:
    """numpy f16 / uint16 array -> contiguous uint16 view."""
    x = np.ascontiguousarray(x)
    if x.dtype == np.float16:
        return x.view(np.uint16)
    assert x.dtype == np.uint16, f"{what}: expected float16 or uint16 bit patterns, got {x.dtype}"
    return x


def _ptr(x) -> int:
    if x is None:
        return 0
    if _is_torch(x):
        return x.data_ptr()
    return x.ctypes.data


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _numel(x) -> int:
    return x.numel() if _is_torch(x) else x.size


# --------------------------------------------------------------------------- weights

class Q4Weights:
    """4-bit weights resident on the GPU in the prepacked unit layout.
    Mirrors Q4Weights (src/kernels/q4/weights.rs:26-271, quantize.rs:29-81)."""

    def __init__(self, handle, params: Q4Params):
        self._h, self._params = handle, params

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            lib().smeg_q4_destroy(h)

    @staticmethod
    def new(quants, scales, n: int, k: int) -> "Q4Weights":
        return Q4Weights.with_params(quants, scales, None, n, k, Q4Params())

    @staticmethod
    def with_params(quants, scales, mins, n: int, k: int, p: Q4Params) -> "Q4Weights":
        quants = np.ascontiguousarray(quants, dtype=np.uint8)
        scales = _np_bits(scales, "scales")
        nbk = -(-k // p.block())
        assert quants.size == (k * n + 1) // 2, "quants is ceil(k*n/2) bytes"
        assert scales.size == n * nbk, "scales is n*ceil(k/block)"
        if p.is_affine():
            assert mins is not None, "Q4Form::Affine requires a mins array"
            mins = _np_bits(mins, "mins")
            assert mins.size == n * nbk, "mins is n*ceil(k/block)"
        else:
            assert mins is None, "Q4Form::Scale takes no mins array"
        h = C.c_void_p()
        check("smeg_q4_create", lib().smeg_q4_create(_ptr(quants), _ptr(scales), _ptr(mins), n, k, p.block(), C.byref(h)))
        return Q4Weights(h, p)

    @staticmethod
    def quantize(w, layout: WeightLayout, n: int, k: int, p: Q4Params | None = None) -> "Q4Weights":
        p = p or Q4Params()
        w = np.ascontiguousarray(w, dtype=np.float32).reshape(-1)
        assert w.size == n * k, "w holds n * k weights"
        h = C.c_void_p()
        check("smeg_q4_quantize", lib().smeg_q4_quantize(_ptr(w), int(layout), n, k, p.block(), int(p.is_affine()), C.byref(h)))
        return Q4Weights(h, p)

    @staticmethod
    def from_band(nibbles, scales, n: int, k: int, p: Q4Params | None = None) -> "Q4Weights":
        """From the band-major arrays the reference's own Q4Weights holds."""
        p = p or Q4Params()
        nibbles = np.ascontiguousarray(nibbles, dtype=np.uint8)
        scales = _np_bits(scales, "scales")
        h = C.c_void_p()
        check("smeg_q4_from_band", lib().smeg_q4_from_band(_ptr(nibbles), _ptr(scales), None, n, k, p.block(), C.byref(h)))
        return Q4Weights(h, p)

    def n(self) -> int:
        return lib().smeg_q4_n(self._h)

    def k(self) -> int:
        return lib().smeg_q4_k(self._h)

    def params(self) -> Q4Params:
        return self._params

    def device_bytes(self) -> int:
        return lib().smeg_q4_device_bytes(self._h)

    def unpack(self):
        """(quants, scales) in the constructor's input layout, read back from the device."""
        n, k = self.n(), self.k()
        nbk = -(-k // self._params.block())
        quants = np.zeros((k * n + 1) // 2, np.uint8)
        scales = np.zeros(n * nbk, np.uint16)
        check("smeg_q4_unpack", lib().smeg_q4_unpack(self._h, _ptr(quants), _ptr(scales)))
        return quants, scales


class _LowbitWeights:
    def __init__(self, handle):
        self._h = handle

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            lib().smeg_lowbit_destroy(h)

    def n(self) -> int:
        return lib().smeg_lowbit_n(self._h)

    def k(self) -> int:
        return lib().smeg_lowbit_k(self._h)

    def block(self) -> int:
        return lib().smeg_lowbit_block(self._h)

    def device_bytes(self) -> int:
        return lib().smeg_lowbit_device_bytes(self._h)

    def unpack(self):
        n, k = self.n(), self.k()
        nbk = -(-k // self.block())
        per = 4 if lib().smeg_lowbit_bits(self._h) == 2 else 8
        bits = np.zeros((k * n + per - 1) // per, np.uint8)
        scales = np.zeros(n * nbk, np.uint16)
        check("smeg_lowbit_unpack", lib().smeg_lowbit_unpack(self._h, _ptr(bits), _ptr(scales)))
        return bits, scales


class Q2Weights(_LowbitWeights):
    """2-bit weights (src/kernels/lowbit/q2.rs:31-186)."""

    def __init__(self, handle, params: Q2Params):
        super().__init__(handle)
        self._params = params

    @staticmethod
    def new(codes, scales, n: int, k: int, p: Q2Params | None = None) -> "Q2Weights":
        p = p or Q2Params()
        codes = np.ascontiguousarray(codes, dtype=np.uint8)
        scales = _np_bits(scales, "scales")
        assert codes.size == (k * n + 3) // 4, "codes is ceil(k*n/4) bytes"
        assert scales.size == n * (-(-k // p.block())), "scales is n*ceil(k/block)"
        cb = np.asarray(p.codebook(), np.int8)
        h = C.c_void_p()
        check("smeg_q2_create", lib().smeg_q2_create(_ptr(codes), _ptr(scales), n, k, p.block(), _ptr(cb), C.byref(h)))
        return Q2Weights(h, p)

    @staticmethod
    def quantize(w, layout: WeightLayout, n: int, k: int, p: Q2Params | None = None) -> "Q2Weights":
        p = p or Q2Params()
        w = np.ascontiguousarray(w, dtype=np.float32).reshape(-1)
        assert w.size == n * k, "w holds n * k weights"
        cb = np.asarray(p.codebook(), np.int8)
        assert np.abs(cb.astype(np.int32)).max() > 0, "q2 codebook is all zeros"
        h = C.c_void_p()
        check("smeg_q2_quantize", lib().smeg_q2_quantize(_ptr(w), int(layout), n, k, p.block(), _ptr(cb), C.byref(h)))
        return Q2Weights(h, p)

    @staticmethod
    def from_band(codes, scales, n: int, k: int, p: Q2Params | None = None) -> "Q2Weights":
        p = p or Q2Params()
        codes = np.ascontiguousarray(codes, dtype=np.uint8)
        scales = _np_bits(scales, "scales")
        cb = np.asarray(p.codebook(), np.int8)
        h = C.c_void_p()
        check("smeg_q2_from_band", lib().smeg_q2_from_band(_ptr(codes), _ptr(scales), n, k, p.block(), _ptr(cb), C.byref(h)))
        return Q2Weights(h, p)

    def params(self) -> Q2Params:
        return self._params


class Q1Weights(_LowbitWeights):
    """1-bit weights (src/kernels/lowbit/q1.rs:23-233)."""

    @staticmethod
    def new(signs, scales, layout: WeightLayout, n: int, k: int, block: int) -> "Q1Weights":
        assert block & (block - 1) == 0 and 16 <= block <= 1 << 16, \
            f"q1 block size must be a power of two from 16 to 65536, got {block}"
        signs = np.ascontiguousarray(signs, dtype=np.uint8)
        scales = _np_bits(scales, "scales")
        assert signs.size == (k * n + 7) // 8, "signs is ceil(k*n/8) bytes"
        assert scales.size == n * (-(-k // block)), "scales is n*ceil(k/block)"
        h = C.c_void_p()
        check("smeg_q1_create", lib().smeg_q1_create(_ptr(signs), _ptr(scales), int(layout), n, k, block, C.byref(h)))
        return Q1Weights(h)

    @staticmethod
    def quantize(w, layout: WeightLayout, n: int, k: int, block: int) -> "Q1Weights":
        assert block & (block - 1) == 0 and 16 <= block <= 1 << 16, \
            f"q1 block size must be a power of two from 16 to 65536, got {block}"
        w = np.ascontiguousarray(w, dtype=np.float32).reshape(-1)
        assert w.size == n * k, "w holds n * k weights"
        h = C.c_void_p()
        check("smeg_q1_quantize", lib().smeg_q1_quantize(_ptr(w), int(layout), n, k, block, C.byref(h)))
        return Q1Weights(h)

    @staticmethod
    def from_band(signs, scales, n: int, k: int, block: int) -> "Q1Weights":
        signs = np.ascontiguousarray(signs, dtype=np.uint8)
        scales = _np_bits(scales, "scales")
        h = C.c_void_p()
        check("smeg_q1_from_band", lib().smeg_q1_from_band(_ptr(signs), _ptr(scales), n, k, block, C.byref(h)))
        return Q1Weights(h)

    @staticmethod
    def interleave(gate: "Q1Weights", up: "Q1Weights") -> "Q1Weights":
        """gate and up as one 2n-column set, 32 columns at a time
        (Q1Weights::interleave, src/kernels/lowbit/q1.rs:149-186)."""
        n, k, block = gate.n(), gate.k(), gate.block()
        assert (up.n(), up.k(), up.block()) == (n, k, block), "gate and up have the same shape and block size"
        nbk = -(-k // block)
        gs, gsc = gate.unpack()
        us, usc = up.unpack()
        gb = np.unpackbits(gs, bitorder="little")[: n * k].reshape(n, k)
        ub = np.unpackbits(us, bitorder="little")[: n * k].reshape(n, k)
        gsc, usc = gsc.reshape(n, nbk), usc.reshape(n, nbk)
        rows, srows = [], []
        for c0 in range(0, n, 32):
            c1 = min(c0 + 32, n)
            rows += [gb[c0:c1], ub[c0:c1]]
            srows += [gsc[c0:c1], usc[c0:c1]]
        bits = np.packbits(np.concatenate(rows).reshape(-1), bitorder="little")
        return Q1Weights.new(bits, np.concatenate(srows).reshape(-1), WeightLayout.OutIn, 2 * n, k, block)


# --------------------------------------------------------------------------- epilogue

_OPS = dict(add_scalar=0, mul_scalar=1, add_row=2, mul_row=3, add_col=4, mul_col=5, add_tensor=6, mul_tensor=7,
            act=8, max=9, min=10, sub_scalar=11, sub_row=12, sub_col=13, sub_tensor=14, div_scalar=15, div_row=16,
            div_col=17, div_tensor=18, max_row=19, max_col=20, max_tensor=21, min_row=22, min_col=23, min_tensor=24)
_ROW_OPS = {2, 3, 12, 16, 19, 22}
_COL_OPS = {4, 5, 13, 17, 20, 23}
_TENSOR_OPS = {6, 7, 14, 18, 21, 24}
_ACTS = dict(relu=1, gelu=2, silu=3, tanh=4, sigmoid=5, leaky_relu=6, relu6=7, hardsigmoid=8, hardswish=9, abs=10,
             neg=11, square=12, sign=13, sqrt=14, softsign=15, recip=16, rsqrt=17, exp=18, log=19, elu=20, selu=21,
             softplus=22, mish=23, gelu_exact=24)


def _round_scalar(v: float, dtype: str) -> float:
    """Scalars are given in the element type T and carried as f32
    (push_scalar, src/epilogue/graph.rs:84-95)."""
    if dtype == "bf16":
        u = np.asarray([v], np.float32).view(np.uint32).astype(np.uint64)
        u = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
        return float(u.astype(np.uint32).view(np.float32)[0])
    with np.errstate(over="ignore"):
        return float(np.float32(np.float16(v)))


class Epilogue:
    """The fused epilogue as an ordered op-graph (src/epilogue/graph.rs:33-432).

    Methods push nodes in call order, except relu / gelu / silu / tanh / sigmoid,
    which set a TRAILING activation applied last whatever the call order
    (graph.rs:38-42,185-223)."""

    def __init__(self, dtype: str = "f16"):
        assert dtype in ("f16", "bf16")
        self.dtype = dtype
        self.nodes = []   # (op, aux, scalar, operand, ld)
        self.act = None

    @staticmethod
    def new(dtype: str = "f16") -> "Epilogue":
        return Epilogue(dtype)

    def _push(self, op, aux=0, scalar=0.0, operand=None, ld=0):
        self.nodes.append((op, aux, float(scalar), operand, int(ld)))
        return self

    # scalar ops
    def add_scalar(self, v): return self._push(0, scalar=_round_scalar(v, self.dtype))
    def mul_scalar(self, v): return self._push(1, scalar=_round_scalar(v, self.dtype))
    def sub_scalar(self, v): return self._push(11, scalar=_round_scalar(v, self.dtype))
    def div_scalar(self, v): return self._push(15, scalar=_round_scalar(v, self.dtype))
    def max(self, lo): return self._push(9, scalar=_round_scalar(lo, self.dtype))
    def min(self, hi): return self._push(10, scalar=_round_scalar(hi, self.dtype))
    def clamp(self, lo, hi): return self.max(lo).min(hi)
    # vector / tensor ops
    def add_row(self, v): return self._push(2, operand=v)
    def mul_row(self, v): return self._push(3, operand=v)
    def sub_row(self, v): return self._push(12, operand=v)
    def div_row(self, v): return self._push(16, operand=v)
    def max_row(self, v): return self._push(19, operand=v)
    def min_row(self, v): return self._push(22, operand=v)
    def add_col(self, v): return self._push(4, operand=v)
    def mul_col(self, v): return self._push(5, operand=v)
    def sub_col(self, v): return self._push(13, operand=v)
    def div_col(self, v): return self._push(17, operand=v)
    def max_col(self, v): return self._push(20, operand=v)
    def min_col(self, v): return self._push(23, operand=v)
    def add_tensor(self, v): return self._push(6, operand=v)
    def mul_tensor(self, v): return self._push(7, operand=v)
    def sub_tensor(self, v): return self._push(14, operand=v)
    def div_tensor(self, v): return self._push(18, operand=v)
    def max_tensor(self, v): return self._push(21, operand=v)
    def min_tensor(self, v): return self._push(24, operand=v)
    def add_tensor_strided(self, v, ld): return self._push(6, operand=v, ld=ld)
    def mul_tensor_strided(self, v, ld): return self._push(7, operand=v, ld=ld)
    def sub_tensor_strided(self, v, ld): return self._push(14, operand=v, ld=ld)
    def div_tensor_strided(self, v, ld): return self._push(18, operand=v, ld=ld)
    def max_tensor_strided(self, v, ld): return self._push(21, operand=v, ld=ld)
    def min_tensor_strided(self, v, ld): return self._push(24, operand=v, ld=ld)
    # trailing activations
    def relu(self): self.act = 1; return self
    def gelu(self): self.act = 2; return self
    def silu(self): self.act = 3; return self
    def tanh(self): self.act = 4; return self
    def sigmoid(self): self.act = 5; return self
    # in-order activations
    def leaky_relu(self, alpha): return self._push(8, aux=6, scalar=np.float32(alpha))
    def relu6(self): return self._push(8, aux=7)
    def hardsigmoid(self): return self._push(8, aux=8)
    def hardswish(self): return self._push(8, aux=9)
    def abs(self): return self._push(8, aux=10)
    def neg(self): return self._push(8, aux=11)
    def square(self): return self._push(8, aux=12)
    def sign(self): return self._push(8, aux=13)
    def sqrt(self): return self._push(8, aux=14)
    def softsign(self): return self._push(8, aux=15)
    def recip(self): return self._push(8, aux=16)
    def rsqrt(self): return self._push(8, aux=17)
    def exp(self): return self._push(8, aux=18)
    def log(self): return self._push(8, aux=19)
    def elu(self, alpha): return self._push(8, aux=20, scalar=np.float32(alpha))
    def selu(self): return self._push(8, aux=21)
    def softplus(self): return self._push(8, aux=22)
    def mish(self): return self._push(8, aux=23)
    def gelu_exact(self): return self._push(8, aux=24)

    def with_leading(self, lead: "Epilogue") -> "Epilogue":
        """lead's nodes ahead of this graph's, this graph's activation kept
        (with_leading, src/epilogue/graph.rs:149-157)."""
        out = Epilogue(self.dtype)
        out.nodes = list(lead.nodes) + list(self.nodes)
        out.act = self.act
        return out

    def resolved(self):
        """Node list as the FFI sees it (resolve_nodes, src/exec/scalar.rs:28-53)."""
        items = list(self.nodes)
        if self.act is not None:
            items.append((8, self.act, 0.0, None, 0))
        return items

    def validate(self, m: int, n: int) -> None:
        """validate_ep, src/exec/guard.rs:112-150."""
        for op, _aux, _s, operand, ld in self.nodes:
            if op in _ROW_OPS:
                assert _numel(operand) == m, "row operand is per-M (length m)"
            elif op in _COL_OPS:
                assert _numel(operand) == n, "col operand is per-N (length n)"
            elif op in _TENSOR_OPS:
                ldv = ld or n
                assert ldv >= n, "tensor row stride must be >= n"
                assert m == 0 or _numel(operand) >= (m - 1) * ldv + n, "tensor must hold m*n elements (stride ld)"

    def _desc(self, device: bool):
        """(EpDesc16 or None, keep-alive list) with host or device operand pointers."""
        items = self.resolved()
        if not items:
            return None, []
        arr = (EpNode * len(items))()
        keep = [arr]
        for i, (op, aux, scalar, operand, ld) in enumerate(items):
            p = None
            if operand is not None:
                if device:
                    assert _is_torch(operand) and operand.is_cuda, "device call needs CUDA tensor operands"
                    operand = operand.contiguous()
                    want = torch.bfloat16 if self.dtype == "bf16" else torch.float16
                    assert operand.dtype == want, f"operand dtype {operand.dtype} != {want}"
                else:
                    assert not _is_torch(operand), "host call needs numpy operands"
                    operand = _np_bits(operand, "epilogue operand")
                keep.append(operand)
                p = _ptr(operand)
            arr[i] = EpNode(op, aux, scalar, p, ld)
        desc = EpDesc16(len(items), arr)
        keep.append(desc)
        return desc, keep


# --------------------------------------------------------------------------- matmuls

def _check_io(a, c, m, n, k):
    assert _numel(a) == m * k, "a is m*k"
    assert _numel(c) == m * n, "c is m*n"


def _run_q4(a, w: Q4Weights, c, m: int, ep: Epilogue | None, bf16: bool) -> None:
    n, k = w.n(), w.k()
    _check_io(a, c, m, n, k)
    if ep is not None:
        assert ep.dtype == ("bf16" if bf16 else "f16")
        ep.validate(m, n)
    if m == 0 or n == 0:
        return
    L = lib()
    if _is_torch(a):
        assert a.is_cuda and c.is_cuda and a.is_contiguous() and c.is_contiguous()
        want = torch.bfloat16 if bf16 else torch.float16
        assert a.dtype == want and c.dtype == want
        desc, keep = ep._desc(True) if ep is not None else (None, [])
        fn = L.smeg_matmul_q4_bf16_dev if bf16 else L.smeg_matmul_q4_f16_dev
        check(fn.__name__, fn(w._h, _ptr(a), _ptr(c), m, C.byref(desc) if desc else None, _stream()))
        del keep
    else:
        ab = _np_bits(a, "a")
        assert isinstance(c, np.ndarray) and c.flags.c_contiguous and c.dtype in (np.float16, np.uint16)
        desc, keep = ep._desc(False) if ep is not None else (None, [])
        fn = L.smeg_matmul_q4_bf16 if bf16 else L.smeg_matmul_q4_f16
        check(fn.__name__, fn(w._h, _ptr(ab), _ptr(c), m, C.byref(desc) if desc else None))
        del keep


def matmul_q4(a, w: Q4Weights, c, m: int) -> None:
    """C = A @ dequant(W), f16 (matmul_q4, src/kernels/q4/matmul.rs:33-35)."""
    _run_q4(a, w, c, m, None, False)


def matmul_q4_ep(a, w: Q4Weights, c, m: int, ep: Epilogue) -> None:
    """matmul_q4_ep, src/kernels/q4/matmul.rs:21-23."""
    _run_q4(a, w, c, m, ep, False)


def matmul_q4_bf16(a, w: Q4Weights, c, m: int) -> None:
    """matmul_q4_bf16, src/kernels/q4/matmul.rs:178-186."""
    _run_q4(a, w, c, m, None, True)


def matmul_q4_bf16_ep(a, w: Q4Weights, c, m: int, ep: Epilogue) -> None:
    """matmul_q4_bf16_ep, src/kernels/q4/matmul.rs:188-196."""
    _run_q4(a, w, c, m, ep, True)


def _run_lowbit(a, w: _LowbitWeights, c, m: int, ep: Epilogue | None, mopa: bool = False) -> None:
    n, k = w.n(), w.k()
    _check_io(a, c, m, n, k)
    if ep is not None:
        assert ep.dtype == "f16"
        ep.validate(m, n)
    if m == 0 or n == 0:
        return
    L = lib()
    if _is_torch(a):
        assert a.is_cuda and c.is_cuda and a.is_contiguous() and c.is_contiguous()
        assert a.dtype == torch.float16 and c.dtype == torch.float16
        desc, keep = ep._desc(True) if ep is not None else (None, [])
        name = "smeg_matmul_lowbit_f16_dev" if mopa else "smeg_matmul_lowbit_dev"
        check(name, getattr(L, name)(w._h, _ptr(a), _ptr(c), m, C.byref(desc) if desc else None, _stream()))
        del keep
    else:
        ab = _np_bits(a, "a")
        assert isinstance(c, np.ndarray) and c.flags.c_contiguous and c.dtype in (np.float16, np.uint16)
        desc, keep = ep._desc(False) if ep is not None else (None, [])
        name = "smeg_matmul_lowbit_f16" if mopa else "smeg_matmul_lowbit"
        check(name, getattr(L, name)(w._h, _ptr(ab), _ptr(c), m, C.byref(desc) if desc else None))
        del keep


def matmul_q2(a, w: Q2Weights, c, m: int) -> None:
    """matmul_q2, src/kernels/lowbit/matmul.rs:38-40."""
    _run_lowbit(a, w, c, m, None)


def matmul_q2_ep(a, w: Q2Weights, c, m: int, ep: Epilogue) -> None:
    """matmul_q2_ep, src/kernels/lowbit/matmul.rs:48-50."""
    _run_lowbit(a, w, c, m, ep)


def matmul_q1(a, w: Q1Weights, c, m: int) -> None:
    """matmul_q1, src/kernels/lowbit/matmul.rs:70-72."""
    _run_lowbit(a, w, c, m, None)


def matmul_q1_ep(a, w: Q1Weights, c, m: int, ep: Epilogue) -> None:
    """matmul_q1_ep, src/kernels/lowbit/matmul.rs:79-81."""
    _run_lowbit(a, w, c, m, ep)


# --------------------------------------------------------------------------- dense weights: the Gemm builder

class Packed:
    """Pre-packed dense weights (Packed<f16> / Packed<bf16>): B is k x n row-major in the element
    type; the device copy is K-major for the tensor cores.  Built by prepack_f16 / prepack_bf16."""

    def __init__(self, h, n, k, dtype):
        self._h, self.n, self.k, self.dtype = h, n, k, dtype

    def __del__(self):
        try:
            if self._h:
                lib().smeg_dense_destroy(self._h)
                self._h = None
        except Exception:
            pass


def _prepack(b, n: int, k: int, dtype: str) -> Packed:
    bits = _np_bits(b, "b")
    assert bits.size == k * n, "b is k*n (row-major)"
    h = C.c_void_p()
    check("smeg_dense_create", lib().smeg_dense_create(_ptr(bits), n, k, 1 if dtype == "bf16" else 0, C.byref(h)))
    return Packed(h, n, k, dtype)


def prepack_f16(b, n: int, k: int) -> Packed:
    """prepack_f16, src/kernels/f16.rs:212: b is the k x n row-major f16 matrix."""
    return _prepack(b, n, k, "f16")


def prepack_bf16(b, n: int, k: int) -> Packed:
    """prepack_bf16, src/kernels/bf16.rs: b holds bf16 bit patterns (uint16), k x n row-major."""
    return _prepack(b, n, k, "bf16")


class Gemm:
    """Gemm::new(a, &packed, m).add_col(bias).gelu().run(&mut c) (src/exec/builder.rs:220-227,
    428-813): C = ep( T(beta * (A @ B)) ).  Every op method of Epilogue is available with the same
    meaning (and the same trailing-activation rule), plus beta(), col_major_output() and run()."""

    def __init__(self, a, packed: Packed, m: int):
        self._a, self._p, self._m = a, packed, m
        self._beta = 1.0
        self._col_major = False
        self._ep = Epilogue(packed.dtype)

    @staticmethod
    def new(a, packed: Packed, m: int) -> "Gemm":
        return Gemm(a, packed, m)

    def __getattr__(self, name):
        fn = getattr(Epilogue, name, None)
        if fn is None or name.startswith("_") or name in ("new", "resolved", "validate", "with_leading"):
            raise AttributeError(name)

        def forward(*args):
            getattr(self._ep, name)(*args)
            return self
        return forward

    def beta(self, beta: float) -> "Gemm":
        self._beta = _round_scalar(beta, self._p.dtype)
        return self

    def col_major_output(self) -> "Gemm":
        self._col_major = True
        return self

    def run(self, c) -> None:
        m, n, k = self._m, self._p.n, self._p.k
        _check_io(self._a, c, m, n, k)
        self._ep.validate(m, n)
        if m == 0 or n == 0:
            return
        if self._p.dtype == "bf16":
            beta_bits = int(np.asarray([self._beta], np.float32).view(np.uint32)[0] >> 16)
        else:
            beta_bits = int(np.asarray([self._beta], np.float16).view(np.uint16)[0])
        L = lib()
        has_ep = bool(self._ep.nodes) or self._ep.act is not None
        if _is_torch(self._a):
            a = self._a
            assert a.is_cuda and c.is_cuda and a.is_contiguous() and c.is_contiguous()
            desc, keep = self._ep._desc(True) if has_ep else (None, [])
            check("smeg_gemm_dense_dev", L.smeg_gemm_dense_dev(self._p._h, _ptr(a), _ptr(c), m, beta_bits, int(self._col_major),
                                                               C.byref(desc) if desc else None, _stream()))
            del keep
        else:
            ab = _np_bits(self._a, "a")
            desc, keep = self._ep._desc(False) if has_ep else (None, [])
            check("smeg_gemm_dense", L.smeg_gemm_dense(self._p._h, _ptr(ab), _ptr(c), m, beta_bits, int(self._col_major),
                                                       C.byref(desc) if desc else None))
            del keep


def matmul_q2_mopa(a, w: Q2Weights, c, m: int) -> None:
    """matmul_q2_mopa, src/kernels/lowbit/matmul.rs:100-102: f16 activations, no int8 step."""
    _run_lowbit(a, w, c, m, None, mopa=True)


def matmul_q2_mopa_ep(a, w: Q2Weights, c, m: int, ep: Epilogue) -> None:
    """matmul_q2_mopa_ep, src/kernels/lowbit/matmul.rs:108-116."""
    _run_lowbit(a, w, c, m, ep, mopa=True)


def matmul_q1_mopa(a, w: Q1Weights, c, m: int) -> None:
    """matmul_q1_mopa, src/kernels/lowbit/matmul.rs:123-125."""
    _run_lowbit(a, w, c, m, None, mopa=True)


def matmul_q1_mopa_ep(a, w: Q1Weights, c, m: int, ep: Epilogue) -> None:
    """matmul_q1_mopa_ep, src/kernels/lowbit/matmul.rs:131-139."""
    _run_lowbit(a, w, c, m, ep, mopa=True)


def matmul_lowbit_debug(a, w: _LowbitWeights, m: int):
    """Device call that also returns the int8 activations, their scales and the
    exact int32 block sums (torch CUDA tensors), for the bit-exactness tests."""
    n, k = w.n(), w.k()
    nbk = -(-k // w.block())
    assert _is_torch(a) and a.is_cuda and a.dtype == torch.float16 and a.numel() == m * k
    c = torch.empty((m, n), dtype=torch.float16, device=a.device)
    q = torch.empty((m, k), dtype=torch.int8, device=a.device)
    sa = torch.empty((m, nbk), dtype=torch.float32, device=a.device)
    sums = torch.zeros((m, n, nbk), dtype=torch.int32, device=a.device)
    check("smeg_matmul_lowbit_debug_dev",
          lib().smeg_matmul_lowbit_debug_dev(w._h, _ptr(a), _ptr(c), m, _ptr(q), _ptr(sa), _ptr(sums), _stream()))
    return c, q, sa, sums


# --------------------------------------------------------------------------- model blocks

def interleave_gate_up(g, u, layout: WeightLayout, n: int, k: int) -> np.ndarray:
    """[gate | up] as k x 2n row-major (InOut), 32 columns at a time
    (interleave, src/linear.rs:603-617)."""
    g = np.asarray(g).reshape(n, k).T if layout == WeightLayout.OutIn else np.asarray(g).reshape(k, n)
    u = np.asarray(u).reshape(n, k).T if layout == WeightLayout.OutIn else np.asarray(u).reshape(k, n)
    parts = []
    for c0 in range(0, n, 32):
        c1 = min(c0 + 32, n)
        parts += [g[:, c0:c1], u[:, c0:c1]]
    return np.ascontiguousarray(np.concatenate(parts, axis=1))


class Linear:
    """A projection on Q4, 2-bit, 1-bit or dense f16 weights with an optional bias (a leading AddCol) and an optional
    folded RMS norm of its input (a leading MulRow of rms_scales) -- Linear, src/linear.rs:133-155, 440-463; kernel
    routing by rows as run_ep, src/linear.rs:535-552.

    The reference switches Q4 from its GEMV to the f16 panel at PANEL_ROWS = 8 rows and opted-in low-bit weights to
    the f16 MOPA path at LOWBIT_MOPA_ROWS = 64 (measured on M5).  Here the Q4 switch between the decode kernels and
    the tensor-core GEMM sits inside the library (17 rows on B200); the low-bit opt-in keeps the reference's constant."""

    PANEL_ROWS = 8
    LOWBIT_MOPA_ROWS = 64

    def __init__(self, q4: "Q4Weights | None" = None, bias=None, *, q2: "Q2Weights | None" = None,
                 q1: "Q1Weights | None" = None, f16: "Packed | None" = None):
        given = [w for w in (q4, q2, q1, f16) if w is not None]
        assert len(given) == 1, "a Linear holds exactly one weight set"
        self.q4, self.q2, self.q1, self.f16, self.bias = q4, q2, q1, f16, bias
        self.mopa = False
        self.rms_eps = None

    @staticmethod
    def quantize(w, layout: WeightLayout, n: int, k: int, p: Q4Params | None = None, bias=None) -> "Linear":
        return Linear(Q4Weights.quantize(w, layout, n, k, p), bias)

    @staticmethod
    def from_q4(q4: Q4Weights, bias=None) -> "Linear":
        return Linear(q4, bias)

    @staticmethod
    def from_q2(q2: Q2Weights, bias=None) -> "Linear":
        """Linear::from_q2, src/linear.rs:214."""
        return Linear(None, bias, q2=q2)

    @staticmethod
    def from_q1(q1: Q1Weights, bias=None) -> "Linear":
        """Linear::from_q1, src/linear.rs:234."""
        return Linear(None, bias, q1=q1)

    @staticmethod
    def from_f16(packed: "Packed", bias=None) -> "Linear":
        assert packed.dtype == "f16"
        return Linear(None, bias, f16=packed)

    def lowbit_mopa(self, on: bool = True) -> "Linear":
        """Opt 2-bit / 1-bit weights into the f16 tensor-core path from LOWBIT_MOPA_ROWS rows (Linear::lowbit_mopa)."""
        self.mopa = bool(on)
        return self

    def rms_norm_input(self, eps: float) -> "Linear":
        """The layer computes rms_norm(x) @ W for weights whose rows were scaled by the norm's gamma beforehand
        (WeightLayout::scale_inputs): the per-row 1 / rms rides as a leading MulRow (src/linear.rs:305-308, 452-457)."""
        self.rms_eps = float(eps)
        return self

    def _w(self):
        return self.q4 or self.q2 or self.q1 or self.f16

    def n(self) -> int:
        w = self._w()
        return w.n if isinstance(w, Packed) else w.n()

    def k(self) -> int:
        w = self._w()
        return w.k if isinstance(w, Packed) else w.k()

    def _lead(self, x, m: int):
        """with_lead, src/linear.rs:440-463: the RMS row scale of x, then the bias."""
        if self.rms_eps is None and self.bias is None:
            return None
        lead = Epilogue()
        if self.rms_eps is not None:
            k = self.k()
            assert _numel(x) == m * k, "x is m*k"
            if _is_torch(x):
                r = torch.empty(m, dtype=torch.float16, device=x.device)
                check("smeg_rms_scales_dev", lib().smeg_rms_scales_dev(_ptr(r), _ptr(x), m, k, self.rms_eps, _stream()))
            else:
                xd = torch.from_numpy(np.ascontiguousarray(_np_bits(x, "x")).view(np.float16)).cuda()
                rd = torch.empty(m, dtype=torch.float16, device="cuda")
                check("smeg_rms_scales_dev", lib().smeg_rms_scales_dev(_ptr(rd), _ptr(xd), m, k, self.rms_eps, _stream()))
                r = rd.cpu().numpy()
            lead = lead.mul_row(r)
        if self.bias is not None:
            lead = lead.add_col(self.bias)
        return lead

    def forward_ep(self, x, y, m: int, ep: Epilogue | None = None) -> None:
        lead = self._lead(x, m)
        if lead is not None:
            ep = (ep or Epilogue()).with_leading(lead)
        if self.q4 is not None:
            _run_q4(x, self.q4, y, m, ep, False)
        elif self.f16 is not None:
            g = Gemm(x, self.f16, m)
            if ep is not None:
                g._ep = ep
            g.run(y)
        else:
            w = self.q2 if self.q2 is not None else self.q1
            _run_lowbit(x, w, y, m, ep, mopa=self.mopa and m >= Linear.LOWBIT_MOPA_ROWS)

    def forward(self, x, y, m: int) -> None:
        self.forward_ep(x, y, m, None)

    def accumulate(self, x, y, m: int) -> None:
        """y (f32) += f32(forward(x)) -- Linear::accumulate, src/linear.rs:425-432.  Device tensors."""
        assert _is_torch(x) and _numel(y) == m * self.n(), "y is m*n"
        out = torch.empty((m, self.n()), dtype=torch.float16, device=x.device)
        self.forward(x, out, m)
        check("smeg_add_f16_to_f32_dev", lib().smeg_add_f16_to_f32_dev(_ptr(y), _ptr(out), m * self.n(), _stream()))

    def partial(self, x, partial, m: int) -> None:
        """partial (m x n f32) = the un-rounded sums x @ W: one rank's share of a projection whose input width is split
        over ranks (the rounding and the residual add follow the sum over ranks).  Q4 weights without bias or norm."""
        assert self.q4 is not None and self.bias is None and self.rms_eps is None, "a partial product takes plain Q4 weights"
        assert _is_torch(x) and x.dtype == torch.float16 and _numel(x) == m * self.k(), "x is m*k f16 on the device"
        assert partial.dtype == torch.float32 and _numel(partial) == m * self.n(), "partial is m*n f32"
        check("smeg_matmul_q4_partial_dev", lib().smeg_matmul_q4_partial_dev(self.q4._h, _ptr(x), _ptr(partial), m, _stream()))


class GatedLinear:
    """act(x @ W_gate) * (x @ W_up) from one interleaved 2n-column Q4 matrix
    (GatedLinear, src/linear.rs:603-656,779-835)."""

    def __init__(self, inner: Linear, gate: Gate):
        self.inner, self.gate = inner, gate

    @staticmethod
    def quantize(w_gate, w_up, layout: WeightLayout, n: int, k: int, gate: Gate, p: Q4Params | None = None):
        w = interleave_gate_up(np.asarray(w_gate, np.float32), np.asarray(w_up, np.float32), layout, n, k)
        return GatedLinear(Linear.quantize(w, WeightLayout.InOut, 2 * n, k, p), gate)

    @staticmethod
    def from_q1(gate: Q1Weights, up: Q1Weights, act: Gate) -> "GatedLinear":
        """GatedLinear::from_q1, src/linear.rs:686: 1-bit gate and up projections as one interleaved layer."""
        return GatedLinear(Linear.from_q1(Q1Weights.interleave(gate, up)), act)

    def n(self) -> int:
        return self.inner.n() // 2

    def k(self) -> int:
        return self.inner.k()

    def forward(self, x, y, m: int) -> None:
        n = self.n()
        assert _numel(y) == m * n, "y is m*n"
        if _is_torch(x):
            both = torch.empty((m, 2 * n), dtype=torch.float16, device=x.device)
            self.inner.forward(x, both, m)
            check("smeg_glu_f16_dev", lib().smeg_glu_f16_dev(_ptr(y), _ptr(both), m, n, int(self.gate), _stream()))
        else:
            both = np.zeros((m, 2 * n), np.float16)
            self.inner.forward(x, both, m)
            lib().neon_glu_f16(_ptr(y), _ptr(both), m, n, int(self.gate))


class Mlp:
    """y += down(act(up(x))) (Mlp::new) or y += down(act(x @ W_gate) * (x @ W_up)) (Mlp::gated); accumulate,
    src/mlp.rs:67-146.  The gated Q4 form without biases or folded norms runs as one library call (fused kernels
    above 64 rows); every other form runs its layers one after the other exactly as the reference's three-call path."""

    def __init__(self, up, down: Linear, act: "Gate | None" = None):
        gated = isinstance(up, GatedLinear)
        assert down.k() == up.n(), "down takes up's outputs"
        assert gated or act is not None, "a plain MLP names its activation"
        self.up, self.down, self.act = up, down, act
        self._h = None
        inner = up.inner if gated else None
        if (gated and inner.q4 is not None and down.q4 is not None and inner.bias is None and down.bias is None
                and inner.rms_eps is None and down.rms_eps is None):
            h = C.c_void_p()
            check("smeg_mlp_create", lib().smeg_mlp_create(inner.q4._h, down.q4._h, int(up.gate), C.byref(h)))
            self._h = h

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            lib().smeg_mlp_destroy(h)

    @staticmethod
    def new(up: Linear, act: Gate, down: Linear) -> "Mlp":
        """Mlp::new, src/mlp.rs:67: the plain MLP of GPT-2, y += down(act(up(x)))."""
        return Mlp(up, down, act)

    @staticmethod
    def gated(up: GatedLinear, down: Linear) -> "Mlp":
        return Mlp(up, down)

    def k(self) -> int:
        return self.up.k()

    def n(self) -> int:
        return self.down.n()

    def hidden(self) -> int:
        return self.down.k()

    def accumulate(self, x, y, m: int) -> None:
        assert _numel(x) == m * self.k(), "x is m*k"
        assert _numel(y) == m * self.n(), "y is m*n"
        if self._h is not None:
            if _is_torch(x):
                assert x.dtype == torch.float16 and y.dtype == torch.float32 and x.is_contiguous() and y.is_contiguous()
                check("smeg_mlp_accumulate_dev", lib().smeg_mlp_accumulate_dev(self._h, _ptr(x), _ptr(y), m, _stream()))
            else:
                xb = _np_bits(x, "x")
                assert y.dtype == np.float32 and y.flags.c_contiguous
                check("smeg_mlp_accumulate", lib().smeg_mlp_accumulate(self._h, _ptr(xb), _ptr(y), m))
            return
        # the three-call path of src/mlp.rs:133-146 on device tensors
        assert _is_torch(x) and x.dtype == torch.float16 and y.dtype == torch.float32
        hid = torch.empty((m, self.hidden()), dtype=torch.float16, device=x.device)
        if isinstance(self.up, GatedLinear):
            self.up.forward(x, hid, m)
        else:
            ep = Epilogue().gelu() if self.act == Gate.Gelu else Epilogue().silu()
            self.up.forward_ep(x, hid, m, ep)
        self.down.accumulate(hid, y, m)

    def partial(self, x, partial, m: int) -> None:
        """This rank's f32 partial sums of the down projection (tensor parallel)."""
        assert self._h is not None, "the tensor-parallel halves exist for the gated Q4 block"
        assert _is_torch(x) and partial.dtype == torch.float32 and partial.numel() == m * self.n()
        check("smeg_mlp_partial_dev", lib().smeg_mlp_partial_dev(self._h, _ptr(x), _ptr(partial), m, _stream()))

    @staticmethod
    def finish(y, total) -> None:
        """y += f32(f16(total)): the f16 store of the down projection, then the residual add."""
        check("smeg_mlp_finish_dev", lib().smeg_mlp_finish_dev(_ptr(y), _ptr(total), y.numel(), _stream()))


class Norm:
    """A norm layer with its parameters: layer_norm (Norm::layer) or rms_norm (Norm::rms), src/nn.rs:163-230.
    forward takes f32 rows on the device and writes f16 (or f32) rows."""

    def __init__(self, weight, bias, eps: float, rms: bool):
        w = np.ascontiguousarray(weight, np.float32)
        assert w.size > 0, "a norm needs at least one feature"
        if bias is not None:
            assert np.asarray(bias).size == w.size, "bias holds weight.len() values"
        self.weight = torch.from_numpy(w).cuda()
        self.bias = None if bias is None else torch.from_numpy(np.ascontiguousarray(bias, np.float32)).cuda()
        self.eps, self.is_rms = float(eps), bool(rms)

    @staticmethod
    def layer(weight, bias, eps: float) -> "Norm":
        return Norm(weight, bias, eps, False)

    @staticmethod
    def rms(weight, eps: float) -> "Norm":
        return Norm(weight, None, eps, True)

    def width(self) -> int:
        return self.weight.numel()

    def forward(self, x, y) -> None:
        dim = self.width()
        assert _is_torch(x) and x.dtype == torch.float32 and x.numel() % dim == 0, "x holds whole rows of weight.len()"
        assert y.numel() == x.numel(), "y is the same shape as x"
        y16 = _ptr(y) if y.dtype == torch.float16 else None
        y32 = _ptr(y) if y.dtype == torch.float32 else None
        assert y16 or y32
        check("smeg_norm_rows_dev", lib().smeg_norm_rows_dev(y16, y32, _ptr(x), _ptr(self.weight), _ptr(self.bias), x.numel() // dim,
                                                             dim, self.eps, int(self.is_rms), _stream()))


class KvCache:
    """An f16 key/value cache for one attention layer, on the device, with the attention against it (KvCache,
    src/kernels/kv_attention.rs:354-581): rows of kv_heads * head_dim values, one per position, appended in order;
    queries have `heads` heads (a multiple of kv_heads: grouped-query attention); the score scale defaults to
    1 / sqrt(head_dim)."""

    def __init__(self, heads: int, kv_heads: int, head_dim: int, capacity: int):
        assert head_dim % 8 == 0 and 8 <= head_dim <= 256, "head_dim must be a multiple of 8 in 8..=256"
        assert kv_heads > 0 and heads > 0 and heads % kv_heads == 0, "heads must be a positive multiple of kv_heads"
        self._heads, self._kv_heads, self._head_dim, self._capacity = heads, kv_heads, head_dim, capacity
        self._k = torch.zeros((max(capacity, 1), kv_heads * head_dim), dtype=torch.float16, device="cuda")
        self._v = torch.zeros_like(self._k)
        self._len = 0
        self._scale = float(np.float32(1.0) / np.sqrt(np.float32(head_dim)))

    def with_scale(self, scale: float) -> "KvCache":
        self._scale = float(np.float32(scale))
        return self

    def len(self) -> int:
        return self._len

    def is_empty(self) -> bool:
        return self._len == 0

    def capacity(self) -> int:
        return self._capacity

    def row_len(self) -> int:
        return self._kv_heads * self._head_dim

    def query_len(self) -> int:
        return self._heads * self._head_dim

    def heads(self) -> int:
        return self._heads

    def kv_heads(self) -> int:
        return self._kv_heads

    def head_dim(self) -> int:
        return self._head_dim

    def scale(self) -> float:
        return self._scale

    def clear(self) -> None:
        self._len = 0

    def truncate(self, n: int) -> None:
        self._len = min(self._len, n)

    def keys(self):
        return self._k[: self._len]

    def values(self):
        return self._v[: self._len]

    def extend_from(self, src, stride: int, k_off: int, v_off: int, rows: int) -> None:
        """Appends `rows` key and value rows taken from rows of the f16 device tensor `src` (stride elements apart,
        keys at element k_off, values at v_off of a row): what a fused [q | k | v] projection produced."""
        assert self._len + rows <= self._capacity, f"KvCache full: {self._len} + {rows} rows over capacity {self._capacity}"
        check("smeg_kv_append_dev", lib().smeg_kv_append_dev(_ptr(self._k), _ptr(self._v), _ptr(src), stride, k_off, v_off,
                                                            self.row_len(), self._len, rows, _stream()))
        self._len += rows

    def extend(self, k, v) -> None:
        """KvCache::extend: whole rows of f16 keys and values (device tensors)."""
        row = self.row_len()
        assert _numel(k) == _numel(v) and _numel(k) % row == 0 and _numel(k) > 0, \
            "k and v hold the same whole number of kv_heads * head_dim rows"
        rows = _numel(k) // row
        assert self._len + rows <= self._capacity, f"KvCache full: {self._len} + {rows} rows over capacity {self._capacity}"
        self._k[self._len:self._len + rows].copy_(k.reshape(rows, row))
        self._v[self._len:self._len + rows].copy_(v.reshape(rows, row))
        self._len += rows

    push = extend

    def _attend(self, q, q_stride: int, rows: int, out) -> None:
        q_f32 = 1 if q.dtype == torch.float32 else 0
        check("smeg_attn_kv_causal_dev",
              lib().smeg_attn_kv_causal_dev(_ptr(out), _ptr(q), q_f32, q_stride, _ptr(self._k), _ptr(self._v), self._len - rows, rows,
                                            self._heads, self._kv_heads, self._head_dim, self._scale, _stream()))

    def attend(self, q, out) -> None:
        """One query row of heads * head_dim (f32 or f16) against every cached position; out f32."""
        assert self._len > 0, "attention_kv_f16 needs at least one cached key"
        assert _numel(q) == self.query_len() and _numel(out) == self.query_len(), "q is heads * head_dim"
        self._attend(q, self.query_len(), 1, out)

    def attend_causal(self, q, rows: int, out) -> None:
        """`rows` query rows, row i attending to positions 0..=len - rows + i (the cache already holds the block)."""
        assert rows <= self._len, f"attend_causal: {rows} rows but {self._len} cached"
        assert _numel(q) == rows * self.query_len() and _numel(out) == rows * self.query_len(), "q is rows * heads * head_dim"
        self._attend(q, self.query_len(), rows, out)


class SelfAttention:
    """A transformer self-attention block added into a residual stream (SelfAttention, src/self_attention.rs:66-231, its
    separate-steps path): the fused qkv projection ([q | k | v] in head order), the new positions' keys and values
    appended to a KvCache, causal attention over the cache, and the out projection: y += out(attention(q, K, V)).  No
    rotary embedding, as there."""

    def __init__(self, qkv: Linear, out: Linear, heads: int, kv_heads: int, head_dim: int):
        assert kv_heads > 0 and heads > 0 and heads % kv_heads == 0, "heads must be a positive multiple of kv_heads"
        assert qkv.n() == (heads + 2 * kv_heads) * head_dim, "qkv has (heads + 2 * kv_heads) * head_dim outputs"
        assert out.k() == heads * head_dim, "out takes heads * head_dim inputs"
        self.qkv, self.out, self._heads, self._kv_heads, self._head_dim = qkv, out, heads, kv_heads, head_dim

    @staticmethod
    def new(qkv: Linear, out: Linear, heads: int, kv_heads: int, head_dim: int) -> "SelfAttention":
        return SelfAttention(qkv, out, heads, kv_heads, head_dim)

    def width(self) -> int:
        return self.qkv.k()

    def out_width(self) -> int:
        return self.out.n()

    def cache(self, capacity: int) -> KvCache:
        return KvCache(self._heads, self._kv_heads, self._head_dim, capacity)

    def attend(self, x, cache: KvCache, m: int):
        """The block up to the out projection: m rows of f16 x projected, their keys and values appended to the cache,
        and the attention outputs of the block's heads as m x (heads * head_dim) f16."""
        d = self.width()
        assert _is_torch(x) and x.dtype == torch.float16 and _numel(x) == m * d, "x is m * width"
        assert cache.heads() == self._heads and cache.kv_heads() == self._kv_heads and cache.head_dim() == self._head_dim, \
            "the cache's heads match the block's"
        assert cache.len() + m <= cache.capacity(), f"{m} rows do not fit in the cache"
        q_len, kv_len = self._heads * self._head_dim, self._kv_heads * self._head_dim
        w = q_len + 2 * kv_len
        qkv = torch.empty((m, w), dtype=torch.float16, device=x.device)
        self.qkv.forward(x, qkv, m)
        cache.extend_from(qkv, w, q_len, q_len + kv_len, m)
        att = torch.empty((m, q_len), dtype=torch.float32, device=x.device)
        cache._attend(qkv, w, m, att)                       # the queries are the first q_len values of each projected row
        att16 = torch.empty((m, q_len), dtype=torch.float16, device=x.device)
        check("smeg_f32_to_f16_dev", lib().smeg_f32_to_f16_dev(_ptr(att16), _ptr(att), m * q_len, _stream()))
        return att16

    def accumulate(self, x, cache: KvCache, y, m: int) -> None:
        """y (m x out.n f32) += out(attention(qkv(x))) for m rows of f16 x at the cache's next positions, which this appends."""
        assert _numel(y) == m * self.out.n(), "y is m * out.n()"
        self.out.accumulate(self.attend(x, cache, m), y, m)


class Block:
    """A pre-norm transformer layer over an f32 residual stream: x += attn(norm1(x)), then x += mlp(norm2(x))
    (Block, src/block.rs:40-106).  Block(norm2, mlp) is the MLP half alone, for callers that run attention themselves."""

    def __init__(self, *parts):
        if len(parts) == 2:
            norm1, attn, (norm2, mlp) = None, None, parts
        else:
            norm1, attn, norm2, mlp = parts
        d = norm2.width()
        assert mlp.k() == d and mlp.n() == d and (attn is None or (norm1.width() == d and attn.width() == d and attn.out_width() == d)), \
            "the norms, attention and MLP share the residual's width"
        self.norm1, self.attn, self.norm2, self.mlp = norm1, attn, norm2, mlp

    @staticmethod
    def new(norm1: Norm, attn: SelfAttention, norm2: Norm, mlp: Mlp) -> "Block":
        return Block(norm1, attn, norm2, mlp)

    def width(self) -> int:
        return self.norm2.width()

    def cache(self, capacity: int) -> KvCache:
        return self.attn.cache(capacity)

    def accumulate(self, x, *args) -> None:
        """accumulate(x, cache, rows): both halves at the cache's next positions; accumulate(x, rows): the MLP half."""
        cache, rows = (None, args[0]) if len(args) == 1 else args
        assert _is_torch(x) and x.dtype == torch.float32 and x.numel() == rows * self.width(), "x is rows * width"
        h = torch.empty((rows, self.width()), dtype=torch.float16, device=x.device)
        if cache is not None:
            assert self.attn is not None, "this block was built without its attention half"
            self.norm1.forward(x, h)
            self.attn.accumulate(h, cache, x, rows)
        self.norm2.forward(x, h)
        self.mlp.accumulate(h, x, rows)


def last_status() -> int:
    return int(lib().smeg_last_status())


def device_info():
    sm, mem = C.c_int(), C.c_size_t()
    check("smeg_device_info", lib().smeg_device_info(C.byref(sm), C.byref(mem)))
    return sm.value, mem.value
