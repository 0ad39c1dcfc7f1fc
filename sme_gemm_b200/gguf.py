"""GGUF v3 files as weight sets of this library (host side; numpy only until a handle is made).

Mirrors the reader of the reference's Bonsai example (examples/bonsai/gguf.rs: metadata, tensor directory,
the bytes of each tensor; examples/bonsai/model.rs:134-160: the named Q1_0 tensors' rows stacked as one
Q1Weights) and adds the block formats whose arithmetic this library's weight kinds hold exactly:

    Q1_0  (type 41)  128 weights: f16 scale, 16 bytes of sign bits            -> Q1Weights, block 128
    Q4_0  (type 2)    32 weights: f16 scale d, 16 bytes of nibbles q, d (q-8) -> Q4Weights, block 32
    Q4_1  (type 3)    32 weights: f16 d, f16 m, 16 bytes of nibbles q, d q + m -> Q4Weights, block 32, affine form
    TQ2_0 (type 35)  256 weights: 64 bytes of 2-bit codes q, f16 d, d (q-1)   -> Q2Weights, block 256, codebook -1 0 1
    F32 / F16                                                                 -> numpy arrays

A GGUF tensor of dims [k, n] (innermost first) is n rows of k weights, blocks running along k: the OutIn layout.
Errors are ValueError with the reference's messages.
"""
from __future__ import annotations

import struct
from dataclasses import dataclass

import numpy as np

F32, F16, Q4_0, Q4_1, TQ2_0, Q1_0 = 0, 1, 2, 3, 35, 41

# (weights per block, bytes per block)
_BLOCK = {F32: (1, 4), F16: (1, 2), Q4_0: (32, 18), Q4_1: (32, 20), TQ2_0: (256, 66), Q1_0: (128, 18)}


@dataclass
class Tensor:
    dims: list          # innermost first, as GGUF stores them
    ty: int
    begin: int
    end: int


class _Reader:
    def __init__(self, b: bytes):
        self.b, self.at = b, 0

    def take(self, n: int) -> bytes:
        end = self.at + n
        if n < 0 or end > len(self.b):
            raise ValueError("truncated GGUF header")
        s = self.b[self.at:end]
        self.at = end
        return s

    def u32(self) -> int:
        return struct.unpack("<I", self.take(4))[0]

    def u64(self) -> int:
        return struct.unpack("<Q", self.take(8))[0]

    def string(self) -> str:
        return self.take(self.u64()).decode("utf-8", errors="replace")

    def value(self, ty: int):
        if ty == 0:
            return self.take(1)[0]
        if ty == 1:
            return struct.unpack("<b", self.take(1))[0]
        if ty == 2:
            return struct.unpack("<H", self.take(2))[0]
        if ty == 3:
            return struct.unpack("<h", self.take(2))[0]
        if ty == 4:
            return self.u32()
        if ty == 5:
            return struct.unpack("<i", self.take(4))[0]
        if ty == 6:
            return float(struct.unpack("<f", self.take(4))[0])
        if ty == 7:
            return self.take(1)[0] != 0
        if ty == 8:
            return self.string()
        if ty == 9:
            ety, n = self.u32(), self.u64()
            return [self.value(ety) for _ in range(n)]
        if ty == 10:
            return self.u64()
        if ty == 11:
            return struct.unpack("<q", self.take(8))[0]
        if ty == 12:
            return float(struct.unpack("<d", self.take(8))[0])
        raise ValueError(f"unknown GGUF value type {ty}")


class Gguf:
    """A loaded file: `meta` (key -> int / float / bool / str / list), `tensors` (name -> Tensor)."""

    def __init__(self, data: bytes):
        self.data = data
        r = _Reader(data)
        if r.take(4) != b"GGUF":
            raise ValueError("not a GGUF file")
        version = r.u32()
        if version != 3:
            raise ValueError(f"GGUF version {version}, expected 3")
        n_tensors, n_kv = r.u64(), r.u64()
        self.meta = {}
        for _ in range(n_kv):
            key = r.string()
            self.meta[key] = r.value(r.u32())
        infos = []
        for _ in range(n_tensors):
            name = r.string()
            dims = [r.u64() for _ in range(r.u32())]
            infos.append((name, dims, r.u32(), r.u64()))
        align = self.meta.get("general.alignment", 32)
        if not isinstance(align, int) or isinstance(align, bool) or align <= 0:
            raise ValueError("bad alignment")
        start = -(-r.at // align) * align
        self.tensors = {}
        for name, dims, ty, offset in infos:
            if ty not in _BLOCK:
                raise ValueError(f"{name}: unsupported ggml type {ty}")
            per, nbytes = _BLOCK[ty]
            elems = int(np.prod(dims, dtype=np.uint64)) if dims else 1
            if elems % per != 0:
                raise ValueError(f"{name}: {elems} values is not whole blocks")
            begin = start + offset
            end = begin + elems // per * nbytes
            if end > len(data):
                raise ValueError(f"{name}: data past the end of the file")
            self.tensors[name] = Tensor(dims, ty, begin, end)

    @staticmethod
    def load(path) -> "Gguf":
        with open(path, "rb") as f:
            return Gguf(f.read())

    def tensor(self, name: str):
        t = self.tensors.get(name)
        if t is None:
            raise ValueError(f"missing tensor {name}")
        return t, np.frombuffer(self.data, np.uint8, t.end - t.begin, t.begin)

    def int(self, key: str) -> int:
        v = self.meta.get(key)
        if not isinstance(v, int) or isinstance(v, bool):
            raise ValueError(f"missing integer {key}")
        if v < 0:
            raise ValueError(f"{key} < 0")
        return v

    def float(self, key: str) -> float:
        v = self.meta.get(key)
        if not isinstance(v, float):
            raise ValueError(f"missing float {key}")
        return v

    def str(self, key: str):
        v = self.meta.get(key)
        return v if isinstance(v, str) else None

    def strings(self, key: str) -> list:
        """An array of strings (tokenizer.ggml.tokens, tokenizer.ggml.merges)."""
        v = self.meta.get(key)
        if not isinstance(v, list):
            raise ValueError(f"missing {key}")
        if not all(isinstance(s, str) for s in v):
            raise ValueError("non-string " + ("token" if key.endswith("tokens") else "merge"))
        return v

    def f32(self, name: str) -> np.ndarray:
        """An F32 or F16 tensor as f32, shape = dims reversed (outermost first)."""
        t, b = self.tensor(name)
        if t.ty == F32:
            a = b.view("<f4").astype(np.float32)
        elif t.ty == F16:
            a = b.view("<f2").astype(np.float32)
        else:
            raise ValueError(f"{name}: expected an F32 or F16 tensor")
        return a.reshape(list(reversed(t.dims)))


# --------------------------------------------------------------------------- block formats -> logical arrays

def _rows(g: Gguf, names, ty: int, what: str):
    """The named 2-D tensors of one block type, their rows stacked: (blocks[n][k / per][bytes], n, k)."""
    per, nbytes = _BLOCK[ty]
    parts, n, k = [], 0, None
    for name in names:
        t, b = g.tensor(name)
        if t.ty != ty or len(t.dims) != 2:
            raise ValueError(f"{name}: expected a 2-D {what} tensor")
        if k is None:
            k = t.dims[0]
        if k != t.dims[0]:
            raise ValueError(f"{name}: input width differs")
        if k % per != 0:
            raise ValueError(f"{name}: rows of {k} values are not whole blocks")
        n += t.dims[1]
        parts.append(b.reshape(t.dims[1], k // per, nbytes))
    k = 0 if k is None else k
    blocks = np.concatenate(parts, axis=0) if parts else np.zeros((0, 0, nbytes), np.uint8)
    return blocks, n, k


def q1_arrays(g: Gguf, names):
    """Q1_0 tensors (examples/bonsai/model.rs:134-160) -> (signs, scales, n, k) for Q1Weights.new(.., OutIn, n, k, 128):
    sign bits in row order, low bit first; one f16 scale per 128 weights at [j * (k / 128) + blk]."""
    blocks, n, k = _rows(g, names, Q1_0, "Q1_0")
    scales = np.ascontiguousarray(blocks[:, :, 0:2]).view("<u2").reshape(-1).astype(np.uint16)
    signs = np.ascontiguousarray(blocks[:, :, 2:18]).reshape(-1)
    return signs, scales, n, k


def q4_0_arrays(g: Gguf, names):
    """Q4_0 tensors -> (quants, scales, n, k) for Q4Weights.new(quants, scales, n, k) (block 32).  A block holds
    weight i of its 32 in the low nibble of byte i (i < 16) or the high nibble of byte i - 16, as q = code + 8; the
    logical array wants the signed code of weight (d, j) at nibble d * n + j, low nibble first."""
    blocks, n, k = _rows(g, names, Q4_0, "Q4_0")
    scales = np.ascontiguousarray(blocks[:, :, 0:2]).view("<u2").reshape(-1).astype(np.uint16)
    qs = blocks[:, :, 2:18]
    nib = np.concatenate([qs & 0x0F, qs >> 4], axis=2).reshape(n, k)          # [j][d], q = code + 8
    code = (nib ^ 8).astype(np.uint8)                                          # two's-complement nibble of q - 8
    flat = np.ascontiguousarray(code.T).reshape(-1)                            # index d * n + j
    if flat.size % 2:
        flat = np.concatenate([flat, np.zeros(1, np.uint8)])
    quants = (flat[0::2] | (flat[1::2] << 4)).astype(np.uint8)
    return quants, scales, n, k


def q4_1_arrays(g: Gguf, names):
    """Q4_1 tensors -> (quants, scales, mins, n, k) for Q4Weights.with_params(.., Q4Params(32).affine()).  The file's
    weight is d * q + m with q in 0..15; the affine form of this library (src/kernels/q4/mod.rs:39-48) is
    scale * code + min with code in -8..7, so scale = d, code = q - 8 and min = m + 8 d.  That offset is stored as f16:
    where m + 8 d is not an f16 number it is rounded once (the f32 sum to f16, nearest even), and the block's weights
    move by that rounding, at most half a unit in the last place of the offset."""
    blocks, n, k = _rows(g, names, Q4_1, "Q4_1")
    d = np.ascontiguousarray(blocks[:, :, 0:2]).view("<f2")
    m = np.ascontiguousarray(blocks[:, :, 2:4]).view("<f2")
    scales = d.view("<u2").reshape(-1).astype(np.uint16)
    off = (m.astype(np.float32) + np.float32(8.0) * d.astype(np.float32)).astype(np.float32)
    with np.errstate(over="ignore"):
        mins = off.astype("<f2").view("<u2").reshape(-1).astype(np.uint16)
    qs = blocks[:, :, 4:20]
    nib = np.concatenate([qs & 0x0F, qs >> 4], axis=2).reshape(n, k)          # [j][d], q = code + 8
    code = (nib ^ 8).astype(np.uint8)
    flat = np.ascontiguousarray(code.T).reshape(-1)
    if flat.size % 2:
        flat = np.concatenate([flat, np.zeros(1, np.uint8)])
    quants = (flat[0::2] | (flat[1::2] << 4)).astype(np.uint8)
    return quants, scales, mins, n, k


def tq2_0_arrays(g: Gguf, names):
    """TQ2_0 tensors -> (codes, scales, n, k) for Q2Weights.new(codes, scales, n, k, Q2Params(256) with codebook
    [-1, 0, 1, 0]).  A block is 64 bytes of codes then its f16 scale; weight 128 h + 32 l + i (h < 2, l < 4, i < 32) is
    bits 2l, 2l+1 of byte 32 h + i, and its value is (q - 1) * d."""
    blocks, n, k = _rows(g, names, TQ2_0, "TQ2_0")
    scales = np.ascontiguousarray(blocks[:, :, 64:66]).view("<u2").reshape(-1).astype(np.uint16)
    qs = blocks[:, :, 0:64].reshape(n, -1, 2, 1, 32)                           # [j][blk][h][.][i]
    shifts = (2 * np.arange(4, dtype=np.uint8)).reshape(1, 1, 1, 4, 1)
    q = ((qs >> shifts) & 3).reshape(n, k)                                     # [j][d], order h, l, i within a block
    flat = np.ascontiguousarray(q.T).reshape(-1).astype(np.uint8)              # index d * n + j
    pad = (-flat.size) % 4
    if pad:
        flat = np.concatenate([flat, np.zeros(pad, np.uint8)])
    codes = (flat[0::4] | (flat[1::4] << 2) | (flat[2::4] << 4) | (flat[3::4] << 6)).astype(np.uint8)
    return codes, scales, n, k


TQ2_CODEBOOK = [-1, 0, 1, 0]


def dequant(g: Gguf, name: str) -> np.ndarray:
    """Any supported tensor as f32 [rows][k] in the formats' own arithmetic (f32 product of the f16 scale and the
    small integer): what a loaded weight set must reproduce."""
    t, b = g.tensor(name)
    if t.ty in (F32, F16):
        return g.f32(name)
    per, nbytes = _BLOCK[t.ty]
    k = t.dims[0]
    rows = int(np.prod(t.dims[1:], dtype=np.uint64)) if len(t.dims) > 1 else 1
    blocks = b.reshape(rows, k // per, nbytes)
    if t.ty == Q1_0:
        d = np.ascontiguousarray(blocks[:, :, 0:2]).view("<f2").astype(np.float32)
        bits = np.unpackbits(np.ascontiguousarray(blocks[:, :, 2:18]), axis=2, bitorder="little")
        return (np.where(bits == 1, 1.0, -1.0).astype(np.float32) * d).reshape(rows, k)
    if t.ty == Q4_0:
        d = np.ascontiguousarray(blocks[:, :, 0:2]).view("<f2").astype(np.float32)
        qs = blocks[:, :, 2:18]
        nib = np.concatenate([qs & 0x0F, qs >> 4], axis=2).astype(np.float32)
        return ((nib - 8.0) * d).reshape(rows, k)
    if t.ty == Q4_1:
        d = np.ascontiguousarray(blocks[:, :, 0:2]).view("<f2").astype(np.float32)
        m = np.ascontiguousarray(blocks[:, :, 2:4]).view("<f2").astype(np.float32)
        qs = blocks[:, :, 4:20]
        nib = np.concatenate([qs & 0x0F, qs >> 4], axis=2).astype(np.float32)
        return (nib * d + m).reshape(rows, k)
    d = np.ascontiguousarray(blocks[:, :, 64:66]).view("<f2").astype(np.float32)
    qs = blocks[:, :, 0:64].reshape(rows, -1, 2, 1, 32)
    shifts = (2 * np.arange(4, dtype=np.uint8)).reshape(1, 1, 1, 4, 1)
    q = ((qs >> shifts) & 3).astype(np.float32).reshape(rows, k // 256, 256)
    return ((q - 1.0) * d).reshape(rows, k)


# --------------------------------------------------------------------------- weight sets (need the CUDA library)

def q1(g: Gguf, names):
    from .host import Q1Weights, WeightLayout
    signs, scales, n, k = q1_arrays(g, names)
    return Q1Weights.new(signs, scales, WeightLayout.OutIn, n, k, 128)


def q4_0(g: Gguf, names):
    from .host import Q4Weights
    quants, scales, n, k = q4_0_arrays(g, names)
    return Q4Weights.new(quants, scales, n, k)


def q4_1(g: Gguf, names):
    from .host import Q4Params, Q4Weights
    quants, scales, mins, n, k = q4_1_arrays(g, names)
    return Q4Weights.with_params(quants, scales, mins, n, k, Q4Params(32).affine())


def tq2_0(g: Gguf, names):
    from .host import Q2Params, Q2Weights
    codes, scales, n, k = tq2_0_arrays(g, names)
    return Q2Weights.new(codes, scales, n, k, Q2Params(256).with_codebook(TQ2_CODEBOOK))
