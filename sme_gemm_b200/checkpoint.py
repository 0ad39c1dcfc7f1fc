"""A safetensors checkpoint as named f32 tensors, and its matrices as Q4 `Linear`s.

Mirrors `Checkpoint` of the reference's nanoGPT example (examples/shakespeare/model.rs:28-70: every tensor must be F32;
`get` gives a tensor's values, `matrix` a 2-D tensor with its rows and columns in torch's [out][in] layout) and the
`linear` step of its model loader (:84-91: the matrix quantised to Q4 with the chosen K-block, OutIn).  The file format
is the published one: an 8-byte little-endian header length, a JSON header mapping each name to its dtype, shape and
byte range in the data section that follows (the reference reads it with the `safetensors` crate).
"""
from __future__ import annotations

import json
import struct

import numpy as np


class Checkpoint:
    def __init__(self, data: bytes, where: str = "<bytes>"):
        def bad(msg):
            return ValueError(f"{where}: {msg}")
        if len(data) < 8:
            raise bad("header too small")
        (n,) = struct.unpack("<Q", data[:8])
        if n > len(data) - 8:
            raise bad("invalid header length")
        try:
            header = json.loads(data[8:8 + n].decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise bad(f"invalid header: {e}") from None
        body = memoryview(data)[8 + n:]
        self._t = {}
        for name, info in header.items():
            if name == "__metadata__":
                continue
            if info["dtype"] != "F32":
                raise bad(f"{name} is {info['dtype']}, not F32")
            shape = [int(x) for x in info["shape"]]
            b, e = info["data_offsets"]
            count = int(np.prod(shape, dtype=np.int64)) if shape else 1
            if e < b or e > len(body) or e - b != 4 * count:
                raise bad(f"{name}: byte range does not match its shape")
            self._t[name] = (shape, np.frombuffer(body[b:e], "<f4").astype(np.float32))

    @staticmethod
    def load(path) -> "Checkpoint":
        with open(path, "rb") as f:
            return Checkpoint(f.read(), str(path))

    def names(self):
        return list(self._t)

    def get(self, name: str) -> np.ndarray:
        if name not in self._t:
            raise ValueError(f"the checkpoint has no {name}")
        return self._t[name][1]

    def matrix(self, name: str):
        """(values, rows, columns) of a 2-D tensor."""
        if name not in self._t:
            raise ValueError(f"the checkpoint has no {name}")
        shape, v = self._t[name]
        if len(shape) != 2:
            raise ValueError(f"{name} is {shape}, not a matrix")
        return v, shape[0], shape[1]

    def linear(self, name: str, q4_block: int = 32):
        """The matrix `name` ([out][in]) quantised to Q4 with q4_block-deep K-blocks (needs the CUDA library)."""
        from .host import Linear, Q4Params, Q4Weights, WeightLayout
        w, rows, cols = self.matrix(name)
        return Linear.from_q4(Q4Weights.quantize(w, WeightLayout.OutIn, rows, cols, Q4Params(q4_block)))

    def norm(self, name: str, eps: float = 1e-5):
        from .host import Norm
        return Norm.layer(self.get(name), None, eps)
