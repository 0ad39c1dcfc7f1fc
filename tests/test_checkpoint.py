"""The safetensors checkpoint reader (sme_gemm_b200/checkpoint.py) on files written here, after
examples/shakespeare/model.rs:28-70: F32 only, values and shapes by name, the error messages."""
import json
import struct

import numpy as np
import pytest

from sme_gemm_b200.checkpoint import Checkpoint


def write_safetensors(tensors, metadata=None) -> bytes:
    header, body = {}, b""
    if metadata:
        header["__metadata__"] = metadata
    for name, (dtype, arr) in tensors.items():
        raw = arr.tobytes()
        header[name] = {"dtype": dtype, "shape": list(arr.shape), "data_offsets": [len(body), len(body) + len(raw)]}
        body += raw
    h = json.dumps(header).encode()
    h += b" " * ((-len(h)) % 8)
    return struct.pack("<Q", len(h)) + h + body


def test_tensors_by_name_and_matrices():
    rng = np.random.default_rng(0)
    w = rng.standard_normal((12, 8)).astype("<f4")
    g = rng.standard_normal(8).astype("<f4")
    ck = Checkpoint(write_safetensors({"transformer.h.0.attn.c_attn.weight": ("F32", w), "transformer.h.0.ln_1.weight": ("F32", g)},
                                      {"format": "pt"}))
    assert sorted(ck.names()) == ["transformer.h.0.attn.c_attn.weight", "transformer.h.0.ln_1.weight"]
    v, rows, cols = ck.matrix("transformer.h.0.attn.c_attn.weight")
    assert (rows, cols) == (12, 8) and np.array_equal(v, w.reshape(-1))
    assert np.array_equal(ck.get("transformer.h.0.ln_1.weight"), g)
    with pytest.raises(ValueError, match="the checkpoint has no lm_head.weight"):
        ck.get("lm_head.weight")
    with pytest.raises(ValueError, match=r"transformer.h.0.ln_1.weight is \[8\], not a matrix"):
        ck.matrix("transformer.h.0.ln_1.weight")


def test_refusals():
    h = np.zeros((2, 2), "<f2")
    with pytest.raises(ValueError, match="w is F16, not F32"):
        Checkpoint(write_safetensors({"w": ("F16", h)}))
    with pytest.raises(ValueError, match="header too small"):
        Checkpoint(b"\x00\x00")
    with pytest.raises(ValueError, match="invalid header length"):
        Checkpoint(struct.pack("<Q", 1000) + b"{}")
    with pytest.raises(ValueError, match="invalid header"):
        Checkpoint(struct.pack("<Q", 4) + b"{{{{")
    good = write_safetensors({"w": ("F32", np.zeros((2, 2), "<f4"))})
    with pytest.raises(ValueError, match="w: byte range does not match its shape"):
        Checkpoint(good[:-4])
