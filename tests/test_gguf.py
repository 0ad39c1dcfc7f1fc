"""The GGUF v3 reader and the block formats it turns into weight sets (sme_gemm_b200/gguf.py), on synthetic files written
here: metadata of every value type, alignment, the reference reader's error cases (examples/bonsai/gguf.rs:110-165), and
Q1_0 / Q4_0 / TQ2_0 tensors whose logical arrays must dequantise (through the oracle) to the formats' own values."""
import struct

import numpy as np
import pytest

import oracle as orc
from sme_gemm_b200 import gguf


def _s(x: str) -> bytes:
    b = x.encode()
    return struct.pack("<Q", len(b)) + b


def _val(ty, v) -> bytes:
    fmt = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<B", 10: "<Q", 11: "<q", 12: "<d"}
    if ty == 8:
        return _s(v)
    if ty == 9:
        ety, items = v
        return struct.pack("<IQ", ety, len(items)) + b"".join(_val(ety, i) for i in items)
    return struct.pack(fmt[ty], v)


def write_gguf(meta, tensors, align=32, version=3, magic=b"GGUF") -> bytes:
    """meta: [(key, type id, value)]; tensors: [(name, dims innermost first, ggml type, bytes)]."""
    head = magic + struct.pack("<IQQ", version, len(tensors), len(meta))
    for key, ty, v in meta:
        head += _s(key) + struct.pack("<I", ty) + _val(ty, v)
    body, infos = b"", b""
    for name, dims, ty, data in tensors:
        pad = (-len(body)) % align
        body += b"\0" * pad
        infos += _s(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims) + struct.pack("<IQ", ty, len(body))
        body += data
    head += infos
    head += b"\0" * ((-len(head)) % align)
    return head + body


def q1_blocks(rng, n, k):
    sc = rng.uniform(0.01, 0.05, (n, k // 128)).astype("<f2")
    signs = rng.integers(0, 256, (n, k // 128, 16)).astype(np.uint8)
    return np.concatenate([sc.view(np.uint8).reshape(n, -1, 2), signs], axis=2).tobytes(), sc, signs


def q4_blocks(rng, n, k):
    sc = rng.uniform(0.01, 0.05, (n, k // 32)).astype("<f2")
    qs = rng.integers(0, 256, (n, k // 32, 16)).astype(np.uint8)
    return np.concatenate([sc.view(np.uint8).reshape(n, -1, 2), qs], axis=2).tobytes()


def q4_1_blocks(rng, n, k, exact=False):
    """exact: offsets m = -8 d + (a small multiple of d's unit), so that m + 8 d is an f16 number."""
    sc = rng.uniform(0.01, 0.05, (n, k // 32)).astype("<f2")
    if exact:
        mn = (np.float32(-8.0) * sc.astype(np.float32)).astype("<f2")
        sc = (mn.astype(np.float32) / np.float32(-8.0)).astype("<f2")          # d = -m / 8 exactly: m + 8 d = 0
    else:
        mn = rng.uniform(-0.4, 0.1, (n, k // 32)).astype("<f2")
    qs = rng.integers(0, 256, (n, k // 32, 16)).astype(np.uint8)
    return np.concatenate([sc.view(np.uint8).reshape(n, -1, 2), mn.view(np.uint8).reshape(n, -1, 2), qs], axis=2).tobytes()


def tq2_blocks(rng, n, k):
    q = rng.integers(0, 3, (n, k // 256, 64, 4)).astype(np.uint8)          # codes 0..2 only
    qs = (q[..., 0] | (q[..., 1] << 2) | (q[..., 2] << 4) | (q[..., 3] << 6)).astype(np.uint8)
    sc = rng.uniform(0.01, 0.05, (n, k // 256)).astype("<f2")
    return np.concatenate([qs, sc.view(np.uint8).reshape(n, -1, 2)], axis=2).tobytes()


def test_metadata_directory_and_alignment():
    rng = np.random.default_rng(1)
    a = rng.standard_normal((3, 8)).astype("<f4")
    h = rng.standard_normal((2, 4)).astype("<f2")
    meta = [("a.u8", 0, 200), ("a.i8", 1, -3), ("a.u16", 2, 60000), ("a.i16", 3, -300), ("a.u32", 4, 4000000000),
            ("a.i32", 5, -7), ("a.f32", 6, 0.5), ("a.bool", 7, 1), ("general.name", 8, "synthetic"),
            ("tokenizer.ggml.tokens", 9, (8, ["a", "b", "ab"])), ("a.u64", 10, 1 << 40), ("a.i64", 11, -(1 << 40)),
            ("a.f64", 12, 0.25), ("general.alignment", 4, 64), ("ints", 9, (5, [1, -2, 3]))]
    for align in (64,):
        g = gguf.Gguf(write_gguf(meta, [("w.a", [8, 3], gguf.F32, a.tobytes()), ("w.h", [4, 2], gguf.F16, h.tobytes())], align))
        assert g.meta["a.u8"] == 200 and g.meta["a.i8"] == -3 and g.meta["a.u16"] == 60000 and g.meta["a.i16"] == -300
        assert g.meta["a.u32"] == 4000000000 and g.meta["a.i32"] == -7 and g.meta["a.bool"] is True
        assert g.meta["a.u64"] == 1 << 40 and g.meta["a.i64"] == -(1 << 40) and g.meta["ints"] == [1, -2, 3]
        assert g.float("a.f32") == 0.5 and g.float("a.f64") == 0.25 and g.str("general.name") == "synthetic"
        assert g.strings("tokenizer.ggml.tokens") == ["a", "b", "ab"] and g.int("a.u16") == 60000
        assert g.tensors["w.a"].begin % 64 == 0 and g.tensors["w.h"].begin % 64 == 0
        assert np.array_equal(g.f32("w.a"), a) and np.array_equal(g.f32("w.h"), h.astype(np.float32))
    # default alignment is 32
    g = gguf.Gguf(write_gguf([], [("x", [4], gguf.F32, np.arange(4, dtype="<f4").tobytes())]))
    assert g.tensors["x"].begin % 32 == 0 and np.array_equal(g.f32("x"), np.arange(4, dtype=np.float32))


def test_error_cases_of_the_reader():
    ok = [("x", [4], gguf.F32, np.zeros(4, "<f4").tobytes())]
    with pytest.raises(ValueError, match="not a GGUF file"):
        gguf.Gguf(write_gguf([], ok, magic=b"GGML"))
    with pytest.raises(ValueError, match="GGUF version 2, expected 3"):
        gguf.Gguf(write_gguf([], ok, version=2))
    with pytest.raises(ValueError, match="truncated GGUF header"):
        gguf.Gguf(write_gguf([("k", 8, "v")], ok)[:20])
    with pytest.raises(ValueError, match="x: unsupported ggml type 12"):
        gguf.Gguf(write_gguf([], [("x", [4], 12, b"\0" * 16)]))
    with pytest.raises(ValueError, match="x: 100 values is not whole blocks"):
        gguf.Gguf(write_gguf([], [("x", [100], gguf.Q1_0, b"\0" * 18)]))
    with pytest.raises(ValueError, match="x: data past the end of the file"):
        gguf.Gguf(write_gguf([], ok)[:-4])
    with pytest.raises(ValueError, match="unknown GGUF value type 13"):
        gguf.Gguf(b"GGUF" + struct.pack("<IQQ", 3, 0, 1) + _s("k") + struct.pack("<I", 13))
    g = gguf.Gguf(write_gguf([("n", 5, -1), ("s", 8, "t")], ok))
    with pytest.raises(ValueError, match="missing tensor y"):
        g.tensor("y")
    with pytest.raises(ValueError, match="n < 0"):
        g.int("n")
    with pytest.raises(ValueError, match="missing integer s"):
        g.int("s")
    with pytest.raises(ValueError, match="missing float n"):
        g.float("n")
    assert g.str("n") is None
    with pytest.raises(ValueError, match="expected a 2-D Q1_0 tensor"):
        gguf.q1_arrays(g, ["x"])


def test_q1_0_rows_stack_into_one_weight_set():
    """examples/bonsai/model.rs:134-160: scales and sign bytes of the named tensors, rows in order."""
    rng = np.random.default_rng(2)
    k = 256
    b0, sc0, sg0 = q1_blocks(rng, 5, k)
    b1, sc1, sg1 = q1_blocks(rng, 3, k)
    g = gguf.Gguf(write_gguf([], [("q", [k, 5], gguf.Q1_0, b0), ("kv", [k, 3], gguf.Q1_0, b1)]))
    signs, scales, n, kk = gguf.q1_arrays(g, ["q", "kv"])
    assert (n, kk) == (8, k)
    assert np.array_equal(scales, np.concatenate([sc0.view(np.uint16).reshape(-1), sc1.view(np.uint16).reshape(-1)]))
    assert np.array_equal(signs, np.concatenate([sg0.reshape(-1), sg1.reshape(-1)]))
    # the weights these arrays mean (bit 1 = +scale, low bit first, OutIn) are the format's own
    want = np.concatenate([gguf.dequant(g, "q"), gguf.dequant(g, "kv")], axis=0)
    bits = np.unpackbits(signs, bitorder="little").reshape(n, k)
    got = np.where(bits == 1, 1.0, -1.0) * orc.f16_bits_to_f32(scales).reshape(n, k // 128).repeat(128, axis=1)
    assert np.array_equal(got.astype(np.float32), want)
    with pytest.raises(ValueError, match="input width differs"):
        g2 = gguf.Gguf(write_gguf([], [("a", [k, 2], gguf.Q1_0, q1_blocks(rng, 2, k)[0]), ("b", [128, 2], gguf.Q1_0, q1_blocks(rng, 2, 128)[0])]))
        gguf.q1_arrays(g2, ["a", "b"])


def test_q4_0_arrays_dequantise_to_the_formats_values():
    rng = np.random.default_rng(3)
    n, k = 7, 96
    g = gguf.Gguf(write_gguf([], [("w", [k, n], gguf.Q4_0, q4_blocks(rng, n, k))]))
    quants, scales, nn, kk = gguf.q4_0_arrays(g, ["w"])
    assert (nn, kk) == (n, k) and quants.size == (n * k + 1) // 2 and scales.size == n * (k // 32)
    deq = orc.f16_bits_to_f32(orc.q4_dequant(quants, scales, None, n, k, 32)).reshape(k, n)      # [d][j], rounded to f16
    want = gguf.dequant(g, "w")                                                                   # [j][d], f32 product
    assert np.array_equal(deq.T, orc.f16_bits_to_f32(orc.f32_to_f16_bits(want)).reshape(n, k))


def test_q4_1_arrays_are_the_affine_form():
    """d q + m = d (q - 8) + (m + 8 d): codes and scales are the file's, the offset is rounded to f16 once."""
    rng = np.random.default_rng(5)
    n, k = 6, 128
    for exact in (True, False):
        g = gguf.Gguf(write_gguf([], [("w", [k, n], gguf.Q4_1, q4_1_blocks(rng, n, k, exact))]))
        quants, scales, mins, nn, kk = gguf.q4_1_arrays(g, ["w"])
        assert (nn, kk) == (n, k) and scales.size == mins.size == n * (k // 32)
        deq = orc.f16_bits_to_f32(orc.q4_dequant(quants, scales, mins, n, k, 32)).reshape(k, n).T     # [j][d]
        want = gguf.dequant(g, "w")
        want16 = orc.f16_bits_to_f32(orc.f32_to_f16_bits(want)).reshape(n, k)
        if exact:
            assert np.array_equal(deq, want16)
        else:
            # the offset moved by at most half its last place (|m + 8 d| < 0.5: 2^-12), then one f16 rounding of a value < 1
            assert np.max(np.abs(deq - want)) <= 2.0 ** -12 + 2.0 ** -11
    g0 = gguf.Gguf(write_gguf([], [("x", [32, 1], gguf.Q4_0, q4_blocks(rng, 1, 32))]))
    with pytest.raises(ValueError, match="x: expected a 2-D Q4_1 tensor"):
        gguf.q4_1_arrays(g0, ["x"])


def test_tq2_0_arrays_hold_the_formats_codes():
    rng = np.random.default_rng(4)
    n, k = 3, 512
    g = gguf.Gguf(write_gguf([], [("w", [k, n], gguf.TQ2_0, tq2_blocks(rng, n, k))]))
    codes, scales, nn, kk = gguf.tq2_0_arrays(g, ["w"])
    assert (nn, kk) == (n, k) and codes.size == n * k // 4 and scales.size == n * (k // 256)
    q = np.stack([(codes >> s) & 3 for s in (0, 2, 4, 6)], axis=1).reshape(k, n)                 # code of (d, j)
    cb = np.asarray(gguf.TQ2_CODEBOOK, np.float32)
    got = cb[q].T * orc.f16_bits_to_f32(scales).reshape(n, k // 256).repeat(256, axis=1)
    assert np.array_equal(got.astype(np.float32), gguf.dequant(g, "w"))
