"""Host-side preparation (quantisers + GPU prepack) checked on the CPU:
bit equality of the library's quantisers with the oracle's, pack/unpack
identity on the reference's ragged shapes, and the documented position of every
code inside the packed units (an independent restatement of the layout)."""
import ctypes as C

import numpy as np
import pytest

import oracle as orc
import sme_gemm_b200 as sg
from refgen import data

L = sg.lib()


def p(a):
    return None if a is None else a.ctypes.data


def host_pack(bits, wbits, layout, scales, n, k, block):
    codes = np.zeros(L.smeg_packed_code_bytes(bits, n, k), np.uint8)
    sc = np.zeros(L.smeg_packed_scale_elems(bits, n, k, block), np.uint16)
    assert L.smeg_host_pack(bits, p(wbits), layout, p(scales), n, k, block, p(codes), p(sc)) == 0
    return codes, sc


def host_unpack(bits, codes, sc, n, k, block):
    per = {4: 2, 2: 4, 1: 8}[bits]
    nbk = -(-k // block)
    wbits = np.zeros((k * n + per - 1) // per, np.uint8)
    scales = np.zeros(n * nbk, np.uint16)
    assert L.smeg_host_unpack(bits, p(codes), p(sc), n, k, block, p(wbits), p(scales)) == 0
    return wbits, scales


@pytest.mark.parametrize("n,k,block,layout", [(33, 64, 32, 0), (40, 100, 32, 1), (8, 96, 64, 1), (17, 130, 16, 0), (5, 9, 2, 1)])
def test_q4_quantizer_equals_oracle(n, k, block, layout):
    w = (np.random.default_rng(n + k).standard_normal(n * k) * 0.02).astype(np.float32)
    w[::13] = 0
    nbk = -(-k // block)
    q = np.zeros((k * n + 1) // 2, np.uint8)
    s = np.zeros(n * nbk, np.uint16)
    assert L.smeg_host_q4_quantize(p(w), layout, n, k, block, p(q), p(s)) == 0
    qo, so, _ = orc.q4_quantize(w, layout, n, k, block)
    assert np.array_equal(q, qo) and np.array_equal(s, so)


@pytest.mark.parametrize("n,k,block,layout", [(70, 300, 64, 0), (33, 37, 16, 1)])
def test_q2_q1_quantizers_equal_oracle(n, k, block, layout):
    w = np.random.default_rng(n).standard_normal(n * k).astype(np.float32)
    nbk = -(-k // block)
    for cb in ([-1, 0, 1, 0], [-2, -1, 1, 2]):
        codes = np.zeros((k * n + 3) // 4, np.uint8)
        s = np.zeros(n * nbk, np.uint16)
        cba = np.asarray(cb, np.int8)
        assert L.smeg_host_q2_quantize(p(w), layout, n, k, block, p(cba), p(codes), p(s)) == 0
        co, so = orc.q2_quantize(w, layout, n, k, block, cb)
        assert np.array_equal(codes, co) and np.array_equal(s, so)
    signs = np.zeros((k * n + 7) // 8, np.uint8)
    s = np.zeros(n * nbk, np.uint16)
    assert L.smeg_host_q1_quantize(p(w), layout, n, k, block, p(signs), p(s)) == 0
    so_, sco = orc.q1_quantize(w, layout, n, k, block)
    assert np.array_equal(signs, so_) and np.array_equal(s, sco)
    zero = np.zeros(4, np.int8)
    assert L.smeg_host_q2_quantize(p(w), layout, n, k, block, p(zero), p(codes), p(s)) == -2


# shapes of the reference's pack round-trip tests (src/kernels/q4/weights.rs:429-438,
# src/kernels/lowbit/q2.rs:198, q1.rs:246) plus unit-boundary cases
Q4_SHAPES = [(1, 1), (3, 5), (32, 32), (33, 31), (48, 1), (17, 64), (64, 65), (31, 96), (130, 257)]


@pytest.mark.parametrize("n,k", Q4_SHAPES)
@pytest.mark.parametrize("block", [1, 16, 32, 128])
def test_q4_pack_unpack_identity(n, k, block):
    quants = data(n * 131 + k * 17, (k * n + 1) // 2)
    if (k * n) % 2:
        quants[-1] &= 0x0F
    nbk = -(-k // block)
    scales = (np.arange(n * nbk) * 7 + 1).astype(np.uint16)
    codes, sc = host_pack(4, quants, 0, scales, n, k, block)
    q2, s2 = host_unpack(4, codes, sc, n, k, block)
    assert np.array_equal(q2, quants) and np.array_equal(s2, scales)


@pytest.mark.parametrize("n,k,block", [(1, 1, 16), (65, 37, 16), (130, 300, 256), (16, 128, 64), (17, 129, 16)])
def test_q2_q1_pack_unpack_identity(n, k, block):
    nbk = -(-k // block)
    scales = (np.arange(n * nbk) * 3 + 5).astype(np.uint16)
    codes_in = ((np.arange((k * n + 3) // 4) * 37) % 251).astype(np.uint8)
    rem = (k * n) % 4
    if rem:
        codes_in[-1] &= (1 << (2 * rem)) - 1
    codes, sc = host_pack(2, codes_in, 1, scales, n, k, block)
    c2, s2 = host_unpack(2, codes, sc, n, k, block)
    assert np.array_equal(c2, codes_in) and np.array_equal(s2, scales)
    signs = ((np.arange((k * n + 7) // 8) * 37) % 251).astype(np.uint8)
    rem = (k * n) % 8
    if rem:
        signs[-1] &= (1 << rem) - 1
    bits = np.unpackbits(signs, bitorder="little")[: k * n]
    for layout in (0, 1):
        codes, sc = host_pack(1, signs, layout, scales, n, k, block)
        back, s2 = host_unpack(1, codes, sc, n, k, block)   # OutIn order
        want = bits.reshape(n, k) if layout == 0 else bits.reshape(k, n).T
        got = np.unpackbits(back, bitorder="little")[: k * n].reshape(n, k)
        assert np.array_equal(got, want) and np.array_equal(s2, scales)


def test_q4_unit_layout_is_the_documented_mma_fragment_order():
    """Independent restatement of the Q4 unit layout: lane 4g+t, word ks, nibble
    order (0,4,1,5 | 2,6,3,7) = column g depths +0..+3 | column g+8 depths +0..+3."""
    n, k, block = 32, 128, 32
    rng = np.random.default_rng(0)
    code = rng.integers(-8, 8, (k, n))
    flat = (code.reshape(-1) & 0xF).astype(np.uint8)
    quants = (flat[0::2] | (flat[1::2] << 4)).astype(np.uint8)
    scales = np.arange(n * (k // block), dtype=np.uint16)
    codes, sc = host_pack(4, quants, 0, scales, n, k, block)
    # [column group][unit][32 lanes][4 words]; the 2 real column groups are padded to 8 (128 columns)
    words = codes.view(np.uint32).reshape(8, k // 64, 32, 4)
    assert (words[2:] == 0x88888888).all()   # padding = code 0
    for cg in range(n // 16):
        for u in range(k // 64):
            for lane in range(32):
                g, t = lane >> 2, lane & 3
                for ks in range(4):
                    w = int(words[cg, u, lane, ks])
                    d = 64 * u + 32 * (ks >> 1) + 8 * t + 4 * (ks & 1)
                    nib = [(w >> (4 * i)) & 0xF for i in range(8)]
                    got_lo = [nib[0] - 8, nib[4] - 8, nib[1] - 8, nib[5] - 8]
                    got_hi = [nib[2] - 8, nib[6] - 8, nib[3] - 8, nib[7] - 8]
                    assert got_lo == list(code[d:d + 4, 16 * cg + g])
                    assert got_hi == list(code[d:d + 4, 16 * cg + g + 8])
    # scales: [column group][block][16 slots], column c in slot 2*(c % 8) + c // 8
    assert sc.reshape(8, k // block, 16)[1, 2, 2 * 5] == scales[(16 + 5) * (k // block) + 2]
    assert sc.reshape(8, k // block, 16)[0, 1, 2 * 3 + 1] == scales[11 * (k // block) + 1]


def test_q2_q1_unit_layouts_are_the_documented_fragment_order():
    n, k = 16, 256
    rng = np.random.default_rng(1)
    c2 = rng.integers(0, 4, (k, n))
    flat = c2.reshape(-1).astype(np.uint8)
    codes_in = (flat[0::4] | (flat[1::4] << 2) | (flat[2::4] << 4) | (flat[3::4] << 6)).astype(np.uint8)
    scales = np.zeros(n * 1, np.uint16)
    codes, _ = host_pack(2, codes_in, 1, scales, n, k, 256)
    words = codes.view(np.uint32).reshape(1, k // 128, 32, 4)
    for u in range(k // 128):
        for lane in range(32):
            g, t = lane >> 2, lane & 3
            for ks in range(4):
                w = int(words[0, u, lane, ks])
                d = 128 * u + 32 * ks + 8 * t
                for f in range(16):
                    assert (w >> (2 * f)) & 3 == c2[d + (f >> 1), g + 8 * (f & 1)]
    s1 = rng.integers(0, 2, (n, k))   # OutIn [j][d]
    signs = np.packbits(s1.reshape(-1).astype(np.uint8), bitorder="little")
    codes, _ = host_pack(1, signs, 0, scales, n, k, 256)
    words = codes.view(np.uint32).reshape(1, 1, 32, 4)
    for lane in range(32):
        g, t = lane >> 2, lane & 3
        for wd in range(4):
            w = int(words[0, 0, lane, wd])
            for b in range(32):
                s = 2 * wd + ((b & 7) >> 2)
                d = 32 * s + 8 * t + 4 * ((b >> 1) & 1) + (b >> 3)
                assert (w >> b) & 1 == s1[g + 8 * (b & 1), d]


def test_band_major_import_round_trips_through_the_reference_layouts():
    """smeg_*_from_band reads the reference's own packed arrays; checked on the
    host by importing what the oracle's restated reference packers produce."""
    # exercised through the host pack of the re-imported logical arrays: the import
    # itself needs a device, so only the size contracts are checked here
    assert orc.lib().orc_q4_band_nibble_bytes(130, 70) == 2 * 70 * 64
    assert orc.lib().orc_q2_band_code_bytes(65, 37) == 2 * 48 * 16
    assert orc.lib().orc_q1_band_sign_bytes(65, 37) == 2 * 48 * 8
