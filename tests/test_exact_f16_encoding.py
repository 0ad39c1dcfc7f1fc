"""The integer block sums of the int8-activation kernels are formed on the f16 tensor-core path.  These tests restate, in
numpy, the encodings lowbit_mma.cu / lowbit_tc.cu rely on and check that they are exact:
  * a weight as the f16 whose bit pattern is a small unsigned integer u (u * 2^-24), an activation code as the f16 integer q;
  * 1-bit weights used where they lie in a packed word: bit b of a half word is 2^(b-24) for b < 12, and the activation
    codes of the matching depths are scaled by the inverse power of two (act_quant_kernel, qh_perm = 2), so that the sums of
    a lane's two columns carry 2^-16 and 2^-15.
The tensor cores multiply f16 exactly and add in f32; every partial sum here is a multiple of 2^-24 below 2^0..2^8, which
f32 holds exactly -- the numpy check sums in f64 and verifies that bound."""
import numpy as np

MASKS_LO = (0x00010001, 0x01000100, 0x00040004, 0x04000400)      # column g: positions (0,1) (2,3) (4,5) (6,7) of a run of 8
MASKS_HI = (0x00020002, 0x02000200, 0x00080008, 0x08000800)      # column g + 8: one bit higher
POS_SCALE = (256.0, 256.0, 1.0, 1.0, 64.0, 64.0, 0.25, 0.25)     # what act_quant_kernel multiplies the codes by
PERM = (0, 2, 1, 3, 4, 6, 5, 7)                                  # depth held at each position


def f16_of_bits(bits):
    return np.array(bits, np.uint16).view(np.float16).astype(np.float64)


def test_a_bit_of_a_half_word_is_a_power_of_two():
    for b in range(12):
        assert f16_of_bits([1 << b])[0] == 2.0 ** (b - 24)
    # (above that the exponent field no longer counts in steps of one: the kernels never use those bits in place)
    assert f16_of_bits([1 << 12])[0] != 2.0 ** (12 - 24)


def test_subnormal_coded_weights_times_integer_codes_are_exact():
    rng = np.random.default_rng(1)
    u = rng.integers(0, 256, 512)                                 # 2-bit: codebook value + 128; 1-bit: the sign bit
    q = rng.integers(-128, 128, 512)
    w = f16_of_bits(u.astype(np.uint16))                          # u * 2^-24
    assert np.array_equal(w, u * 2.0 ** -24)
    qh = q.astype(np.float16).astype(np.float64)
    assert np.array_equal(qh, q)
    acc = np.cumsum(w * qh)                                       # the order of a depth-ordered accumulation
    units = acc * 2.0 ** 24
    assert np.array_equal(units, np.round(units)) and np.max(np.abs(units)) < 2 ** 24      # exact in f32 as well
    assert int(units[-1]) == int(np.sum(u * q))


def test_sign_bits_used_in_place_give_the_scaled_integer_sums():
    rng = np.random.default_rng(2)
    for _ in range(50):
        # one lane's word for one 32-deep step after the kernels' shift: bits 0..3, 8..11, 16..19, 24..27 are in use.
        # bit (0 | 8 | 16 | 24) + (0 | 2) + hi: depth (0 | 1 | 2 | 3) + (0 | 4) of column g (hi = 0) or g + 8 (hi = 1)
        v = int(rng.integers(0, 1 << 32))
        q = rng.integers(-128, 128, 8)                            # the lane's eight activation codes, depth order
        scaled = np.array([q[PERM[p]] * POS_SCALE[p] for p in range(8)])
        assert np.array_equal(scaled.astype(np.float16).astype(np.float64), scaled)        # still exact f16 numbers
        for masks, unit in ((MASKS_LO, 2.0 ** -16), (MASKS_HI, 2.0 ** -15)):
            hi = 0 if masks is MASKS_LO else 1
            acc = 0.0
            for r, mk in enumerate(masks):                        # register r holds positions 2r (low half), 2r + 1 (high half)
                reg = v & mk
                lo, hh = f16_of_bits([reg & 0xffff])[0], f16_of_bits([reg >> 16])[0]
                acc += lo * scaled[2 * r] + hh * scaled[2 * r + 1]
            # the sum the kernels mean: the sign bits of the eight depths times the codes
            bit_of_depth = {0: 0, 1: 8, 2: 16, 3: 24, 4: 2, 5: 10, 6: 18, 7: 26}
            want = sum(((v >> (bit_of_depth[d] + hi)) & 1) * int(q[d]) for d in range(8))
            assert acc == want * unit
