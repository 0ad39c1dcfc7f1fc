"""Input generators of the reference's own tests, restated so its test inputs
can be regenerated bit for bit (tests/correctness/main.rs:36-46 `fill`;
the byte stream of tests/correctness/q4.rs:18-21 and
src/kernels/lowbit/matmul.rs:409-417 `data`)."""
import numpy as np

_M = (1 << 64) - 1
_A = 6364136223846793005
_C = 1442695040888963407


class Lcg:
    def __init__(self, seed: int):
        self.s = seed & _M

    def fill(self, n: int) -> np.ndarray:
        """`fill`: f16(u - 0.5), u = (s >> 40) / 2^24, increment 1442695040888963407."""
        out = np.empty(n, np.float32)
        s = self.s
        for i in range(n):
            s = (s * _A + _C) & _M
            out[i] = np.float32(s >> 40) / np.float32(1 << 24) - np.float32(0.5)
        self.s = s
        return out.astype(np.float16)

    def bytes(self, n: int) -> np.ndarray:
        """byte stream: s = s*A + 1; (s >> 40) as u8."""
        out = np.empty(n, np.uint8)
        s = self.s
        for i in range(n):
            s = (s * _A + 1) & _M
            out[i] = (s >> 40) & 0xFF
        self.s = s
        return out


def data(seed: int, n: int) -> np.ndarray:
    return Lcg(seed).bytes(n)
