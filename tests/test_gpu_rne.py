"""The device's f32 -> bf16 rounding against the engine's integer rule (reference src/core/bf16.rs:13-23), over bit
patterns chosen to hit every case of the rule: ties with an even and an odd kept bit, one below and one above a tie,
the carry into the exponent and into infinity, zeros, subnormals, both signs, every exponent. The kernels convert
with the hardware instruction; the rule is (bits + 0x7fff + lsb) >> 16. NaN inputs are outside the contract."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def integer_rule(bits: np.ndarray) -> np.ndarray:
    b = bits.astype(np.uint64)
    return ((b + 0x7FFF + ((b >> 16) & 1)) >> 16).astype(np.uint16)


def test_hardware_rounding_is_the_integer_rule(ctx):
    rng = np.random.default_rng(7)
    low17 = np.array([0x00000, 0x00001, 0x07FFF, 0x08000, 0x08001, 0x0FFFF, 0x10000, 0x10001, 0x17FFF, 0x18000, 0x18001, 0x1FFFF], dtype=np.uint32)
    parts = []
    for sign in (0, 1):
        for exp in range(0, 255):  # 255 = Inf / NaN: Inf is added below, NaN is outside the contract
            hi6 = rng.integers(0, 64, size=(8, 1), dtype=np.uint32)  # the mantissa bits above the kept bit's neighbours
            hi6[0, 0], hi6[1, 0] = 0, 63  # all zeros; all ones (the carry into the exponent)
            pat = (np.uint32(sign) << 31) | (np.uint32(exp) << 23) | (hi6 << 17) | low17[None, :]
            parts.append(pat.reshape(-1))
    parts.append(np.array([0x7F800000, 0xFF800000, 0x7F7FFFFF, 0xFF7FFFFF, 0x7F7F8000, 0x7F7F7FFF], dtype=np.uint32))
    rnd = rng.integers(0, 1 << 32, size=1 << 22, dtype=np.uint64).astype(np.uint32)
    rnd = rnd[(rnd & 0x7F800000) != 0x7F800000]
    parts.append(rnd)
    bits = np.concatenate(parts)
    n = 4096
    bits = np.concatenate([bits, np.zeros((-len(bits)) % n, dtype=np.uint32)])
    m = len(bits) // n
    d_acc, d_y = ctx.to_device(bits), ctx.alloc(len(bits) * 2)
    ctx.epilogue(n, 0)(m, d_acc, d_y)
    ctx.sync()
    got = d_y.download(np.uint16, (len(bits),))
    want = integer_rule(bits)
    bad = np.nonzero(got != want)[0]
    assert len(bad) == 0, [(hex(int(bits[i])), hex(int(got[i])), hex(int(want[i]))) for i in bad[:8]]
