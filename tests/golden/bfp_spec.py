"""The frozen block-float spec in exact integer / rational arithmetic, written independently of the C oracle
and of the CUDA kernels (no floating-point operation decides a result).  Used by the known-answer generator
and by the oracle's own tests.

Published description: docs/public/dataformats.rst:59-89 of the reference (shared exponent = largest exponent
of the 16 values; sign + 7 / 3 / 1 magnitude bits without an implied one).  Frozen choices: round to nearest,
ties to even; a round-up past the largest magnitude saturates; zero / denormal inputs encode as 0; Inf / NaN
encode the largest magnitude; a zero magnitude is stored with sign 0; datum i occupies bits [i*(m+1), (i+1)*(m+1))
of the block's little-endian bit string; decode (-1)^s * q * 2^(E-127-(m-1)), q = 0 -> +0.0.
"""
import math
import struct
from fractions import Fraction

SPEC_VERSION = 1


def f2b(x: float) -> int:
    return struct.unpack("<I", struct.pack("<f", x))[0]


def encode_block(bits16, m):
    """16 binary32 bit patterns -> (shared exponent byte, bytes of the 16 datums)."""
    exps = [(b >> 23) & 0xFF for b in bits16]
    E = max(exps)
    qmax = (1 << m) - 1
    datums = []
    for b, e in zip(bits16, exps):
        sign = b >> 31
        if e == 0:
            q = 0
        elif e == 255:
            q = qmax
        else:
            mag = Fraction((b & 0x7FFFFF) | 0x800000, 1 << 23) * Fraction(2) ** (e - 127)
            v = mag * Fraction(2) ** (m - 1) / Fraction(2) ** (E - 127)
            fl = math.floor(v)
            rem = v - fl
            if rem > Fraction(1, 2) or (rem == Fraction(1, 2) and fl % 2 == 1):
                fl += 1
            q = min(fl, qmax)
        datums.append(((sign << m) | q) if q else 0)
    w = m + 1
    bitstring = 0
    for i, d in enumerate(datums):
        bitstring |= d << (w * i)
    return E, bitstring.to_bytes(2 * w, "little")


def decode_block(E, data: bytes, m):
    """-> 16 binary32 bit patterns (overflow gives infinity, as the conversion to binary32 does)."""
    w = m + 1
    word = int.from_bytes(data, "little")
    out = []
    for i in range(16):
        dat = (word >> (w * i)) & ((1 << w) - 1)
        q, s = dat & ((1 << m) - 1), dat >> m
        if q == 0:
            out.append(0)
            continue
        k = E - 127 - (m - 1)
        # q * 2^k as binary32: q has at most 7 bits, so the value is exact unless it overflows or is subnormal
        top = q.bit_length() - 1 + k
        if top > 127:
            bits = 0x7F800000
        elif top >= -126:
            bits = ((top + 127) << 23) | ((q << (23 - (q.bit_length() - 1))) & 0x7FFFFF)
        else:
            shift = k + 149          # value = q * 2^k = (q << shift) * 2^-149
            bits = (q << shift) if shift >= 0 else 0
            assert shift >= 0, "a decoded value is never below the smallest subnormal"
        out.append(bits | (s << 31))
    return out
