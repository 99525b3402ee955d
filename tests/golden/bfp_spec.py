"""The frozen block-float spec in exact integer / rational arithmetic, written independently of the C oracle
and of the CUDA kernels (no floating-point operation decides a result).  Used by the known-answer generator
and by the oracle's own tests.

Published description: docs/public/dataformats.rst:59-89 of the reference (shared exponent = largest exponent
of the 16 values; sign + 7 / 3 / 1 magnitude bits without an implied one).  Frozen choices: round to nearest,
ties to even; a round-up past the largest magnitude saturates; zero / denormal inputs encode as 0; Inf / NaN
encode the largest magnitude; a zero magnitude is stored with sign 0; datum i occupies bits [i*(m+1), (i+1)*(m+1))
of the block's little-endian bit string; decode (-1)^s * q * 2^(E-127-(m-1)), q = 0 -> +0.0.

The choices that change bytes are also available the other way round (Policy): truncation, or "add half, then truncate"
(nearest, ties away from zero), instead of rounding to nearest even; a
shared exponent raised by one instead of saturation, another face order, and exponents / datums counted from the top
end of each 32-bit word.  The default Policy() is the frozen spec above.
"""
import math
import struct
from fractions import Fraction

SPEC_VERSION = 1


class Policy:
    def __init__(self, rounding=0, overflow=0, face_order=(0, 1, 2, 3), exponent_order=0, datum_order=0):
        self.rounding = rounding              # 0 nearest even, 1 truncate, 2 nearest with ties away from zero (add half, then truncate)
        self.overflow = overflow              # 0 saturate, 1 raise the shared exponent by one
        self.face_order = tuple(face_order)   # face stored first, second, third, fourth
        self.exponent_order = exponent_order  # 0: exponent of block k in byte k, 1: in byte k ^ 3
        self.datum_order = datum_order        # 0: datum i in the i-th field from the bottom, 1: fields of each 32-bit word from the top

    def as_tuple(self):
        return (self.rounding, self.overflow) + self.face_order + (self.exponent_order, self.datum_order)


DEFAULT = Policy()


def f2b(x: float) -> int:
    return struct.unpack("<I", struct.pack("<f", x))[0]


def _quantise(bits16, exps, E, m, policy):
    """Magnitudes of the block against shared exponent E, before saturation (None marks Inf / NaN)."""
    qs = []
    for b, e in zip(bits16, exps):
        if e == 0:
            qs.append(0)
        elif e == 255:
            qs.append(None)
        else:
            mag = Fraction((b & 0x7FFFFF) | 0x800000, 1 << 23) * Fraction(2) ** (e - 127)
            v = mag * Fraction(2) ** (m - 1) / Fraction(2) ** (E - 127)
            fl = math.floor(v)
            rem = v - fl
            if policy.rounding == 0 and (rem > Fraction(1, 2) or (rem == Fraction(1, 2) and fl % 2 == 1)):
                fl += 1
            elif policy.rounding == 2 and rem >= Fraction(1, 2):
                fl += 1
            qs.append(fl)
    return qs


def _field_position(i, w, policy):
    """Bit offset of datum i in the block's bytes read as little-endian 32-bit words."""
    per_word = 32 // w
    word, field = divmod(i, per_word)
    if policy.datum_order:
        field = per_word - 1 - field
    return word * 32 + field * w


def encode_block(bits16, m, policy=DEFAULT):
    """16 binary32 bit patterns -> (shared exponent byte, bytes of the 16 datums)."""
    exps = [(b >> 23) & 0xFF for b in bits16]
    E = max(exps)
    qmax = (1 << m) - 1
    qs = _quantise(bits16, exps, E, m, policy)
    if policy.overflow and E < 255 and any(q is not None and q > qmax for q in qs):
        E += 1
        qs = _quantise(bits16, exps, E, m, policy)
    datums = []
    for b, q in zip(bits16, qs):
        q = qmax if q is None else min(q, qmax)
        datums.append((((b >> 31) << m) | q) if q else 0)
    w = m + 1
    bitstring = 0
    for i, d in enumerate(datums):
        bitstring |= d << _field_position(i, w, policy)
    return E, bitstring.to_bytes(2 * w, "little")


def encode_tile(bits32x32, m, policy=DEFAULT):
    """One 32x32 tile (rows of binary32 bit patterns) -> its record: 64 exponent bytes, then the datum bytes of the
    64 blocks; block k = the face at position k // 16, face row k % 16."""
    w = m + 1
    exps = bytearray(64)
    data = bytearray(64 * 2 * w)
    for pos, face in enumerate(policy.face_order):
        for fr in range(16):
            r, c = (face >> 1) * 16 + fr, (face & 1) * 16
            E, d = encode_block([int(v) for v in bits32x32[r][c:c + 16]], m, policy)
            k = pos * 16 + fr
            exps[k ^ 3 if policy.exponent_order else k] = E
            data[k * 2 * w:(k + 1) * 2 * w] = d
    return bytes(exps) + bytes(data)


def decode_block(E, data: bytes, m, policy=DEFAULT):
    """-> 16 binary32 bit patterns (overflow gives infinity, as the conversion to binary32 does)."""
    w = m + 1
    word = int.from_bytes(data, "little")
    out = []
    for i in range(16):
        dat = (word >> _field_position(i, w, policy)) & ((1 << w) - 1)
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


# ------------------------------------------------------------------------------------------------------------------
# Lf8: 1 sign, 5 exponent, 2 mantissa bits per element, no shared exponent (docs/public/dataformats.rst:24 of the
# reference).  Frozen reading (the reference has no host conversion to compare with): the IEEE-754 rules for those
# field widths -- bias 15, subnormals, code 0x7c = infinity, 0x7d-0x7f = NaN -- and round to nearest, ties to the
# even code.  Stated here as "the nearest representable value", by exact comparison against the whole value table.
# ------------------------------------------------------------------------------------------------------------------
def lf8_value(code: int) -> Fraction:
    """Exact value of a finite, non-negative code (0 .. 0x7b)."""
    e, m = (code >> 2) & 31, code & 3
    assert code < 0x7C
    if e == 0:
        return Fraction(m, 4) * Fraction(2) ** (-14)
    return (1 + Fraction(m, 4)) * Fraction(2) ** (e - 15)


_LF8_TABLE = [lf8_value(c) for c in range(0x7C)]
# the value code 0x7c would have if the exponent range went on: deciding between the largest finite value and infinity
_LF8_NEXT = Fraction(2) ** 16


def lf8_encode_bits(b: int) -> int:
    """binary32 bit pattern -> Lf8 code."""
    sign = (b >> 24) & 0x80
    e, frac = (b >> 23) & 0xFF, b & 0x7FFFFF
    if e == 255:
        return sign | (0x7F if frac else 0x7C)
    mag = Fraction(frac, 1 << 23) * Fraction(2) ** (-126) if e == 0 else Fraction(frac | 0x800000, 1 << 23) * Fraction(2) ** (e - 127)
    table = _LF8_TABLE + [_LF8_NEXT]
    lo = max(c for c in range(len(table)) if table[c] <= mag) if mag >= 0 else 0
    if lo == len(table) - 1:
        return sign | 0x7C
    down, up = mag - table[lo], table[lo + 1] - mag
    code = lo if down < up else lo + 1 if up < down else (lo if lo % 2 == 0 else lo + 1)
    return sign | code


def lf8_decode_bits(code: int) -> int:
    """Lf8 code -> binary32 bit pattern of the same value (exact; NaN keeps its two mantissa bits on top)."""
    sign = (code & 0x80) << 24
    c = code & 0x7F
    if c >= 0x7C:
        return sign | 0x7F800000 | ((c & 3) << 21)
    v = lf8_value(c)
    if v == 0:
        return sign
    return sign | f2b(float(v))
