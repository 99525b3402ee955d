"""Writes tests/golden/lf8_kat.npz: binary32 bit patterns and the Lf8 codes the exact-arithmetic spec
(bfp_spec.lf8_encode_bits) gives them, plus the decode of all 256 codes.  Run from the repository root:

    python tests/golden/gen_lf8_kat.py
"""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import bfp_spec as S  # noqa: E402


def hand_picked():
    f = S.f2b
    vals = [0.0, -0.0, 1.0, -1.0, 1.125, 1.25, 1.375, 1.5, 1.625, 1.75, 1.875, 2.0,      # ties both ways around 1.x
            57344.0, 61439.996, 61440.0, 61440.004, 65504.0, 65536.0, 1e9, -1e9,      # largest finite, the tie to infinity
            2.0 ** -14, 2.0 ** -15, 2.0 ** -16, 2.0 ** -17, 2.0 ** -17 * 1.0001, 2.0 ** -18,   # subnormal range and its ties
            1.5 * 2.0 ** -16, 2.5 * 2.0 ** -16, 3.5 * 2.0 ** -16, 3.75 * 2.0 ** -16, 1e-30, 1e-45]
    bits = [f(v) for v in vals]
    bits += [0x7F800000, 0xFF800000, 0x7FC00000, 0xFFC00001, 0x7F800001, 0x00000001, 0x007FFFFF, 0x80000001]
    return bits


def main():
    rng = np.random.default_rng(20240607)
    bits = hand_picked()
    # every bfloat16 pattern whose exponent is in or next to the Lf8 range, a spread of others, and random binary32
    for hb in range(0, 65536, 1):
        e = (hb >> 7) & 0xFF
        if 108 <= e <= 145 or hb % 97 == 0:
            bits.append(hb << 16)
    bits += [int(v) for v in rng.integers(0, 2 ** 32, size=3000, dtype=np.uint64)]
    near = (rng.standard_normal(3000) * np.exp(rng.uniform(-13, 12, 3000))).astype(np.float32).view(np.uint32)
    bits += [int(v) for v in near]
    bits = np.array(bits, dtype=np.uint32)
    codes = np.array([S.lf8_encode_bits(int(b)) for b in bits], dtype=np.uint8)
    decode = np.array([S.lf8_decode_bits(c) for c in range(256)], dtype=np.uint32)
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "lf8_kat.npz")
    np.savez_compressed(out, bits=bits, codes=codes, decode=decode, spec_version=np.array([S.SPEC_VERSION]))
    print("wrote", out, len(bits), "vectors")


if __name__ == "__main__":
    main()
