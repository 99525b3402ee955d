"""Writes tests/golden/bfp_kat.npz: known-answer vectors of the frozen block-float spec, computed by the
exact-arithmetic restatement in bfp_spec.py (not by the C oracle, not by the CUDA kernels), and
tests/golden/bfp_kat_policies.npz: the tile records of the same values under each of the other layout policies.

    python tests/golden/gen_bfp_kat.py

256 blocks of 16 values = four 32x32 tiles: hand-picked edge cases first (all zero, lone values, ties, an outlier
flattening its block, saturation on round-up, denormals, signed zeros, Inf / NaN, the ends of the exponent range),
then seeded random blocks of six kinds.  For every block and every mantissa width (7, 3, 1): the shared exponent, the
datum bytes, and the decoded binary32 bit patterns."""
import os
import random

import numpy as np

from bfp_spec import SPEC_VERSION, Policy, decode_block, encode_block, encode_tile, f2b

HERE = os.path.dirname(os.path.abspath(__file__))


def hand_picked():
    inf, nan = 0x7F800000, 0x7FC00000
    z = [0] * 16
    blocks = [
        z,
        [f2b(1.0)] + [0] * 15,
        [f2b(v) for v in (1.0, -1.5, 1.984375, 1.9999)] + [0] * 12,
        [f2b(v) for v in (1000.0, 1.0, 4.0, -8.0, 12.0)] + [0] * 11,
        [f2b(1e-40), 0x80000000, 0x00800000] + [0] * 13,
        [inf, inf | 0x80000000, nan, f2b(3.0e38)] + [0] * 12,
        [f2b(v) for v in (64.0, 0.5, -0.5, 1.5, -1.5, 2.5, -2.5, 3.5, 0.25, 0.75, 1.25, 1.75, 63.5, -63.5, 63.75, -64.0)],
        [0x00800000 + i for i in range(16)],                          # smallest normals: E = 1
        [0x7F7FFFFF - i * 0x10000 for i in range(16)],                # largest finite values: E = 254
        [0x00000001, 0x807FFFFF] + [0] * 14,                          # only denormals: encodes as zero, E = 0
        [f2b(2.0 ** -120 * (i + 1)) for i in range(16)],              # shared exponent below the mantissa width
        [f2b((-1.0) ** i * 2.0 ** (i - 8)) for i in range(16)],       # one value per binade
        [f2b(1.0 + i / 128.0) for i in range(16)],                    # ties at the 7-bit boundary
        [f2b(-(1.0 + (2 * i + 1) / 256.0)) for i in range(16)],
        [nan | 0x80000000] * 16,
        [f2b(0.1 * (i - 8)) for i in range(16)],
    ]
    return blocks


def random_blocks(n, seed):
    rng = random.Random(seed)
    out = []
    for t in range(n):
        kind = t % 6
        if kind == 0:
            vals = [rng.gauss(0, 1) for _ in range(16)]
        elif kind == 1:
            vals = [rng.gauss(0, 1) * 10.0 ** rng.randint(-30, 30) for _ in range(16)]
        elif kind == 2:
            vals = [64.0] + [rng.randint(-9, 9) * 0.5 for _ in range(15)]
        elif kind == 3:
            out.append([rng.getrandbits(32) for _ in range(16)])
            continue
        elif kind == 4:
            vals = [rng.gauss(0, 1) * 2.0 ** -124 for _ in range(16)]
        else:
            vals = [rng.gauss(0, 1) * 2.0 ** 126 for _ in range(16)]
        bits = []
        for v in vals:
            try:
                bits.append(f2b(v))
            except OverflowError:
                bits.append(0x7F800000 | (0x80000000 if v < 0 else 0))
        out.append(bits)
    return out


def main():
    blocks = hand_picked()
    blocks += random_blocks(256 - len(blocks), seed=20240)
    arrays = {"spec_version": np.array([SPEC_VERSION]), "x": np.array(blocks, dtype=np.uint32)}
    for m in (7, 3, 1):
        Es, datas, decs = [], [], []
        for b in blocks:
            E, data = encode_block(b, m)
            Es.append(E)
            datas.append(list(data))
            decs.append(decode_block(E, data, m))
        arrays[f"E{m}"] = np.array(Es, dtype=np.uint8)
        arrays[f"data{m}"] = np.array(datas, dtype=np.uint8)
        arrays[f"decoded{m}"] = np.array(decs, dtype=np.uint32)
    np.savez_compressed(os.path.join(HERE, "bfp_kat.npz"), **arrays)
    print(f"{len(blocks)} blocks written")
    write_policy_vectors(blocks)


# every switch on its own, then combinations; the columns are (rounding, overflow, face order x4, exponent order, datum order)
POLICIES = [
    Policy(rounding=1),
    Policy(overflow=1),
    Policy(datum_order=1),
    Policy(exponent_order=1),
    Policy(face_order=(0, 2, 1, 3)),
    Policy(rounding=1, overflow=1, face_order=(3, 1, 2, 0), exponent_order=1, datum_order=1),
    Policy(rounding=0, overflow=1, face_order=(1, 0, 3, 2), exponent_order=1, datum_order=1),
    Policy(rounding=2),
    Policy(rounding=2, overflow=1, face_order=(2, 3, 0, 1), datum_order=1),
]


def tiles_of(blocks):
    """The 256 blocks as the face rows of four 32x32 tiles, faces in the natural order (as the tests lay them out)."""
    tiles = np.zeros((4, 32, 32), dtype=np.uint32)
    for b, vals in enumerate(blocks):
        t, blk = divmod(b, 64)
        face, fr = divmod(blk, 16)
        tiles[t, (face >> 1) * 16 + fr, (face & 1) * 16:(face & 1) * 16 + 16] = vals
    return tiles


def write_policy_vectors(blocks):
    tiles = tiles_of(blocks)
    arrays = {"spec_version": np.array([SPEC_VERSION]),
              "policies": np.array([p.as_tuple() for p in POLICIES], dtype=np.uint8)}
    for m in (7, 3, 1):
        recs = [[list(encode_tile(tiles[t].tolist(), m, p)) for t in range(4)] for p in POLICIES]
        arrays[f"records{m}"] = np.array(recs, dtype=np.uint8)       # [policy, tile, record bytes]
    np.savez_compressed(os.path.join(HERE, "bfp_kat_policies.npz"), **arrays)
    print(f"{len(POLICIES)} policies x 3 formats x 4 tiles written")


if __name__ == "__main__":
    main()
