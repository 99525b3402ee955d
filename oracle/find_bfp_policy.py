"""Which block-float layout policy reproduces a given queue image?

Test infrastructure, like the rest of this directory.  When tile bytes written by the reference's own converter are at
hand (a .tbin of a device image archive, pybuda/pybuda/tti/archive.py:52-66, together with the tensor it was made from),
this packs the tensor with the CPU oracle under every combination of the policy switches -- 3 roundings x 2 overflow
rules x 24 face orders x 2 exponent orders x 2 datum orders = 576 -- and reports the combinations whose bytes equal the
image (several when the data does not exercise a switch, e.g. no value rounds up past the largest magnitude), or the
closest ones.  The winning combination is then set once per process with buda_set_bfp_policy / ref_set_bfp_policy.

    python oracle/find_bfp_policy.py tensor.npy image.tbin Bfp8_b [--header] [--grid R C] [--ublock RT CT] [--order 0|1]
"""
import argparse
import itertools
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from oracle import budaref as R  # noqa: E402


def all_policies():
    for rounding, overflow, faces, eo, do in itertools.product((0, 1, 2), (0, 1), itertools.permutations(range(4)), (0, 1), (0, 1)):
        yield (rounding, overflow, faces, eo, do)


def rank_policies(tensor, image, df, geom=None, with_header=False, src_df=None):
    """[(mismatching bytes, policy tuple)] over all 576 combinations, best first.  tensor: numpy array of up to 4 dims
    (bfloat16 as uint16 with src_df=R.Float16_b); image: the queue image as a uint8 array."""
    image = np.ascontiguousarray(image, dtype=np.uint8).reshape(-1)
    out = []
    try:
        for pol in all_policies():
            R.set_bfp_policy(R.BfpPolicy(pol[0], pol[1], pol[2], pol[3], pol[4]))
            got = R.tilize_pack(tensor, df, geom, with_header, src_df=src_df)
            if got.size != image.size:
                raise ValueError(f"the image holds {image.size} bytes, this tensor packs to {got.size}")
            out.append((int(np.count_nonzero(got != image)), pol))
    finally:
        R.set_bfp_policy(None)
    out.sort(key=lambda t: t[0])
    return out


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("tensor", help=".npy file: the row-major tensor (float32; uint16 = bfloat16 bits)")
    ap.add_argument("image", help="the queue image bytes (.tbin / .bin)")
    ap.add_argument("format", help="Bfp8_b, Bfp4_b, Bfp2_b, Bfp8, Bfp4, Bfp2")
    ap.add_argument("--header", action="store_true", help="records carry the 32-byte header")
    ap.add_argument("--grid", type=int, nargs=2, default=(1, 1))
    ap.add_argument("--ublock", type=int, nargs=2, default=(1, 1))
    ap.add_argument("--order", type=int, default=0, help="ublock scan order: 0 = row major, 1 = column major")
    args = ap.parse_args()
    R.build()
    x = np.load(args.tensor)
    src_df = R.Float16_b if x.dtype == np.uint16 else None
    df = getattr(R, args.format)
    shape = [1] * (4 - x.ndim) + list(x.shape)
    geom = R.Geom.for_shape(shape, tuple(args.grid), tuple(args.ublock), args.order)
    image = np.fromfile(args.image, dtype=np.uint8)
    ranked = rank_policies(x, image, df, geom, args.header, src_df)
    exact = [p for n, p in ranked if n == 0]
    names = "(rounding, overflow, face order, exponent order, datum order)"
    if exact:
        print(f"{len(exact)} of 576 combinations reproduce the image byte for byte {names}:")
        for p in exact:
            print("  ", p)
    else:
        print(f"no combination reproduces the image; closest {names}, mismatching bytes of {image.size}:")
        for n, p in ranked[:8]:
            print("  ", p, n)


if __name__ == "__main__":
    main()
