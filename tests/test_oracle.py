"""CPU tests that pin the oracle: against the reference's golden quantise outputs, against the
reference's own tile-order round-trip property, against its byte-size tables, and (for the
unpinned Bfp encoding) against hand-worked blocks and an independent pure-Python statement of the
frozen spec."""
import itertools
import math
import os
import struct

import numpy as np
import pytest
import torch


# ------------------------------------------------------------------------------------------------
# quantise ops vs the reference's golden vectors (tests/golden/gen_quant_golden.py)
# ------------------------------------------------------------------------------------------------
def test_quantize_matches_reference_golden(oracle, golden):
    g = golden
    assert np.array_equal(oracle.quantize(g["a_x"], g["a_scale"], float(g["a_zp"])), g["a_q"])
    assert np.array_equal(oracle.quantize(g["b_x"], g["b_scale_last"], -5, axis=-1), g["b_q_last"])
    assert np.array_equal(oracle.quantize(g["b_x"], g["b_scale_mid"], 7, axis=1), g["b_q_mid"])
    # BudaQuantize takes a pre-broadcast reciprocal scale: row 0 of it is the per-column vector
    assert np.array_equal(oracle.quantize(g["b_x"], g["c_recip"][0, 0], 2, axis=-1, buda=True), g["c_q"])


def test_dequantize_matches_reference_golden(oracle, golden):
    g = golden
    bits = lambda a: np.ascontiguousarray(a).view(np.uint32)
    assert np.array_equal(bits(oracle.dequantize(g["a_q"], g["a_scale"], 3)), bits(g["a_dq"]))
    assert np.array_equal(bits(oracle.dequantize(g["b_q_last"], g["b_scale_last"], -5, axis=-1)), bits(g["b_dq_last"]))
    assert np.array_equal(bits(oracle.dequantize(g["b_q_mid"], g["b_scale_mid"], 7, axis=1)), bits(g["b_dq_mid"]))
    assert np.array_equal(bits(oracle.dequantize(g["c_q"], g["b_scale_last"], 2, axis=-1)), bits(g["c_dq"]))


def test_requantize_matches_reference_golden(oracle, golden):
    g = golden
    ones = np.ones(128, np.float32)
    assert np.array_equal(oracle.requantize(g["d_acc"], g["d_scales"], ones, 0), g["d_rq"])
    assert np.array_equal(oracle.requantize(g["d_acc"], g["d_scales"], ones, 11), g["d_rq_zp11"])
    assert np.array_equal(oracle.requantize(g["d_acc"], g["d_scales"], g["d_out_scale"], -3), g["d_rq_div_zpm3"])
    assert np.array_equal(oracle.buda_requantize(g["d_acc"], g["d_scales"], 0), g["d_brq"])
    assert np.array_equal(oracle.requantize(g["d_acc"], g["d_scales_mid"], np.ones(32, np.float32), 5, axis=1),
                          g["d_rq_mid_zp5"])


def test_quantize_saturates_and_rounds_half_even(oracle):
    x = np.array([0.025, 0.075, 0.125, -0.025, -0.075, 1e9, -1e9, np.nan, np.inf, -np.inf], np.float32)
    q = oracle.quantize(x, np.array([0.05], np.float32), 0)
    # 0.025/0.05 = 0.5 in binary32 arithmetic rounds to even 0; 0.075/0.05 = 1.5 -> 2; 2.5 -> 2
    assert list(q) == [0, 2, 2, 0, -2, 127, -128, 0, 127, -128]


# ------------------------------------------------------------------------------------------------
# sizes: pybuda/csrc/lower_to_buda/common.cpp:167-190, pybuda/csrc/balancer/balancer_utils.hpp:24-51
# ------------------------------------------------------------------------------------------------
def test_tile_and_format_sizes(oracle):
    R = oracle
    expect = {R.Float32: 4096, R.Float16: 2048, R.Float16_b: 2048, R.Bfp8: 1088, R.Bfp8_b: 1088, R.Bfp4: 576,
              R.Bfp4_b: 576, R.Bfp2: 320, R.Bfp2_b: 320, R.Lf8: 1024, R.UInt16: 2048, R.Int8: 1024, R.Int32: 4096,
              R.RawUInt8: 1024, R.RawUInt16: 2048, R.RawUInt32: 4096}
    for df, n in expect.items():
        assert R.tile_bytes(df, False) == n
        assert R.tile_bytes(df, True) == n + 32
        assert R.lib().ref_data_format_byte_size(df, 1024) == n
    assert R.tile_bytes(R.Invalid) == -1


# ------------------------------------------------------------------------------------------------
# tile order: the reference's exhaustive round trip (balancer/tests/test_tile_layout.cpp:250-281),
# on a reduced range so it runs in seconds, plus direct checks of the address formula
# ------------------------------------------------------------------------------------------------
def _factors(n):
    return [f for f in range(1, n + 1) if n % f == 0]


def test_tile_layout_round_trip(oracle):
    R = oracle
    count = 0
    for tdim, rdim, cdim in itertools.product((1, 3), (1, 4, 6), (1, 4, 6)):
        for grid_r in _factors(rdim):
            for grid_c in _factors(cdim):
                for ur in _factors(rdim // grid_r):
                    for uc in _factors(cdim // grid_c):
                        for order in (0, 1):
                            g = R.Geom(grid_r, grid_c, rdim // (grid_r * ur), cdim // (grid_c * uc), ur, uc, tdim, order)
                            seen = set()
                            for t in range(tdim):
                                for r in range(rdim):
                                    for c in range(cdim):
                                        cr, cc, addr = R.tile_map(g, t, r, c)
                                        assert R.tile_unmap(g, cr, cc, addr) == (t, r, c)
                                        seen.add((cr, cc, addr))
                            assert len(seen) == tdim * rdim * cdim  # a bijection
                            count += 1
    assert count > 200


def test_tile_layout_formula(oracle):
    R = oracle
    # grid 2x1, mblock 2x3, ublock 2x2, t = 2
    g = R.Geom(2, 1, 2, 3, 2, 2, 2, 0)
    # tile (t=1, r=5, c=3): core row 5 // 4 = 1; inside the core r=1, c=3 -> m=0, n=1, u=(1,1)
    cr, cc, addr = R.tile_map(g, 1, 5, 3)
    assert (cr, cc) == (1, 0)
    assert addr == 1 * (2 * 3 * 4) + (0 * 3 + 1) * 4 + 1 * 2 + 1
    gc = R.Geom(2, 1, 2, 3, 2, 2, 2, 1)
    _, _, addr_c = R.tile_map(gc, 1, 5, 3)
    assert addr_c == 1 * (2 * 3 * 4) + (1 * 2 + 0) * 4 + 1 * 2 + 1


# ------------------------------------------------------------------------------------------------
# Bfp encoding: hand-worked blocks and an independent restatement in exact rational arithmetic
# ------------------------------------------------------------------------------------------------
def f2b(x):
    return struct.unpack("<I", struct.pack("<f", x))[0]


def spec_encode_block(bits16, m):
    """The frozen spec in exact integer/rational arithmetic, written independently of the C code:
    q = round_half_even(|x| * 2^(m-1) / 2^(E-127)), saturated; zero/denormal -> 0; Inf/NaN -> max."""
    from fractions import Fraction

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
    return E, np.frombuffer(bitstring.to_bytes(2 * w, "little"), dtype=np.uint8)


def test_bfp8_hand_worked_blocks(oracle):
    R = oracle
    # all zero
    E, d = R.bfp_pack_block(np.zeros(16, np.uint32), 7)
    assert E == 0 and not d.any()
    # 1.0 alone: exponent 127, magnitude 64 (1.0 * 2^6)
    v = [1.0] + [0.0] * 15
    E, d = R.bfp_pack_block([f2b(x) for x in v], 7)
    assert E == 127 and d[0] == 0x40 and not d[1:].any()
    # equal exponents: 1.0, -1.5, 1.984375 (= 127/64), 1.9999 (rounds up to 128 -> saturates to 127)
    v = [1.0, -1.5, 1.984375, 1.9999] + [0.0] * 12
    E, d = R.bfp_pack_block([f2b(x) for x in v], 7)
    assert E == 127 and list(d[:4]) == [0x40, 0x80 | 0x60, 0x7F, 0x7F]
    # an outlier x1000 flattens the rest: 1000 = 1.953125 * 2^9 -> E = 136; 1.0 * 2^6 / 2^9 = 0.125 -> 0
    v = [1000.0, 1.0, 4.0, -8.0, 12.0] + [0.0] * 11
    E, d = R.bfp_pack_block([f2b(x) for x in v], 7)
    assert E == 136
    assert d[0] == 125            # 1000 / 2^9 * 64 = 125
    assert d[1] == 0              # 0.125 rounds to 0 (and loses its sign slot)
    assert d[2] == 0              # 4 / 512 * 64 = 0.5: tie, rounds to even 0
    assert d[3] == 0x80 | 1       # 8 / 512 * 64 = 1.0, negative
    assert d[4] == 2              # 12 / 512 * 64 = 1.5: tie, rounds to even 2
    # denormal input flushes; -0.0 stores +0
    v = [1e-40, -0.0, 2.0 ** -126] + [0.0] * 13
    E, d = R.bfp_pack_block([f2b(x) for x in v], 7)
    assert E == 1 and list(d[:3]) == [0, 0, 0x40]
    # Inf / NaN take the largest magnitude and keep their sign; finite values vanish next to them
    v = [float("inf"), float("-inf"), float("nan"), 3.0e38] + [0.0] * 12
    E, d = R.bfp_pack_block([f2b(x) for x in v], 7)
    assert E == 255 and list(d[:3]) == [0x7F, 0xFF, 0x7F]
    assert d[3] == 56  # 3e38 = 1.7632 * 2^127: 1.7632 * 64 / 2 = 56.4


def test_bfp4_bfp2_sub_byte_order(oracle):
    R = oracle
    v = [1.0, -1.0, 0.5, 0.25] + [0.0] * 12
    E, d = R.bfp_pack_block([f2b(x) for x in v], 3)
    # datums: 1.0 -> 4, -1.0 -> 8|4, 0.5 -> 2, 0.25 -> 1; datum 0 in the low nibble
    assert E == 127 and d[0] == (0xC << 4 | 0x4) and d[1] == (0x1 << 4 | 0x2)
    E, d = R.bfp_pack_block([f2b(x) for x in v], 1)
    # one magnitude bit: 1.0 -> 1, -1.0 -> 2|1, 0.5 -> tie 0.5 -> even 0, 0.25 -> 0
    assert E == 127 and d[0] == (0b11 << 2 | 0b01)


@pytest.mark.parametrize("m", [7, 3, 1])
def test_bfp_oracle_matches_rational_spec(oracle, m):
    rng = np.random.default_rng(100 + m)
    for trial in range(300):
        kind = trial % 6
        if kind == 0:
            x = rng.standard_normal(16).astype(np.float32)
        elif kind == 1:
            x = (rng.standard_normal(16) * 10.0 ** rng.integers(-30, 30, 16)).astype(np.float32)
        elif kind == 2:   # exact ties: small integers against a large power of two
            x = (rng.integers(-9, 10, 16) * 0.5).astype(np.float32)
            x[0] = 64.0
        elif kind == 3:   # raw bit patterns: denormals, NaN, Inf included
            x = rng.integers(0, 2 ** 32, 16, dtype=np.uint64).astype(np.uint32).view(np.float32)
        elif kind == 4:   # tiny blocks (shared exponent below the mantissa width)
            x = (rng.standard_normal(16) * 2.0 ** -124).astype(np.float32)
        else:             # huge blocks
            x = (rng.standard_normal(16) * 2.0 ** 126).astype(np.float32)
        bits = x.view(np.uint32)
        E, d = oracle.bfp_pack_block(bits, m)
        E2, d2 = spec_encode_block([int(b) for b in bits], m)
        assert E == E2 and np.array_equal(d, d2), (trial, x)
        # decode: q * 2^(E-127-(m-1)), exact
        y = oracle.bfp_unpack_block(E, d, m)
        w = m + 1
        word = int.from_bytes(d.tobytes(), "little")
        for i in range(16):
            dat = (word >> (w * i)) & ((1 << w) - 1)
            q, s = dat & ((1 << m) - 1), dat >> m
            with np.errstate(over="ignore"):
                want = np.float32(math.ldexp(q, E - 127 - (m - 1))) if q else np.float32(0.0)
            want = -want if (s and q) else want
            assert y[i].view(np.uint32) == np.float32(want).view(np.uint32)


@pytest.mark.parametrize("df_name", ["Bfp8_b", "Bfp4_b", "Bfp2_b"])
def test_pack_is_idempotent_and_sized(oracle, df_name):
    R = oracle
    df = getattr(R, df_name)
    x = np.random.default_rng(7).standard_normal((2, 3, 64, 96)).astype(np.float32)
    g = R.Geom.for_shape(x.shape, grid=(2, 1), ublock=(1, 3), ublock_order=1)
    for hdr in (False, True):
        img = R.tilize_pack(x, df, geom=g, with_header=hdr)
        assert img.size == 2 * 3 * 2 * 3 * R.tile_bytes(df, hdr)
        y = R.unpack_untilize(img, df, x.shape, geom=g, with_header=hdr)
        assert np.array_equal(R.tilize_pack(y, df, geom=g, with_header=hdr), img)
    # bfloat16 source = same bytes as its widened binary32
    xb = (x.view(np.uint32) >> 16).astype(np.uint16)
    xw = (xb.astype(np.uint32) << 16).view(np.float32)
    assert np.array_equal(R.tilize_pack(xb, df, src_df=R.Float16_b), R.tilize_pack(xw, df))


def test_face_order_and_plain_layout(oracle):
    R = oracle
    x = np.arange(32 * 32, dtype=np.float32).reshape(1, 1, 32, 32)
    img = R.tilize_pack(x, R.Float32).view(np.float32)
    # F0 = rows 0-15 x cols 0-15, F1 = rows 0-15 x cols 16-31, F2 = rows 16-31 x cols 0-15, F3
    assert np.array_equal(img[:256].reshape(16, 16), x[0, 0, :16, :16])
    assert np.array_equal(img[256:512].reshape(16, 16), x[0, 0, :16, 16:])
    assert np.array_equal(img[512:768].reshape(16, 16), x[0, 0, 16:, :16])
    assert np.array_equal(img[768:].reshape(16, 16), x[0, 0, 16:, 16:])
    for dt, df in ((np.int8, R.Int8), (np.int32, R.Int32), (np.float16, R.Float16)):
        a = np.random.default_rng(1).integers(-100, 100, (1, 2, 64, 64)).astype(dt)
        assert np.array_equal(R.unpack_untilize(R.tilize_pack(a, df), df, a.shape, dst_dtype=dt), a)


def test_config1_size(oracle):
    R = oracle
    # [1,1,1024,1024] -> 1024 tiles -> 1,114,112 bytes of Bfp8_b
    g = R.Geom.for_shape([1, 1, 1024, 1024])
    n = R.lib().ref_tilized_bytes(g, (np.ctypeslib.ctypes.c_uint32 * 4)(1, 1, 1024, 1024), R.Bfp8_b, 0)
    assert n == 1114112


@pytest.mark.parametrize("m", [7, 3, 1])
def test_bfp_a_oracle_matches_rational_spec(oracle, m):
    """The "a" formats: 5-bit shared exponent of binary16 sources, same datum rules."""
    from fractions import Fraction

    rng = np.random.default_rng(200 + m)
    for trial in range(200):
        if trial % 3 == 0:
            h = rng.standard_normal(16).astype(np.float16).view(np.uint16)
        elif trial % 3 == 1:
            h = rng.integers(0, 2 ** 16, 16, dtype=np.uint32).astype(np.uint16)   # raw patterns: denormals, Inf, NaN
        else:
            h = (rng.integers(-9, 10, 16) * 0.5).astype(np.float16)
            h[0] = np.float16(64.0)
            h = h.view(np.uint16)
        E, d = oracle.bfp_a_pack_block(h, m)
        exps = [(int(x) >> 10) & 31 for x in h]
        assert E == max(exps)
        qmax, w = (1 << m) - 1, m + 1
        word = int.from_bytes(d.tobytes(), "little")
        for i, (x, e) in enumerate(zip(h, exps)):
            x = int(x)
            if e == 0:
                q = 0
            elif e == 31:
                q = qmax
            else:
                v = Fraction((x & 0x3FF) | 0x400, 1 << 10) * Fraction(2) ** (e - 15) * Fraction(2) ** (m - 1) / Fraction(2) ** (E - 15)
                fl = math.floor(v)
                rem = v - fl
                if rem > Fraction(1, 2) or (rem == Fraction(1, 2) and fl % 2 == 1):
                    fl += 1
                q = min(fl, qmax)
            want = (((x >> 15) << m) | q) if q else 0
            assert (word >> (w * i)) & ((1 << w) - 1) == want, (trial, i)
        y = oracle.bfp_a_unpack_block(E, d, m)
        for i in range(16):
            dat = (word >> (w * i)) & ((1 << w) - 1)
            q, s = dat & qmax, dat >> m
            val = math.ldexp(q, E - 15 - (m - 1)) * (-1 if s and q else 1)
            assert float(y[i]) == val


def test_bfp_a_tilize_round_trip(oracle):
    R = oracle
    x = (np.random.default_rng(3).standard_normal((2, 1, 64, 96)) * 5).astype(np.float16)
    for df in (R.Bfp8, R.Bfp4, R.Bfp2):
        img = R.tilize_pack(x, df)
        assert img.size == 2 * 2 * 3 * R.tile_bytes(df)
        y16 = R.unpack_untilize(img, df, x.shape, dst_dtype=np.float16)
        y32 = R.unpack_untilize(img, df, x.shape)
        assert np.array_equal(y16.astype(np.float32), y32)          # decoded values are exact in binary16
        assert np.array_equal(R.tilize_pack(y16, df), img)           # idempotent


def test_i8_matmul_oracle_matches_the_golden_chain(oracle):
    """int8 matmul -> int32 (op/eval/common.py:50-65), then requantization / dequantization of the result
    (csrc/graph_lib/python_bindings.cpp:655-676, op/eval/buda/quantize.py:35-53), against torch."""
    g = torch.Generator().manual_seed(9)
    a = torch.randint(-128, 128, (96, 128), generator=g, dtype=torch.int8)
    w = torch.randint(-128, 128, (128, 256), generator=g, dtype=torch.int8)
    img = oracle.tilize_pack(w.reshape(1, 1, 128, 256).numpy(), oracle.Int8)
    assert img.size == 4 * 8 * 1024                      # 32 Int8 tiles of 1024 bytes, no exponent sections
    acc = a.int() @ w.int()
    # the reference evaluates the matmul in float32: identical while the sums stay below 2^24
    assert torch.equal((a.float() @ w.float()).to(torch.int32), acc)
    assert np.array_equal(oracle.i8_matmul(a.numpy(), img, 128, 256), acc.numpy())
    for scale in (torch.tensor([3e-4]), torch.rand(256, generator=g) * 1e-3 + 1e-5):
        want_q = torch.clamp(torch.round(acc.float() * scale + 3.0), -128, 127).to(torch.int8)
        assert np.array_equal(oracle.i8_matmul(a.numpy(), img, 128, 256, scale.numpy(), 3.0, 1), want_q.numpy())
        want_f = (acc.float() - 3.0) * scale
        assert np.array_equal(oracle.i8_matmul(a.numpy(), img, 128, 256, scale.numpy(), 3.0, 2), want_f.numpy())


@pytest.mark.parametrize("th", [1, 2, 4, 8, 16])
def test_tiny_tiles_equal_zero_padded_full_tiles(oracle, th):
    """A tile of a tiny-tile queue (TileDim, csrc/lower_to_buda/common.hpp:80-90; rows per tile as in
    op/eval/buda/tilizer.py:40-52) holds `th` tensor rows in a full-size record: the image equals that of the
    tensor with every group of `th` rows padded with zero rows to 32."""
    rng = np.random.default_rng(th)
    rt = 3
    x = rng.standard_normal((2, 2, rt * th, 96)).astype(np.float32)
    g = oracle.Geom.for_shape(x.shape, tile_height=th)
    xp = np.zeros((2, 2, rt * 32, 96), np.float32)
    for r in range(rt):
        xp[:, :, r * 32:r * 32 + th] = x[:, :, r * th:(r + 1) * th]
    for df in (oracle.Bfp8_b, oracle.Bfp2_b, oracle.Float32):
        img = oracle.tilize_pack(x, df, g)
        assert img.size == 2 * 2 * rt * 3 * oracle.tile_bytes(df)
        assert np.array_equal(img, oracle.tilize_pack(xp, df))
        back = oracle.unpack_untilize(img, df, x.shape, geom=g)
        full = oracle.unpack_untilize(img, df, xp.shape)
        for r in range(rt):
            assert np.array_equal(back[:, :, r * th:(r + 1) * th].view(np.uint32), full[:, :, r * 32:r * 32 + th].view(np.uint32))


def _kat():
    import os
    return np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "bfp_kat.npz"))


@pytest.mark.parametrize("m", [7, 3, 1])
def test_oracle_matches_committed_known_answers(oracle, m):
    """tests/golden/bfp_kat.npz was computed in exact rational arithmetic (tests/golden/bfp_spec.py), independently of
    the C oracle: 256 blocks incl. ties, saturation, denormals, Inf / NaN and both ends of the exponent range."""
    k = _kat()
    assert int(k["spec_version"][0]) == 1
    for i in range(k["x"].shape[0]):
        E, d = oracle.bfp_pack_block(k["x"][i], m)
        assert E == int(k[f"E{m}"][i]) and np.array_equal(d, k[f"data{m}"][i]), i
        y = oracle.bfp_unpack_block(E, d, m)
        assert np.array_equal(y.view(np.uint32), k[f"decoded{m}"][i]), i


def test_known_answer_generator_is_reproducible():
    """The committed fixture is what the committed generator writes."""
    import importlib.util, os, sys
    gdir = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
    sys.path.insert(0, gdir)
    try:
        spec = importlib.util.spec_from_file_location("gen_bfp_kat", os.path.join(gdir, "gen_bfp_kat.py"))
        gen = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(gen)
        blocks = gen.hand_picked() + gen.random_blocks(256 - len(gen.hand_picked()), seed=20240)
        k = _kat()
        assert np.array_equal(np.array(blocks, dtype=np.uint32), k["x"])
        from bfp_spec import encode_block
        for i in (0, 3, 5, 17, 100, 255):
            E, data = encode_block(blocks[i], 7)
            assert E == int(k["E7"][i]) and list(data) == list(k["data7"][i])
    finally:
        sys.path.remove(gdir)



# ------------------------------------------------------------------------------------------------
# Layout policies: the switches for what the published format description leaves open
# ------------------------------------------------------------------------------------------------
def _policy_kat():
    import os
    return np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "bfp_kat_policies.npz"))


def _kat_tiles():
    """The 256 known-answer blocks laid out as the face rows of four 32x32 tiles side by side: [1,1,32,128]."""
    k = _kat()
    x = np.zeros((1, 1, 32, 128), np.uint32)
    for b in range(256):
        t, blk = divmod(b, 64)
        face, fr = divmod(blk, 16)
        x[0, 0, (face >> 1) * 16 + fr, t * 32 + (face & 1) * 16: t * 32 + (face & 1) * 16 + 16] = k["x"][b]
    return x


def _spec_decode_tiles(records, m, policy_row):
    """What the exact-arithmetic spec decodes from four tile records laid side by side: [1,1,32,128] bit patterns."""
    import os, sys
    gdir = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
    sys.path.insert(0, gdir)
    try:
        from bfp_spec import Policy, decode_block
    finally:
        sys.path.remove(gdir)
    pol = Policy(int(policy_row[0]), int(policy_row[1]), tuple(int(v) for v in policy_row[2:6]), int(policy_row[6]), int(policy_row[7]))
    w = m + 1
    rec = 64 + 64 * 2 * w
    out = np.zeros((1, 1, 32, 128), np.uint32)
    records = np.asarray(records, np.uint8).reshape(4, rec)
    for t in range(4):
        for pos, face in enumerate(pol.face_order):
            for fr in range(16):
                k = pos * 16 + fr
                E = int(records[t, k ^ 3 if pol.exponent_order else k])
                data = records[t, 64 + k * 2 * w: 64 + (k + 1) * 2 * w].tobytes()
                r, c = (face >> 1) * 16 + fr, t * 32 + (face & 1) * 16
                out[0, 0, r, c:c + 16] = decode_block(E, data, m, pol)
    return out


@pytest.mark.parametrize("df_name,m", [("Bfp8_b", 7), ("Bfp4_b", 3), ("Bfp2_b", 1)])
def test_oracle_matches_known_answers_of_every_policy(oracle, df_name, m):
    """tests/golden/bfp_kat_policies.npz holds the tile records of the known-answer values under each non-default
    policy, computed by the exact-arithmetic spec; the C oracle with the same switches must write the same bytes,
    and read them back to what the spec decodes."""
    kp = _policy_kat()
    x = _kat_tiles().view(np.float32)
    try:
        for pi, row in enumerate(kp["policies"]):
            pol = oracle.BfpPolicy(int(row[0]), int(row[1]), tuple(int(v) for v in row[2:6]), int(row[6]), int(row[7]))
            oracle.set_bfp_policy(pol)
            img = oracle.tilize_pack(x, getattr(oracle, df_name))
            want = kp[f"records{m}"][pi].reshape(-1)
            assert np.array_equal(img, want), (pi, row.tolist(), int(np.argmax(img != want)))
            back = oracle.unpack_untilize(img, getattr(oracle, df_name), x.shape).view(np.uint32)
            assert np.array_equal(back, _spec_decode_tiles(want, m, row)), (pi, "decode")
    finally:
        oracle.set_bfp_policy(None)


def test_policy_switches_one_by_one(oracle):
    """Each switch does what its name says, on hand-worked blocks."""
    from oracle import budaref as R
    f = lambda v: np.array([v], np.float32).view(np.uint32)[0]
    try:
        # rounding: 1.9921875 = 255/128 -> 7-bit magnitude 127.5: nearest-even saturates at 127, truncation gives 127;
        # 1.0234375 = 65.5/64 -> nearest even 66 (65.5 -> 66), truncation 65
        blk = np.zeros(16, np.uint32)
        blk[0], blk[1] = f(1.0), f(1.0234375)
        E, d = R.bfp_pack_block(blk, 7)
        assert (E, d[0], d[1]) == (127, 64, 66)
        R.set_bfp_policy(R.BfpPolicy(rounding=1))
        E, d = R.bfp_pack_block(blk, 7)
        assert (E, d[0], d[1]) == (127, 64, 65)
        # "add half, then truncate": a tie goes away from zero whatever the kept bit: 1.0078125 = 64.5/64 -> 65 (nearest even: 64),
        # 1.0234375 = 65.5/64 -> 66 either way, and anything below the tie still goes down
        blk[2], blk[3] = f(1.0078125), f(-1.00390625)
        R.set_bfp_policy(None)
        E, d = R.bfp_pack_block(blk, 7)
        assert (E, d[0], d[1], d[2], d[3]) == (127, 64, 66, 64, 0x80 | 64)
        R.set_bfp_policy(R.BfpPolicy(rounding=2))
        E, d = R.bfp_pack_block(blk, 7)
        assert (E, d[0], d[1], d[2], d[3]) == (127, 64, 66, 65, 0x80 | 64)
        # overflow: 1.99609375 rounds up to 128 > 127: saturate keeps E, bump raises E and halves every magnitude
        blk[:] = 0
        blk[0], blk[1] = f(1.99609375), f(-1.0)
        R.set_bfp_policy(None)
        E, d = R.bfp_pack_block(blk, 7)
        assert (E, d[0], d[1]) == (127, 127, 0x80 | 64)
        R.set_bfp_policy(R.BfpPolicy(overflow=1))
        E, d = R.bfp_pack_block(blk, 7)
        assert (E, d[0], d[1]) == (128, 64, 0x80 | 32)
        # truncation never overflows, so the two switches together leave E alone
        R.set_bfp_policy(R.BfpPolicy(rounding=1, overflow=1))
        E, d = R.bfp_pack_block(blk, 7)
        assert (E, d[0], d[1]) == (127, 127, 0x80 | 64)
        # datum order: Bfp4 datums 0..7 share the first 32-bit word; big order puts datum 0 in the top nibble of byte 3
        blk[:] = 0
        blk[0] = f(1.0)      # 3-bit magnitude 4
        R.set_bfp_policy(None)
        _, d = R.bfp_pack_block(blk, 3)
        assert d[0] == 0x04 and not d[1:].any()
        R.set_bfp_policy(R.BfpPolicy(datum_order=1))
        _, d = R.bfp_pack_block(blk, 3)
        assert d[3] == 0x40 and not d[:3].any() and not d[4:].any()
        # face order and exponent order on one tile: a single 2.0 in face 2 (row 16, column 0)
        x = np.zeros((1, 1, 32, 32), np.float32)
        x[0, 0, 16, 0] = 2.0
        R.set_bfp_policy(None)
        img = R.tilize_pack(x, R.Bfp8_b)
        assert img[32] == 128 and img[64 + 32 * 16] == 64
        R.set_bfp_policy(R.BfpPolicy(face_order=(2, 0, 1, 3), exponent_order=1))
        img = R.tilize_pack(x, R.Bfp8_b)
        assert img[0 ^ 3] == 128 and img[64] == 64           # face 2 is stored first; its exponent sits in byte 3 of word 0
        assert np.array_equal(R.unpack_untilize(img, R.Bfp8_b, x.shape), x)
        with pytest.raises(ValueError):
            R.set_bfp_policy(R.BfpPolicy(face_order=(0, 0, 1, 2)))
    finally:
        R.set_bfp_policy(None)


# ------------------------------------------------------------------------------------------------
# Runtime tensor transforms: the numpy restatements against vectors the reference's own functions produced
# ------------------------------------------------------------------------------------------------
def _transform_golden():
    import os
    return np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "transform_golden.npz"))


def test_transform_restatements_match_the_reference_vectors(oracle):
    g = _transform_golden()
    k = 0
    while f"emb{k}_in" in g.files:
        n, w, q_rt, q_ct = (int(v) for v in g[f"emb{k}_meta"])
        got = oracle.embedding_index(g[f"emb{k}_in"], n, q_rt)
        assert got.shape == g[f"emb{k}_out"].shape == (w, 1, q_rt * 32, q_ct * 32)
        assert np.array_equal(got, g[f"emb{k}_out"]), ("embedding index", k)
        k += 1
    assert k == 5
    k = 0
    while f"pre{k}_in" in g.files:
        got = oracle.prestride_act(g[f"pre{k}_in"], int(g[f"pre{k}_stride"][0]))
        assert np.array_equal(got, g[f"pre{k}_out"]), ("prestride", k)
        k += 1
    assert k == 4
    k = 0
    while f"pad{k}_in" in g.files:
        x, bc, want = g[f"pad{k}_in"], list(g[f"pad{k}_bcast"]), g[f"pad{k}_out"]
        x4 = x.reshape((1,) * (4 - x.ndim) + x.shape)
        got = oracle.pad_to_tiles(x4, replicate_rows=(2 in bc or -2 in bc), replicate_cols=(3 in bc or -1 in bc))
        assert np.array_equal(got.reshape(want.shape), want), ("pad", k)
        k += 1
    assert k == 5


# ------------------------------------------------------------------------------------------------
# Lf8 (1-5-2 float per element).  Parity unpinned: the reference documents the field widths only
# (docs/public/dataformats.rst:24).  The oracle is checked against the exact-arithmetic spec's committed
# vectors and against an independent implementation of the same IEEE-style format (torch.float8_e5m2).
# ------------------------------------------------------------------------------------------------
def _lf8_kat():
    return np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "lf8_kat.npz"))


def test_lf8_oracle_matches_committed_known_answers(oracle):
    kat = _lf8_kat()
    vals = kat["bits"].view(np.float32)
    got = np.array([oracle.lf8_encode(v) for v in vals.astype(np.float64)], dtype=np.uint8)
    nan = np.isnan(vals)
    assert np.array_equal(got[~nan], kat["codes"][~nan])
    assert np.all((got[nan] & 0x7F) == 0x7F)
    for c in range(256):
        want = np.array([kat["decode"][c]], dtype=np.uint32).view(np.float32)[0]
        have = np.float32(oracle.lf8_decode(c))
        assert (np.isnan(want) and np.isnan(have)) or want.view(np.uint32) == have.view(np.uint32), c


def test_lf8_spec_vectors_are_reproducible():
    import importlib.util
    spec = importlib.util.spec_from_file_location("bfp_spec_lf8", os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "bfp_spec.py"))
    S = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(S)
    kat = _lf8_kat()
    for i in list(range(0, 60)) + list(range(60, len(kat["bits"]), 211)):
        assert S.lf8_encode_bits(int(kat["bits"][i])) == int(kat["codes"][i])


def test_lf8_oracle_agrees_with_an_independent_e5m2_conversion(oracle):
    if not hasattr(torch, "float8_e5m2"):
        pytest.skip("this torch has no float8_e5m2")
    bits = (np.arange(65536, dtype=np.uint32) << 16)          # every bfloat16 pattern, widened
    rng = np.random.default_rng(5)
    more = (rng.standard_normal(65536) * np.exp(rng.uniform(-14, 12, 65536))).astype(np.float32).view(np.uint32)
    x = np.concatenate([bits, more]).view(np.float32).reshape(1, 1, 128, 1024)
    img = oracle.tilize_pack(x, oracle.Lf8)
    assert img.size == x.size
    codes = oracle.unpack_untilize(img, oracle.Lf8, x.shape, np.uint8, dst_df=oracle.Lf8)   # relayout back to row-major
    t8 = torch.from_numpy(x.copy()).to(torch.float8_e5m2)
    nan = np.isnan(x)
    assert np.array_equal(codes[~nan], t8.view(torch.uint8).numpy()[~nan])
    back = oracle.unpack_untilize(img, oracle.Lf8, x.shape, np.float32)
    assert np.array_equal(back.view(np.uint32)[~nan], t8.to(torch.float32).numpy().view(np.uint32)[~nan])
    assert np.all(np.isnan(back[nan]))
    # bfloat16 and binary16 sources and destinations
    xb = (x.view(np.uint32) >> 16).astype(np.uint16)          # truncated to bfloat16: compare with its own widening
    img_of_widened = oracle.tilize_pack((xb.astype(np.uint32) << 16).view(np.float32), oracle.Lf8)
    assert np.array_equal(oracle.tilize_pack(xb, oracle.Lf8, src_df=oracle.Float16_b), img_of_widened)
    xh = x.astype(np.float16)
    imgh = oracle.tilize_pack(xh, oracle.Lf8)
    th8 = torch.from_numpy(xh.copy()).to(torch.float8_e5m2)
    nanh = np.isnan(xh)
    codesh = oracle.unpack_untilize(imgh, oracle.Lf8, x.shape, np.uint8, dst_df=oracle.Lf8)
    assert np.array_equal(codesh[~nanh], th8.view(torch.uint8).numpy()[~nanh])
    backh = oracle.unpack_untilize(imgh, oracle.Lf8, x.shape, np.float16)
    assert np.array_equal(backh.view(np.uint16), (codesh.astype(np.uint16) << 8))


def test_policy_finder_recovers_the_policy_an_image_was_written_under(oracle):
    """oracle/find_bfp_policy.py: the search a maintainer runs when real tile bytes of the reference's converter appear."""
    from oracle import find_bfp_policy as F
    rng = np.random.default_rng(11)
    x = rng.standard_normal((1, 1, 64, 64)).astype(np.float32)
    x.reshape(-1)[::37] *= 1e3                     # outliers: blocks with small values next to a large one
    x[0, 0, 0, :16] = 1.99609375                   # a block that rounds up past the largest magnitude (overflow rule shows)
    x[0, 0, 1, :16] = np.float32(1.0078125)        # ties (the three roundings differ)
    want = (2, 1, (2, 0, 3, 1), 1, 0)
    try:
        oracle.set_bfp_policy(oracle.BfpPolicy(*want))
        image = oracle.tilize_pack(x, oracle.Bfp8_b)
    finally:
        oracle.set_bfp_policy(None)
    ranked = F.rank_policies(x, image, oracle.Bfp8_b)
    exact = [p for n, p in ranked if n == 0]
    assert exact == [want]
    # the default image is found as the default policy, and the switches the data cannot show come back as alternatives
    flat = np.full((1, 1, 32, 32), 1.0, np.float32)
    ranked = F.rank_policies(flat, oracle.tilize_pack(flat, oracle.Bfp8_b), oracle.Bfp8_b)
    exact = [p for n, p in ranked if n == 0]
    assert (0, 0, (0, 1, 2, 3), 0, 0) in exact and len(exact) > 1
