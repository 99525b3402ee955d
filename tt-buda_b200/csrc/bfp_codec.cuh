// Block-float (Bfp8_b / Bfp4_b / Bfp2_b) encode and decode of one 16-value block in registers.
//
// Format (published description: docs/public/dataformats.rst:59-89 of the reference, drawings
// docs/public/images/bfp{8,4,2}_blocks.png): the 16 values of a block share one 8-bit exponent E,
// the largest biased binary32 exponent in the block; a datum is sign + M magnitude bits
// (M = 7 / 3 / 1) with no implied one:  q = round(|x| * 2^(M-1) / 2^(E-127)).
// Choices the description leaves open, frozen here and in the CPU oracle alike:
//   round to nearest, ties to even; a round-up past 2^M-1 saturates (E is not bumped);
//   zero / denormal inputs encode as 0; Inf / NaN encode the largest magnitude;
//   a zero magnitude is stored with sign 0; datum i sits in bits [i*(M+1), (i+1)*(M+1)) of the
//   block's little-endian bit string;  q == 0 decodes to +0.0.
//
// The encoder is a floating-point formulation: one fused multiply-add per value computes
// |x| * 2^(M-1+127-E) + 1.5*2^23, whose single rounding IS round-to-nearest-even at integer
// granularity, leaving q in the low mantissa byte; flush-to-zero on the inputs gives the denormal
// policy for free.  Blocks whose scale 2^(M-1+127-E) is not a normal binary32 (E < M-1, or
// E > M+252) take an integer path instead.
#pragma once

#include <stdint.h>

#include "buda_common.cuh"

namespace buda {

constexpr uint32_t kMagicBits = 0x4b400000u;  // 1.5 * 2^23: ulp 1, even

template <int M>
struct BfpTraits {
    static constexpr uint32_t qmax = (1u << M) - 1u;
    static constexpr int words = 16 * (M + 1) / 32;  // 32-bit words of mantissa data per block: 4 / 2 / 1
    static constexpr int bytes = 16 * (M + 1) / 8;   // 16 / 8 / 4
};

// Integer encoder of one value (used for blocks at the ends of the exponent range, and by the general
// kernel flavour after a shared exponent was raised).  rmode: 0 round the dropped bits to nearest even, 1 drop them,
// 2 add half an ulp of the kept width and then drop them (nearest, ties away from zero) -- instead of rounding to
// nearest even.  *over is set when the magnitude of a finite value came out above the largest one.
__device__ __forceinline__ uint32_t bfp_encode_datum_int(uint32_t bits, uint32_t E, int m, int rmode = 0, bool *over = nullptr)
{
    const uint32_t qmax = (1u << m) - 1u;
    uint32_t e = (bits >> 23) & 0xffu, q;
    if (e == 0) {
        q = 0;
    } else if (e == 255) {
        q = qmax;
    } else {
        uint32_t sig = (bits & 0x7fffffu) | 0x800000u;
        uint32_t shift = E - e + 24u - (uint32_t)m;
        if (shift > 25u) {
            q = 0;
        } else {
            uint32_t kept = sig >> shift, rem = sig & ((1u << shift) - 1u), half = 1u << (shift - 1u);
            kept += ((rmode == 0 && (rem > half || (rem == half && (kept & 1u)))) || (rmode == 2 && rem >= half)) ? 1u : 0u;
            if (over && kept > qmax) *over = true;
            q = kept < qmax ? kept : qmax;
        }
    }
    return q ? (((bits >> 31) << m) | q) : 0u;
}

// Reverses the order of the (M + 1)-bit datum fields inside one 32-bit word (its own inverse).
template <int M>
__device__ __forceinline__ uint32_t reverse_datum_fields(uint32_t w)
{
    if (M == 7) return __byte_perm(w, 0u, 0x0123);
    if (M == 3) {
        const uint32_t r = __byte_perm(w, 0u, 0x0123);
        return ((r & 0x0f0f0f0fu) << 4) | ((r >> 4) & 0x0f0f0f0fu);
    }
    const uint32_t r = __brev(w);
    return ((r & 0x55555555u) << 1) | ((r >> 1) & 0x55555555u);
}

// Largest biased binary32 exponent of the 16 values.  The maximum of the magnitudes is taken as floats: the absolute
// values fold into the min/max instructions, three operands at a time.  A NaN operand gives 0x7fffffff, so NaN and
// Inf both end with exponent field 255, as an integer maximum of the magnitude bits would; for every other input
// the two maxima have the same exponent field.
__device__ __forceinline__ uint32_t bfp_block_exponent(const uint32_t (&x)[16])
{
    float mf;
    asm("{\n\t.reg .f32 a<16>, m<7>;\n\t"
        "abs.f32 a0, %1;\n\tabs.f32 a1, %2;\n\tabs.f32 a2, %3;\n\tabs.f32 a3, %4;\n\t"
        "abs.f32 a4, %5;\n\tabs.f32 a5, %6;\n\tabs.f32 a6, %7;\n\tabs.f32 a7, %8;\n\t"
        "abs.f32 a8, %9;\n\tabs.f32 a9, %10;\n\tabs.f32 a10, %11;\n\tabs.f32 a11, %12;\n\t"
        "abs.f32 a12, %13;\n\tabs.f32 a13, %14;\n\tabs.f32 a14, %15;\n\tabs.f32 a15, %16;\n\t"
        "max.NaN.f32 m0, a0, a1, a2;\n\tmax.NaN.f32 m1, a3, a4, a5;\n\tmax.NaN.f32 m2, a6, a7, a8;\n\t"
        "max.NaN.f32 m3, a9, a10, a11;\n\tmax.NaN.f32 m4, a12, a13, a14;\n\t"
        "max.NaN.f32 m5, m0, m1, m2;\n\tmax.NaN.f32 m6, m3, m4, a15;\n\t"
        "max.NaN.f32 %0, m5, m6;\n\t}"
        : "=f"(mf)
        : "f"(__uint_as_float(x[0])), "f"(__uint_as_float(x[1])), "f"(__uint_as_float(x[2])), "f"(__uint_as_float(x[3])),
          "f"(__uint_as_float(x[4])), "f"(__uint_as_float(x[5])), "f"(__uint_as_float(x[6])), "f"(__uint_as_float(x[7])),
          "f"(__uint_as_float(x[8])), "f"(__uint_as_float(x[9])), "f"(__uint_as_float(x[10])), "f"(__uint_as_float(x[11])),
          "f"(__uint_as_float(x[12])), "f"(__uint_as_float(x[13])), "f"(__uint_as_float(x[14])), "f"(__uint_as_float(x[15])));
    return __float_as_uint(mf) >> 23;
}

// |x| * S + 1.5 * 2^23 in one fused multiply-add: rounded to nearest even (R = 0), or toward zero (R = 1: truncation of
// the magnitude, every operand being non-negative).  The magnitude sits in the low bits of the result, unsaturated.
// R = 2, half an ulp added before the truncation: the constant is 1.5 * 2^22 + 0.5, where the unit in the last place is
// one half, so the truncated sum counts floor(2 v + 1) halves and q = floor(v + 0.5) is that count shifted right by
// one; it is handed back on top of 1.5 * 2^23 like the other two.
template <int R>
__device__ __forceinline__ uint32_t bfp_quantise_bits(uint32_t xbits, float S)
{
    float r;
    if (R == 2) {
        asm("{\n\t.reg .f32 t;\n\tabs.ftz.f32 t, %1;\n\tfma.rz.ftz.f32 %0, t, %2, %3;\n\t}"
            : "=f"(r) : "f"(__uint_as_float(xbits)), "f"(S), "f"(6291456.5f));
        return kMagicBits + ((__float_as_uint(r) - 0x4ac00000u) >> 1);
    }
    if (R == 1)
        asm("{\n\t.reg .f32 t;\n\tabs.ftz.f32 t, %1;\n\tfma.rz.ftz.f32 %0, t, %2, %3;\n\t}"
            : "=f"(r) : "f"(__uint_as_float(xbits)), "f"(S), "f"(12582912.0f));
    else
        asm("{\n\t.reg .f32 t;\n\tabs.ftz.f32 t, %1;\n\tfma.rn.ftz.f32 %0, t, %2, %3;\n\t}"
            : "=f"(r) : "f"(__uint_as_float(xbits)), "f"(S), "f"(12582912.0f));
    return __float_as_uint(r);
}

// Signs and saturated magnitudes (y: magic constant + q, one per value) -> the packed datums of the block.
template <int M>
__device__ __forceinline__ void bfp_pack_datums(const uint32_t (&x)[16], const uint32_t (&y)[16], uint32_t (&out)[BfpTraits<M>::words])
{
    uint32_t D[4];
#pragma unroll
    for (int w = 0; w < 4; w++) {
        // Q: the four magnitudes, one per byte.  T: the four sign-carrying top bytes.
        uint32_t Q = __byte_perm(__byte_perm(y[4 * w], y[4 * w + 1], 0x0040),
                                 __byte_perm(y[4 * w + 2], y[4 * w + 3], 0x0040), 0x5410);
        uint32_t T = __byte_perm(__byte_perm(x[4 * w], x[4 * w + 1], 0x0073),
                                 __byte_perm(x[4 * w + 2], x[4 * w + 3], 0x0073), 0x5410);
        if (M == 7) {
            uint32_t nz = (Q + 0x7f7f7f7fu) & 0x80808080u;  // bit 7 of a byte set iff its q > 0
            D[w] = Q | (T & nz);
        } else if (M == 3) {
            uint32_t nz = (Q + 0x07070707u) & 0x08080808u;
            D[w] = Q | ((T >> 4) & nz);
        } else {
            uint32_t nz = (Q + 0x01010101u) & 0x02020202u;
            D[w] = Q | ((T >> 6) & nz);
        }
    }
    if (M == 7) {
#pragma unroll
        for (int w = 0; w < 4; w++) out[w % BfpTraits<M>::words] = D[w];
    } else if (M == 3) {
        // two 4-bit datums per byte: bytes 0 and 2 of (D | D >> 4)
        uint32_t t0 = D[0] | (D[0] >> 4), t1 = D[1] | (D[1] >> 4);
        uint32_t t2 = D[2] | (D[2] >> 4), t3 = D[3] | (D[3] >> 4);
        out[0] = __byte_perm(t0, t1, 0x6420);
        out[1 % BfpTraits<M>::words] = __byte_perm(t2, t3, 0x6420);
    } else {
        // four 2-bit datums per byte: byte 0 of u, u = t | t >> 12, t = D | D >> 6
        uint32_t u[4];
#pragma unroll
        for (int w = 0; w < 4; w++) {
            uint32_t t = D[w] | (D[w] >> 6);
            u[w] = t | (t >> 12);
        }
        out[0] = __byte_perm(__byte_perm(u[0], u[1], 0x0040), __byte_perm(u[2], u[3], 0x0040), 0x5410);
    }
}

// One block through the integer encoder.  Returns true when a finite magnitude rounded up past the largest one.
template <int M>
__device__ __forceinline__ bool bfp_encode16_int(const uint32_t (&x)[16], uint32_t E, int rmode, uint32_t (&out)[BfpTraits<M>::words])
{
    bool over = false;
#pragma unroll
    for (int w = 0; w < BfpTraits<M>::words; w++) out[w] = 0;
#pragma unroll
    for (int i = 0; i < 16; i++) {
        uint32_t d = bfp_encode_datum_int(x[i], E, M, rmode, &over);
        out[(i * (M + 1)) / 32] |= d << ((i * (M + 1)) % 32);
    }
    return over;
}

// Encode one block.  x: the 16 values as binary32 bit patterns.  Returns the shared exponent and
// the packed datums (out[0] holds datums 0.., little-endian).  R: rounding (0 nearest even; 1 truncate, the same
// instruction count: only the rounding mode of the multiply-add differs; 2 half added before the truncation).
template <int M, int R = 0>
__device__ __forceinline__ void bfp_encode16(const uint32_t (&x)[16], uint32_t &E_out,
                                             uint32_t (&out)[BfpTraits<M>::words])
{
    constexpr uint32_t qmax = BfpTraits<M>::qmax;
    const uint32_t E = bfp_block_exponent(x);
    E_out = E;

    if (E + 1u >= (uint32_t)M && E <= (uint32_t)(M + 252)) {
        const float S = __uint_as_float((uint32_t)(M + 253 - (int)E) << 23);  // 2^(M-1+127-E)
        uint32_t y[16];
#pragma unroll
        for (int i = 0; i < 16; i++) y[i] = min(bfp_quantise_bits<R>(x[i], S), kMagicBits + qmax);  // Inf / NaN and round-ups saturate here
        bfp_pack_datums<M>(x, y, out);
    } else {
        (void)bfp_encode16_int<M>(x, E, R, out);
    }
}

// The same under a layout policy (general kernel flavour): truncation instead of rounding, a shared exponent that
// is raised by one when a magnitude rounds up past the largest one (every value of the block is then encoded
// against the raised exponent), and the datum fields of each 32-bit word in reverse order.
// (Inlined on purpose: a call that takes the block by reference would pin the 16 values to local memory for the whole
// kernel, and every access of the hot path would go through it -- measured at 0.65 of the plain kernel's speed.)
template <int M>
__device__ __forceinline__ void bfp_encode16_raised(const uint32_t (&x)[16], uint32_t E, int rmode, uint32_t (&out)[BfpTraits<M>::words])
{
    (void)bfp_encode16_int<M>(x, E, rmode, out);
}

// raise_limit: the shared exponent may be raised while it is below this (255; 143 = 31 + 112 for the widened
// binary16 values of the "a" formats, whose exponent byte has 5 bits).
template <int M>
__device__ __forceinline__ void bfp_encode16_policy(const uint32_t (&x)[16], uint32_t &E_out, uint32_t (&out)[BfpTraits<M>::words],
                                                    const BfpPolicy &pol, uint32_t raise_limit)
{
    constexpr uint32_t qmax = BfpTraits<M>::qmax;
    uint32_t E = bfp_block_exponent(x);
    bool over = false;
    if (E + 1u >= (uint32_t)M && E <= (uint32_t)(M + 252)) {
        const float S = __uint_as_float((uint32_t)(M + 253 - (int)E) << 23);
        uint32_t y[16];
        if (pol.rmode == 1) {
#pragma unroll
            for (int i = 0; i < 16; i++) y[i] = bfp_quantise_bits<1>(x[i], S);
        } else if (pol.rmode == 2) {
#pragma unroll
            for (int i = 0; i < 16; i++) y[i] = bfp_quantise_bits<2>(x[i], S);
        } else {
#pragma unroll
            for (int i = 0; i < 16; i++) y[i] = bfp_quantise_bits<0>(x[i], S);
        }
        uint32_t top = 0;
#pragma unroll
        for (int i = 0; i < 16; i++) {
            top = max(top, y[i]);
            y[i] = min(y[i], kMagicBits + qmax);
        }
        over = top > kMagicBits + qmax;     // below the limit every value of the block is finite
        bfp_pack_datums<M>(x, y, out);
    } else {
        over = bfp_encode16_int<M>(x, E, pol.rmode, out);
    }
    if (pol.bump && over && E < raise_limit) {
        E += 1u;
        bfp_encode16_raised<M>(x, E, pol.rmode, out);
    }
    E_out = E;
    if (pol.datum_be) {
#pragma unroll
        for (int w = 0; w < BfpTraits<M>::words; w++) out[w] = reverse_datum_fields<M>(out[w]);
    }
}

// ------------------------------------------------------------------------------------------------
// bfloat16 sources, two values per 32-bit word.  The torch dtype that feeds a Bfp*_b queue is bfloat16
// (pybuda/pybuda/tensor.py:602-632), so this is the common case for parameters; working on packed pairs
// halves the integer work of the binary32 formulation above (which bounds that kernel: ALU pipe 64 %).
//   |x| pairs: one AND; block maximum: max.u16x2; quantise: fma.rn.bf16x2(|x|, 2^(M-1+127-E), 128.0) -- a bfloat16
//   in [128, 256) has ulp 1, so the single rounding of the fma IS round-to-nearest-even at integer granularity
//   and q sits in the low 7 bits; a round-up to 256, Inf and NaN are caught by min.u16x2 against 128 + qmax.
// Blocks with E < 17 (where a denormal input times the scale could still round to 1) or E > 253 (scale not a
// normal bfloat16 for every M) return false: the caller widens the values and uses bfp_encode16.
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t max_u16x2(uint32_t a, uint32_t b)
{
    uint32_t d;
    asm("max.u16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ uint32_t min_u16x2(uint32_t a, uint32_t b)
{
    uint32_t d;
    asm("min.u16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}

template <int M>
__device__ __forceinline__ bool bfp_encode16_bf16(const uint32_t (&h)[8], uint32_t &E_out, uint32_t (&out)[BfpTraits<M>::words])
{
    constexpr uint32_t qmax = BfpTraits<M>::qmax;
    uint32_t mx;
    // block maximum of the magnitudes as bfloat16 pairs; a NaN gives 0x7fff, i.e. exponent field 255 like Inf
    asm("{\n\t.reg .b32 a<8>, m<6>;\n\t"
        "abs.bf16x2 a0, %1;\n\tabs.bf16x2 a1, %2;\n\tabs.bf16x2 a2, %3;\n\tabs.bf16x2 a3, %4;\n\t"
        "abs.bf16x2 a4, %5;\n\tabs.bf16x2 a5, %6;\n\tabs.bf16x2 a6, %7;\n\tabs.bf16x2 a7, %8;\n\t"
        "max.NaN.bf16x2 m0, a0, a1;\n\tmax.NaN.bf16x2 m1, a2, a3;\n\tmax.NaN.bf16x2 m2, a4, a5;\n\t"
        "max.NaN.bf16x2 m3, a6, a7;\n\tmax.NaN.bf16x2 m4, m0, m1;\n\tmax.NaN.bf16x2 m5, m2, m3;\n\t"
        "max.NaN.bf16x2 %0, m4, m5;\n\t}"
        : "=r"(mx) : "r"(h[0]), "r"(h[1]), "r"(h[2]), "r"(h[3]), "r"(h[4]), "r"(h[5]), "r"(h[6]), "r"(h[7]));
    const uint32_t E = max(mx & 0xffffu, mx >> 16) >> 7;
    E_out = E;
    if (E < 17u || E > 253u) return false;
    const uint32_t S = ((uint32_t)(M + 253) - E) * 0x00800080u;      // 2^(M-1+127-E) as bfloat16, both halves
    uint32_t d2[8];
#pragma unroll
    for (int w = 0; w < 8; w++) {
        uint32_t r;
        asm("{\n\t.reg .b32 t;\n\tabs.bf16x2 t, %1;\n\tfma.rn.bf16x2 %0, t, %2, %3;\n\t}" : "=r"(r) : "r"(h[w]), "r"(S), "r"(0x43004300u));
        r = min_u16x2(r, 0x43004300u + qmax * 0x00010001u);
        const uint32_t q2 = r & (qmax * 0x00010001u);
        const uint32_t sign_bit = (qmax + 1u) * 0x00010001u;            // the datum's sign position in each half
        const uint32_t sgn = (h[w] >> (15 - M)) & sign_bit;
        const uint32_t nz = (q2 + qmax * 0x00010001u) & sign_bit;       // set iff q > 0: a zero magnitude keeps sign 0
        d2[w] = q2 | (sgn & nz);
    }
    if (M == 7) {
#pragma unroll
        for (int k = 0; k < 4; k++) out[k % BfpTraits<M>::words] = __byte_perm(d2[2 * k], d2[2 * k + 1], 0x6420);
    } else if (M == 3) {
        uint32_t t[8];
#pragma unroll
        for (int w = 0; w < 8; w++) t[w] = d2[w] | (d2[w] >> 12);       // byte 0 = datum 2w | datum 2w+1 << 4
        out[0] = __byte_perm(__byte_perm(t[0], t[1], 0x0040), __byte_perm(t[2], t[3], 0x0040), 0x5410);
        out[1 % BfpTraits<M>::words] = __byte_perm(__byte_perm(t[4], t[5], 0x0040), __byte_perm(t[6], t[7], 0x0040), 0x5410);
    } else {
        uint32_t acc = 0;
#pragma unroll
        for (int w = 0; w < 8; w++) acc |= ((d2[w] | (d2[w] >> 14)) & 0xfu) << (4 * w);   // datums 2w, 2w+1: 2 bits each
        out[0] = acc;
    }
    return true;
}

// "a" formats (Bfp8 / Bfp4 / Bfp2): same datums, but the shared exponent is the 5-bit exponent of
// binary16 (bias 15), stored in a byte.  The source is binary16; it is widened to binary32 bit patterns
// so the encoder above can be reused: binary16 zeros / denormals become 0 (flush); Inf / NaN become the
// largest binary32 below 2^17, i.e. exponent field 31 + 112 with a full mantissa, so they round up past
// the largest magnitude and saturate to it while finite neighbours keep their distance 31 - e from the
// block exponent; everything else converts exactly.
__device__ __forceinline__ uint32_t half_bits_to_float_bits(uint32_t h)
{
    const uint32_t hm = h & 0x7fffu;
    uint32_t a = (hm << 13) + 0x38000000u;   // re-bias the exponent by 127 - 15
    a = hm < 0x0400u ? 0u : a;
    a = hm >= 0x7c00u ? 0x47ffffffu : a;
    return a | ((h & 0x8000u) << 16);
}

// ------------------------------------------------------------------------------------------------
// Lf8: a float of 1 sign, 5 exponent and 2 mantissa bits per element, no shared exponent
// (docs/public/dataformats.rst:24 of the reference).  The reference has no host-side conversion for it, so the
// arithmetic is this library's reading: the IEEE-754 rules of a binary format with those field widths (bias 15,
// subnormals, infinities and NaNs), rounding to nearest even -- the upper byte of a binary16.
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t lf8_encode_float_bits(uint32_t u)
{
    const uint32_t a = u & 0x7fffffffu;
    // 2^-14 and above: exponent field and two mantissa bits, rounded to nearest even; a carry out of the mantissa moves
    // up the exponent; past the largest finite value the result is 0x7c = infinity
    const uint32_t r = (a + 0x000fffffu + ((a >> 21) & 1u)) >> 21;
    const uint32_t normal = min(r - (112u << 2), 0x7cu);
    // below 2^-14: multiples of 2^-16, 0 .. 4 (4 = the smallest normal)
    // (one multiply-add into the low bits of 1.5 * 2^23 rounds to nearest even without a conversion instruction)
    const uint32_t subnormal = __float_as_uint(__fmaf_rn(__uint_as_float(min(a, 113u << 23)), 65536.0f, 12582912.0f)) & 7u;
    uint32_t c = a >= (113u << 23) ? normal : subnormal;   // both computed, one selected: no divergence inside a warp
    c = a > 0x7f800000u ? 0x7fu : c;                      // NaN
    return c | ((u >> 24) & 0x80u);
}

__device__ __forceinline__ uint32_t lf8_encode_half_bits(uint32_t h)
{
    const uint32_t a = h & 0x7fffu;
    const uint32_t c = a > 0x7c00u ? 0x7fu : (a + 0x7fu + ((a >> 8) & 1u)) >> 8;   // the same rounding on the binary16 bit pattern
    return c | ((h >> 8) & 0x80u);
}

// exact: every Lf8 value is a binary32 (and a bfloat16: upper half of the result; and a binary16: code << 8)
__device__ __forceinline__ uint32_t lf8_decode_float_bits(uint32_t c)
{
    const uint32_t x = (c & 0x7fu) << 21;                         // exponent and mantissa fields where binary32 has them
    uint32_t a = x + (112u << 23);                                // normal: re-bias by 127 - 15
    a += x >= (0x7cu << 21) ? (112u << 23) : 0u;                  // exponent 31: infinity / NaN (the mantissa bits stay on top)
    // exponent 0: m * 2^-16, m = 0 .. 3
    const uint32_t sub = __float_as_uint(__fmul_rn(__fadd_rn(__uint_as_float(0x4b000000u | (c & 3u)), -8388608.0f), 1.52587890625e-05f));
    a = x < (4u << 21) ? sub : a;
    return a | ((c & 0x80u) << 24);
}

// Two binary32 values -> two Lf8 codes (first value in the low byte) with the hardware's e5m2 conversion, which rounds to
// nearest even and handles subnormals but saturates to the largest finite value; values that round to infinity under the
// IEEE rule (magnitude >= 61440, the midpoint above the largest finite value) and infinities themselves are set right
// afterwards, as are NaNs (0x7f with the sign of the input).
__device__ __forceinline__ uint32_t lf8_encode_float_bits_x2(uint32_t u0, uint32_t u1)
{
    uint16_t d;
    asm("cvt.rn.satfinite.e5m2x2.f32 %0, %1, %2;" : "=h"(d) : "f"(__uint_as_float(u1)), "f"(__uint_as_float(u0)));
    uint32_t c = d;
    const uint32_t a0 = u0 & 0x7fffffffu, a1 = u1 & 0x7fffffffu;
    // 0x47700000 = 61440.0f: from there on infinity, and NaN (sign kept) above the infinity pattern
    if (a0 >= 0x47700000u) c = (c & 0xff00u) | ((u0 >> 24) & 0x80u) | (a0 > 0x7f800000u ? 0x7fu : 0x7cu);
    if (a1 >= 0x47700000u) c = (c & 0x00ffu) | ((((u1 >> 24) & 0x80u) | (a1 > 0x7f800000u ? 0x7fu : 0x7cu)) << 8);
    return c;
}

// binary32 block exponent of widened binary16 data -> the 5-bit exponent byte
__device__ __forceinline__ uint32_t a_exponent_byte(uint32_t e32) { return e32 > 112u ? e32 - 112u : 0u; }

// scale 2^(E5 - 15 - (M-1)) of an "a" block: always a normal binary32
template <int M>
__device__ __forceinline__ float bfp_a_block_scale(uint32_t e5) { return __uint_as_float((e5 + 127u - 15u - (uint32_t)(M - 1)) << 23); }

// Scale of a block: 2^(E - 127 - (M-1)) as a binary32 (denormal when needed).  For M == 1 and
// E == 255 the scale 2^128 is not representable: the caller multiplies by `post` (2.0) as well.
template <int M>
__device__ __forceinline__ float bfp_block_scale(uint32_t E, float &post)
{
    int k = (int)E - 127 - (M - 1);
    post = 1.0f;
    if (k > 127) {
        post = 2.0f;
        k = 127;
    }
    if (k >= -126) return __uint_as_float((uint32_t)(k + 127) << 23);
    return __uint_as_float(1u << (k + 149));
}

// Decode one block to 16 binary32 values (exact; overflow gives infinity).
template <int M, bool AF = false>
__device__ __forceinline__ void bfp_decode16(uint32_t E, const uint32_t (&in)[BfpTraits<M>::words], float (&v)[16])
{
    float post = 1.0f;
    const float sc = AF ? bfp_a_block_scale<M>(E & 31u) : bfp_block_scale<M>(E, post);
#pragma unroll
    for (int i = 0; i < 16; i++) {
        uint32_t q, signbit;
        if (M == 7) {
            const uint32_t w = in[(i / 4) % BfpTraits<M>::words];
            const int j = i % 4;
            // magnitude byte j spliced under the upper three bytes of the magic constant
            q = __byte_perm(w & 0x7f7f7f7fu, kMagicBits, 0x7650 + j);
            signbit = (w << (24 - 8 * j)) & 0x80000000u;
        } else {
            const uint32_t w = in[((i * (M + 1)) / 32) % BfpTraits<M>::words];
            const int sh = (i * (M + 1)) % 32;
            const uint32_t d = w >> sh;
            q = kMagicBits | (d & BfpTraits<M>::qmax);
            signbit = (d << (31 - M)) & 0x80000000u;
        }
        float mag = __fmul_rn(__fadd_rn(__uint_as_float(q), -12582912.0f), sc);
        if (M == 1 && !AF) mag = __fmul_rn(mag, post);
        // (+-0) + (+0) = +0: a zero magnitude decodes to +0.0 whatever its sign bit says
        v[i] = __fadd_rn(__uint_as_float(__float_as_uint(mag) | signbit), 0.0f);
    }
}

// Decode of one block straight to bfloat16 pairs (the default result type of a read from a Bfp*_b queue,
// pybuda/pybuda/tensor.py:730-740): datum pair -> (2^M + q) as bfloat16 (q spliced into the top mantissa bits
// under the exponent of 2^M), then one fma.rn.bf16x2 per pair: (2^M + q) * s - 2^M * s = q * s exactly, with
// s = 2^(E-127-(M-1)); a zero magnitude gives +0.0 whatever its sign bit.  Half the work of decoding to binary32
// and narrowing.  Returns false when s or 2^(M+1) * s is not a normal bfloat16 (E < M or E > 252): the caller uses
// bfp_decode16.  o[p] holds values 2p (low half) and 2p + 1.
template <int M>
__device__ __forceinline__ bool bfp_decode16_bf16(uint32_t E, const uint32_t (&in)[BfpTraits<M>::words], uint32_t (&o)[8])
{
    if (E < (uint32_t)M || E > 252u) return false;
    constexpr uint32_t base = ((uint32_t)(127 + M) << 7) * 0x00010001u;           // 2^M in both halves
    const uint32_t sc = (E - (uint32_t)(M - 1)) * 0x00800080u;                      // s: exponent field E - (M-1)
    const uint32_t off = ((E + 1u) * 0x00800080u) | 0x80008000u;                    // -(2^M * s): exponent field E + 1
    // byte-aligned data: `lane[r]` holds, in byte j, datum (data per byte) * j + r shifted so that its sign is
    // bit 7 and its magnitude starts at bit 6
    constexpr int kPerByte = 8 / (M + 1);                                           // 1 / 2 / 4 data per byte
    uint32_t lane[BfpTraits<M>::words][kPerByte];
#pragma unroll
    for (int w = 0; w < BfpTraits<M>::words; w++) {
#pragma unroll
        for (int r = 0; r < kPerByte; r++)
            lane[w][r] = M == 7 ? in[w] : (in[w] << ((kPerByte - 1 - r) * (M + 1))) & ((0xffu << (7 - M)) & 0xffu) * 0x01010101u;
    }
#pragma unroll
    for (int p = 0; p < 8; p++) {
        // PP: datum 2p in bytes 0 and 1, datum 2p + 1 in bytes 2 and 3
        const int d0 = 2 * p, d1 = 2 * p + 1;
        const int w0 = d0 / (4 * kPerByte);                                         // both data sit in the same word
        const int j0 = (d0 / kPerByte) % 4, j1 = (d1 / kPerByte) % 4;
        const uint32_t A = lane[w0][d0 % kPerByte], B = lane[w0][d1 % kPerByte];
        const uint32_t PP = __byte_perm(A, B, (uint32_t)(j0 | (j0 << 4) | ((4 + j1) << 8) | ((4 + j1) << 12)));
        const uint32_t x = (PP & 0x807f807fu) | base;                                // +-(2^M + q)
        const uint32_t o2 = off ^ (PP & 0x80008000u);                                // -+(2^M * s)
        asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(o[p]) : "r"(x), "r"(sc), "r"(o2));   // +-(q * s); +0 when q is 0
    }
    return true;
}

}  // namespace buda
