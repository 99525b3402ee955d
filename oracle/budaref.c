/*
 * budaref.c -- CPU ORACLE for the TT-Buda data-format path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file is a plain-C restatement of the algorithms on the data-format path of
 * tenstorrent/tt-buda.  It exists so the CUDA kernels can be checked bit-for-bit; it is never
 * linked into, loaded by, or called from the shipped library.  Only tests, the smoke check and
 * the benchmark's CPU-baseline leg may use it.
 *
 * PARITY STATUS
 *   - Tile-level queue ordering: PINNED by the reference's own model, TileLayout::map
 *     (pybuda/csrc/balancer/types.cpp:629-666) and its exhaustive round-trip test
 *     (pybuda/csrc/balancer/tests/test_tile_layout.cpp:250-281), restated in ref_tile_map /
 *     ref_tile_unmap below.
 *   - Quantize / Dequantize / Requantize: PINNED by golden vectors generated from the
 *     reference's own eval (pybuda/pybuda/op/eval/pybuda/quantize.py:55-122,
 *     pybuda/pybuda/op/eval/buda/quantize.py:23-53).
 *   - Byte sizes: PINNED by pybuda/csrc/lower_to_buda/common.cpp:167-190 and
 *     pybuda/csrc/balancer/balancer_utils.hpp:24-51.
 *   - Face order inside a tile and the Bfp byte encoding: PARITY UNPINNED.  The converter that
 *     produces those bytes lives in tenstorrent/tt-budabackend (git submodule
 *     third_party/budabackend, branch main, no pinned commit, directory empty in the reference
 *     checkout).  The restatement follows the published description
 *     (docs/public/dataformats.rst:59-89 and docs/public/images/bfp{8,4,2}_blocks.png) and freezes
 *     every choice the description leaves open; each such choice is marked "POLICY" below, and the ones that
 *     change bytes (rounding, overflow, face / exponent / datum order) are switches (ref_set_bfp_policy) so that a
 *     real converter's bytes can be adopted by setting them.
 *
 * The Bfp encoder here works in integers (shift / mask / explicit round-to-nearest-even) on
 * purpose: the CUDA kernels use a floating-point formulation of the same arithmetic, so agreement
 * between the two is a real check and not the same code compiled twice.
 *
 * Build: see oracle/Makefile  (gcc -O3 -mavx2 -ffp-contract=off -fopenmp).
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

/* DataFormat values: pybuda/csrc/lower_to_buda/common.hpp:92-111 */
enum {
    DF_Float32 = 0, DF_Float16 = 1, DF_Bfp8 = 2, DF_Bfp4 = 3, DF_Bfp2 = 11, DF_Float16_b = 5,
    DF_Bfp8_b = 6, DF_Bfp4_b = 7, DF_Bfp2_b = 15, DF_Lf8 = 10, DF_UInt16 = 12, DF_Int8 = 14,
    DF_Int32 = 8, DF_RawUInt8 = 0xf0, DF_RawUInt16 = 0xf1, DF_RawUInt32 = 0xf2, DF_Invalid = 0xff
};

/* Queue geometry as emitted per queue by the reference compiler
 * (pybuda/csrc/lower_to_buda/netlist.cpp:141-232) and carried by DramIODesc
 * (pybuda/csrc/backend_api/backend_api.cpp:409-426). */
typedef struct {
    uint32_t grid_r, grid_c;       /* bufq_grid_dim_r/c: one buffer per grid core        */
    uint32_t mblock_m, mblock_n;   /* macro-block, in micro-blocks                       */
    uint32_t ublock_rt, ublock_ct; /* micro-block, in tiles                              */
    uint32_t t;                    /* z dimension of one entry                           */
    uint32_t ublock_order;         /* 0 = row-major ublock scan (R), 1 = column-major (C)*/
    uint32_t tile_height;          /* 0 or 32: full tiles; 16/8/4/2/1: tiny tiles (TileDim,
                                      pybuda/csrc/lower_to_buda/common.hpp:80-90; tensor rows per tile as in
                                      pybuda/pybuda/op/eval/buda/tilizer.py:40-52).  POLICY: the record keeps the
                                      full-tile size (balancer_utils.hpp:24-51) and rows >= tile_height are zero */
} ref_geom;

int ref_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* limits the OpenMP team of the following calls (the single-thread CPU baseline); returns the previous limit */
int ref_set_threads(int n)
{
#ifdef _OPENMP
    int prev = omp_get_max_threads();
    if (n > 0) omp_set_num_threads(n);
    return prev;
#else
    (void)n;
    return 1;
#endif
}

/* ---------------------------------------------------------------------------------------------
 * POLICY switches: every choice the published description leaves open for the block-float bytes, as one
 * process-wide record (default: all zero, faces in order 0 1 2 3).  "Truncate bits to fit in the BFP format mantissa
 * size, optionally round before truncation" (docs/public/dataformats.rst:80-81) names truncation and a rounding it does not specify (to nearest even, or half an ulp added before the truncation); the drawings
 * docs/public/images/bfp{8,4,2}_blocks.png show 32-bit rows without saying which end holds the first exponent /
 * datum.  When real tile bytes of the reference's converter are available, the combination that reproduces them
 * is set here and, identically, in the CUDA library.
 * ------------------------------------------------------------------------------------------- */
typedef struct {
    uint32_t rounding;       /* 0 nearest even, 1 truncate, 2 add half an ulp then truncate (nearest, ties away from zero) */
    uint32_t overflow;       /* 0 saturate, 1 raise the block exponent by one and re-encode the block */
    uint8_t face_order[4];   /* face stored at position p of the record */
    uint32_t exponent_order; /* 0: exponent of block k in byte k; 1: in byte k ^ 3 (big-endian 32-bit words) */
    uint32_t datum_order;    /* 0: datum i in bits [i w, (i+1) w) of the block; 1: fields of each 32-bit word reversed */
} ref_bfp_policy;

static ref_bfp_policy g_pol = {0, 0, {0, 1, 2, 3}, 0, 0};

int ref_set_bfp_policy(const ref_bfp_policy *p)
{
    static const ref_bfp_policy def = {0, 0, {0, 1, 2, 3}, 0, 0};
    if (!p) { g_pol = def; return 0; }
    int seen = 0;
    for (int i = 0; i < 4; i++) {
        if (p->face_order[i] > 3) return 1;
        seen |= 1 << p->face_order[i];
    }
    if (seen != 15 || p->rounding > 2 || p->overflow > 1 || p->exponent_order > 1 || p->datum_order > 1) return 1;
    g_pol = *p;
    return 0;
}

/* bit offset of datum i (w bits wide) inside its block's bytes, read as little-endian 32-bit words */
static inline int datum_bit_offset(int i, int w)
{
    int per_word = 32 / w, word = i / per_word, field = i % per_word;
    if (g_pol.datum_order) field = per_word - 1 - field;
    return word * 32 + field * w;
}

static inline void put_datum(uint8_t *out, int i, int w, uint32_t d)
{
    int bit = datum_bit_offset(i, w);
    out[bit >> 3] |= (uint8_t)(d << (bit & 7));
}

static inline uint32_t get_datum(const uint8_t *in, int i, int w)
{
    int bit = datum_bit_offset(i, w);
    return ((uint32_t)in[bit >> 3] >> (bit & 7)) & ((1u << w) - 1u);
}

static inline int exponent_byte_index(int blk) { return g_pol.exponent_order ? (blk ^ 3) : blk; }

/* ---------------------------------------------------------------------------------------------
 * Sizes
 * ------------------------------------------------------------------------------------------- */

/* bytes of one 32x32 tile; follows balancer_utils.hpp:24-51 (header_padding = 32 when asked) */
long ref_tile_bytes(int df, int with_header)
{
    long h = with_header ? 32 : 0;
    switch (df) {
        case DF_Float32: case DF_Int32: case DF_RawUInt32: return 4096 + h;
        case DF_Float16: case DF_Float16_b: case DF_UInt16: case DF_RawUInt16: return 2048 + h;
        case DF_Bfp8: case DF_Bfp8_b: return 1024 + 64 + h;
        case DF_Bfp4: case DF_Bfp4_b: return 512 + 64 + h;
        case DF_Bfp2: case DF_Bfp2_b: return 256 + 64 + h;
        case DF_Lf8: case DF_Int8: case DF_RawUInt8: return 1024 + h;
        default: return -1;
    }
}

/* follows data_format_byte_size, common.cpp:167-190 */
long ref_data_format_byte_size(int df, long elements)
{
    switch (df) {
        case DF_Float32: case DF_Int32: case DF_RawUInt32: return 4 * elements;
        case DF_UInt16: case DF_Float16_b: case DF_Float16: case DF_RawUInt16: return 2 * elements;
        case DF_Bfp8_b: case DF_Bfp8: return elements + elements / 16;
        case DF_Bfp4_b: case DF_Bfp4: return elements / 2 + elements / 16;
        case DF_Bfp2_b: case DF_Bfp2: return elements / 4 + elements / 16;
        case DF_Lf8: case DF_Int8: case DF_RawUInt8: return elements;
        case DF_Invalid: return 0;
        default: return -1;
    }
}

static int bfp_mant_bits(int df)
{
    switch (df) {
        case DF_Bfp8_b: case DF_Bfp8: return 7;
        case DF_Bfp4_b: case DF_Bfp4: return 3;
        case DF_Bfp2_b: case DF_Bfp2: return 1;
        default: return 0;
    }
}

static int elem_bytes(int df)
{
    switch (df) {
        case DF_Float32: case DF_Int32: case DF_RawUInt32: return 4;
        case DF_Float16: case DF_Float16_b: case DF_UInt16: case DF_RawUInt16: return 2;
        case DF_Lf8: case DF_Int8: case DF_RawUInt8: return 1;
        default: return 0;
    }
}

/* ---------------------------------------------------------------------------------------------
 * Tile-level ordering: TileLayout::map, types.cpp:629-648 (forward) and 650-666 (inverse).
 * Canonical coordinate = (t, r, c) in tiles over the whole tensor; linear coordinate = (grid
 * core, tile address inside that core's buffer).
 * ------------------------------------------------------------------------------------------- */
void ref_tile_map(const ref_geom *g, uint32_t t, uint32_t r, uint32_t c, uint32_t *core_r,
                  uint32_t *core_c, uint64_t *addr)
{
    uint32_t block_rt = g->mblock_m * g->ublock_rt;
    uint32_t block_ct = g->mblock_n * g->ublock_ct;
    uint32_t u_r = r % g->ublock_rt, u_c = c % g->ublock_ct;
    uint32_t m = (r / g->ublock_rt) % g->mblock_m;
    uint32_t n = (c / g->ublock_ct) % g->mblock_n;
    uint64_t ublock_vol = (uint64_t)g->ublock_rt * g->ublock_ct;
    uint64_t mblock_vol = (uint64_t)g->mblock_m * g->mblock_n * ublock_vol;
    uint64_t mblock_lin = (g->ublock_order == 0) ? ((uint64_t)m * g->mblock_n + n) * ublock_vol
                                                 : ((uint64_t)n * g->mblock_m + m) * ublock_vol;
    *core_r = r / block_rt;
    *core_c = c / block_ct;
    *addr = (uint64_t)t * mblock_vol + mblock_lin + (uint64_t)u_r * g->ublock_ct + u_c;
}

void ref_tile_unmap(const ref_geom *g, uint32_t core_r, uint32_t core_c, uint64_t addr, uint32_t *t,
                    uint32_t *r, uint32_t *c)
{
    uint64_t ublock_vol = (uint64_t)g->ublock_rt * g->ublock_ct;
    uint64_t mblock_vol = (uint64_t)g->mblock_m * g->mblock_n * ublock_vol;
    uint64_t mblock_off = addr % mblock_vol;
    uint64_t ublock_off = mblock_off % ublock_vol;
    uint64_t num_ublocks = mblock_off / ublock_vol;
    uint32_t m = (g->ublock_order == 0) ? (uint32_t)(num_ublocks / g->mblock_n)
                                        : (uint32_t)(num_ublocks % g->mblock_m);
    uint32_t n = (g->ublock_order == 0) ? (uint32_t)(num_ublocks % g->mblock_n)
                                        : (uint32_t)(num_ublocks / g->mblock_m);
    *t = (uint32_t)(addr / mblock_vol);
    *r = core_r * g->mblock_m * g->ublock_rt + m * g->ublock_rt + (uint32_t)(ublock_off / g->ublock_ct);
    *c = core_c * g->mblock_n * g->ublock_ct + n * g->ublock_ct + (uint32_t)(ublock_off % g->ublock_ct);
}

/* ---------------------------------------------------------------------------------------------
 * Bfp block encode / decode  (dataformats.rst:74-83: steps 3-8)
 *
 * A block is 16 values that share one 8-bit exponent ("_b" formats: the fp32/bf16 exponent
 * itself).  Each datum is sign + m magnitude bits, m = 7 / 3 / 1, with NO implied one.
 * ------------------------------------------------------------------------------------------- */

/* Encode one value against the block exponent.  bits: IEEE-754 binary32 pattern.  *over is set when a finite value's
 * magnitude comes out above the largest one. */
static inline uint32_t bfp_encode_datum(uint32_t bits, uint32_t block_exp, int m, int *over)
{
    uint32_t sign = bits >> 31;
    uint32_t e = (bits >> 23) & 0xffu;
    uint32_t qmax = (1u << m) - 1u;
    uint32_t q;
    if (e == 0) {
        q = 0; /* POLICY: zero and denormal inputs encode as zero (flush) */
    } else if (e == 255) {
        q = qmax; /* POLICY: Inf and NaN encode the largest magnitude, keeping their sign */
    } else {
        /* step 4: make the implied one explicit -> 24-bit significand */
        uint32_t sig = (bits & 0x7fffffu) | 0x800000u;
        /* steps 5-7: shift right by the exponent delta, then keep m bits of the 24 */
        uint32_t shift = (block_exp - e) + (uint32_t)(24 - m);
        if (shift > 25) {
            q = 0; /* less than half of the last kept bit: rounds to zero */
        } else {
            /* POLICY (rounding): to nearest, ties to even, on the dropped bits ("optionally round"), or plain
             * truncation */
            uint32_t kept = sig >> shift;
            uint32_t rem = sig & ((1u << shift) - 1u);
            uint32_t half = 1u << (shift - 1);
            if (!g_pol.rounding && (rem > half || (rem == half && (kept & 1u)))) kept++;
            else if (g_pol.rounding == 2 && rem >= half) kept++;   /* add half, then truncate: ties away from zero */
            /* POLICY (overflow): a round-up past the largest magnitude saturates here; under the other policy the
             * caller raises the block exponent and encodes the block again */
            if (kept > qmax) *over = 1;
            q = kept > qmax ? qmax : kept;
        }
    }
    if (q == 0) sign = 0; /* POLICY: a zero magnitude is stored as +0 */
    return (sign << m) | q;
}

/* Encode one 16-value block.  out receives 16/8/4 bytes for m = 7/3/1.
 * POLICY (datum order, default): datum i of the block occupies the lower-numbered bits first, i.e.
 * Bfp4 datum i -> bits [4(i&1)+3 : 4(i&1)] of byte i/2, Bfp2 datum i -> bits [2(i&3)+1 : 2(i&3)]
 * of byte i/4 (little-endian inside the 32-bit rows drawn in bfp4_blocks.png / bfp2_blocks.png). */
void ref_bfp_pack_block(const uint32_t bits[16], int m, uint8_t *exp_out, uint8_t *out)
{
    uint32_t block_exp = 0;
    for (int i = 0; i < 16; i++) {
        uint32_t e = (bits[i] >> 23) & 0xffu; /* step 3: maximum exponent of the block */
        if (e > block_exp) block_exp = e;
    }
    int w = m + 1;             /* datum width in bits: 8, 4, 2 */
    uint32_t d[16];
    int over = 0;
    for (int i = 0; i < 16; i++) d[i] = bfp_encode_datum(bits[i], block_exp, m, &over);
    if (g_pol.overflow && over && block_exp < 255) {
        block_exp++;
        for (int i = 0; i < 16; i++) d[i] = bfp_encode_datum(bits[i], block_exp, m, &over);
    }
    *exp_out = (uint8_t)block_exp;
    memset(out, 0, 16 * w / 8);
    for (int i = 0; i < 16; i++) put_datum(out, i, w, d[i]);
}

/* Decode: value = (-1)^s * q * 2^(E - 127 - (m-1)), rounded to binary32 (exact unless it
 * overflows, which yields infinity).  q == 0 decodes to +0.0. */
static inline float bfp_decode_datum(uint32_t d, uint32_t block_exp, int m)
{
    uint32_t q = d & ((1u << m) - 1u);
    uint32_t sign = (d >> m) & 1u;
    if (q == 0) return 0.0f;
    double v = ldexp((double)q, (int)block_exp - 127 - (m - 1));
    float f = (float)v;
    return sign ? -f : f;
}

void ref_bfp_unpack_block(uint8_t exp_in, const uint8_t *in, int m, float out[16])
{
    int w = m + 1;
    for (int i = 0; i < 16; i++) out[i] = bfp_decode_datum(get_datum(in, i, w), exp_in, m);
}

/* ---------------------------------------------------------------------------------------------
 * "a" formats (Bfp8 / Bfp4 / Bfp2): the shared exponent is the 5-bit binary16 exponent "padded to 8b"
 * (dataformats.rst:68); the source is binary16 (pybuda/pybuda/device_connector.py:188-192 casts to
 * float16 for these queues).  Same datum rules as the "b" formats, in the binary16 domain:
 * 11-bit significand, zero / denormal -> 0, Inf / NaN (e == 31) -> largest magnitude.
 * decode: (-1)^s * q * 2^(E - 15 - (m-1)).   PARITY UNPINNED like the "b" encoding.
 * ------------------------------------------------------------------------------------------- */
static inline uint32_t bfp_a_encode_datum(uint16_t h, uint32_t block_exp, int m, int *over)
{
    uint32_t sign = h >> 15, e = (h >> 10) & 31u, qmax = (1u << m) - 1u, q;
    if (e == 0) {
        q = 0;
    } else if (e == 31) {
        q = qmax;
    } else {
        uint32_t sig = (h & 0x3ffu) | 0x400u;                 /* 11-bit significand */
        uint32_t shift = (block_exp - e) + (uint32_t)(11 - m);
        if (shift > 12) {
            q = 0;
        } else {
            uint32_t kept = sig >> shift, rem = sig & ((1u << shift) - 1u), half = 1u << (shift - 1);
            if (!g_pol.rounding && (rem > half || (rem == half && (kept & 1u)))) kept++;
            else if (g_pol.rounding == 2 && rem >= half) kept++;   /* add half, then truncate: ties away from zero */
            if (kept > qmax) *over = 1;
            q = kept > qmax ? qmax : kept;
        }
    }
    if (q == 0) sign = 0;
    return (sign << m) | q;
}

void ref_bfp_a_pack_block(const uint16_t h[16], int m, uint8_t *exp_out, uint8_t *out)
{
    uint32_t block_exp = 0;
    for (int i = 0; i < 16; i++) {
        uint32_t e = (h[i] >> 10) & 31u;
        if (e > block_exp) block_exp = e;
    }
    int w = m + 1;
    uint32_t d[16];
    int over = 0;
    for (int i = 0; i < 16; i++) d[i] = bfp_a_encode_datum(h[i], block_exp, m, &over);
    /* an all-Inf/NaN-free block whose exponent is 30 may be raised to 31 */
    if (g_pol.overflow && over && block_exp < 31) {
        block_exp++;
        for (int i = 0; i < 16; i++) d[i] = bfp_a_encode_datum(h[i], block_exp, m, &over);
    }
    *exp_out = (uint8_t)block_exp;
    memset(out, 0, 16 * w / 8);
    for (int i = 0; i < 16; i++) put_datum(out, i, w, d[i]);
}

void ref_bfp_a_unpack_block(uint8_t exp_in, const uint8_t *in, int m, float out[16])
{
    int w = m + 1;
    for (int i = 0; i < 16; i++) {
        uint32_t d = get_datum(in, i, w);
        uint32_t q = d & ((1u << m) - 1u), sign = (d >> m) & 1u;
        float f = q ? (float)ldexp((double)q, (int)(exp_in & 31u) - 15 - (m - 1)) : 0.0f;
        out[i] = (sign && q) ? -f : f;
    }
}

/* binary32 -> binary16, round to nearest even, overflow to infinity */
static inline uint16_t float_to_half_bits(float f)
{
    uint32_t b; memcpy(&b, &f, 4);
    uint32_t sign = (b >> 16) & 0x8000u, a = b & 0x7fffffffu;
    if (a >= 0x7f800000u) return (uint16_t)(sign | 0x7c00u | ((a > 0x7f800000u) ? 0x200u : 0u));
    if (a >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u);            /* rounds to >= 65520: infinity */
    if (a < 0x33000001u) return (uint16_t)sign;                         /* below half the smallest denormal */
    int e = (int)(a >> 23) - 127;
    uint32_t sig = (a & 0x7fffffu) | 0x800000u;
    int shift = (e < -14) ? (13 + (-14 - e)) : 13;                      /* bits dropped from the 24-bit significand */
    uint32_t kept = sig >> shift, rem = sig & ((1u << shift) - 1u), half = 1u << (shift - 1);
    if (rem > half || (rem == half && (kept & 1u))) kept++;
    uint32_t h = (e < -14) ? kept : (((uint32_t)(e + 15) << 10) + (kept - 0x400u));
    return (uint16_t)(sign | h);
}

static int is_bfp_a(int df) { return df == DF_Bfp8 || df == DF_Bfp4 || df == DF_Bfp2; }

/* ---------------------------------------------------------------------------------------------
 * Lf8: "1-bit sign, 5-bit exponent, 2-bit mantissa, no shared exponent, floating point"
 * (docs/public/dataformats.rst:24).  The reference has no host conversion for it and no torch dtype
 * (pybuda/pybuda/tensor.py:563-632 raise), so this is a reading of the format table, PARITY UNPINNED:
 * the IEEE-754 rules for those field widths (bias 15, subnormals, infinities, NaNs), round to nearest
 * even.  Written on values (frexp / ldexp), not on bit patterns, so that it is independent of the
 * device code it checks.
 * ------------------------------------------------------------------------------------------- */
uint8_t ref_lf8_encode(double v)
{
    uint8_t sign = signbit(v) ? 0x80u : 0u;
    if (v != v) return (uint8_t)(sign | 0x7fu);
    double a = fabs(v);
    if (isinf(a)) return (uint8_t)(sign | 0x7cu);
    if (a < ldexp(1.0, -14)) return (uint8_t)(sign | (uint8_t)nearbyint(ldexp(a, 16)));  /* multiples of 2^-16; 4 = 2^-14 */
    int e;
    double m = frexp(a, &e);            /* a = m * 2^e, 0.5 <= m < 1 */
    int q = (int)nearbyint(ldexp(m, 3)) - 4;   /* (2m - 1) * 4 rounded to nearest even: 0..4 */
    e -= 1;
    if (q == 4) { q = 0; e += 1; }
    if (e > 15) return (uint8_t)(sign | 0x7cu);  /* past the largest finite value 1.75 * 2^15 */
    return (uint8_t)(sign | ((e + 15) << 2) | q);
}

double ref_lf8_decode(uint8_t c)
{
    int e = (c >> 2) & 31, m = c & 3;
    double a;
    if (e == 31) a = m ? NAN : INFINITY;
    else if (e == 0) a = ldexp((double)m, -16);
    else a = ldexp(1.0 + m / 4.0, e - 15);
    return (c & 0x80u) ? -a : a;
}

/* binary16 bit pattern -> value (exact) */
static inline double half_bits_to_double(uint16_t h)
{
    int e = (h >> 10) & 31, m = h & 0x3ff;
    double a;
    if (e == 31) a = m ? NAN : INFINITY;
    else if (e == 0) a = ldexp((double)m, -24);
    else a = ldexp(1.0 + m / 1024.0, e - 15);
    return (h & 0x8000u) ? -a : a;
}

static int is_lf8_float_side(int df) { return df == DF_Float32 || df == DF_Float16_b || df == DF_Float16; }

/* ---------------------------------------------------------------------------------------------
 * Element access helpers
 * ------------------------------------------------------------------------------------------- */
static inline uint32_t load_as_f32_bits(const uint8_t *p, int df)
{
    if (df == DF_Float32) { uint32_t v; memcpy(&v, p, 4); return v; }
    /* bfloat16 widens exactly: it is the upper half of a binary32 */
    uint16_t h; memcpy(&h, p, 2); return (uint32_t)h << 16;
}

static inline void store_from_f32(uint8_t *p, int df, float f)
{
    if (df == DF_Float32) { memcpy(p, &f, 4); return; }
    /* every decoded Bfp value has at most 7 significant bits, so the upper half of the
     * binary32 is the exact bfloat16 */
    uint32_t b; memcpy(&b, &f, 4);
    uint16_t h = (uint16_t)(b >> 16);
    memcpy(p, &h, 2);
}

/* Tile record layout (POLICY where marked):
 *   [optional 32-byte header, zero filled (POLICY: contents unknown, balancer_utils.hpp:27)]
 *   Bfp:   [64 exponent bytes: exponent k belongs to block k][mantissas of block 0..63]
 *          block k = face k/16, face row k%16 (POLICY: faces in order F0 F1 F2 F3 =
 *          (rows 0-15, cols 0-15), (rows 0-15, cols 16-31), (rows 16-31, cols 0-15),
 *          (rows 16-31, cols 16-31); rows top-down)
 *   plain: the four faces in the same order, each 16x16 row-major, native element bytes. */

typedef struct {
    const ref_geom *g;
    uint32_t W, Z, R, C;       /* tensor dims; Z must equal g->t                */
    uint32_t th;               /* tensor rows per tile                          */
    uint64_t tiles_per_entry;  /* per core buffer: t * mblock volume            */
    uint64_t tile_bytes;
    uint64_t buf_bytes;        /* one core's buffer: W entries                  */
} layout_ctx;

static int make_ctx(layout_ctx *c, const ref_geom *g, const uint32_t shape[4], int df, int with_header)
{
    long tb = ref_tile_bytes(df, with_header);
    if (tb < 0) return 1;
    c->g = g; c->W = shape[0]; c->Z = shape[1]; c->R = shape[2]; c->C = shape[3];
    c->th = g->tile_height ? g->tile_height : 32;
    if (c->th > 32 || (c->th & (c->th - 1))) return 1;
    if (c->R % c->th || c->C % 32) return 1;
    if (g->t != c->Z) return 1;
    if ((uint64_t)g->grid_r * g->mblock_m * g->ublock_rt * c->th != c->R) return 1;
    if ((uint64_t)g->grid_c * g->mblock_n * g->ublock_ct * 32 != c->C) return 1;
    c->tiles_per_entry = (uint64_t)g->t * g->mblock_m * g->mblock_n * g->ublock_rt * g->ublock_ct;
    c->tile_bytes = (uint64_t)tb;
    c->buf_bytes = (uint64_t)c->W * c->tiles_per_entry * c->tile_bytes;
    return 0;
}

static inline uint64_t tile_offset(const layout_ctx *c, uint32_t w, uint32_t z, uint32_t rt, uint32_t ct)
{
    uint32_t cr, cc; uint64_t addr;
    ref_tile_map(c->g, z, rt, ct, &cr, &cc, &addr);
    uint64_t core = (uint64_t)cr * c->g->grid_c + cc;
    return core * c->buf_bytes + ((uint64_t)w * c->tiles_per_entry + addr) * c->tile_bytes;
}

/* total bytes of the tilized image of a tensor of this shape in this queue */
long long ref_tilized_bytes(const ref_geom *g, const uint32_t shape[4], int df, int with_header)
{
    layout_ctx c;
    if (make_ctx(&c, g, shape, df, with_header)) return -1;
    return (long long)(c.buf_bytes * g->grid_r * g->grid_c);
}

/* ---------------------------------------------------------------------------------------------
 * tilize (+ Bfp pack): row-major [W,Z,R,C] with BYTE strides -> queue image.
 * Restates what tt::backend::tilize_tensor / push_input do for this path
 * (bound at backend_api.cpp:688-704).  Returns 0 on success.
 * ------------------------------------------------------------------------------------------- */
int ref_tilize_pack(const void *src_, int src_df, const uint32_t shape[4], const uint32_t strides[4],
                    const ref_geom *g, int dst_df, int with_header, void *dst_)
{
    const uint8_t *src = (const uint8_t *)src_;
    uint8_t *dst = (uint8_t *)dst_;
    layout_ctx c;
    if (make_ctx(&c, g, shape, dst_df, with_header)) return 1;
    int m = bfp_mant_bits(dst_df);
    int es = elem_bytes(src_df);
    int lf8 = (dst_df == DF_Lf8 && is_lf8_float_side(src_df));   /* element-wise conversion; Lf8 -> Lf8 is a relayout */
    if (lf8) {
        /* nothing more to check */
    } else if (m && is_bfp_a(dst_df)) {
        if (src_df != DF_Float16) return 1;
    } else if (m) {
        if (!(dst_df == DF_Bfp8_b || dst_df == DF_Bfp4_b || dst_df == DF_Bfp2_b)) return 1;
        if (!(src_df == DF_Float32 || src_df == DF_Float16_b)) return 1;
    } else {
        if (es == 0 || es != elem_bytes(dst_df)) return 1; /* layout-only: same element width */
    }
    uint32_t Rt = c.R / c.th, Ct = c.C / 32;
    long hdr = with_header ? 32 : 0;
    long long ntiles = (long long)c.W * c.Z * Rt * Ct;
    static const uint8_t zeros[16 * 4] = {0};
#pragma omp parallel for schedule(static)
    for (long long ti = 0; ti < ntiles; ti++) {
        uint32_t ct = (uint32_t)(ti % Ct);
        uint32_t rt = (uint32_t)((ti / Ct) % Rt);
        uint32_t z = (uint32_t)((ti / ((long long)Ct * Rt)) % c.Z);
        uint32_t w = (uint32_t)(ti / ((long long)Ct * Rt * c.Z));
        uint8_t *rec = dst + tile_offset(&c, w, z, rt, ct);
        if (hdr) memset(rec, 0, 32);
        rec += hdr;
        const uint8_t *base = src + (uint64_t)w * strides[0] + (uint64_t)z * strides[1];
        for (int pos = 0; pos < 4; pos++) {
            int face = g_pol.face_order[pos];                      /* POLICY (face order): the face stored at this position */
            for (int fr = 0; fr < 16; fr++) {
                uint32_t tr = (uint32_t)((face >> 1) * 16 + fr);   /* row inside the tile */
                uint64_t r = (uint64_t)rt * c.th + tr;
                uint64_t col0 = (uint64_t)ct * 32 + (face & 1) * 16;
                const uint8_t *p = base + r * strides[2] + col0 * strides[3];
                uint32_t estride = strides[3];
                if (tr >= c.th) { p = zeros; estride = (uint32_t)es; }   /* rows a tiny tile does not hold */
                int blk = pos * 16 + fr;
                if (lf8) {
                    for (int i = 0; i < 16; i++) {
                        const uint8_t *q = p + (uint64_t)i * estride;
                        double v;
                        if (src_df == DF_Float16) { uint16_t h; memcpy(&h, q, 2); v = half_bits_to_double(h); }
                        else { uint32_t b = load_as_f32_bits(q, src_df); float f; memcpy(&f, &b, 4); v = (double)f; }
                        rec[(long)blk * 16 + i] = ref_lf8_encode(v);
                    }
                } else if (m && is_bfp_a(dst_df)) {
                    uint16_t hv[16];
                    for (int i = 0; i < 16; i++) memcpy(&hv[i], p + (uint64_t)i * estride, 2);
                    int bpb = 16 * (m + 1) / 8;
                    ref_bfp_a_pack_block(hv, m, rec + exponent_byte_index(blk), rec + 64 + (long)blk * bpb);
                } else if (m) {
                    uint32_t bits[16];
                    for (int i = 0; i < 16; i++) bits[i] = load_as_f32_bits(p + (uint64_t)i * estride, src_df);
                    int bpb = 16 * (m + 1) / 8;
                    ref_bfp_pack_block(bits, m, rec + exponent_byte_index(blk), rec + 64 + (long)blk * bpb);
                } else {
                    for (int i = 0; i < 16; i++)
                        memcpy(rec + ((long)blk * 16 + i) * es, p + (uint64_t)i * estride, es);
                }
            }
        }
    }
    return 0;
}

/* inverse: queue image -> row-major [W,Z,R,C] with byte strides (get_output, backend_api.cpp:701).
 * Bfp sources decode to Float32 or Float16_b; plain sources keep their element bytes. */
int ref_unpack_untilize(const void *src_, int src_df, int with_header, const ref_geom *g, void *dst_,
                        int dst_df, const uint32_t shape[4], const uint32_t strides[4])
{
    const uint8_t *src = (const uint8_t *)src_;
    uint8_t *dst = (uint8_t *)dst_;
    layout_ctx c;
    if (make_ctx(&c, g, shape, src_df, with_header)) return 1;
    int m = bfp_mant_bits(src_df);
    int es = elem_bytes(dst_df);
    int lf8 = (src_df == DF_Lf8 && is_lf8_float_side(dst_df));
    if (lf8) {
        /* nothing more to check */
    } else if (m && is_bfp_a(src_df)) {
        if (!(dst_df == DF_Float32 || dst_df == DF_Float16)) return 1;
    } else if (m) {
        if (!(src_df == DF_Bfp8_b || src_df == DF_Bfp4_b || src_df == DF_Bfp2_b)) return 1;
        if (!(dst_df == DF_Float32 || dst_df == DF_Float16_b)) return 1;
    } else {
        if (es == 0 || es != elem_bytes(src_df)) return 1;
    }
    uint32_t Rt = c.R / c.th, Ct = c.C / 32;
    long hdr = with_header ? 32 : 0;
    long long ntiles = (long long)c.W * c.Z * Rt * Ct;
#pragma omp parallel for schedule(static)
    for (long long ti = 0; ti < ntiles; ti++) {
        uint32_t ct = (uint32_t)(ti % Ct);
        uint32_t rt = (uint32_t)((ti / Ct) % Rt);
        uint32_t z = (uint32_t)((ti / ((long long)Ct * Rt)) % c.Z);
        uint32_t w = (uint32_t)(ti / ((long long)Ct * Rt * c.Z));
        const uint8_t *rec = src + tile_offset(&c, w, z, rt, ct) + hdr;
        uint8_t *base = dst + (uint64_t)w * strides[0] + (uint64_t)z * strides[1];
        for (int pos = 0; pos < 4; pos++) {
            int face = g_pol.face_order[pos];
            for (int fr = 0; fr < 16; fr++) {
                uint32_t tr = (uint32_t)((face >> 1) * 16 + fr);
                if (tr >= c.th) continue;                      /* rows a tiny tile does not hold */
                uint64_t r = (uint64_t)rt * c.th + tr;
                uint64_t col0 = (uint64_t)ct * 32 + (face & 1) * 16;
                uint8_t *p = base + r * strides[2] + col0 * strides[3];
                int blk = pos * 16 + fr;
                if (lf8) {
                    for (int i = 0; i < 16; i++) {
                        uint8_t code = rec[(long)blk * 16 + i];
                        uint8_t *q = p + (uint64_t)i * strides[3];
                        if (dst_df == DF_Float16) {
                            uint16_t h = (uint16_t)(code << 8);   /* the code is the upper byte of the binary16 of the same value */
                            memcpy(q, &h, 2);
                        } else {
                            float f = (float)ref_lf8_decode(code);   /* exact */
                            if ((code & 0x7cu) == 0x7cu && (code & 3u)) {   /* NaN: the two mantissa bits go to the top of the wider mantissa */
                                uint32_t b = ((uint32_t)(code & 0x80u) << 24) | 0x7f800000u | ((uint32_t)(code & 3u) << 21);
                                memcpy(&f, &b, 4);
                            }
                            store_from_f32(q, dst_df, f);
                        }
                    }
                } else if (m && is_bfp_a(src_df)) {
                    float vals[16];
                    int bpb = 16 * (m + 1) / 8;
                    ref_bfp_a_unpack_block(rec[exponent_byte_index(blk)], rec + 64 + (long)blk * bpb, m, vals);
                    for (int i = 0; i < 16; i++) {
                        if (dst_df == DF_Float32) {
                            memcpy(p + (uint64_t)i * strides[3], &vals[i], 4);
                        } else {
                            uint16_t hb = float_to_half_bits(vals[i]);
                            memcpy(p + (uint64_t)i * strides[3], &hb, 2);
                        }
                    }
                } else if (m) {
                    float vals[16];
                    int bpb = 16 * (m + 1) / 8;
                    ref_bfp_unpack_block(rec[exponent_byte_index(blk)], rec + 64 + (long)blk * bpb, m, vals);
                    for (int i = 0; i < 16; i++) store_from_f32(p + (uint64_t)i * strides[3], dst_df, vals[i]);
                } else {
                    for (int i = 0; i < 16; i++)
                        memcpy(p + (uint64_t)i * strides[3], rec + ((long)blk * 16 + i) * es, es);
                }
            }
        }
    }
    return 0;
}

/* ---------------------------------------------------------------------------------------------
 * Golden int8 quantisation ops.  Each follows the torch expression of the reference eval, one
 * IEEE binary32 operation per torch operator (this file is compiled with -ffp-contract=off so
 * no multiply-add is fused).  torch.round is round-half-to-even = rintf in the default mode.
 * The scale of element i is scale[(i / inner) % scale_len]: inner = product of the dims after
 * `axis`; scale_len == 1 gives a per-tensor scale (reshape_to_match_input, quantize.py:38-52).
 * The final cast follows torch's float -> integer conversion of an already clamped value
 * (NaN survives clamp and converts to 0).
 * ------------------------------------------------------------------------------------------- */
static inline float clampf(float v, float lo, float hi)
{
    if (v != v) return v;
    return v < lo ? lo : (v > hi ? hi : v);
}

static inline int8_t to_i8(float v) { return (v != v) ? 0 : (int8_t)(int32_t)v; }

/* mode 0: Quantize, quantize.py:56-66      clamp(round(x / scale) + zp, lo, hi)
 * mode 1: BudaQuantize, quantize.py:68-77 and buda/quantize.py:24-33   round(x * scale) + zp */
void ref_quantize(const float *x, long long n, const float *scale, long long scale_len, long long inner,
                  float zp, int mode, float lo, float hi, int8_t *out)
{
#pragma omp parallel for schedule(static)
    for (long long i = 0; i < n; i++) {
        float s = scale[(i / inner) % scale_len];
        float q = (mode == 0) ? (x[i] / s) : (x[i] * s);
        float r = rintf(q) + zp;
        out[i] = to_i8(clampf(r, lo, hi));
    }
}

/* Dequantize, quantize.py:79-93 and buda/quantize.py:35-40      (float(x) - zp) * scale */
void ref_dequantize(const int8_t *x, long long n, const float *scale, long long scale_len, long long inner,
                    float zp, float *out)
{
#pragma omp parallel for schedule(static)
    for (long long i = 0; i < n; i++) {
        float s = scale[(i / inner) % scale_len];
        out[i] = ((float)x[i] - zp) * s;
    }
}

/* mode 0: Requantize, quantize.py:95-110   s = inp_scale / out_scale; round(s * float(x) + zp)
 *         (scale_b = out_scale; the int32 input is promoted to binary32 by the multiply)
 * mode 1: BudaRequantize, quantize.py:112-122 and buda/quantize.py:42-53  round(float(x) * scale + zp)
 *         (scale_b unused) */
void ref_requantize(const int32_t *x, long long n, const float *scale_a, const float *scale_b,
                    long long scale_len, long long inner, float zp, int mode, float lo, float hi, int8_t *out)
{
#pragma omp parallel for schedule(static)
    for (long long i = 0; i < n; i++) {
        long long k = (i / inner) % scale_len;
        float s = (mode == 0) ? (scale_a[k] / scale_b[k]) : scale_a[k];
        float p = s * (float)x[i];
        float r = rintf(p + zp);
        out[i] = to_i8(clampf(r, lo, hi));
    }
}

/* ---------------------------------------------------------------------------------------------
 * Matmul with Bfp8_b weights, golden semantics (op/eval/pybuda/matmul.py:20-33 evaluates
 * torch.matmul on the operand values): C = A @ decode(W), binary32 accumulation in k order.
 * A: bfloat16 row-major [M,K]; W: Bfp8_b queue image of a [K,N] tensor in geometry g;
 * C: binary32 row-major [M,N].  Small sizes only; the tests use it for spot checks.
 * ------------------------------------------------------------------------------------------- */
int ref_bfp8b_matmul(const uint16_t *A, long M, long K, const void *W, const ref_geom *g, long N, float *C)
{
    uint32_t shape[4] = {1, 1, (uint32_t)K, (uint32_t)N};
    uint32_t strides[4] = {(uint32_t)(K * N * 4), (uint32_t)(K * N * 4), (uint32_t)(N * 4), 4};
    float *Wf = (float *)__builtin_malloc((size_t)K * N * 4);
    if (!Wf) return 1;
    if (ref_unpack_untilize(W, DF_Bfp8_b, 0, g, Wf, DF_Float32, shape, strides)) { __builtin_free(Wf); return 1; }
#pragma omp parallel for schedule(static)
    for (long i = 0; i < M; i++) {
        float *c = C + i * N;
        for (long j = 0; j < N; j++) c[j] = 0.0f;
        for (long k = 0; k < K; k++) {
            uint32_t ab = (uint32_t)A[i * K + k] << 16;
            float a; memcpy(&a, &ab, 4);
            const float *wr = Wf + k * N;
            for (long j = 0; j < N; j++) c[j] += a * wr[j];
        }
    }
    __builtin_free(Wf);
    return 0;
}

/* ---------------------------------------------------------------------------------------------
 * int8 matmul with the requantisation / dequantisation that follows it in the reference
 * (csrc/graph_lib/python_bindings.cpp:655-676: a matmul with the "requant" attribute is evaluated,
 * then "requantization" is applied to its result; op/eval/common.py:50-65: an int8 matmul yields int32).
 * A: int8 row-major [M,K]; W: Int8 queue image of a [K,N] tensor in geometry g; acc in int32 (exact;
 * the reference's float32 torch.matmul gives the same integers while partial sums stay below 2^24).
 *   mode 0  out int32  = acc
 *   mode 1  out int8   = clamp(round(float(acc) * scale + zp), -128, 127)   op/eval/buda/quantize.py:42-53
 *   mode 2  out float  = (float(acc) - zp) * scale                            op/eval/buda/quantize.py:35-40
 * scale: 1 value or N values (per output column).
 * ------------------------------------------------------------------------------------------- */
int ref_i8_matmul(const int8_t *A, long M, long K, const void *W, const ref_geom *g, long N, const float *scale, long scale_len,
                  float zp, int mode, void *out)
{
    uint32_t shape[4] = {1, 1, (uint32_t)K, (uint32_t)N};
    uint32_t strides[4] = {(uint32_t)(K * N), (uint32_t)(K * N), (uint32_t)N, 1};
    int8_t *Wi = (int8_t *)__builtin_malloc((size_t)K * N);
    if (!Wi) return 1;
    if (ref_unpack_untilize(W, DF_Int8, 0, g, Wi, DF_Int8, shape, strides)) { __builtin_free(Wi); return 1; }
#pragma omp parallel for schedule(static)
    for (long i = 0; i < M; i++) {
        int32_t *acc = (int32_t *)__builtin_malloc((size_t)N * 4);
        for (long j = 0; j < N; j++) acc[j] = 0;
        for (long k = 0; k < K; k++) {
            const int32_t a = A[i * K + k];
            const int8_t *wr = Wi + k * N;
            for (long j = 0; j < N; j++) acc[j] += a * (int32_t)wr[j];
        }
        for (long j = 0; j < N; j++) {
            const float sc = scale ? scale[scale_len == 1 ? 0 : j] : 1.0f;
            if (mode == 0) {
                ((int32_t *)out)[i * N + j] = acc[j];
            } else if (mode == 1) {
                float f = (float)acc[j] * sc;
                f = f + zp;
                f = nearbyintf(f);
                f = f < -128.0f ? -128.0f : (f > 127.0f ? 127.0f : f);
                ((int8_t *)out)[i * N + j] = (f != f) ? 0 : (int8_t)f;
            } else {
                float f = (float)acc[j] - zp;
                ((float *)out)[i * N + j] = f * sc;
            }
        }
        __builtin_free(acc);
    }
    __builtin_free(Wi);
    return 0;
}
