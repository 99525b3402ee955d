// K4 / K5 / K6: the golden int8 quantisation ops as streaming kernels.
//
// Each kernel evaluates, per element, exactly the chain of binary32 operations of the reference's
// torch expressions (pybuda/pybuda/op/eval/pybuda/quantize.py:55-122 and
// pybuda/pybuda/op/eval/buda/quantize.py:23-53): IEEE division, separate multiply and add (never
// fused), round-half-to-even, clamp, truncating cast; NaN survives the clamp and casts to 0.
//
// Quantise / requantise: a thread owns 16 consecutive elements (four 128-bit streaming loads in
// flight, one 128-bit store).  Dequantise, whose traffic is 4/5 stores: a warp owns 512 consecutive
// elements and a thread takes the groups of 4 at lane, lane + 32, lane + 64, lane + 96, so every
// store instruction of a warp writes one contiguous 512-byte run.  (Measured on B200: each layout
// is the faster one for its kernel.)  The scale of element i is scale[(i / inner) % scale_len].
#include "buda_common.cuh"

namespace buda {

enum ScaleMode : int {
    kScalePerTensor = 0,   // scale_len == 1
    kScaleLastAxis16 = 1,  // inner == 1, scale_len % 16 == 0: 16 consecutive scales per thread
    kScaleChunk = 2,       // inner % 16 == 0: one scale per 16-element chunk
    kScaleGeneral = 3,     // per-element index arithmetic
    // the dequantise kernel deals groups of 4 elements instead of chunks of 16
    kScaleLastAxis4 = 4,   // inner == 1, scale_len % 4 == 0, aligned: 4 consecutive scales per group
    kScaleGroup = 5        // inner % 4 == 0: one scale per group
};

struct ScaleSel {
    int64_t scale_len, inner;
};

template <int SM>
__device__ __forceinline__ void load_scales16(const float *__restrict__ scale, const ScaleSel sel, int64_t i0, int cnt,
                                              float (&s)[16])
{
    if (SM == kScalePerTensor) {
        const float v = __ldg(scale);
#pragma unroll
        for (int k = 0; k < 16; k++) s[k] = v;
    } else if (SM == kScaleLastAxis16) {
        const float4 *p = reinterpret_cast<const float4 *>(scale + (i0 % sel.scale_len));
#pragma unroll
        for (int j = 0; j < 4; j++) {
            float4 v = __ldg(p + j);
            s[4 * j] = v.x; s[4 * j + 1] = v.y; s[4 * j + 2] = v.z; s[4 * j + 3] = v.w;
        }
    } else if (SM == kScaleChunk) {
        const float v = __ldg(scale + (i0 / sel.inner) % sel.scale_len);
#pragma unroll
        for (int k = 0; k < 16; k++) s[k] = v;
    } else {
#pragma unroll
        for (int k = 0; k < 16; k++) s[k] = (k < cnt) ? __ldg(scale + ((i0 + k) / sel.inner) % sel.scale_len) : 1.0f;
    }
}

constexpr int kGroupsPerThread = 4;
constexpr int kThreadsPerBlock = 256;

template <int SM>
__device__ __forceinline__ void load_scales4(const float *__restrict__ scale, const ScaleSel sel, int64_t i0, float (&s)[4])
{
    if (SM == kScalePerTensor) {
        s[0] = s[1] = s[2] = s[3] = __ldg(scale);
    } else if (SM == kScaleLastAxis4) {
        const float4 v = __ldg(reinterpret_cast<const float4 *>(scale + (i0 % sel.scale_len)));
        s[0] = v.x; s[1] = v.y; s[2] = v.z; s[3] = v.w;
    } else if (SM == kScaleGroup) {
        s[0] = s[1] = s[2] = s[3] = __ldg(scale + (i0 / sel.inner) % sel.scale_len);
    } else {
#pragma unroll
        for (int k = 0; k < 4; k++) s[k] = __ldg(scale + ((i0 + k) / sel.inner) % sel.scale_len);
    }
}

// Which groups a thread owns: warp w of the grid covers groups [w*128, w*128 + 128); lane takes
// w*128 + j*32 + lane for j = 0..3.
__device__ __forceinline__ int64_t first_group(int64_t warp_index, int lane) { return warp_index * 128 + lane; }

// torch.round (half to even) of 16 values in place.  Below 2^22 adding and subtracting 1.5 * 2^23 IS
// that rounding (one binary32 add rounds to nearest even at integer granularity) and runs on the
// full-rate pipe; a thread that holds any larger magnitude takes the conversion instruction for its
// chunk instead (one branch per 16 values, rarely taken).  NaN stays NaN on either path.
__device__ __forceinline__ void round_half_even16(float (&t)[16])
{
    bool big = false;
#pragma unroll
    for (int k = 0; k < 16; k++) big = big || (fabsf(t[k]) >= 4194304.0f);
    if (big) {
#pragma unroll
        for (int k = 0; k < 16; k++) t[k] = rintf(t[k]);
    } else {
#pragma unroll
        for (int k = 0; k < 16; k++) t[k] = __fadd_rn(__fadd_rn(t[k], 12582912.0f), -12582912.0f);
    }
}

// clamp (torch.clamp keeps NaN; the cast of NaN gives 0) and cast to int8, returned in the low byte.
// FAST (bounds within +-2^22): the two's-complement low byte of an integer-valued float c is the low
// byte of the bits of c + 1.5 * 2^23, so no float->int conversion instruction is needed.
template <bool FAST>
__device__ __forceinline__ uint32_t clamp_cast_i8(float r, float lo, float hi)
{
    float c = fminf(fmaxf(r, lo), hi);
    c = (r != r) ? 0.0f : c;
    if (FAST) return __float_as_uint(__fadd_rn(c, 12582912.0f));
    return (uint32_t)(int)c;
}

// low bytes of four words -> one word
__device__ __forceinline__ uint32_t pack_i8x4(uint32_t a, uint32_t b, uint32_t c, uint32_t d)
{
    return __byte_perm(__byte_perm(a, b, 0x0040), __byte_perm(c, d, 0x0040), 0x5410);
}

// ------------------------------------------------------------------------------------------------
// quantize: MODE 0 divides by the scale, MODE 1 multiplies by it
// ------------------------------------------------------------------------------------------------
// Division by a scale that a thread meets again in every sweep (hoisted scales) need not be a division
// instruction sequence per element.  With r = RN(1 / s) (correctly rounded reciprocal), q' = RN(x * r) is within
// 1.5 * 2^-23 |x / s| of the true quotient, and the golden result depends on the quotient only through
// round-half-even(RN(x / s)).  So: round q' with the magic-number add; if q' lies farther than `screen` from every
// half-integer, RN(x / s) rounds to the same integer (screen >= 3 * 2^-24 * (B + 2), B = largest magnitude that does
// not saturate in the clamp; beyond B both saturate alike) and the cheap result stands; otherwise -- a few chunks in
// a thousand -- the chunk is redone with the IEEE division.  Bit-identical to the division, at a third of its
// instructions.  The host enables it (screen > 0) only for bounds and zero point within +-2^20, where values of
// magnitude 2^22 and above saturate whatever their rounding.
template <int MODE, int SM, bool VEC, bool FAST>
__global__ void __launch_bounds__(256)
quantize_kernel(const float *__restrict__ x, int64_t n, const float *__restrict__ scale, ScaleSel sel, float zp, float lo,
                float hi, int8_t *__restrict__ out, int hoist, float screen)
{
    const int64_t chunks = (n + 15) >> 4;
    float s[16];
    float r[16];
    bool rcp_ok = false;
    // when the grid stride is a whole number of scale periods a thread meets the same 16 scales in
    // every sweep: fetch them once
    if (hoist) load_scales16<SM>(scale, sel, ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) << 4, 16, s);
    if (MODE == 0 && FAST && hoist && screen > 0.0f) {
        rcp_ok = true;
#pragma unroll
        for (int k = 0; k < 16; k++) {
            r[k] = __frcp_rn(s[k]);
            const float a = fabsf(s[k]);
            rcp_ok = rcp_ok && (a >= 7.8886090522101181e-31f) && (a <= 1.2676506002282294e30f);   // 2^-100 .. 2^100; NaN fails
        }
    }
    for (int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; c < chunks; c += (int64_t)gridDim.x * blockDim.x) {
        const int64_t i0 = c << 4;
        const int cnt = (n - i0 >= 16) ? 16 : (int)(n - i0);
        float v[16];
        if (VEC && cnt == 16) {
            const float4 *p = reinterpret_cast<const float4 *>(x + i0);
#pragma unroll
            for (int j = 0; j < 4; j++) {
                float4 t = __ldcs(p + j);
                v[4 * j] = t.x; v[4 * j + 1] = t.y; v[4 * j + 2] = t.z; v[4 * j + 3] = t.w;
            }
        } else {
#pragma unroll
            for (int k = 0; k < 16; k++) v[k] = (k < cnt) ? x[i0 + k] : 0.0f;
        }
        if (!hoist) load_scales16<SM>(scale, sel, i0, cnt, s);
        uint32_t q[16];
        bool rounded = false;
        if (MODE == 0 && FAST && rcp_ok) {
            float t[16];
            bool risky = false;
#pragma unroll
            for (int k = 0; k < 16; k++) {
                const float qa = __fmul_rn(v[k], r[k]);
                t[k] = __fadd_rn(__fadd_rn(qa, 12582912.0f), -12582912.0f);
                risky = risky || (fabsf(fabsf(__fsub_rn(qa, t[k])) - 0.5f) < screen);
            }
            if (!risky) {
#pragma unroll
                for (int k = 0; k < 16; k++) v[k] = t[k];
                rounded = true;
            }
        }
        if (!rounded) {
#pragma unroll
            for (int k = 0; k < 16; k++) v[k] = (MODE == 0) ? __fdiv_rn(v[k], s[k]) : __fmul_rn(v[k], s[k]);
            round_half_even16(v);
        }
#pragma unroll
        for (int k = 0; k < 16; k++) q[k] = clamp_cast_i8<FAST>(__fadd_rn(v[k], zp), lo, hi);
        if (VEC && cnt == 16) {
            uint4 o = make_uint4(pack_i8x4(q[0], q[1], q[2], q[3]), pack_i8x4(q[4], q[5], q[6], q[7]),
                                 pack_i8x4(q[8], q[9], q[10], q[11]), pack_i8x4(q[12], q[13], q[14], q[15]));
            __stcs(reinterpret_cast<uint4 *>(out + i0), o);
        } else {
#pragma unroll
            for (int k = 0; k < 16; k++)
                if (k < cnt) out[i0 + k] = (int8_t)(q[k] & 0xffu);
        }
    }
}

// The same arithmetic for the commonest case (one scale for the tensor, aligned pointers, int8 bounds, a whole number
// of chunks), one chunk per thread and no loop: the four data loads are issued first, so nothing waits for the scale
// before them, and blocks that live for one sweep are handed out in address order by the hardware.
template <int MODE>
__global__ void __launch_bounds__(256)
quantize_once_kernel(const float *__restrict__ x, int64_t chunks, const float *__restrict__ scale, float zp, float lo, float hi,
                     int8_t *__restrict__ out, float screen)
{
    const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= chunks) return;
    const int64_t i0 = c << 4;
    float v[16];
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const float4 t = __ldcs(reinterpret_cast<const float4 *>(x + i0) + j);
        v[4 * j] = t.x; v[4 * j + 1] = t.y; v[4 * j + 2] = t.z; v[4 * j + 3] = t.w;
    }
    const float sc = __ldg(scale);
    bool rounded = false;
    if (MODE == 0 && screen > 0.0f) {
        const float a = fabsf(sc);
        if (a >= 7.8886090522101181e-31f && a <= 1.2676506002282294e30f) {   // 2^-100 .. 2^100; NaN fails
            const float r = __frcp_rn(sc);
            float t[16];
            bool risky = false;
#pragma unroll
            for (int k = 0; k < 16; k++) {
                const float qa = __fmul_rn(v[k], r);
                t[k] = __fadd_rn(__fadd_rn(qa, 12582912.0f), -12582912.0f);
                risky = risky || (fabsf(fabsf(__fsub_rn(qa, t[k])) - 0.5f) < screen);
            }
            if (!risky) {
#pragma unroll
                for (int k = 0; k < 16; k++) v[k] = t[k];
                rounded = true;
            }
        }
    }
    if (!rounded) {
#pragma unroll
        for (int k = 0; k < 16; k++) v[k] = (MODE == 0) ? __fdiv_rn(v[k], sc) : __fmul_rn(v[k], sc);
        round_half_even16(v);
    }
    uint32_t q[16];
#pragma unroll
    for (int k = 0; k < 16; k++) q[k] = clamp_cast_i8<true>(__fadd_rn(v[k], zp), lo, hi);
    __stcs(reinterpret_cast<uint4 *>(out + i0), make_uint4(pack_i8x4(q[0], q[1], q[2], q[3]), pack_i8x4(q[4], q[5], q[6], q[7]),
                                                            pack_i8x4(q[8], q[9], q[10], q[11]), pack_i8x4(q[12], q[13], q[14], q[15])));
}

// ------------------------------------------------------------------------------------------------
// dequantize
// ------------------------------------------------------------------------------------------------
template <int SM>
__global__ void __launch_bounds__(kThreadsPerBlock)
dequantize_vec_kernel(const int8_t *__restrict__ x, int64_t groups, const float *__restrict__ scale, ScaleSel sel, float zp,
                      float *__restrict__ out)
{
    const int lane = threadIdx.x & 31;
    const int64_t warps = (int64_t)gridDim.x * (kThreadsPerBlock / 32);
    for (int64_t w = (int64_t)blockIdx.x * (kThreadsPerBlock / 32) + (threadIdx.x >> 5); w * 128 < groups; w += warps) {
        const int64_t g0 = first_group(w, lane);
        uint32_t xw[kGroupsPerThread];
#pragma unroll
        for (int j = 0; j < kGroupsPerThread; j++) {
            const int64_t g = g0 + j * 32;
            xw[j] = (g < groups) ? __ldcs(reinterpret_cast<const uint32_t *>(x) + g) : 0u;
        }
#pragma unroll
        for (int j = 0; j < kGroupsPerThread; j++) {
            const int64_t g = g0 + j * 32;
            if (g < groups) {
                float s[4], r[4];
                load_scales4<SM>(scale, sel, g * 4, s);
                // int8 -> float without a conversion instruction: byte + 128 spliced under 1.5 * 2^23, minus the bias
                const uint32_t b = xw[j] ^ 0x80808080u;
#pragma unroll
                for (int k = 0; k < 4; k++) {
                    const float xf = __fadd_rn(__uint_as_float(__byte_perm(b, 0x4b400000u, 0x7650 + k)), -12583040.0f);
                    r[k] = __fmul_rn(__fsub_rn(xf, zp), s[k]);
                }
                __stcs(reinterpret_cast<float4 *>(out) + g, make_float4(r[0], r[1], r[2], r[3]));
            }
        }
    }
}

__global__ void __launch_bounds__(kThreadsPerBlock)
dequantize_scalar_kernel(const int8_t *__restrict__ x, int64_t first, int64_t n, const float *__restrict__ scale, ScaleSel sel,
                         float zp, float *__restrict__ out)
{
    for (int64_t i = first + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        out[i] = __fmul_rn(__fsub_rn((float)x[i], zp), scale[(i / sel.inner) % sel.scale_len]);
}

// ------------------------------------------------------------------------------------------------
// requantize: MODE 0 uses inp_scale / out_scale, MODE 1 uses scale_a alone
// ------------------------------------------------------------------------------------------------
template <int MODE, int SM, bool VEC, bool FAST>
__global__ void __launch_bounds__(256)
requantize_kernel(const int32_t *__restrict__ x, int64_t n, const float *__restrict__ scale_a,
                  const float *__restrict__ scale_b, ScaleSel sel, float zp, float lo, float hi, int8_t *__restrict__ out,
                  int hoist)
{
    const int64_t chunks = (n + 15) >> 4;
    float s[16];
    // when the grid stride is a whole number of scale periods a thread meets the same 16 scales in
    // every sweep: fetch (and, for Requantize, divide) them once
    if (hoist) {
        const int64_t i00 = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) << 4;
        load_scales16<SM>(scale_a, sel, i00, 16, s);
        if (MODE == 0) {
            float sb[16];
            load_scales16<SM>(scale_b, sel, i00, 16, sb);
#pragma unroll
            for (int k = 0; k < 16; k++) s[k] = __fdiv_rn(s[k], sb[k]);
        }
    }
    for (int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; c < chunks; c += (int64_t)gridDim.x * blockDim.x) {
        const int64_t i0 = c << 4;
        const int cnt = (n - i0 >= 16) ? 16 : (int)(n - i0);
        int xi[16];
        if (VEC && cnt == 16) {
            const int4 *p = reinterpret_cast<const int4 *>(x + i0);
#pragma unroll
            for (int j = 0; j < 4; j++) {
                int4 t = __ldcs(p + j);
                xi[4 * j] = t.x; xi[4 * j + 1] = t.y; xi[4 * j + 2] = t.z; xi[4 * j + 3] = t.w;
            }
        } else {
#pragma unroll
            for (int k = 0; k < 16; k++) xi[k] = (k < cnt) ? x[i0 + k] : 0;
        }
        if (!hoist) {
            load_scales16<SM>(scale_a, sel, i0, cnt, s);
            if (MODE == 0) {
                float sb[16];
                load_scales16<SM>(scale_b, sel, i0, cnt, sb);
#pragma unroll
                for (int k = 0; k < 16; k++) s[k] = __fdiv_rn(s[k], sb[k]);
            }
        }
        uint32_t q[16];
        float pz[16];
#pragma unroll
        for (int k = 0; k < 16; k++) {
            // the int32 operand is promoted to binary32 (round to nearest even) by the multiply
            pz[k] = __fadd_rn(__fmul_rn(s[k], __int2float_rn(xi[k])), zp);
        }
        round_half_even16(pz);
#pragma unroll
        for (int k = 0; k < 16; k++) q[k] = clamp_cast_i8<FAST>(pz[k], lo, hi);
        if (VEC && cnt == 16) {
            uint4 o = make_uint4(pack_i8x4(q[0], q[1], q[2], q[3]), pack_i8x4(q[4], q[5], q[6], q[7]),
                                 pack_i8x4(q[8], q[9], q[10], q[11]), pack_i8x4(q[12], q[13], q[14], q[15]));
            __stcs(reinterpret_cast<uint4 *>(out + i0), o);
        } else {
#pragma unroll
            for (int k = 0; k < 16; k++)
                if (k < cnt) out[i0 + k] = (int8_t)(q[k] & 0xffu);
        }
    }
}

// One chunk per thread and no loop (see quantize_once_kernel): one scale for the tensor, aligned pointers, int8 bounds,
// a whole number of chunks.
template <int MODE, int SM>
__global__ void __launch_bounds__(256)
requantize_once_kernel(const int32_t *__restrict__ x, int64_t chunks, const float *__restrict__ scale_a,
                       const float *__restrict__ scale_b, ScaleSel sel, float zp, float lo, float hi, int8_t *__restrict__ out)
{
    const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= chunks) return;
    const int64_t i0 = c << 4;
    int xi[16];
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const int4 t = __ldcs(reinterpret_cast<const int4 *>(x + i0) + j);
        xi[4 * j] = t.x; xi[4 * j + 1] = t.y; xi[4 * j + 2] = t.z; xi[4 * j + 3] = t.w;
    }
    float s[16];
    load_scales16<SM>(scale_a, sel, i0, 16, s);
    if (MODE == 0) {
        float sb[16];
        load_scales16<SM>(scale_b, sel, i0, 16, sb);
#pragma unroll
        for (int k = 0; k < 16; k++) s[k] = __fdiv_rn(s[k], sb[k]);
    }
    float pz[16];
#pragma unroll
    for (int k = 0; k < 16; k++) pz[k] = __fadd_rn(__fmul_rn(s[k], __int2float_rn(xi[k])), zp);
    round_half_even16(pz);
    uint32_t q[16];
#pragma unroll
    for (int k = 0; k < 16; k++) q[k] = clamp_cast_i8<true>(pz[k], lo, hi);
    __stcs(reinterpret_cast<uint4 *>(out + i0), make_uint4(pack_i8x4(q[0], q[1], q[2], q[3]), pack_i8x4(q[4], q[5], q[6], q[7]),
                                                            pack_i8x4(q[8], q[9], q[10], q[11]), pack_i8x4(q[12], q[13], q[14], q[15])));
}

// ------------------------------------------------------------------------------------------------
// host launchers
// ------------------------------------------------------------------------------------------------
static int pick_scale_mode(int64_t scale_len, int64_t inner, const void *sa, const void *sb)
{
    if (scale_len == 1) return kScalePerTensor;
    const bool al = ((reinterpret_cast<uintptr_t>(sa) | reinterpret_cast<uintptr_t>(sb)) & 15u) == 0;
    if (inner == 1 && (scale_len % 16) == 0 && al) return kScaleLastAxis16;
    if ((inner % 16) == 0) return kScaleChunk;
    return kScaleGeneral;
}

static unsigned grid_for_groups(int64_t groups, int sm_count)
{
    const int64_t per_block = (int64_t)(kThreadsPerBlock / 32) * 128;  // groups one block covers per sweep
    int64_t blocks = (groups + per_block - 1) / per_block;
    // No resident-wave cap here: this kernel is four fifths stores, and short-lived blocks handed out in address
    // order ran 3.6 % faster than 64 blocks per SM striding over the tensor (6240 vs 6020 GB/s at 2^27 elements).
    (void)sm_count;
    const int64_t cap = 0x7fffffff;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return (unsigned)blocks;
}

static unsigned grid_for_tail(int64_t n)
{
    int64_t blocks = (n + kThreadsPerBlock - 1) / kThreadsPerBlock;
    if (blocks > 65535) blocks = 65535;
    if (blocks < 1) blocks = 1;
    return (unsigned)blocks;
}

// One resident wave of blocks (8 x 256 threads per SM) sweeps the tensor, so a thread does several sweeps and what it
// fetched or derived once (per-axis scales, the reciprocal of the scale) pays off.  Measured: per-axis always faster
// this way; per-tensor 15 % faster at the 2^25-element size (30.3 vs 34.8 us), 1.4 % slower than many short-lived
// blocks at 2^27, hence the switch.
static unsigned grid_for(int64_t n, int sm_count, bool per_axis)
{
    const int64_t chunks = (n + 15) >> 4;
    int64_t blocks = (chunks + 255) / 256;
    const int64_t cap = (int64_t)sm_count * ((per_axis || n <= (int64_t(1) << 26)) ? 8 : 64);
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return (unsigned)blocks;
}

#define BUDA_SM_SWITCH(sm, CALL)                      \
    switch (sm) {                                     \
        case kScalePerTensor: CALL(kScalePerTensor); break;   \
        case kScaleLastAxis16: CALL(kScaleLastAxis16); break; \
        case kScaleChunk: CALL(kScaleChunk); break;   \
        default: CALL(kScaleGeneral); break;          \
    }

cudaError_t launch_quantize(const float *x, int64_t n, const float *scale, int64_t scale_len, int64_t inner, float zp,
                            int mode, float lo, float hi, int8_t *out, int sm_count, cudaStream_t stream)
{
    const ScaleSel sel{scale_len, inner};
    const int sm = pick_scale_mode(scale_len, inner, scale, nullptr);
    const bool vec = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out)) & 15u) == 0;
    const unsigned grid = grid_for(n, sm_count, sm != kScalePerTensor);
    const bool fast = lo >= -4194304.0f && hi <= 4194304.0f;
    // same scales in every sweep of the grid?  (per-tensor: trivially; last axis: stride a multiple of the period)
    const int hoist = (sm == kScalePerTensor || (sm == kScaleLastAxis16 && ((int64_t)grid * 256 * 16) % scale_len == 0)) ? 1 : 0;
    // screened-reciprocal division (see quantize_kernel): only where magnitudes of 2^22 and above saturate for sure
    float screen = 0.0f;
    if (mode == 0 && lo >= -1048576.0f && hi <= 1048576.0f && fabsf(zp) <= 1048576.0f) {
        const float B = fmaxf(fabsf(lo), fabsf(hi)) + fabsf(zp);
        screen = (B + 2.0f) * 2.384185791015625e-07f;   // (B + 2) * 2^-22
    }
    if (vec && fast && sm == kScalePerTensor && (n & 15) == 0 && n > 0) {
        const int64_t chunks = n >> 4;
        const unsigned once_grid = (unsigned)((chunks + 255) / 256);
        if (mode == 0) quantize_once_kernel<0><<<once_grid, 256, 0, stream>>>(x, chunks, scale, zp, lo, hi, out, screen);
        else quantize_once_kernel<1><<<once_grid, 256, 0, stream>>>(x, chunks, scale, zp, lo, hi, out, screen);
        return cudaGetLastError();
    }
#define CALL(SMV)                                                                                                     \
    if (mode == 0) {                                                                                                  \
        if (vec && fast) quantize_kernel<0, SMV, true, true><<<grid, 256, 0, stream>>>(x, n, scale, sel, zp, lo, hi, out, hoist, screen);   \
        else if (vec) quantize_kernel<0, SMV, true, false><<<grid, 256, 0, stream>>>(x, n, scale, sel, zp, lo, hi, out, hoist, screen);     \
        else quantize_kernel<0, SMV, false, false><<<grid, 256, 0, stream>>>(x, n, scale, sel, zp, lo, hi, out, hoist, screen);             \
    } else {                                                                                                          \
        if (vec && fast) quantize_kernel<1, SMV, true, true><<<grid, 256, 0, stream>>>(x, n, scale, sel, zp, lo, hi, out, hoist, screen);   \
        else if (vec) quantize_kernel<1, SMV, true, false><<<grid, 256, 0, stream>>>(x, n, scale, sel, zp, lo, hi, out, hoist, screen);     \
        else quantize_kernel<1, SMV, false, false><<<grid, 256, 0, stream>>>(x, n, scale, sel, zp, lo, hi, out, hoist, screen);             \
    }
    BUDA_SM_SWITCH(sm, CALL)
#undef CALL
    return cudaGetLastError();
}

cudaError_t launch_dequantize(const int8_t *x, int64_t n, const float *scale, int64_t scale_len, int64_t inner, float zp,
                              float *out, int sm_count, cudaStream_t stream)
{
    const ScaleSel sel{scale_len, inner};
    int sm = kScaleGeneral;
    if (scale_len == 1) sm = kScalePerTensor;
    else if (inner == 1 && (scale_len % 4) == 0 && (reinterpret_cast<uintptr_t>(scale) & 15u) == 0) sm = kScaleLastAxis4;
    else if ((inner % 4) == 0) sm = kScaleGroup;
    // the vector kernel takes the aligned body in groups of 4; a scalar kernel finishes the tail, or does
    // everything when a base pointer is not aligned for the vector accesses
    const bool vec = ((reinterpret_cast<uintptr_t>(x) & 3u) | (reinterpret_cast<uintptr_t>(out) & 15u)) == 0;
    const int64_t groups = vec ? n / 4 : 0;
    if (groups > 0) {
        const unsigned grid = grid_for_groups(groups, sm_count);
        switch (sm) {
            case kScalePerTensor: dequantize_vec_kernel<kScalePerTensor><<<grid, kThreadsPerBlock, 0, stream>>>(x, groups, scale, sel, zp, out); break;
            case kScaleLastAxis4: dequantize_vec_kernel<kScaleLastAxis4><<<grid, kThreadsPerBlock, 0, stream>>>(x, groups, scale, sel, zp, out); break;
            case kScaleGroup: dequantize_vec_kernel<kScaleGroup><<<grid, kThreadsPerBlock, 0, stream>>>(x, groups, scale, sel, zp, out); break;
            default: dequantize_vec_kernel<kScaleGeneral><<<grid, kThreadsPerBlock, 0, stream>>>(x, groups, scale, sel, zp, out); break;
        }
    }
    const int64_t first = groups * 4;
    if (first < n)
        dequantize_scalar_kernel<<<grid_for_tail(n - first), kThreadsPerBlock, 0, stream>>>(x, first, n, scale, sel, zp, out);
    return cudaGetLastError();
}

cudaError_t launch_requantize(const int32_t *x, int64_t n, const float *scale_a, const float *scale_b, int64_t scale_len,
                              int64_t inner, float zp, int mode, float lo, float hi, int8_t *out, int sm_count,
                              cudaStream_t stream)
{
    const ScaleSel sel{scale_len, inner};
    const int sm = pick_scale_mode(scale_len, inner, scale_a, mode == 0 ? scale_b : nullptr);
    const bool vec = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out)) & 15u) == 0;
    const unsigned grid = grid_for(n, sm_count, sm != kScalePerTensor);
    const bool fast = lo >= -4194304.0f && hi <= 4194304.0f;
    // same scales in every sweep of the grid?  (per-tensor: trivially; last axis: stride a multiple of the period)
    const int hoist = (sm == kScalePerTensor || (sm == kScaleLastAxis16 && ((int64_t)grid * 256 * 16) % scale_len == 0)) ? 1 : 0;
    // (with scales along the last axis the resident blocks that fetch their 16 scales once stay faster: 6070 vs 5070 GB/s for
    // one chunk per short-lived thread, and 3840 GB/s at the 2^25-element size for short-lived blocks of four runs of 256
    // chunks whose threads fetch their scales once -- at ~100 registers only two such blocks fit an SM)
    if (vec && fast && sm == kScalePerTensor && (n & 15) == 0 && n > 0) {
        const int64_t chunks = n >> 4;
        const unsigned once_grid = (unsigned)((chunks + 255) / 256);
        if (mode == 0)
            requantize_once_kernel<0, kScalePerTensor><<<once_grid, 256, 0, stream>>>(x, chunks, scale_a, scale_b, sel, zp, lo, hi, out);
        else
            requantize_once_kernel<1, kScalePerTensor><<<once_grid, 256, 0, stream>>>(x, chunks, scale_a, scale_b, sel, zp, lo, hi, out);
        return cudaGetLastError();
    }
#define CALL(SMV)                                                                                                                 \
    if (mode == 0) {                                                                                                              \
        if (vec && fast) requantize_kernel<0, SMV, true, true><<<grid, 256, 0, stream>>>(x, n, scale_a, scale_b, sel, zp, lo, hi, out, hoist);  \
        else if (vec) requantize_kernel<0, SMV, true, false><<<grid, 256, 0, stream>>>(x, n, scale_a, scale_b, sel, zp, lo, hi, out, hoist);    \
        else requantize_kernel<0, SMV, false, false><<<grid, 256, 0, stream>>>(x, n, scale_a, scale_b, sel, zp, lo, hi, out, hoist);            \
    } else {                                                                                                                      \
        if (vec && fast) requantize_kernel<1, SMV, true, true><<<grid, 256, 0, stream>>>(x, n, scale_a, scale_b, sel, zp, lo, hi, out, hoist);  \
        else if (vec) requantize_kernel<1, SMV, true, false><<<grid, 256, 0, stream>>>(x, n, scale_a, scale_b, sel, zp, lo, hi, out, hoist);    \
        else requantize_kernel<1, SMV, false, false><<<grid, 256, 0, stream>>>(x, n, scale_a, scale_b, sel, zp, lo, hi, out, hoist);            \
    }
    BUDA_SM_SWITCH(sm, CALL)
#undef CALL
    return cudaGetLastError();
}

}  // namespace buda
