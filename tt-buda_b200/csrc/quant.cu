// K4 / K5 / K6: the golden int8 quantisation ops as streaming kernels.
//
// Each kernel evaluates, per element, exactly the chain of binary32 operations of the reference's
// torch expressions (pybuda/pybuda/op/eval/pybuda/quantize.py:55-122 and
// pybuda/pybuda/op/eval/buda/quantize.py:23-53): IEEE division, separate multiply and add (never
// fused), round-half-to-even, clamp, truncating cast; NaN survives the clamp and casts to 0.
//
// A thread owns 16 consecutive elements: four 128-bit streaming loads in flight, one 128-bit store
// (quantise / requantise) or four (dequantise).  The scale of element i is
// scale[(i / inner) % scale_len].
#include "buda_common.cuh"

namespace buda {

enum ScaleMode : int {
    kScalePerTensor = 0,   // scale_len == 1
    kScaleLastAxis16 = 1,  // inner == 1, scale_len % 16 == 0: 16 consecutive scales per thread
    kScaleChunk = 2,       // inner % 16 == 0: one scale per 16-element chunk
    kScaleGeneral = 3      // per-element index arithmetic
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
template <int MODE, int SM, bool VEC, bool FAST>
__global__ void __launch_bounds__(256)
quantize_kernel(const float *__restrict__ x, int64_t n, const float *__restrict__ scale, ScaleSel sel, float zp, float lo,
                float hi, int8_t *__restrict__ out)
{
    const int64_t chunks = (n + 15) >> 4;
    for (int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; c < chunks; c += (int64_t)gridDim.x * blockDim.x) {
        const int64_t i0 = c << 4;
        const int cnt = (n - i0 >= 16) ? 16 : (int)(n - i0);
        float v[16], s[16];
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
        load_scales16<SM>(scale, sel, i0, cnt, s);
        uint32_t q[16];
#pragma unroll
        for (int k = 0; k < 16; k++) v[k] = (MODE == 0) ? __fdiv_rn(v[k], s[k]) : __fmul_rn(v[k], s[k]);
        round_half_even16(v);
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

// ------------------------------------------------------------------------------------------------
// dequantize
// ------------------------------------------------------------------------------------------------
template <int SM, bool VEC>
__global__ void __launch_bounds__(256)
dequantize_kernel(const int8_t *__restrict__ x, int64_t n, const float *__restrict__ scale, ScaleSel sel, float zp,
                  float *__restrict__ out)
{
    const int64_t chunks = (n + 15) >> 4;
    for (int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; c < chunks; c += (int64_t)gridDim.x * blockDim.x) {
        const int64_t i0 = c << 4;
        const int cnt = (n - i0 >= 16) ? 16 : (int)(n - i0);
        float xf[16];
        float s[16];
        if (VEC && cnt == 16) {
            const uint4 t = __ldcs(reinterpret_cast<const uint4 *>(x + i0));
            const uint32_t w[4] = {t.x ^ 0x80808080u, t.y ^ 0x80808080u, t.z ^ 0x80808080u, t.w ^ 0x80808080u};
            // int8 -> float without a conversion instruction: byte + 128 spliced under 1.5 * 2^23, minus the bias
#pragma unroll
            for (int k = 0; k < 16; k++)
                xf[k] = __fadd_rn(__uint_as_float(__byte_perm(w[k >> 2], 0x4b400000u, 0x7650 + (k & 3))), -12583040.0f);
        } else {
#pragma unroll
            for (int k = 0; k < 16; k++) xf[k] = (k < cnt) ? (float)x[i0 + k] : 0.0f;
        }
        load_scales16<SM>(scale, sel, i0, cnt, s);
        float r[16];
#pragma unroll
        for (int k = 0; k < 16; k++) r[k] = __fmul_rn(__fsub_rn(xf[k], zp), s[k]);
        if (VEC && cnt == 16) {
            float4 *o = reinterpret_cast<float4 *>(out + i0);
#pragma unroll
            for (int j = 0; j < 4; j++) __stcs(o + j, make_float4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]));
        } else {
#pragma unroll
            for (int k = 0; k < 16; k++)
                if (k < cnt) out[i0 + k] = r[k];
        }
    }
}

// ------------------------------------------------------------------------------------------------
// requantize: MODE 0 uses inp_scale / out_scale, MODE 1 uses scale_a alone
// ------------------------------------------------------------------------------------------------
template <int MODE, int SM, bool VEC, bool FAST>
__global__ void __launch_bounds__(256)
requantize_kernel(const int32_t *__restrict__ x, int64_t n, const float *__restrict__ scale_a,
                  const float *__restrict__ scale_b, ScaleSel sel, float zp, float lo, float hi, int8_t *__restrict__ out)
{
    const int64_t chunks = (n + 15) >> 4;
    for (int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; c < chunks; c += (int64_t)gridDim.x * blockDim.x) {
        const int64_t i0 = c << 4;
        const int cnt = (n - i0 >= 16) ? 16 : (int)(n - i0);
        int xi[16];
        float s[16];
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
        load_scales16<SM>(scale_a, sel, i0, cnt, s);
        if (MODE == 0) {
            float sb[16];
            load_scales16<SM>(scale_b, sel, i0, cnt, sb);
#pragma unroll
            for (int k = 0; k < 16; k++) s[k] = __fdiv_rn(s[k], sb[k]);
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

static unsigned grid_for(int64_t n, int sm_count)
{
    const int64_t chunks = (n + 15) >> 4;
    int64_t blocks = (chunks + 255) / 256;
    const int64_t cap = (int64_t)sm_count * 64;
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
    const unsigned grid = grid_for(n, sm_count);
    const bool fast = lo >= -4194304.0f && hi <= 4194304.0f;
#define CALL(SMV)                                                                                                     \
    if (mode == 0) {                                                                                                  \
        if (vec && fast) quantize_kernel<0, SMV, true, true><<<grid, 256, 0, stream>>>(x, n, scale, sel, zp, lo, hi, out);   \
        else if (vec) quantize_kernel<0, SMV, true, false><<<grid, 256, 0, stream>>>(x, n, scale, sel, zp, lo, hi, out);     \
        else quantize_kernel<0, SMV, false, false><<<grid, 256, 0, stream>>>(x, n, scale, sel, zp, lo, hi, out);             \
    } else {                                                                                                          \
        if (vec && fast) quantize_kernel<1, SMV, true, true><<<grid, 256, 0, stream>>>(x, n, scale, sel, zp, lo, hi, out);   \
        else if (vec) quantize_kernel<1, SMV, true, false><<<grid, 256, 0, stream>>>(x, n, scale, sel, zp, lo, hi, out);     \
        else quantize_kernel<1, SMV, false, false><<<grid, 256, 0, stream>>>(x, n, scale, sel, zp, lo, hi, out);             \
    }
    BUDA_SM_SWITCH(sm, CALL)
#undef CALL
    return cudaGetLastError();
}

cudaError_t launch_dequantize(const int8_t *x, int64_t n, const float *scale, int64_t scale_len, int64_t inner, float zp,
                              float *out, int sm_count, cudaStream_t stream)
{
    const ScaleSel sel{scale_len, inner};
    const int sm = pick_scale_mode(scale_len, inner, scale, nullptr);
    const bool vec = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out)) & 15u) == 0;
    const unsigned grid = grid_for(n, sm_count);
#define CALL(SMV)                                                                                   \
    if (vec) dequantize_kernel<SMV, true><<<grid, 256, 0, stream>>>(x, n, scale, sel, zp, out);     \
    else dequantize_kernel<SMV, false><<<grid, 256, 0, stream>>>(x, n, scale, sel, zp, out);
    BUDA_SM_SWITCH(sm, CALL)
#undef CALL
    return cudaGetLastError();
}

cudaError_t launch_requantize(const int32_t *x, int64_t n, const float *scale_a, const float *scale_b, int64_t scale_len,
                              int64_t inner, float zp, int mode, float lo, float hi, int8_t *out, int sm_count,
                              cudaStream_t stream)
{
    const ScaleSel sel{scale_len, inner};
    const int sm = pick_scale_mode(scale_len, inner, scale_a, mode == 0 ? scale_b : nullptr);
    const bool vec = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out)) & 15u) == 0;
    const unsigned grid = grid_for(n, sm_count);
    const bool fast = lo >= -4194304.0f && hi <= 4194304.0f;
#define CALL(SMV)                                                                                                                 \
    if (mode == 0) {                                                                                                              \
        if (vec && fast) requantize_kernel<0, SMV, true, true><<<grid, 256, 0, stream>>>(x, n, scale_a, scale_b, sel, zp, lo, hi, out);  \
        else if (vec) requantize_kernel<0, SMV, true, false><<<grid, 256, 0, stream>>>(x, n, scale_a, scale_b, sel, zp, lo, hi, out);    \
        else requantize_kernel<0, SMV, false, false><<<grid, 256, 0, stream>>>(x, n, scale_a, scale_b, sel, zp, lo, hi, out);            \
    } else {                                                                                                                      \
        if (vec && fast) requantize_kernel<1, SMV, true, true><<<grid, 256, 0, stream>>>(x, n, scale_a, scale_b, sel, zp, lo, hi, out);  \
        else if (vec) requantize_kernel<1, SMV, true, false><<<grid, 256, 0, stream>>>(x, n, scale_a, scale_b, sel, zp, lo, hi, out);    \
        else requantize_kernel<1, SMV, false, false><<<grid, 256, 0, stream>>>(x, n, scale_a, scale_b, sel, zp, lo, hi, out);            \
    }
    BUDA_SM_SWITCH(sm, CALL)
#undef CALL
    return cudaGetLastError();
}

}  // namespace buda
