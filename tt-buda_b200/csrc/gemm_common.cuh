// Pieces shared by the tensor-core matmul kernels: shared-memory matrix descriptors, TMA tile loads,
// tcgen05 fences / loads / commits, cluster helpers, the bfloat16 decode of one Bfp8_b block, and the
// host-side tensor-map encoder lookup.
#pragma once

#include <cuda.h>

#include "buda_common.cuh"

namespace buda {
namespace gemm {

constexpr int kRecord = 1088;   // Bfp8_b tile record, no header
constexpr int kMaxDst = 8;      // destinations one epilogue can write (this device + peers)

__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes)
{
    // start address, leading / stride byte offsets in 16-byte units, descriptor version 1, 128B swizzle
    return (uint64_t)((addr >> 4) & 0x3fffu) | ((uint64_t)((lbo_bytes >> 4) & 0x3fffu) << 16) |
           ((uint64_t)((sbo_bytes >> 4) & 0x3fffu) << 32) | (1ull << 46) | (2ull << 61);
}

__device__ __forceinline__ void tma_load_2d(void *smem_dst, const CUtensorMap *tmap, int x, int y, uint64_t *bar)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
            smem_u32(smem_dst)),
        "l"(reinterpret_cast<uint64_t>(tmap)), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}

// One tile of shared memory (laid out as the tensor map's box, 128-byte swizzle) to global memory, this device's or a
// peer's; completion is tracked by the issuing thread's bulk group.  x * element size is a multiple of 16 bytes at every
// call site, and no coordinate is negative.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap *tmap, const void *smem_src, int x, int y)
{
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];" ::"l"(reinterpret_cast<uint64_t>(tmap)),
                 "r"(x), "r"(y), "r"(smem_u32(smem_src))
                 : "memory");
}

// Tensor maps of the output matrix on every destination (this device first, then peers)
struct alignas(64) OutMaps {
    CUtensorMap m[kMaxDst];
};

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// arrive on an mbarrier once every tcgen05.mma issued so far by this thread has completed
__device__ __forceinline__ void umma_commit(uint64_t *bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// 32 consecutive accumulator columns of this thread's lane; the values are valid after tmem_ld_wait()
__device__ __forceinline__ void tmem_ld32_issue(uint32_t taddr, uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, "
        "[%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32])
{
    tmem_ld32_issue(taddr, r);
    tmem_ld_wait();
}

__device__ __forceinline__ uint32_t fma_bf16x2(uint32_t a, uint32_t b, uint32_t c)
{
    uint32_t d;
    asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi)
{
    uint32_t d;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
    return d;
}


// ------------------------------------------------------------------------------------------------
// Thread-block clusters (CTA pairs)
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}

// every thread of every CTA in the cluster; orders shared-memory initialisation before remote use
__device__ __forceinline__ void cluster_sync_all()
{
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// shared::cluster address of `local_addr` (a shared::cta address) in the CTA of rank `rank`
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_addr, uint32_t rank)
{
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
    return r;
}

// arrive on an mbarrier that may live in the peer CTA (address from map_to_cta).  The data this signals is
// read by the tensor cores through the async proxy, after the writers' own fence.proxy.async; the arrive
// itself carries the default (release, CTA scope) ordering.  Cluster-scope release / acquire forms were
// measured to add roughly 0.4 us to every k-block of the pair kernel's issue loop.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr)
{
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait_parked_cluster(uint64_t *bar, uint32_t parity, uint32_t hint_ns)
{
    return mbar_try_wait_parked(bar, parity, hint_ns);
}

// Bounded wait on a barrier whose arrivals come from both CTAs of a pair.
__device__ __forceinline__ bool mbar_wait_bounded_cluster(uint64_t *bar, uint32_t parity, volatile int *abort_flag,
                                                          unsigned int *status, unsigned int code)
{
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = global_timer_ns();
    while (true) {
        if (mbar_try_wait_parked_cluster(bar, parity, 20000u)) return true;
        if (*abort_flag) return false;
        if (global_timer_ns() - t0 > kWaitLimitNs) {
            *abort_flag = 1;
            report_status(status, code);
            return false;
        }
    }
}

// ------------------------------------------------------------------------------------------------
// Decode of one Bfp8_b block (16 values: fixed k, 16 consecutive n, one shared exponent) to bfloat16,
// written into an N-major ("MN-major") 128B-swizzled operand tile whose 64-column x 8-deep atoms
// (1024 B) are laid out [k / 8][n / 64]; kAtomsN = atoms along n (4 for a 256-column stage, 2 for 128).
// ------------------------------------------------------------------------------------------------
template <int kAtomsN>
__device__ __forceinline__ void decode_block_to_operand(const uint4 mant, const uint32_t exponent, uint8_t *stage, int k_local,
                                                        int n_local)
{
    // scale 2^(E-133) as bfloat16 bits (exponent field E-6) in both halves; -128 * scale beside it.
    // Blocks below 2^-126 (E < 7) flush to zero.
    const uint32_t e6 = max(exponent, 6u) - 6u;
    const uint32_t sc = e6 * 0x00800080u;
    const uint32_t off = e6 ? sc + 0x83808380u : 0u;
    const uint32_t w[4] = {mant.x, mant.y, mant.z, mant.w};
    uint32_t o[8];
#pragma unroll
    for (int q = 0; q < 4; q++) {
        const uint32_t mg = w[q] & 0x7f7f7f7fu, sg = w[q] & 0x80808080u;
        // (128 + m) as bfloat16 is 0x4300 | m: splice each magnitude byte under 0x43
        const uint32_t p01 = __byte_perm(mg, 0x43434343u, 0x4140);
        const uint32_t p23 = __byte_perm(mg, 0x43434343u, 0x4342);
        o[2 * q] = fma_bf16x2(p01, sc, off) | __byte_perm(sg, 0u, 0x1404);
        o[2 * q + 1] = fma_bf16x2(p23, sc, off) | __byte_perm(sg, 0u, 0x3424);
    }
    const int kr = k_local & 7, c0 = (n_local & 63) >> 3;
    uint8_t *dst = stage + ((k_local >> 3) * kAtomsN + (n_local >> 6)) * 1024 + kr * 128;
    *reinterpret_cast<uint4 *>(dst + ((c0 ^ kr) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
    *reinterpret_cast<uint4 *>(dst + (((c0 + 1) ^ kr) << 4)) = make_uint4(o[4], o[5], o[6], o[7]);
}

// rounds 32 binary32 accumulator values of one row to bfloat16 and stores them to every destination
__device__ __forceinline__ void store_row32(const uint32_t (&v)[32], uint16_t *const *dst, int n_dst, int64_t elem_offset)
{
    uint4 o[4];
#pragma unroll
    for (int q = 0; q < 4; q++) {
        o[q].x = pack_bf16x2(__uint_as_float(v[8 * q]), __uint_as_float(v[8 * q + 1]));
        o[q].y = pack_bf16x2(__uint_as_float(v[8 * q + 2]), __uint_as_float(v[8 * q + 3]));
        o[q].z = pack_bf16x2(__uint_as_float(v[8 * q + 4]), __uint_as_float(v[8 * q + 5]));
        o[q].w = pack_bf16x2(__uint_as_float(v[8 * q + 6]), __uint_as_float(v[8 * q + 7]));
    }
    for (int d = 0; d < n_dst; d++) {
        uint4 *out = reinterpret_cast<uint4 *>(dst[d] + elem_offset);
#pragma unroll
        for (int q = 0; q < 4; q++) out[q] = o[q];
    }
}

struct Params;
__device__ __forceinline__ void store_row32_i8(const uint32_t (&v)[32], const Params &p, int64_t elem_offset, int col);

struct Params {
    const uint8_t *W;         // weight image: record (kt, nt) at (kt * Nt + nt) * record bytes
    uint16_t *C[kMaxDst];     // destinations (this device first, then peers), row stride ldc ELEMENTS of the output type
    int n_dst;
    uint16_t *C_mc;           // multicast address of the same matrix on every device of the group (NVSwitch replicates
                              // one store to all of them), or null
    int64_t M, N, K, ldc;
    uint32_t m_tiles, n_tiles, k_blocks, Nt;
    uint32_t raster_m;        // pair kernel: output tiles are walked in groups of this many tile rows (see tile_coords)
    int tma_epilogue;         // pair kernel, Bfp8 kind: output tiles leave through shared memory and bulk tensor stores
    unsigned int *status;
    // int8 kind only: what the epilogue does with the int32 accumulators
    int out_mode;             // BUDA_I8_OUT_*
    const float *scale;       // per column (scale_len == N) or one value (scale_len == 1); unused for int32 output
    int64_t scale_len;
    float zero_point, lo, hi;
};

// Which output tile the t-th work unit is.  Tiles are walked in groups of raster_m tile rows: down the rows of a group,
// then along the columns, then the next group.  The pairs that run at the same time then share a few tile rows of the
// activations, which stay in L2 for the whole sweep over the columns, instead of streaming all of A once per wave.
__device__ __forceinline__ void tile_coords(const Params &p, uint32_t t, uint32_t &m_blk, uint32_t &n_blk)
{
    const uint32_t per_group = p.raster_m * p.n_tiles;
    const uint32_t group = t / per_group, within = t - group * per_group;
    const uint32_t m0 = group * p.raster_m;
    const uint32_t rows = min(p.raster_m, p.m_tiles - m0);      // the last group may be shorter
    n_blk = within / rows;
    m_blk = m0 + (within - n_blk * rows);
}

// Requantisation of 32 consecutive columns of one row (first column `col`) to int8, four values per word.
__device__ __forceinline__ void requant_row32(const uint32_t (&v)[32], const Params &p, int col, uint32_t (&packed)[8])
{
    const bool per_col = p.scale_len != 1;
    const float s0 = __ldg(p.scale);
    const float4 *scv = reinterpret_cast<const float4 *>(p.scale + (per_col ? col : 0));
    // clamp, then round: the bounds are integers and rounding is monotone, so this equals the golden
    // round-then-clamp; after the clamp |c| <= 128, where adding 1.5 * 2^23 rounds half to even and leaves the
    // two's-complement result in the low byte of the sum's bits -- no round or float->int conversion instruction
    // (those run at a quarter of the rate and were the epilogue's bottleneck: 0.124 ms of a 0.468 ms launch).
#pragma unroll
    for (int q = 0; q < 8; q++) {
        const float4 sc = per_col ? __ldg(scv + q) : make_float4(s0, s0, s0, s0);
        const float s4[4] = {sc.x, sc.y, sc.z, sc.w};
        uint32_t b4[4];
#pragma unroll
        for (int b = 0; b < 4; b++) {
            const float f = __fadd_rn(__fmul_rn(__int2float_rn((int)v[4 * q + b]), s4[b]), p.zero_point);
            float c = fminf(fmaxf(f, p.lo), p.hi);
            c = (f != f) ? 0.0f : c;                      // NaN (e.g. 0 * inf) becomes 0, as in the stand-alone quantise kernels
            b4[b] = __float_as_uint(__fadd_rn(c, 12582912.0f));
        }
        packed[q] = __byte_perm(__byte_perm(b4[0], b4[1], 0x0040), __byte_perm(b4[2], b4[3], 0x0040), 0x5410);
    }
}

// Epilogue of the int8 matmul for 32 consecutive columns of one row (first column `col`): the int32
// accumulators as they are, requantised to int8, or dequantised to float32.  The arithmetic is the golden
// evaluation's, operation by operation (separate multiply and add, round half to even, clamp, cast):
//   requantise  clamp(round(float(acc) * scale + zero_point), lo, hi)      pybuda/pybuda/op/eval/buda/quantize.py:42-53
//   dequantise  (float(acc) - zero_point) * scale                            pybuda/pybuda/op/eval/buda/quantize.py:35-40
__device__ __forceinline__ void store_row32_i8(const uint32_t (&v)[32], const Params &p, int64_t elem_offset, int col)
{
    if (p.out_mode == BUDA_I8_OUT_INT32) {
        uint32_t *out = reinterpret_cast<uint32_t *>(p.C[0]) + elem_offset;
#pragma unroll
        for (int q = 0; q < 8; q++)
            reinterpret_cast<uint4 *>(out)[q] = make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
        return;
    }
    const bool per_col = p.scale_len != 1;
    const float s0 = __ldg(p.scale);
    const float4 *scv = reinterpret_cast<const float4 *>(p.scale + (per_col ? col : 0));
    if (p.out_mode == BUDA_I8_OUT_DEQUANT_F32) {
        float *out = reinterpret_cast<float *>(p.C[0]) + elem_offset;
#pragma unroll
        for (int q = 0; q < 8; q++) {
            const float4 sc = per_col ? __ldg(scv + q) : make_float4(s0, s0, s0, s0);
            float4 f;
            f.x = __fmul_rn(__fsub_rn(__int2float_rn((int)v[4 * q]), p.zero_point), sc.x);
            f.y = __fmul_rn(__fsub_rn(__int2float_rn((int)v[4 * q + 1]), p.zero_point), sc.y);
            f.z = __fmul_rn(__fsub_rn(__int2float_rn((int)v[4 * q + 2]), p.zero_point), sc.z);
            f.w = __fmul_rn(__fsub_rn(__int2float_rn((int)v[4 * q + 3]), p.zero_point), sc.w);
            reinterpret_cast<float4 *>(out)[q] = f;
        }
        return;
    }
    uint32_t packed[8];
    requant_row32(v, p, col, packed);
    uint8_t *out = reinterpret_cast<uint8_t *>(p.C[0]) + elem_offset;
    reinterpret_cast<uint4 *>(out)[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
    reinterpret_cast<uint4 *>(out)[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn()
{
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
    return fn;
}


}  // namespace gemm
}  // namespace buda
