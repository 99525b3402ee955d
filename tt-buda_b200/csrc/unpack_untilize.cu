// K2 / K3 (inverse): queue image of 32x32 tiles -> row-major tensor, fused with the
// Bfp8_b / Bfp4_b / Bfp2_b decode to binary32 or bfloat16 (or a plain relayout).
//
// Device counterpart of the conversion the reference performs inside tt::backend::get_output
// (bound at pybuda/csrc/backend_api/backend_api.cpp:701).
//
// Mirror image of the pack kernels: the staged kernel brings whole tile records into shared
// memory with bulk async copies (one per tile), a thread decodes one 16-value block and writes it
// into a padded row-major band in shared memory, and the band leaves with plain coalesced stores
// (lanes along the row, 512 contiguous bytes per warp instruction; measured 11-15 % faster than one
// bulk async store per row, whose completion the next band had to wait for).  The direct kernel
// (any alignment) gives each block to four lanes.
// As on the pack side every kernel has a plain flavour (a batch of tensors of one shape, default byte layout) and a
// general one (template flag G: a table with one entry per tensor, and the layout policy's face / exponent / datum order).
#include "bfp_codec.cuh"
#include <atomic>

#include "buda_common.cuh"
#include "work_slots_cuda.cuh"

namespace buda {

constexpr int kUConsumerWarps = 8;
constexpr int kUConsumerThreads = kUConsumerWarps * 32;
constexpr int kUStagedThreads = kUConsumerThreads + 32;

struct UItemMeta {
    uint32_t b, w, z, rt, ct0, ntiles, pad0, pad1;
};

template <int M, int ES>
struct UnpackCfg {
    static constexpr int box = unpack_box_tiles_for(ES, M > 0);
    static constexpr int row_bytes = box * 32 * ES;
    static constexpr int pitch = row_bytes + 16;
    static constexpr int out_buf_bytes = 32 * pitch;
    static constexpr int payload = (M > 0) ? (64 + 1024 * (M + 1) / 8) : (1024 * ES);
    static constexpr int rec_max = payload + 32;
    static constexpr int in_stage_bytes = box * rec_max;
    static constexpr int stages = box > kBoxTiles ? 2 : 4;   // 16-tile items: two stages keep two CTAs per SM
    static constexpr int out_bufs = 2;
    static constexpr int smem_bytes = stages * in_stage_bytes + out_bufs * out_buf_bytes + stages * (int)sizeof(UItemMeta) +
                                      2 * stages * 8 + 16;
    // general flavour: a copy of the table entry in use, the first work item of every entry, and per stage where the
    // item's band starts in the row-major tensor and its row stride (worked out by the producer, which holds the entry)
    static constexpr int gen_extra_bytes = 136 + (kMaxGen + 1) * 4 + 4 + stages * 2 * 8;
    template <bool G>
    static constexpr int smem_for() { return smem_bytes + (G ? gen_extra_bytes : 0); }
};

__device__ __forceinline__ void decode_uitem(const TileJob &job, uint32_t item, UItemMeta &m)
{
    uint32_t cb = item % job.boxes_per_band;
    uint32_t q = item / job.boxes_per_band;
    m.rt = q % job.Rt;
    q /= job.Rt;
    m.z = q % job.Z;
    q /= job.Z;
    m.w = q % job.W;
    m.b = q / job.W;
    m.ct0 = cb * job.box_tiles;
    m.ntiles = min(job.box_tiles, job.Ct - m.ct0);
}

// In this file PtrTable.src is the queue image and PtrTable.dst the row-major tensor.
__device__ __forceinline__ uint32_t pack_half2(float lo, float hi)
{
    uint32_t d;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));  // exact for decoded values; overflow gives infinity
    return d;
}

// General flavour.  Kernel parameters are slow to read with a run-time index, so the table is touched as little as
// possible: every entry's first work item is copied to shared memory once per CTA, the entry a work item belongs to is
// found there by bisection, and the entry itself is copied to shared memory when the producer moves on to it.
struct UGenCache {
    GenEntry e;                       // 128 bytes
    uint32_t loaded, pad;             // index of the entry held in e
};
static_assert(sizeof(UGenCache) == 136, "shared-memory plan of the general flavour");

__device__ __forceinline__ void ugen_load_starts(const GenTable &tab, uint32_t total_items, uint32_t *starts, int tid, int nthreads)
{
    for (uint32_t i = (uint32_t)tid; i <= tab.n; i += (uint32_t)nthreads) starts[i] = i < tab.n ? tab.e[i].item_start : total_items;
}

// whole producer warp; returns with *cache holding the entry of `item`
__device__ __forceinline__ void ugen_find_entry(const GenTable &tab, const uint32_t *starts, uint32_t item, UGenCache *cache, int lane)
{
    const uint32_t idx = cache->loaded;
    if (idx >= tab.n || item < starts[idx] || item >= starts[idx + 1u]) {
        uint32_t lo = 0, hi = tab.n;          // largest index with starts[index] <= item
        while (hi - lo > 1u) {
            const uint32_t mid = (lo + hi) >> 1;
            if (starts[mid] <= item) lo = mid; else hi = mid;
        }
        __syncwarp();
        const uint32_t *src = reinterpret_cast<const uint32_t *>(&tab.e[lo]);
        reinterpret_cast<uint32_t *>(&cache->e)[lane] = src[lane];   // 32 lanes x 4 bytes = the entry
        if (lane == 31) cache->loaded = lo;
        __syncwarp();
    }
}

__device__ __forceinline__ void decode_uitem_gen(const UGenCache *cache, const TileJob &common, uint32_t item, UItemMeta &m)
{
    const GenEntry &e = cache->e;
    // divisions by this entry's own numbers as multiply-and-shift; one slice and one entry (the usual case) need none
    const uint32_t q0 = item - e.item_start;
    const uint32_t q1 = fast_div(q0, e.bpb_magic, e.bpb_shift);
    const uint32_t cb = q0 - q1 * e.boxes_per_band;
    const uint32_t q2 = fast_div(q1, e.bands_magic, e.bands_shift);
    const uint32_t k = q1 - q2 * e.bands;
    m.rt = e.band_first + k * e.band_step;
    if (e.Z == 1u) {
        m.z = 0;
        m.w = q2;
    } else {
        m.w = q2 / e.Z;
        m.z = q2 - m.w * e.Z;
    }
    m.b = cache->loaded;
    m.ct0 = cb * common.box_tiles;
    m.ntiles = min(common.box_tiles, e.Ct - m.ct0);
}

static __device__ WorkCounter g_unpack_work[kWorkSlots];

template <bool G> struct UTableOf { using type = PtrTable; };
template <> struct UTableOf<true> { using type = GenTable; };

// P: the launch honours a non-default layout policy (see the pack kernel)
template <int M, int ES, bool AF, bool G, bool P>
__global__ void __launch_bounds__(kUStagedThreads)
unpack_staged_kernel(const __grid_constant__ TileJob job, const __grid_constant__ typename UTableOf<G>::type ptrs, unsigned int *status)
{
    using Cfg = UnpackCfg<M, ES>;
    constexpr int S = Cfg::stages;
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t *in_stage = smem;
    uint8_t *out_buf = smem + S * Cfg::in_stage_bytes;
    UItemMeta *meta = reinterpret_cast<UItemMeta *>(out_buf + Cfg::out_bufs * Cfg::out_buf_bytes);
    uint64_t *full = reinterpret_cast<uint64_t *>(meta + S);
    uint64_t *empty = full + S;
    volatile int *abort_flag = reinterpret_cast<volatile int *>(empty + S);
    // general flavour only (see UnpackCfg::gen_extra_bytes)
    UGenCache *gcache = reinterpret_cast<UGenCache *>(reinterpret_cast<uint8_t *>(empty + S) + 16);
    uint32_t *gstarts = reinterpret_cast<uint32_t *>(gcache + 1);
    uint64_t *gband = reinterpret_cast<uint64_t *>(gstarts + kMaxGen + 2);   // [stage][band start, row stride]

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t rec = job.tile_bytes, hdr = job.header_bytes;

    if (tid == 0) {
        for (int s = 0; s < S; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        *abort_flag = 0;
        if constexpr (G) gcache->loaded = 0xffffffffu;
        mbar_fence_init();
    }
    if constexpr (G) ugen_load_starts(ptrs, job.total_items, gstarts, tid, kUStagedThreads);
    __syncthreads();

    if (warp == kUConsumerWarps) {
        // ---------------------------------------------------------------- producer warp
        WorkCounter *wc = &g_unpack_work[job.work_slot];
        uint32_t it = 0;
        bool ok = true;
        uint32_t item = work_fetch_get(work_fetch_issue(wc, lane));
        for (; item < job.total_items; ++it) {
            const uint32_t next_issued = work_fetch_issue(wc, lane);   // asked for now, read after this item's copies are on their way
            const int s = it % S;
            const uint32_t ph = (it / S) & 1u;
            UItemMeta m;
            const uint8_t *src = nullptr;
            uint64_t band_start = 0, band_stride = 0;
            if constexpr (G) {
                // table look-up and address arithmetic first: they hide behind the wait for a free stage
                ugen_find_entry(ptrs, gstarts, item, gcache, lane);
                decode_uitem_gen(gcache, job, item, m);
                const GenEntry &e = gcache->e;
                if ((uint32_t)lane < m.ntiles) {
                    TileJob ej;
                    job_of_entry(job, e, ej);
                    src = e.q + tile_record_offset(ej, m.w, m.z, m.rt, m.ct0 + lane);
                }
                band_stride = e.stride_r;
                band_start = reinterpret_cast<uint64_t>(e.rm) + (uint64_t)m.w * e.stride_w + (uint64_t)m.z * e.stride_z +
                             (uint64_t)m.rt * 32u * e.stride_r + (uint64_t)m.ct0 * 32u * ES;
            }
            if (!mbar_wait_bounded(&empty[s], ph ^ 1u, abort_flag, status, BUDA_DEVSTAT_UNPACK_EMPTY_WAIT)) {
                ok = false;
                break;
            }
            if constexpr (G) {
                if (lane == 0) {
                    gband[2 * s] = band_start;
                    gband[2 * s + 1] = band_stride;
                }
            }
            if constexpr (!G) {
                decode_uitem(job, item, m);
                if ((uint32_t)lane < m.ntiles) src = ptrs.src[m.b] + tile_record_offset(job, m.w, m.z, m.rt, m.ct0 + lane);
            }
            if (lane == 0) {
                meta[s] = m;
                mbar_arrive_expect_tx(&full[s], m.ntiles * rec);
            }
            __syncwarp();
            if ((uint32_t)lane < m.ntiles) bulk_g2s(in_stage + s * Cfg::in_stage_bytes + lane * rec, src, rec, &full[s]);
            item = work_fetch_get(next_issued);
        }
        if (ok) {
            // no items left: an empty item in the next stage tells the consumer warps to leave
            const int s = it % S;
            if (mbar_wait_bounded(&empty[s], ((it / S) & 1u) ^ 1u, abort_flag, status, BUDA_DEVSTAT_UNPACK_EMPTY_WAIT)) {
                if (lane == 0) {
                    meta[s].ntiles = 0;
                    mbar_arrive(&full[s]);
                }
            } else {
                ok = false;
            }
        }
        if (lane == 0) work_leave(wc);
        if (!ok || *abort_flag) {
            const uint32_t back = it < (uint32_t)S ? it : (uint32_t)S;
            for (uint32_t k = 1; k <= back; k++) {
                const uint32_t j = it - k;
                uint64_t t0 = global_timer_ns();
                while (!mbar_try_wait(&full[j % S], (j / S) & 1u) && global_timer_ns() - t0 < 100000000ull) {}
            }
        }
        return;
    }

    // -------------------------------------------------------------------- consumer warps
    const int fr = lane & 15;
    uint32_t it = 0;
    for (;; ++it) {
        const int s = it % S;
        const uint32_t ph = (it / S) & 1u;
        const bool ok = mbar_wait_bounded(&full[s], ph, abort_flag, status, BUDA_DEVSTAT_UNPACK_FULL_WAIT);
        const UItemMeta m = meta[s];
        if (ok && m.ntiles == 0) break;   // the producer's end marker: the same for every consumer thread
        uint64_t g_start = 0, g_stride = 0;   // general flavour: read while the stage is still ours
        if constexpr (G) {
            if (ok) {
                g_start = gband[2 * s];
                g_stride = gband[2 * s + 1];
            }
        }
        uint8_t *ob = out_buf + (it % Cfg::out_bufs) * Cfg::out_buf_bytes;
        const uint8_t *stage = in_stage + s * Cfg::in_stage_bytes;

        if (!ok) {
            // fall through to the barrier below so the whole CTA leaves together
        } else if (M > 0) {
#pragma unroll
          for (int bc = warp; bc < 2 * Cfg::box; bc += kUConsumerWarps) {  // face column: tile bc/2, left/right face bc%2
            const int tile_in_box = bc >> 1;
            const int face = ((lane >> 4) << 1) | (bc & 1);
            if ((uint32_t)tile_in_box < m.ntiles) {
                constexpr int MM = M > 0 ? M : 7;
                const uint8_t *r = stage + tile_in_box * rec + hdr;
                const int blk = (P ? (int)job.pol.face_pos[face] : face) * 16 + fr;
                const uint32_t E = r[(P && job.pol.exp_be) ? (blk ^ 3) : blk];
                const uint8_t *q = r + 64 + blk * BfpTraits<MM>::bytes;
                uint32_t d[BfpTraits<MM>::words];
                if (MM == 7) {
                    uint4 t = *reinterpret_cast<const uint4 *>(q);
                    d[0] = t.x; d[1 % BfpTraits<MM>::words] = t.y; d[2 % BfpTraits<MM>::words] = t.z; d[3 % BfpTraits<MM>::words] = t.w;
                } else if (MM == 3) {
                    uint2 t = *reinterpret_cast<const uint2 *>(q);
                    d[0] = t.x; d[1 % BfpTraits<MM>::words] = t.y;
                } else {
                    d[0] = *reinterpret_cast<const uint32_t *>(q);
                }
                if (P && job.pol.datum_be) {
#pragma unroll
                    for (int w = 0; w < BfpTraits<MM>::words; w++) d[w] = reverse_datum_fields<MM>(d[w]);
                }
                uint8_t *p = ob + lane * Cfg::pitch + bc * 16 * ES;
                uint32_t h[8];
                if (ES == 2 && !AF && bfp_decode16_bf16<MM>(E, d, h)) {
                    // bfloat16 destination: decoded as packed pairs (false at the ends of the exponent range)
                    *reinterpret_cast<uint4 *>(p) = make_uint4(h[0], h[1], h[2], h[3]);
                    *reinterpret_cast<uint4 *>(p + 16) = make_uint4(h[4], h[5], h[6], h[7]);
                } else {
                    float v[16];
                    bfp_decode16<MM, AF>(E, d, v);
                    if (ES == 4) {
#pragma unroll
                        for (int j = 0; j < 4; j++)
                            *reinterpret_cast<float4 *>(p + 16 * j) = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                    } else {
                        // at most 7 significant bits: the upper half of the binary32 is the exact bfloat16
#pragma unroll
                        for (int j = 0; j < 8; j++)
                            h[j] = AF ? pack_half2(v[2 * j], v[2 * j + 1])
                                      : __byte_perm(__float_as_uint(v[2 * j]), __float_as_uint(v[2 * j + 1]), 0x7632);
                        *reinterpret_cast<uint4 *>(p) = make_uint4(h[0], h[1], h[2], h[3]);
                        *reinterpret_cast<uint4 *>(p + 16) = make_uint4(h[4], h[5], h[6], h[7]);
                    }
                }
            }
          }
        } else {
            constexpr int cpr = ES;
            constexpr int chunks_per_tile = 64 * cpr;
            const int nchunks = (int)m.ntiles * chunks_per_tile;
            for (int c = tid; c < nchunks; c += kUConsumerThreads) {
                const int t = c / chunks_per_tile, k = c % chunks_per_tile;
                const int r16 = (k / cpr) % 16, part = k % cpr;
                const int f = P ? (int)job.pol.face_at[k / (16 * cpr)] : k / (16 * cpr);   // the face stored at this position
                const int row = (f >> 1) * 16 + r16;
                const uint4 v = *reinterpret_cast<const uint4 *>(stage + t * rec + hdr + k * 16);
                *reinterpret_cast<uint4 *>(ob + row * Cfg::pitch + t * 32 * ES + (f & 1) * 16 * ES + part * 16) = v;
            }
        }
        // Every block of the band is decoded: the band leaves with plain coalesced stores, four rows per warp,
        // lanes along the row (one warp instruction = 512 contiguous bytes).  The next item decodes into the other
        // band buffer; this one is overwritten two items later, after the next item's barrier, by which time every
        // warp has finished copying it out.
        if (named_bar_or(1, kUConsumerThreads, !ok)) break;
        if (tid == 0) mbar_arrive(&empty[s]);
        {
            const int chunks = (int)m.ntiles * 2 * ES;   // 16-byte chunks per row piece
            uint8_t *dst0;
            uint64_t stride_r;
            if constexpr (G) {
                stride_r = g_stride;
                dst0 = reinterpret_cast<uint8_t *>(g_start);
            } else {
                stride_r = job.stride_r;
                dst0 = ptrs.dst[m.b] + (uint64_t)m.w * job.stride_w + rm_z_offset(job, m.z) +
                       (uint64_t)m.rt * 32u * stride_r + (uint64_t)m.ct0 * 32u * ES;
            }
#pragma unroll
            for (int rr = 0; rr < 32 / kUConsumerWarps; rr++) {
                const int row = warp * (32 / kUConsumerWarps) + rr;
                const uint8_t *src = ob + row * Cfg::pitch;
                uint8_t *dst = dst0 + (uint64_t)row * stride_r;
                for (int c = lane; c < chunks; c += 32)
                    __stcs(reinterpret_cast<uint4 *>(dst + c * 16), *reinterpret_cast<const uint4 *>(src + c * 16));
            }
        }
    }
}

// ------------------------------------------------------------------------------------------------
// direct kernel
// ------------------------------------------------------------------------------------------------
template <int M, int ES, bool AF, bool G>
__global__ void __launch_bounds__(256)
unpack_direct_kernel(const __grid_constant__ TileJob job, const __grid_constant__ PtrTable ptrs, int batch, int vec_ok)
{
    const int lane = threadIdx.x & 31;
    const uint64_t warps_total = (uint64_t)gridDim.x * (blockDim.x >> 5);
    const uint64_t warp_id = (uint64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const uint64_t tiles = (uint64_t)batch * job.W * job.Z * job.Rt * job.Ct;
    const uint32_t hdr = job.header_bytes;
    // A warp takes a whole tile per iteration: the tile's position is worked out once, and the record reads of all
    // eight 8-row pieces (4 faces x 2 halves) are issued before the first is decoded.
    for (uint64_t tt = warp_id; tt < tiles; tt += warps_total) {
        uint64_t t = tt;
        const uint32_t ct = (uint32_t)(t % job.Ct); t /= job.Ct;
        const uint32_t rt = (uint32_t)(t % job.Rt); t /= job.Rt;
        const uint32_t z = (uint32_t)(t % job.Z); t /= job.Z;
        const uint32_t w = (uint32_t)(t % job.W);
        const uint32_t b = (uint32_t)(t / job.W);
        uint8_t *tile_dst = ptrs.dst[b] + (uint64_t)w * job.stride_w + rm_z_offset(job, z) +
                            (uint64_t)rt * job.tile_h * job.stride_r + ((uint64_t)ct * 32u + (lane & 3) * 4u) * ES;
        const uint8_t *r = ptrs.src[b] + tile_record_offset(job, w, z, rt, ct) + hdr;
        constexpr int MM = (M > 0 && M < kLf8) ? M : 7;
        constexpr int kRaw = (M == 0 && ES == 4) ? 4 : (M == 0 && ES == 2) ? 2 : 1;
        uint32_t raw[8][kRaw];
        uint32_t ex[8];
#pragma unroll
        for (int hf = 0; hf < 8; hf++) {
            const uint32_t face = hf >> 1, half = hf & 1u;
            const uint32_t fr = half * 8u + (lane >> 2);
            const uint32_t tr = (face >> 1) * 16u + fr;            // row inside the tile
            const uint32_t blk = (G ? (uint32_t)job.pol.face_pos[face] : face) * 16u + fr;   // position in the record
            ex[hf] = 0;
#pragma unroll
            for (int i = 0; i < kRaw; i++) raw[hf][i] = 0;
            if (tr >= job.tile_h) continue;                       // tiny tiles: only tile_h rows of a record belong to the tensor
            if (M == kLf8) {
                raw[hf][0] = reinterpret_cast<const uint32_t *>(r + blk * 16u)[lane & 3];   // four 1-5-2 floats, no exponent section
            } else if (M > 0) {
                ex[hf] = r[(G && job.pol.exp_be) ? (blk ^ 3u) : blk];
                const uint8_t *q = r + 64 + blk * BfpTraits<MM>::bytes;
                int part = lane & 3;
                if (G && job.pol.datum_be) part ^= (MM == 3) ? 1 : (MM == 1) ? 3 : 0;   // reversed fields: see the pack kernel
                uint32_t pk;
                if (MM == 7) pk = reinterpret_cast<const uint32_t *>(q)[part];
                else if (MM == 3) pk = reinterpret_cast<const uint16_t *>(q)[part];
                else pk = q[part];
                if (G && job.pol.datum_be) {
                    if (MM == 7) pk = __byte_perm(pk, 0u, 0x0123);
                    else if (MM == 3) pk = ((pk & 0xfu) << 12) | ((pk & 0xf0u) << 4) | ((pk >> 4) & 0xf0u) | ((pk >> 12) & 0xfu);
                    else pk = ((pk & 3u) << 6) | ((pk & 0xcu) << 2) | ((pk >> 2) & 0xcu) | ((pk >> 6) & 3u);
                }
                raw[hf][0] = pk;
            } else {
                const uint8_t *q = r + ((uint64_t)blk * 16u + (lane & 3) * 4u) * ES;
                if (ES == 4) {
                    const uint4 v = *reinterpret_cast<const uint4 *>(q);
                    raw[hf][0] = v.x; raw[hf][kRaw > 1 ? 1 : 0] = v.y; raw[hf][kRaw > 2 ? 2 : 0] = v.z; raw[hf][kRaw > 3 ? 3 : 0] = v.w;
                } else if (ES == 2) {
                    const uint2 v = *reinterpret_cast<const uint2 *>(q);
                    raw[hf][0] = v.x; raw[hf][kRaw > 1 ? 1 : 0] = v.y;
                } else {
                    raw[hf][0] = *reinterpret_cast<const uint32_t *>(q);
                }
            }
        }
#pragma unroll
        for (int hf = 0; hf < 8; hf++) {
            const uint32_t face = hf >> 1, half = hf & 1u;
            const uint32_t tr = (face >> 1) * 16u + half * 8u + (lane >> 2);
            if (tr >= job.tile_h) continue;
            uint8_t *p = tile_dst + (uint64_t)tr * job.stride_r + (face & 1u) * 16u * ES;
            uint32_t x[4];
            if (M == kLf8) {
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const uint32_t c = (raw[hf][0] >> (8 * i)) & 0xffu;
                    // exact in every destination: binary16 holds the code as its upper byte, bfloat16 is the upper half of the binary32
                    x[i] = (ES == 2 && AF) ? (c << 8) : (ES == 2 ? lf8_decode_float_bits(c) >> 16 : lf8_decode_float_bits(c));
                }
            } else if (M > 0) {
                const uint32_t E = ex[hf];
                const uint32_t packed = raw[hf][0];
                float post = 1.0f;
                const float sc = AF ? bfp_a_block_scale<MM>(E & 31u) : bfp_block_scale<MM>(E, post);
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const uint32_t d = packed >> (i * (MM + 1));
                    const uint32_t qb = kMagicBits | (d & BfpTraits<MM>::qmax);
                    const uint32_t signbit = (d << (31 - MM)) & 0x80000000u;
                    float val;
                    if (MM == 1 && !AF) {
                        // the scale may need a second factor (2^128 is not a binary32): multiply twice, then sign and +0
                        float mag = __fmul_rn(__fmul_rn(__fadd_rn(__uint_as_float(qb), -12582912.0f), sc), post);
                        val = __fadd_rn(__uint_as_float(__float_as_uint(mag) | signbit), 0.0f);
                    } else {
                        // q * (+-scale) + (+0): the sign rides on the scale, and the +0 addend turns a zero magnitude with its
                        // sign bit set into +0.0; one multiply-add where a multiply, an OR and an add stood
                        val = __fmaf_rn(__fadd_rn(__uint_as_float(qb), -12582912.0f), __uint_as_float(__float_as_uint(sc) ^ signbit), 0.0f);
                    }
                    x[i] = __float_as_uint(val);
                    if (ES == 2) x[i] = AF ? (pack_half2(val, 0.0f) & 0xffffu) : (x[i] >> 16);
                }
            } else if (ES == 4) {
                x[0] = raw[hf][0]; x[1] = raw[hf][kRaw > 1 ? 1 : 0]; x[2] = raw[hf][kRaw > 2 ? 2 : 0]; x[3] = raw[hf][kRaw > 3 ? 3 : 0];
            } else if (ES == 2) {
                const uint32_t v0 = raw[hf][0], v1 = raw[hf][kRaw > 1 ? 1 : 0];
                x[0] = v0 & 0xffffu; x[1] = v0 >> 16; x[2] = v1 & 0xffffu; x[3] = v1 >> 16;
            } else {
                const uint32_t v = raw[hf][0];
                x[0] = v & 0xffu; x[1] = (v >> 8) & 0xffu; x[2] = (v >> 16) & 0xffu; x[3] = v >> 24;
            }
            if (ES == 4) {
                if (vec_ok) {
                    *reinterpret_cast<uint4 *>(p) = make_uint4(x[0], x[1], x[2], x[3]);
                } else if ((reinterpret_cast<uintptr_t>(p) & 3u) == 0) {
#pragma unroll
                    for (int i = 0; i < 4; i++) reinterpret_cast<uint32_t *>(p)[i] = x[i];
                } else {
#pragma unroll
                    for (int i = 0; i < 16; i++) p[i] = (uint8_t)(x[i >> 2] >> (8 * (i & 3)));
                }
            } else if (ES == 2) {
                if (vec_ok) {
                    *reinterpret_cast<uint2 *>(p) = make_uint2(x[0] | (x[1] << 16), x[2] | (x[3] << 16));
                } else if ((reinterpret_cast<uintptr_t>(p) & 1u) == 0) {
#pragma unroll
                    for (int i = 0; i < 4; i++) reinterpret_cast<uint16_t *>(p)[i] = (uint16_t)x[i];
                } else {
#pragma unroll
                    for (int i = 0; i < 8; i++) p[i] = (uint8_t)(x[i >> 1] >> (8 * (i & 1)));
                }
            } else {
#pragma unroll
                for (int i = 0; i < 4; i++) p[i] = (uint8_t)x[i];
            }
        }
    }
}

// ------------------------------------------------------------------------------------------------
// host launchers
// ------------------------------------------------------------------------------------------------
static DeviceWorkSlots g_unpack_slots[64];   // per device: which work counter the next staged launch takes

template <int M, int ES, bool AF, bool G, bool P = false>
static cudaError_t launch_ustaged(const TileJob &job, const typename UTableOf<G>::type &table, int sm_count, cudaStream_t stream,
                                  unsigned int *status)
{
    using Cfg = UnpackCfg<M, ES>;
    static std::atomic<int> per_sm_cache[64];   // 0 = not yet looked up on this device (concurrent first calls store the same value)
    int dev = 0;
    cudaGetDevice(&dev);
    dev &= 63;
    int per_sm = per_sm_cache[dev].load(std::memory_order_acquire);
    if (per_sm == 0) {
        cudaError_t e = cudaFuncSetAttribute(unpack_staged_kernel<M, ES, AF, G, P>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             Cfg::template smem_for<G>());
        if (e != cudaSuccess) return e;
        int n = 0;
        e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, unpack_staged_kernel<M, ES, AF, G, P>, kUStagedThreads,
                                                          Cfg::template smem_for<G>());
        if (e != cudaSuccess) return e;
        per_sm = n < 1 ? 1 : (n > 4 ? 4 : n);
        per_sm_cache[dev].store(per_sm, std::memory_order_release);
    }
    TileJob launch_job = job;
    typename UTableOf<G>::type launch_table = table;
    if constexpr (G) {
        if (!finalize_table(launch_table, launch_job, Cfg::box)) return cudaErrorInvalidValue;
    } else {
        if (!set_box_tiles(launch_job, Cfg::box)) return cudaErrorInvalidValue;   // more than 2^31 work items: split the batch
    }
    if (launch_job.total_items == 0) return cudaSuccess;
    uint32_t grid = (uint32_t)(sm_count * per_sm);
    if (grid > launch_job.total_items) grid = launch_job.total_items;
    bool tracked = false;
    const int slot = take_work_slot(g_unpack_slots[dev], stream, &tracked);
    if (slot < 0) return cudaErrorLaunchOutOfResources;   // the counters reserved for graph capture are used up
    launch_job.work_slot = (uint32_t)slot;
    // (A programmatic dependent launch -- the next conversion's CTAs becoming resident and running their prologue while
    // this one drains -- was measured on back-to-back launches of the 64-tensor batch: 6.5 % slower, not kept.)
    unpack_staged_kernel<M, ES, AF, G, P><<<grid, kUStagedThreads, Cfg::template smem_for<G>(), stream>>>(launch_job, launch_table, status);
    const cudaError_t e = cudaGetLastError();
    work_slot_launched(g_unpack_slots[dev], slot, stream, tracked);
    return e;
}

template <int M, int ES, bool AF, bool G>
static cudaError_t launch_udirect(const TileJob &job, const PtrTable &ptrs, int batch, int vec_ok, int sm_count,
                                  cudaStream_t stream)
{
    const uint64_t tiles = (uint64_t)batch * job.W * job.Z * job.Rt * job.Ct;   // one warp iteration each
    uint64_t blocks = (tiles + 7) / 8;
    const uint64_t cap = (uint64_t)sm_count * 32;
    if (blocks > cap) blocks = cap;
    unpack_direct_kernel<M, ES, AF, G><<<(unsigned)blocks, 256, 0, stream>>>(job, ptrs, batch, vec_ok);
    return cudaGetLastError();
}

#define BUDA_FOR_EACH_UNPACK_KIND(X) \
    X(7, 4, false) X(3, 4, false) X(1, 4, false) X(7, 2, false) X(3, 2, false) X(1, 2, false) \
    X(7, 4, true) X(3, 4, true) X(1, 4, true) X(7, 2, true) X(3, 2, true) X(1, 2, true)       \
    X(0, 4, false) X(0, 2, false) X(0, 1, false)
// conversions only the direct kernel performs (Lf8 to binary32, bfloat16 and binary16)
#define BUDA_FOR_EACH_DIRECT_ONLY_UNPACK_KIND(X) X(kLf8, 4, false) X(kLf8, 2, false) X(kLf8, 2, true)

// mant_bits 7/3/1 = Bfp decode, 0 = plain relayout; es = destination element bytes; a_format: 5-bit
// shared exponent (destination binary16 when es == 2).  Plain flavour.
cudaError_t launch_untilize(const TileJob &job, const PtrTable &ptrs, int batch, int mant_bits, int es, int a_format, int path,
                            int vec_ok, int sm_count, cudaStream_t stream, unsigned int *status)
{
#define BUDA_DISPATCH(MM, EE, AA)                                                                          \
    if (mant_bits == MM && es == EE && (a_format != 0) == AA)                                              \
        return path == 0 ? launch_ustaged<MM, EE, AA, false>(job, ptrs, sm_count, stream, status)          \
                         : launch_udirect<MM, EE, AA, false>(job, ptrs, batch, vec_ok, sm_count, stream);
    BUDA_FOR_EACH_UNPACK_KIND(BUDA_DISPATCH)
#undef BUDA_DISPATCH
#define BUDA_DISPATCH(MM, EE, AA) \
    if (mant_bits == MM && es == EE && (a_format != 0) == AA && path != 0) \
        return launch_udirect<MM, EE, AA, false>(job, ptrs, batch, vec_ok, sm_count, stream);
    BUDA_FOR_EACH_DIRECT_ONLY_UNPACK_KIND(BUDA_DISPATCH)
#undef BUDA_DISPATCH
    return cudaErrorInvalidValue;
}

// General flavour, staged kernel: one table entry per tensor.
cudaError_t launch_untilize_table(const TileJob &job, const GenTable &table, int mant_bits, int es, int a_format, int sm_count,
                                  cudaStream_t stream, unsigned int *status)
{
#define BUDA_DISPATCH(MM, EE, AA) \
    if (mant_bits == MM && es == EE && (a_format != 0) == AA)                                                            \
        return policy_is_default(job.pol) ? launch_ustaged<MM, EE, AA, true, false>(job, table, sm_count, stream, status) \
                                          : launch_ustaged<MM, EE, AA, true, true>(job, table, sm_count, stream, status);
    BUDA_FOR_EACH_UNPACK_KIND(BUDA_DISPATCH)
#undef BUDA_DISPATCH
    return cudaErrorInvalidValue;
}

// General flavour, direct kernel: a batch of one shape under job.pol.
cudaError_t launch_untilize_direct_policy(const TileJob &job, const PtrTable &ptrs, int batch, int mant_bits, int es, int a_format,
                                          int vec_ok, int sm_count, cudaStream_t stream)
{
#define BUDA_DISPATCH(MM, EE, AA) \
    if (mant_bits == MM && es == EE && (a_format != 0) == AA) return launch_udirect<MM, EE, AA, true>(job, ptrs, batch, vec_ok, sm_count, stream);
    BUDA_FOR_EACH_UNPACK_KIND(BUDA_DISPATCH)
    BUDA_FOR_EACH_DIRECT_ONLY_UNPACK_KIND(BUDA_DISPATCH)
#undef BUDA_DISPATCH
    return cudaErrorInvalidValue;
}

}  // namespace buda
