// K1 / K3: row-major tensor -> queue image of 32x32 tiles (four 16x16 faces), fused with the
// Bfp8_b / Bfp4_b / Bfp2_b block-float pack (or a plain relayout for same-width formats).
//
// Device counterpart of the conversion the reference performs inside tt::backend::tilize_tensor
// and push_input (bound at pybuda/csrc/backend_api/backend_api.cpp:688-704).
//
// Two kernels:
//   pack_staged_kernel  (16-byte aligned rows; the hot path)
//     A persistent CTA per SM slot walks work items; an item is a band of 32 rows x up to 8 tiles
//     (256 columns).  One producer warp stages the band in shared memory with 32 bulk async
//     copies (one per row, TMA engine, completion on an mbarrier) one item ahead; eight
//     consumer warps then each own 16-column face columns of the band: lane = row, so a thread
//     reads one whole 16-value block (one face row) from shared memory, encodes it in registers
//     and drops its 16/8/4 mantissa bytes plus the exponent byte into the tile record being
//     assembled in shared memory.  Finished records leave with one bulk async store per tile.
//     Row pitch in shared memory is row bytes + 16, which makes the 16-byte reads of the 32 lanes
//     (32 different rows) conflict free.
//   pack_direct_kernel  (any alignment / stride; the general path)
//     Four lanes own one block: each loads 4 values (one 128-bit load when aligned), the shared
//     exponent is a 4-lane-wide warp-shuffle maximum, and a warp covers 8 consecutive rows of one
//     face so its stores form one contiguous run of the record.
// Each kernel exists in two flavours (template flag G).  The plain one serves a batch of tensors of one shape with the
// default byte layout.  The general one takes a table with one entry per tensor (own shape, strides, queue geometry,
// selection of tile rows) and honours a layout policy (rounding, overflow, face / exponent / datum order).
#include "bfp_codec.cuh"
#include <atomic>

#include "buda_common.cuh"
#include "work_slots_cuda.cuh"

namespace buda {

// ------------------------------------------------------------------------------------------------
// staged kernel
// ------------------------------------------------------------------------------------------------
constexpr int kConsumerWarps = 8;
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kStagedThreads = kConsumerThreads + 32;  // + one producer warp

struct ItemMeta {
    uint32_t b, w, z, rt, ct0, ntiles, pad0, pad1;
};

template <int M, int ES>
struct PackCfg {
    static constexpr int box = pack_box_tiles_for(ES, M);
    static constexpr int row_bytes = box * 32 * ES;
    static constexpr int pitch = row_bytes + 16;
    static constexpr int in_stage_bytes = 32 * pitch;
    static constexpr int payload = (M > 0) ? (64 + 1024 * (M + 1) / 8) : (1024 * ES);
    static constexpr int rec_max = payload + 32;
    static constexpr int out_buf_bytes = box * rec_max;
    static constexpr int stages = 2;  // depth comes from the CTAs resident per SM, not from stages per CTA
    static constexpr int smem_bytes = stages * in_stage_bytes + 2 * out_buf_bytes + stages * (int)sizeof(ItemMeta) +
                                      2 * stages * 8 + 16;
    // general flavour: a copy of the table entry in use, the first work item of every entry, and per stage the
    // destination of each tile of the item (worked out by the producer, which holds the entry)
    static constexpr int gen_extra_bytes = 136 + (kMaxGen + 1) * 4 + 4 + stages * 16 * 8;
    template <bool G>
    static constexpr int smem_for() { return smem_bytes + (G ? gen_extra_bytes : 0); }
};

__device__ __forceinline__ void decode_item(const TileJob &job, uint32_t item, ItemMeta &m)
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

// General flavour.  Kernel parameters are slow to read with a run-time index, so the table is touched as little as
// possible: every entry's first work item is copied to shared memory once per CTA, the entry a work item belongs to is
// found there by bisection, and the entry itself is copied to shared memory when the producer moves on to it.
struct GenCache {
    GenEntry e;                       // 128 bytes
    uint32_t loaded, pad;             // index of the entry held in e
};
static_assert(sizeof(GenCache) == 136, "shared-memory plan of the general flavour");

__device__ __forceinline__ void gen_load_starts(const GenTable &tab, uint32_t total_items, uint32_t *starts, int tid, int nthreads)
{
    for (uint32_t i = (uint32_t)tid; i <= tab.n; i += (uint32_t)nthreads) starts[i] = i < tab.n ? tab.e[i].item_start : total_items;
}

// whole producer warp; returns with *cache holding the entry of `item`
__device__ __forceinline__ void gen_find_entry(const GenTable &tab, const uint32_t *starts, uint32_t item, GenCache *cache, int lane)
{
    uint32_t idx = cache->loaded;
    if (idx >= tab.n || item < starts[idx] || item >= starts[idx + 1u]) {
        uint32_t lo = 0, hi = tab.n;          // largest idx with starts[idx] <= item
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

__device__ __forceinline__ void decode_item_gen(const GenCache *cache, const TileJob &common, uint32_t item, ItemMeta &m)
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

static __device__ WorkCounter g_pack_work[kWorkSlots];

template <bool G> struct TableOf { using type = PtrTable; };
template <> struct TableOf<true> { using type = GenTable; };

// The general flavour is held to the register budget of the plain one (five CTAs of 288 threads per SM for the 8-bit
// formats): what it spills sits on the policy-only paths.
// P: the launch honours a non-default layout policy (general flavour only).  A job table under the default policy -- the
// usual case: parameter sets, layers of a model -- runs the plain flavour's consumer code.
template <int M, int ES, bool AF, bool G, bool P>
__global__ void __launch_bounds__(kStagedThreads, (G && M == 7 && ES == 4) ? 5 : 0)
pack_staged_kernel(const __grid_constant__ TileJob job, const __grid_constant__ typename TableOf<G>::type ptrs, unsigned int *status)
{
    using Cfg = PackCfg<M, ES>;
    constexpr int S = Cfg::stages;
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t *in_stage = smem;
    uint8_t *out_buf = smem + S * Cfg::in_stage_bytes;
    ItemMeta *meta = reinterpret_cast<ItemMeta *>(out_buf + 2 * Cfg::out_buf_bytes);
    uint64_t *full = reinterpret_cast<uint64_t *>(meta + S);
    uint64_t *empty = full + S;
    volatile int *abort_flag = reinterpret_cast<volatile int *>(empty + S);
    // general flavour only (see PackCfg::gen_extra_bytes)
    GenCache *gcache = reinterpret_cast<GenCache *>(reinterpret_cast<uint8_t *>(empty + S) + 16);
    uint32_t *gstarts = reinterpret_cast<uint32_t *>(gcache + 1);
    uint64_t *gdst = reinterpret_cast<uint64_t *>(gstarts + kMaxGen + 2);

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
    if constexpr (G) gen_load_starts(ptrs, job.total_items, gstarts, tid, kStagedThreads);
    // header bytes of the staged records are written once: they stay zero for every item
    for (int i = tid; i < 2 * Cfg::out_buf_bytes / 4; i += kStagedThreads) reinterpret_cast<uint32_t *>(out_buf)[i] = 0;
    fence_async_smem();
    __syncthreads();

    if (warp == kConsumerWarps) {
        // ---------------------------------------------------------------- producer warp
        WorkCounter *wc = &g_pack_work[job.work_slot];
        uint32_t it = 0;
        bool ok = true;
        uint32_t item = work_fetch_get(work_fetch_issue(wc, lane));
        for (; item < job.total_items; ++it) {
            const uint32_t next_issued = work_fetch_issue(wc, lane);   // asked for now, read after this item's copies are on their way
            const int s = it % S;
            const uint32_t ph = (it / S) & 1u;
            ItemMeta m;
            const uint8_t *src;
            uint8_t *tile_dst = nullptr;
            if constexpr (G) {
                // table look-up and index arithmetic first: they hide behind the wait for a free stage
                gen_find_entry(ptrs, gstarts, item, gcache, lane);
                decode_item_gen(gcache, job, item, m);
                const GenEntry &e = gcache->e;
                src = e.rm + (uint64_t)m.w * e.stride_w + (uint64_t)m.z * e.stride_z + ((uint64_t)m.rt * 32u + lane) * e.stride_r +
                      (uint64_t)m.ct0 * 32u * ES;
                if ((uint32_t)lane < m.ntiles) {
                    TileJob ej;
                    job_of_entry(job, e, ej);
                    tile_dst = e.q + tile_record_offset(ej, m.w, m.z, m.rt, m.ct0 + lane);
                }
            }
            if (!mbar_wait_bounded(&empty[s], ph ^ 1u, abort_flag, status, BUDA_DEVSTAT_PACK_EMPTY_WAIT)) {
                ok = false;
                break;
            }
            if constexpr (G) {
                if ((uint32_t)lane < m.ntiles) gdst[s * 16 + lane] = reinterpret_cast<uint64_t>(tile_dst);
            }
            if constexpr (!G) {
                decode_item(job, item, m);
                src = ptrs.src[m.b] + (uint64_t)m.w * job.stride_w + rm_z_offset(job, m.z) +
                      ((uint64_t)m.rt * 32u + lane) * job.stride_r + (uint64_t)m.ct0 * 32u * ES;
            }
            const uint32_t row_copy = m.ntiles * 32u * ES;
            if (lane == 0) {
                meta[s] = m;
                mbar_arrive_expect_tx(&full[s], 32u * row_copy);
            }
            __syncwarp();
            bulk_g2s(in_stage + s * Cfg::in_stage_bytes + lane * Cfg::pitch, src, row_copy, &full[s]);
            item = work_fetch_get(next_issued);
        }
        if (ok) {
            // no items left: an empty item in the next stage tells the consumer warps to leave
            const int s = it % S;
            if (mbar_wait_bounded(&empty[s], ((it / S) & 1u) ^ 1u, abort_flag, status, BUDA_DEVSTAT_PACK_EMPTY_WAIT)) {
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
            // gave up: let the copies already issued land before the CTA releases its shared memory
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
    // A thread always meets the same face: the face column bc advances by the (even) number of consumer warps, so
    // bc % 2 stays warp % 2.  Its block's place in the record is therefore fixed for the whole launch.
    const int my_face = ((lane >> 4) << 1) | (warp & 1);
    const int blk = (P ? (int)job.pol.face_pos[my_face] : my_face) * 16 + fr;
    const int exp_idx = (P && job.pol.exp_be) ? (blk ^ 3) : blk;
    // general flavour (all uniform over the launch): only a raised exponent needs the policy encoder; truncation is the
    // plain encoder with another rounding mode, a reversed datum order one permute per word afterwards
    const bool plain_codec = !P || !job.pol.bump;
    const int rmode = P ? (int)job.pol.rmode : 0;
    const bool datum_be = P && job.pol.datum_be;
    uint32_t it = 0;
    for (;; ++it) {
        const int s = it % S;
        const uint32_t ph = (it / S) & 1u;
        const bool ok = mbar_wait_bounded(&full[s], ph, abort_flag, status, BUDA_DEVSTAT_PACK_FULL_WAIT);
        const ItemMeta m = meta[s];
        if (ok && m.ntiles == 0) break;   // the producer's end marker: the same for every consumer thread
        uint64_t my_dst = 0;              // general flavour: where this lane's tile record goes (read while the stage is still ours)
        if constexpr (G) {
            if (ok && warp == 0 && (uint32_t)lane < m.ntiles) my_dst = gdst[s * 16 + lane];
        }
        uint8_t *ob = out_buf + (it & 1u) * Cfg::out_buf_bytes;
        const uint8_t *stage = in_stage + s * Cfg::in_stage_bytes;

        if (!ok) {
            // fall through to the barrier below so the whole CTA leaves together
        } else if (M > 0) {
#pragma unroll
          for (int bc = warp; bc < 2 * Cfg::box; bc += kConsumerWarps) {  // face column: tile bc/2, left/right face bc%2
            const int tile_in_box = bc >> 1;
            if ((uint32_t)tile_in_box < m.ntiles) {
                uint32_t x[16];
                const uint8_t *p = stage + lane * Cfg::pitch + bc * 16 * ES;
                constexpr int MM = M > 0 ? M : 7;
                uint32_t E, d[BfpTraits<MM>::words];
                bool encoded = false;
                if (ES == 4) {
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        uint4 v = *reinterpret_cast<const uint4 *>(p + 16 * j);
                        x[4 * j] = v.x; x[4 * j + 1] = v.y; x[4 * j + 2] = v.z; x[4 * j + 3] = v.w;
                    }
                } else {
                    const uint4 v0 = *reinterpret_cast<const uint4 *>(p), v1 = *reinterpret_cast<const uint4 *>(p + 16);
                    const uint32_t h[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
                    // packed-pair encoder; false at the ends of the exponent range
                    if (!AF && plain_codec && rmode == 0) encoded = bfp_encode16_bf16<MM>(h, E, d);
                    if (!encoded) {
#pragma unroll
                        for (int k = 0; k < 8; k++) {
                            if (AF) {  // binary16 source of the "a" formats
                                x[2 * k] = half_bits_to_float_bits(h[k] & 0xffffu);
                                x[2 * k + 1] = half_bits_to_float_bits(h[k] >> 16);
                            } else {   // bfloat16 widens exactly: it is the upper half
                                x[2 * k] = h[k] << 16;
                                x[2 * k + 1] = h[k] & 0xffff0000u;
                            }
                        }
                    }
                }
                if (!encoded) {
                    if (!plain_codec) bfp_encode16_policy<MM>(x, E, d, job.pol, AF ? 143u : 255u);
                    else if (rmode == 1) bfp_encode16<MM, 1>(x, E, d);
                    else if (rmode == 2) bfp_encode16<MM, 2>(x, E, d);
                    else bfp_encode16<MM, 0>(x, E, d);
                }
                if (plain_codec && datum_be) {
#pragma unroll
                    for (int w = 0; w < BfpTraits<MM>::words; w++) d[w] = reverse_datum_fields<MM>(d[w]);
                }
                uint8_t *r = ob + tile_in_box * rec + hdr;
                r[exp_idx] = (uint8_t)(AF ? a_exponent_byte(E) : E);
                uint8_t *q = r + 64 + blk * BfpTraits<MM>::bytes;
                if (MM == 7) *reinterpret_cast<uint4 *>(q) = make_uint4(d[0], d[1 % BfpTraits<MM>::words], d[2 % BfpTraits<MM>::words], d[3 % BfpTraits<MM>::words]);
                else if (MM == 3) *reinterpret_cast<uint2 *>(q) = make_uint2(d[0], d[1 % BfpTraits<MM>::words]);
                else *reinterpret_cast<uint32_t *>(q) = d[0];
            }
          }
        } else {
            // plain relayout: the record is moved as 16-byte chunks; chunk c of a record is face
            // c / (16*cpr), face row (c / cpr) % 16, part c % cpr  (cpr = chunks per 16-value face row)
            constexpr int cpr = ES;                   // 16 * ES / 16
            constexpr int chunks_per_tile = 64 * cpr; // 1024 * ES / 16
            const int nchunks = (int)m.ntiles * chunks_per_tile;
            for (int c = tid; c < nchunks; c += kConsumerThreads) {
                const int t = c / chunks_per_tile, k = c % chunks_per_tile;
                const int r16 = (k / cpr) % 16, part = k % cpr;
                const int f = P ? (int)job.pol.face_at[k / (16 * cpr)] : k / (16 * cpr);   // the face stored at this position
                const int row = (f >> 1) * 16 + r16;
                const uint4 v = *reinterpret_cast<const uint4 *>(stage + row * Cfg::pitch + t * 32 * ES +
                                                                 (f & 1) * 16 * ES + part * 16);
                *reinterpret_cast<uint4 *>(ob + t * rec + hdr + k * 16) = v;
            }
        }
        fence_async_smem();
        if (warp == 0 && lane < Cfg::box) bulk_wait_read_all();  // the previous item's stores have left shared memory
        if (named_bar_or(1, kConsumerThreads, !ok)) break;
        if (tid == 0) mbar_arrive(&empty[s]);
        if (warp == 0 && (uint32_t)lane < m.ntiles) {
            uint8_t *dst;
            if constexpr (G) dst = reinterpret_cast<uint8_t *>(my_dst);
            else dst = ptrs.dst[m.b] + tile_record_offset(job, m.w, m.z, m.rt, m.ct0 + lane);
            bulk_s2g(dst, ob + lane * rec, rec);
            bulk_commit();
        }
    }
    if (warp == 0 && lane < Cfg::box) bulk_wait_all();
}

// ------------------------------------------------------------------------------------------------
// direct kernel: 4 lanes per block, warp-shuffle exponent reduction, any alignment
// ------------------------------------------------------------------------------------------------
// Bits of max(|a|, |b|, |c|, |d|) as floats; a NaN operand gives 0x7fffffff, so the exponent field is 255 for
// NaN and Inf alike, as with an integer maximum of the magnitudes.  The absolute values fold into the
// min/max instructions.
__device__ __forceinline__ uint32_t absmax4_bits(const uint32_t (&x)[4])
{
    float m;
    asm("{\n\t.reg .f32 a0, a1, a2, a3, m0;\n\t"
        "abs.f32 a0, %1;\n\tabs.f32 a1, %2;\n\tabs.f32 a2, %3;\n\tabs.f32 a3, %4;\n\t"
        "max.NaN.f32 m0, a0, a1, a2;\n\t"
        "max.NaN.f32 %0, m0, a3;\n\t}"
        : "=f"(m)
        : "f"(__uint_as_float(x[0])), "f"(__uint_as_float(x[1])), "f"(__uint_as_float(x[2])), "f"(__uint_as_float(x[3])));
    return __float_as_uint(m);
}

// The exponents next to 0 and 255, where the scale of the fast path is not a normal float: integer arithmetic,
// kept out of line because almost no block takes it.
__device__ __noinline__ uint32_t encode4_any_exp(uint32_t x0, uint32_t x1, uint32_t x2, uint32_t x3, uint32_t E, int m,
                                                 int rmode = 0, bool *over = nullptr)
{
    return bfp_encode_datum_int(x0, E, m, rmode, over) | (bfp_encode_datum_int(x1, E, m, rmode, over) << (m + 1)) |
           (bfp_encode_datum_int(x2, E, m, rmode, over) << (2 * (m + 1))) | (bfp_encode_datum_int(x3, E, m, rmode, over) << (3 * (m + 1)));
}

// Four data of one block, shared exponent E already known, packed at (M + 1) bits each.  In the usual exponent
// range the magnitudes come out of one fused multiply-add each (round to nearest even into the low bits of
// 1.5 * 2^23) and everything after it works on the four data at once, one byte each: saturation is per element,
// then the sign bits are gathered with byte permutes and dropped where the magnitude is zero.
// rmode / over: general flavour only (another rounding of the dropped bits; *over reports a finite magnitude above the largest).
template <int M>
__device__ __forceinline__ uint32_t encode4_shared_exp(const uint32_t (&x)[4], uint32_t E, int rmode = 0, bool *over = nullptr)
{
    constexpr uint32_t qmax = BfpTraits<M>::qmax;
    const bool fast = (E + 1u >= (uint32_t)M) && (E <= (uint32_t)(M + 252));
    if (fast) {
        const float S = __uint_as_float((uint32_t)(M + 253 - (int)E) << 23);
        uint32_t r[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const uint32_t y = rmode == 1 ? bfp_quantise_bits<1>(x[i], S) : rmode == 2 ? bfp_quantise_bits<2>(x[i], S) : bfp_quantise_bits<0>(x[i], S);
            if (over && y > kMagicBits + qmax) *over = true;
            r[i] = min(y, kMagicBits + qmax);   // low byte = magnitude (the constant's low byte is 0)
        }
        const uint32_t Q = __byte_perm(__byte_perm(r[0], r[1], 0x0040), __byte_perm(r[2], r[3], 0x0040), 0x5410);
        const uint32_t SG = __byte_perm(__byte_perm(x[0], x[1], 0x0073), __byte_perm(x[2], x[3], 0x0073), 0x5410);
        constexpr uint32_t kSignBit = 0x01010101u << M;
        const uint32_t nz = Q + qmax * 0x01010101u;              // bit M of a byte is set where its magnitude is not 0
        const uint32_t D = Q | ((SG >> (7 - M)) & nz & kSignBit);
        if (M == 7) return D;
        if (M == 3) {
            const uint32_t t = D | (D >> 4);
            return (t & 0xffu) | ((t >> 8) & 0xff00u);
        }
        const uint32_t t = D | (D >> 6);
        return (t | (t >> 12)) & 0xffu;
    }
    return encode4_any_exp(x[0], x[1], x[2], x[3], E, M, rmode, over);
}

template <int ES>
__device__ __forceinline__ void load4(const uint8_t *p, bool vec, uint32_t (&x)[4])
{
    if (ES == 4) {
        if (vec) {
            uint4 v = *reinterpret_cast<const uint4 *>(p);
            x[0] = v.x; x[1] = v.y; x[2] = v.z; x[3] = v.w;
        } else if ((reinterpret_cast<uintptr_t>(p) & 3u) == 0) {
#pragma unroll
            for (int i = 0; i < 4; i++) x[i] = *reinterpret_cast<const uint32_t *>(p + 4 * i);
        } else {
#pragma unroll
            for (int i = 0; i < 4; i++)
                x[i] = (uint32_t)p[4 * i] | ((uint32_t)p[4 * i + 1] << 8) | ((uint32_t)p[4 * i + 2] << 16) |
                       ((uint32_t)p[4 * i + 3] << 24);
        }
    } else if (ES == 2) {
        if (vec) {
            uint2 v = *reinterpret_cast<const uint2 *>(p);
            x[0] = v.x & 0xffffu; x[1] = v.x >> 16; x[2] = v.y & 0xffffu; x[3] = v.y >> 16;
        } else if ((reinterpret_cast<uintptr_t>(p) & 1u) == 0) {
#pragma unroll
            for (int i = 0; i < 4; i++) x[i] = *reinterpret_cast<const uint16_t *>(p + 2 * i);
        } else {
#pragma unroll
            for (int i = 0; i < 4; i++) x[i] = (uint32_t)p[2 * i] | ((uint32_t)p[2 * i + 1] << 8);
        }
    } else {
#pragma unroll
        for (int i = 0; i < 4; i++) x[i] = p[i];
    }
}

// One element of the row-major side under a source view (see SourceView); r, c are coordinates in the tile-aligned
// shape the queue covers.  base is the tensor's first byte.
template <int ES>
__device__ __forceinline__ uint32_t fetch_view_elem(const TileJob &j, const uint8_t *base, uint32_t w, uint32_t z, uint32_t r, uint32_t c)
{
    const SourceView &v = j.view;
    const uint8_t *p;
    if (v.mode == kSrcPadded) {
        if (v.bcast_r) r = 0;
        if (v.bcast_c) c = 0;
        if (r >= v.valid_r || c >= v.valid_c) return 0u;
        p = base + (uint64_t)w * j.stride_w + rm_z_offset(j, z) + (uint64_t)r * j.stride_r + (uint64_t)c * ES;
    } else if (v.mode == kSrcEmbedding) {
        const uint64_t a = (uint64_t)(c >> 5) * 32u + (r & 31u);
        if (a * 32u >= v.emb_group) return 0u;
        const uint64_t flat = (uint64_t)(r >> 5) * v.emb_group + a * 32u + (c & 31u);
        if (flat >= v.emb_count) return ES == 4 ? 0xffffffffu : ES == 2 ? 0xffffu : 0xffu;
        p = base + (uint64_t)w * j.stride_w + flat * ES;
    } else {
        if (r >= v.ps_noff * v.ps_z || c >= v.ps_hs * v.ps_ws) return 0u;
        const uint32_t k = r / v.ps_z, zc = r - k * v.ps_z;
        const uint32_t hr = c / v.ps_ws, wc = c - hr * v.ps_ws;
        const uint32_t y = hr * v.ps_stride + (uint32_t)v.ps_y[k], x = wc * v.ps_stride + (uint32_t)v.ps_x[k];
        if (y >= v.ps_h || x >= v.ps_w) return 0u;
        p = base + (uint64_t)w * j.stride_w + (uint64_t)zc * j.stride_z + (uint64_t)y * j.stride_r + (uint64_t)x * ES;
    }
    if (ES == 4) {
        if ((reinterpret_cast<uintptr_t>(p) & 3u) == 0) return *reinterpret_cast<const uint32_t *>(p);
        return (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24);
    }
    if (ES == 2) {
        if ((reinterpret_cast<uintptr_t>(p) & 1u) == 0) return *reinterpret_cast<const uint16_t *>(p);
        return (uint32_t)p[0] | ((uint32_t)p[1] << 8);
    }
    return p[0];
}

// Encode (or relayout) the four elements a lane holds of block `blk` and store them into tile record `r`.
// blk is the block's position in the record (face position * 16 + face row).
template <int M, int ES, bool AF, bool G>
__device__ __forceinline__ void direct_encode_store(uint32_t (&x)[4], uint32_t blk, uint8_t *r, int lane, const BfpPolicy &pol)
{
    if constexpr (M == kLf8) {
        // element-wise 1-5-2 float: no exponent section, one byte per element; AF marks a binary16 source
        uint32_t packed;
        if (ES == 2 && AF) {
            packed = lf8_encode_half_bits(x[0]) | (lf8_encode_half_bits(x[1]) << 8) | (lf8_encode_half_bits(x[2]) << 16) |
                     (lf8_encode_half_bits(x[3]) << 24);
        } else {
            if (ES == 2) {
#pragma unroll
                for (int i = 0; i < 4; i++) x[i] <<= 16;   // bfloat16 widens exactly
            }
            packed = lf8_encode_float_bits_x2(x[0], x[1]) | (lf8_encode_float_bits_x2(x[2], x[3]) << 16);
        }
        reinterpret_cast<uint32_t *>(r + blk * 16u)[lane & 3] = packed;
    } else if (M > 0) {
        constexpr int MM = (M > 0 && M < kLf8) ? M : 7;
        if (ES == 2) {
#pragma unroll
            for (int i = 0; i < 4; i++) x[i] = AF ? half_bits_to_float_bits(x[i]) : (x[i] << 16);
        }
        uint32_t mx = absmax4_bits(x);
        mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, 1, 4));
        mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, 2, 4));
        uint32_t E = mx >> 23;
        uint32_t packed;
        if constexpr (G) {
            bool over = false;
            packed = encode4_shared_exp<MM>(x, E, (int)pol.rmode, &over);
            // the block spans four lanes: any of them rounding up raises the exponent for all
            uint32_t ov = over ? 1u : 0u;
            ov |= __shfl_xor_sync(0xffffffffu, ov, 1, 4);
            ov |= __shfl_xor_sync(0xffffffffu, ov, 2, 4);
            if (pol.bump && ov && E < (AF ? 143u : 255u)) {
                E += 1u;
                packed = encode4_any_exp(x[0], x[1], x[2], x[3], E, MM, (int)pol.rmode);
            }
        } else {
            packed = encode4_shared_exp<MM>(x, E);
        }
        int part = lane & 3;
        if (G && pol.datum_be) {
            // the lane's four datums in reverse order; which quarter of which word they land in is reversed as well
            if (MM == 7) packed = __byte_perm(packed, 0u, 0x0123);
            else if (MM == 3) packed = ((packed & 0xfu) << 12) | ((packed & 0xf0u) << 4) | ((packed >> 4) & 0xf0u) | ((packed >> 12) & 0xfu);
            else packed = ((packed & 3u) << 6) | ((packed & 0xcu) << 2) | ((packed >> 2) & 0xcu) | ((packed >> 6) & 3u);
            if (MM == 3) part ^= 1;        // two lanes share a 32-bit word
            else if (MM == 1) part ^= 3;   // four lanes share a 32-bit word
        }
        if ((lane & 3) == 0) r[(G && pol.exp_be) ? (blk ^ 3u) : blk] = (uint8_t)(AF ? a_exponent_byte(E) : E);
        uint8_t *q = r + 64 + blk * BfpTraits<MM>::bytes;
        if (MM == 7) reinterpret_cast<uint32_t *>(q)[part] = packed;
        else if (MM == 3) reinterpret_cast<uint16_t *>(q)[part] = (uint16_t)packed;
        else q[part] = (uint8_t)packed;
    } else {
        uint8_t *q = r + ((uint64_t)blk * 16u + (lane & 3) * 4u) * ES;
        if (ES == 4) *reinterpret_cast<uint4 *>(q) = make_uint4(x[0], x[1], x[2], x[3]);
        else if (ES == 2) *reinterpret_cast<uint2 *>(q) = make_uint2(x[0] | (x[1] << 16), x[2] | (x[3] << 16));
        else *reinterpret_cast<uint32_t *>(q) = x[0] | (x[1] << 8) | (x[2] << 16) | (x[3] << 24);
    }
}

template <int M, int ES, bool AF, bool G>
__global__ void __launch_bounds__(256)
pack_direct_kernel(const __grid_constant__ TileJob job, const __grid_constant__ PtrTable ptrs, int batch, int vec_ok)
{
    const int lane = threadIdx.x & 31;
    const uint64_t warps_total = (uint64_t)gridDim.x * (blockDim.x >> 5);
    const uint64_t warp_id = (uint64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const uint64_t tiles = (uint64_t)batch * job.W * job.Z * job.Rt * job.Ct;
    const uint32_t hdr = job.header_bytes;
    constexpr int GR = 8;   // pieces whose loads are issued before the first is encoded
    // A warp takes a whole tile per iteration: the tile's position is worked out once (the divisions by the run-time
    // tensor dims were most of the instructions when a warp took an eighth of a tile).  A tile is eight pieces of
    // 8 rows of one face (piece = face * 2 + half); with rows that allow vector loads, the loads of G pieces are
    // issued before the first is encoded.  The element-wise loads of unaligned rows stay a rolled loop: unrolled,
    // their code no longer fits the instruction cache.
    for (uint64_t tt = warp_id; tt < tiles; tt += warps_total) {
        uint64_t t = tt;
        const uint32_t ct = (uint32_t)(t % job.Ct); t /= job.Ct;
        const uint32_t rt = (uint32_t)(t % job.Rt); t /= job.Rt;
        const uint32_t z = (uint32_t)(t % job.Z); t /= job.Z;
        const uint32_t w = (uint32_t)(t % job.W);
        const uint32_t b = (uint32_t)(t / job.W);
        const uint8_t *tile_src = ptrs.src[b] + (uint64_t)w * job.stride_w + rm_z_offset(job, z) +
                                  (uint64_t)rt * job.tile_h * job.stride_r + ((uint64_t)ct * 32u + (lane & 3) * 4u) * ES;
        uint8_t *r = ptrs.dst[b] + tile_record_offset(job, w, z, rt, ct);
        if (hdr && lane < 8) reinterpret_cast<uint32_t *>(r)[lane] = 0;
        r += hdr;
        if (G && job.view.mode != kSrcDense) {
            // the source is read through a view: element by element, each with its own address or fill value
#pragma unroll 1
            for (uint32_t hf = 0; hf < 8; hf++) {
                const uint32_t face = hf >> 1, half = hf & 1u;
                const uint32_t tr = (face >> 1) * 16u + half * 8u + (lane >> 2);
                const uint32_t c0 = ct * 32u + (face & 1u) * 16u + (lane & 3) * 4u;
                uint32_t x[4];
#pragma unroll
                for (int i = 0; i < 4; i++) x[i] = fetch_view_elem<ES>(job, ptrs.src[b], w, z, rt * 32u + tr, c0 + i);
                const uint32_t pos = (uint32_t)job.pol.face_pos[face];
                direct_encode_store<M, ES, AF, G>(x, pos * 16u + half * 8u + (lane >> 2), r, lane, job.pol);
            }
        } else if (vec_ok) {
#pragma unroll 1
            for (int g = 0; g < 8; g += GR) {
                uint32_t xs[GR][4];
#pragma unroll
                for (int j = 0; j < GR; j++) {
                    const uint32_t face = (uint32_t)(g + j) >> 1, half = (uint32_t)(g + j) & 1u;
                    const uint32_t tr = (face >> 1) * 16u + half * 8u + (lane >> 2);   // row inside the tile
                    xs[j][0] = xs[j][1] = xs[j][2] = xs[j][3] = 0u;                    // tiny tiles: rows >= tile_h stay zero
                    if (tr < job.tile_h) load4<ES>(tile_src + (uint64_t)tr * job.stride_r + (face & 1u) * 16u * ES, true, xs[j]);
                }
#pragma unroll
                for (int j = 0; j < GR; j++) {
                    const uint32_t face = (uint32_t)(g + j) >> 1, half = (uint32_t)(g + j) & 1u;
                    const uint32_t pos = G ? (uint32_t)job.pol.face_pos[face] : face;
                    direct_encode_store<M, ES, AF, G>(xs[j], pos * 16u + half * 8u + (lane >> 2), r, lane, job.pol);
                }
            }
        } else {
#pragma unroll 1
            for (uint32_t hf = 0; hf < 8; hf++) {
                const uint32_t face = hf >> 1, half = hf & 1u;
                const uint32_t tr = (face >> 1) * 16u + half * 8u + (lane >> 2);
                uint32_t x[4] = {0u, 0u, 0u, 0u};
                if (tr < job.tile_h) load4<ES>(tile_src + (uint64_t)tr * job.stride_r + (face & 1u) * 16u * ES, false, x);
                const uint32_t pos = G ? (uint32_t)job.pol.face_pos[face] : face;
                direct_encode_store<M, ES, AF, G>(x, pos * 16u + half * 8u + (lane >> 2), r, lane, job.pol);
            }
        }
    }
}

// ------------------------------------------------------------------------------------------------
// host launchers
// ------------------------------------------------------------------------------------------------
static DeviceWorkSlots g_pack_slots[64];   // per device: which work counter the next staged launch takes

template <int M, int ES, bool AF, bool G, bool P = false>
static cudaError_t launch_staged(const TileJob &job, const typename TableOf<G>::type &table, int sm_count, cudaStream_t stream,
                                 unsigned int *status)
{
    using Cfg = PackCfg<M, ES>;
    static std::atomic<int> per_sm_cache[64];   // 0 = not yet looked up on this device (concurrent first calls store the same value)
    int dev = 0;
    cudaGetDevice(&dev);
    dev &= 63;
    int per_sm = per_sm_cache[dev].load(std::memory_order_acquire);
    if (per_sm == 0) {
        cudaError_t e = cudaFuncSetAttribute(pack_staged_kernel<M, ES, AF, G, P>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             Cfg::template smem_for<G>());
        if (e != cudaSuccess) return e;
        int n = 0;
        e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, pack_staged_kernel<M, ES, AF, G, P>, kStagedThreads,
                                                          Cfg::template smem_for<G>());
        if (e != cudaSuccess) return e;
        per_sm = n < 1 ? 1 : (n > 5 ? 5 : n);
        per_sm_cache[dev].store(per_sm, std::memory_order_release);
    }
    TileJob launch_job = job;
    typename TableOf<G>::type launch_table = table;
    if constexpr (G) {
        if (!finalize_table(launch_table, launch_job, Cfg::box)) return cudaErrorInvalidValue;
    } else {
        if (!set_box_tiles(launch_job, Cfg::box)) return cudaErrorInvalidValue;   // more than 2^31 work items: split the batch
    }
    if (launch_job.total_items == 0) return cudaSuccess;
    uint32_t grid = (uint32_t)(sm_count * per_sm);
    if (grid > launch_job.total_items) grid = launch_job.total_items;
    bool tracked = false;
    const int slot = take_work_slot(g_pack_slots[dev], stream, &tracked);
    if (slot < 0) return cudaErrorLaunchOutOfResources;   // the counters reserved for graph capture are used up
    launch_job.work_slot = (uint32_t)slot;
    // (A programmatic dependent launch -- the next conversion's CTAs becoming resident and running their prologue while
    // this one drains -- was measured on back-to-back launches of the 64-tensor batch: 6.5 % slower, not kept.)
    pack_staged_kernel<M, ES, AF, G, P><<<grid, kStagedThreads, Cfg::template smem_for<G>(), stream>>>(launch_job, launch_table, status);
    const cudaError_t e = cudaGetLastError();
    work_slot_launched(g_pack_slots[dev], slot, stream, tracked);
    return e;
}

template <int M, int ES, bool AF, bool G>
static cudaError_t launch_direct(const TileJob &job, const PtrTable &ptrs, int batch, int vec_ok, int sm_count,
                                 cudaStream_t stream)
{
    const uint64_t tiles = (uint64_t)batch * job.W * job.Z * job.Rt * job.Ct;   // one warp iteration each
    uint64_t blocks = (tiles + 7) / 8;
    const uint64_t cap = (uint64_t)sm_count * 32;
    if (blocks > cap) blocks = cap;
    pack_direct_kernel<M, ES, AF, G><<<(unsigned)blocks, 256, 0, stream>>>(job, ptrs, batch, vec_ok);
    return cudaGetLastError();
}

#define BUDA_FOR_EACH_PACK_KIND(X) \
    X(7, 4, false) X(3, 4, false) X(1, 4, false) X(7, 2, false) X(3, 2, false) X(1, 2, false) \
    X(7, 2, true) X(3, 2, true) X(1, 2, true) X(0, 4, false) X(0, 2, false) X(0, 1, false)
// conversions only the direct kernel performs (Lf8 from binary32, bfloat16 and binary16)
#define BUDA_FOR_EACH_DIRECT_ONLY_PACK_KIND(X) X(kLf8, 4, false) X(kLf8, 2, false) X(kLf8, 2, true)

// mant_bits 7/3/1 = Bfp pack, 0 = plain relayout; es = source element bytes; a_format: 5-bit shared
// exponent with a binary16 source.  path: 0 = staged (needs 16-byte aligned rows), 1 = direct.
// Plain flavour: a batch of tensors of one shape, default byte layout.
cudaError_t launch_tilize(const TileJob &job, const PtrTable &ptrs, int batch, int mant_bits, int es, int a_format, int path,
                          int vec_ok, int sm_count, cudaStream_t stream, unsigned int *status)
{
#define BUDA_DISPATCH(MM, EE, AA)                                                                         \
    if (mant_bits == MM && es == EE && (a_format != 0) == AA)                                             \
        return path == 0 ? launch_staged<MM, EE, AA, false>(job, ptrs, sm_count, stream, status)          \
                         : launch_direct<MM, EE, AA, false>(job, ptrs, batch, vec_ok, sm_count, stream);
    BUDA_FOR_EACH_PACK_KIND(BUDA_DISPATCH)
#undef BUDA_DISPATCH
#define BUDA_DISPATCH(MM, EE, AA) \
    if (mant_bits == MM && es == EE && (a_format != 0) == AA && path != 0) \
        return launch_direct<MM, EE, AA, false>(job, ptrs, batch, vec_ok, sm_count, stream);
    BUDA_FOR_EACH_DIRECT_ONLY_PACK_KIND(BUDA_DISPATCH)
#undef BUDA_DISPATCH
    return cudaErrorInvalidValue;
}

// General flavour, staged kernel: one table entry per tensor; job carries what the entries share (record size,
// header, layout policy).
cudaError_t launch_tilize_table(const TileJob &job, const GenTable &table, int mant_bits, int es, int a_format, int sm_count,
                                cudaStream_t stream, unsigned int *status)
{
#define BUDA_DISPATCH(MM, EE, AA) \
    if (mant_bits == MM && es == EE && (a_format != 0) == AA)                                                           \
        return policy_is_default(job.pol) ? launch_staged<MM, EE, AA, true, false>(job, table, sm_count, stream, status) \
                                          : launch_staged<MM, EE, AA, true, true>(job, table, sm_count, stream, status);
    BUDA_FOR_EACH_PACK_KIND(BUDA_DISPATCH)
#undef BUDA_DISPATCH
    return cudaErrorInvalidValue;
}

// General flavour, direct kernel: a batch of one shape under job.pol.
cudaError_t launch_tilize_direct_policy(const TileJob &job, const PtrTable &ptrs, int batch, int mant_bits, int es, int a_format,
                                        int vec_ok, int sm_count, cudaStream_t stream)
{
#define BUDA_DISPATCH(MM, EE, AA) \
    if (mant_bits == MM && es == EE && (a_format != 0) == AA) return launch_direct<MM, EE, AA, true>(job, ptrs, batch, vec_ok, sm_count, stream);
    BUDA_FOR_EACH_PACK_KIND(BUDA_DISPATCH)
    BUDA_FOR_EACH_DIRECT_ONLY_PACK_KIND(BUDA_DISPATCH)
#undef BUDA_DISPATCH
    return cudaErrorInvalidValue;
}

}  // namespace buda
