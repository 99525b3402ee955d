// Shared device/host helpers for the sm_100a data-format kernels: data-format tables, the tile
// order of a queue, mbarrier + bulk-copy (TMA) wrappers with BOUNDED waits, and the device status
// word that records a wait that gave up.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/buda_cuda.h"

namespace buda {

// ------------------------------------------------------------------------------------------------
// Data formats (values: reference enum DataFormat, pybuda/csrc/lower_to_buda/common.hpp:92-111)
// ------------------------------------------------------------------------------------------------
__host__ __device__ inline int bfp_mant_bits(int df)
{
    switch (df) {
        case BUDA_DF_Bfp8_b: case BUDA_DF_Bfp8: return 7;
        case BUDA_DF_Bfp4_b: case BUDA_DF_Bfp4: return 3;
        case BUDA_DF_Bfp2_b: case BUDA_DF_Bfp2: return 1;
        default: return 0;
    }
}

// Value of the kernels' mantissa-bits parameter that selects the element-wise conversion to / from Lf8 (7 / 3 / 1 are
// the block-float formats, 0 a relayout that keeps the element bytes).
constexpr int kLf8 = 8;

__host__ __device__ inline int plain_elem_bytes(int df)
{
    switch (df) {
        case BUDA_DF_Float32: case BUDA_DF_Int32: case BUDA_DF_RawUInt32: return 4;
        case BUDA_DF_Float16: case BUDA_DF_Float16_b: case BUDA_DF_UInt16: case BUDA_DF_RawUInt16: return 2;
        case BUDA_DF_Lf8: case BUDA_DF_Int8: case BUDA_DF_RawUInt8: return 1;
        default: return 0;
    }
}

// ------------------------------------------------------------------------------------------------
// Launch-time description of one tilize/untilize job (uniform over a batch of tensors)
// ------------------------------------------------------------------------------------------------
constexpr int kMaxBatch = 64;    // tensors per launch (pointer table lives in kernel parameters)
// A work item is a 32-row band of up to this many tiles.  8 (1 KiB row pieces per bulk copy) with two
// stages and two resident CTAs per SM measured 6.26 TB/s on the Bfp8_b pack; 4 tiles with three stages 5.3.
constexpr int kBoxTiles = 8;
// Tiles per work item of the staged kernels.  Unpack: what matters is the 1 KiB row piece it writes, so a block-float
// conversion to 2-byte elements takes twice as many tiles per band as one to 4-byte elements.  (Plain relayouts keep 8:
// their tile records are as large as the rows, and 16 of them would leave room for one CTA per SM only.)  Pack: since
// work items are started in address order, neighbouring 512-byte row pieces are fetched at about the same time anyway,
// and for the 8-bit formats half-size items with five CTAs per SM instead of two are 3.4 % faster (7050 vs 6818 GB/s on
// 32 fp32 tensors); the 4- and 2-bit formats, whose records are smaller, lose 7-14 % that way and keep the full size.
// Plain relayouts: 4-byte elements take half-size items in the pack direction (8 of their 4 KiB records per stage leave
// room for one CTA per SM only), 1-byte elements take double-size items both ways (a row piece of 8 tiles is 256 bytes).
__host__ __device__ constexpr int unpack_box_tiles_for(int es, bool block_float)
{
    return ((block_float && es < 4) || (!block_float && es == 1)) ? 2 * kBoxTiles : kBoxTiles;
}
__host__ __device__ constexpr int pack_box_tiles_for(int es, int mant_bits)
{
    return mant_bits == 7 ? unpack_box_tiles_for(es, true) / 2
                          : (mant_bits == 0 && es == 4) ? kBoxTiles / 2 : unpack_box_tiles_for(es, mant_bits > 0);
}
__host__ __device__ constexpr int box_tiles_for(int es, bool block_float) { return unpack_box_tiles_for(es, block_float); }

// The choices of the block-float byte layout that the published format description leaves open
// (docs/public/dataformats.rst:59-89 of the reference: "truncate bits ..., optionally round before truncation";
// the drawings docs/public/images/bfp{8,4,2}_blocks.png do not say which end of a 32-bit word holds datum 0).
// All zero = the layout this library writes by default.  Only the general kernel flavour reads it.
struct BfpPolicy {
    uint8_t rmode;        // rounding of the dropped mantissa bits: 0 nearest even, 1 truncate, 2 half an ulp added before the truncation
    uint8_t bump;         // a round-up past the largest magnitude: 0 saturates, 1 raises the shared exponent by one
    uint8_t exp_be;       // exponent section: 0 block k in byte k, 1 big-endian inside each 32-bit word (byte k ^ 3)
    uint8_t datum_be;     // mantissa section: 0 datum i in bits [i(m+1), (i+1)(m+1)) of the block, 1 the fields of each 32-bit word reversed
    uint8_t face_pos[4];  // where face f (0 = top left, 1 = top right, 2 = bottom left, 3 = bottom right) sits in the record
    uint8_t face_at[4];   // the inverse: which face sits at position p
};
__host__ __device__ inline BfpPolicy default_policy()
{
    BfpPolicy p = {0, 0, 0, 0, {0, 1, 2, 3}, {0, 1, 2, 3}};
    return p;
}
__host__ __device__ inline bool policy_is_default(const BfpPolicy &p)
{
    return !p.rmode && !p.bump && !p.exp_be && !p.datum_be && p.face_pos[0] == 0 && p.face_pos[1] == 1 && p.face_pos[2] == 2 &&
           p.face_pos[3] == 3;
}

// How the general flavour of the direct pack kernel reads the row-major side when that is not a dense tensor of whole
// tiles: the runtime tensor transforms of the reference's push path, done in the kernel's index arithmetic instead
// of as separate passes over the data.  Element (w, z, r, c) of the tile-aligned shape the queue covers comes from
//   kSrcPadded     the tensor itself where r < valid_r and c < valid_c, zero elsewhere (tile padding of
//                  pad_pytorch_tensor_to_buda, pybuda/pybuda/tensor.py:805-877); with bcast_r / bcast_c the single row /
//                  column of a tile-broadcast dimension stands for every row / column of its tile
//   kSrcEmbedding  a vector of row indices laid out for an embedding op (pybuda/pybuda/tensor.py:1382-1405): with
//                  group = indices per queue tile row, a = (c / 32) * 32 + r % 32 and flat = (r / 32) * group + a * 32 +
//                  c % 32: zero where a >= group / 32, all ones where flat >= count, else indices[w][flat]
//   kSrcPrestride  a convolution activation [w, ps_z, ps_h, ps_w] cut into its stride phases
//                  (pybuda/pybuda/op/eval/pybuda/tm.py:316-335): r = k * ps_z + zc, c = hr * ps_ws + wc ->
//                  act[w, zc, hr * s + y_k, wc * s + x_k], zero outside the activation or past the last phase / pixel
enum : uint32_t { kSrcDense = 0, kSrcPadded = 1, kSrcEmbedding = 2, kSrcPrestride = 3 };
struct SourceView {
    uint32_t mode;
    uint32_t valid_r, valid_c;
    uint32_t bcast_r, bcast_c;
    uint64_t emb_count, emb_group;
    uint32_t ps_stride, ps_noff, ps_z, ps_h, ps_w, ps_hs, ps_ws;
    int8_t ps_x[64], ps_y[64];
};

struct TileJob {
    // row-major side
    uint32_t W, Z, Rt, Ct;              // entries, t, tile rows, tile columns
    uint64_t stride_w, stride_z, stride_r;  // bytes
    uint32_t box_tiles;                 // tiles per work item: box_tiles_for(row-major element size, block-float queue)
    uint32_t boxes_per_band;            // ceil(Ct / box_tiles)
    uint32_t total_items;               // batch * W * Z * Rt * boxes_per_band  (< 2^31)
    uint32_t items_per_tensor;
    // queue side
    buda_queue_geom g;
    uint32_t tile_bytes;                // record size including the optional header
    uint32_t header_bytes;              // 0 or 32
    uint64_t tiles_per_entry;           // per grid core
    uint64_t buf_bytes;                 // bytes of one grid core's buffer (all W entries)
    int trivial_geom;                   // grid 1x1, ublock 1x1, order R: address = (z*Rt + rt)*Ct + ct
    uint32_t slots, slot0;              // ring queue: entry w lives in slot (slot0 + w) % slots; slots == 0: dense image
    // Row-major side, optional split of z into (outer, middle, inner) with their own strides: how the
    // hstack / vstack host transforms place the t slices of a queue entry.  zn1 == 0: plain z * stride_z.
    uint32_t zn1, zn2;
    uint64_t stride_z_mid, stride_z_out;
    uint32_t tile_h;                    // tensor rows per tile: 32, or 16 / 8 / 4 / 2 / 1 for tiny tiles (direct kernels only)
    uint32_t work_slot;                 // staged kernels: which work counter this launch draws its items from
    BfpPolicy pol;                      // general kernel flavour only
    SourceView view;                    // general flavour of the direct pack kernel only
};

// Re-derives the work-item fields of a job for `box` tiles per item; false when the launch would have 2^31 items or more.
inline bool set_box_tiles(TileJob &j, uint32_t box)
{
    const uint64_t batch = j.items_per_tensor ? j.total_items / j.items_per_tensor : 1;
    j.box_tiles = box;
    j.boxes_per_band = (j.Ct + box - 1) / box;
    const uint64_t per_tensor = (uint64_t)j.W * j.Z * j.Rt * j.boxes_per_band;
    if (per_tensor * batch >= (1ull << 31)) return false;
    j.items_per_tensor = (uint32_t)per_tensor;
    j.total_items = (uint32_t)(per_tensor * batch);
    return true;
}

// byte offset of slice z on the row-major side
__host__ __device__ inline uint64_t rm_z_offset(const TileJob &j, uint32_t z)
{
    if (j.zn1 == 0) return (uint64_t)z * j.stride_z;
    return (uint64_t)(z % j.zn1) * j.stride_z + (uint64_t)((z / j.zn1) % j.zn2) * j.stride_z_mid +
           (uint64_t)(z / (j.zn1 * j.zn2)) * j.stride_z_out;
}

// Work items of a staged kernel are handed out in address order from a counter in device memory: a CTA that finishes
// an item takes the next one, so the set of items in flight stays one compact, advancing window of the tensors.
// With a fixed assignment (item = CTA + k * grid) the CTAs drift apart and the window spreads; on a stream that is
// mostly stores that costs 15 % of the bandwidth (measured with a bare 1-byte-in / 4-bytes-out kernel on 32-row x
// 1 KiB bands: 5.69 TB/s fixed, 6.63 TB/s from a counter, the same as one short-lived block per band).
// A launch takes one of kWorkSlots counters round-robin and leaves it zeroed: the CTA that leaves last resets it.
// Two launches share a counter only if kWorkSlots other launches were issued while the first still runs.
struct WorkCounter {
    unsigned int next, done;
};
constexpr int kWorkSlots = 1024;

#ifdef __CUDACC__
// Lane 0 asks for the next item; the answer is only waited for where work_fetch_get() uses it, so a producer warp
// asks before it issues the current item's copies and reads the answer after them.
__device__ __forceinline__ uint32_t work_fetch_issue(WorkCounter *wc, int lane)
{
    uint32_t v = 0;
    if (lane == 0) v = atomicAdd(&wc->next, 1u);
    return v;
}
__device__ __forceinline__ uint32_t work_fetch_get(uint32_t issued) { return __shfl_sync(0xffffffffu, issued, 0); }
// one thread per CTA, after the CTA's last fetch, on every way out of the kernel
__device__ __forceinline__ void work_leave(WorkCounter *wc)
{
    __threadfence();
    if (atomicAdd(&wc->done, 1u) == gridDim.x - 1u) {
        wc->next = 0u;
        wc->done = 0u;
        __threadfence();
    }
}
#endif

struct PtrTable {
    const uint8_t *src[kMaxBatch];
    uint8_t *dst[kMaxBatch];
};

// ------------------------------------------------------------------------------------------------
// Job table of the general kernel flavour: every tensor of a launch has its own shape, strides, queue
// geometry and (optionally) its own selection of tile rows, so a whole set of differently shaped
// parameters is ONE launch, and so is the share of one tensor's tile-row bands that a GPU owns.
// Work items are numbered tensor after tensor (item_start), so they are still started in address order.
// The table travels in the kernel parameters.
// ------------------------------------------------------------------------------------------------
constexpr int kMaxGen = 192;
struct GenEntry {
    const uint8_t *rm;                  // row-major tensor
    uint8_t *q;                         // queue image (pack writes it, unpack reads it)
    uint64_t stride_w, stride_z, stride_r;
    uint64_t tiles_per_entry;           // per grid core: t * macro-block volume
    uint64_t buf_bytes;                 // one grid core's buffer
    uint32_t W, Z, Rt, Ct;              // entries, t, tile rows, tile columns of the whole tensor
    uint32_t item_start;                // first work item of this tensor
    uint32_t boxes_per_band;
    uint32_t band_first, band_step, bands;   // tile rows taken: band_first + k * band_step, k < bands
    uint32_t slots, slot0;
    uint32_t bpb_magic, bands_magic;    // n / boxes_per_band and n / bands as a multiply and a shift (n < 2^31)
    uint16_t grid_r, grid_c, mblock_m, mblock_n, ublock_rt, ublock_ct;
    uint8_t ublock_order, trivial_geom, bpb_shift, bands_shift;
};
static_assert(sizeof(GenEntry) == 128, "one 32-bit word per lane when a warp copies an entry");
struct GenTable {
    uint32_t n, pad;
    GenEntry e[kMaxGen];
};

// floor(n / d) for n < 2^31 as (n * magic) >> shift: magic = ceil(2^(31+s) / d) with s = ceil(log2 d) fits 32 bits.
inline void fast_div_setup(uint32_t d, uint32_t &magic, uint8_t &shift)
{
    uint32_t sft = 0;
    while ((1ull << sft) < d) sft++;
    const uint64_t num = 1ull << (31 + sft);
    magic = (uint32_t)((num + d - 1) / d);
    shift = (uint8_t)(31 + sft);
}
__host__ __device__ inline uint32_t fast_div(uint32_t n, uint32_t magic, uint32_t shift)
{
    return (uint32_t)(((uint64_t)n * magic) >> shift);
}

// Numbers the work items of a table for `box` tiles per item; false when the launch would have 2^31 items or more.
inline bool finalize_table(GenTable &t, TileJob &common, uint32_t box)
{
    uint64_t items = 0;
    common.box_tiles = box;
    for (uint32_t i = 0; i < t.n; i++) {
        GenEntry &e = t.e[i];
        e.boxes_per_band = (e.Ct + box - 1) / box;
        fast_div_setup(e.boxes_per_band, e.bpb_magic, e.bpb_shift);
        fast_div_setup(e.bands, e.bands_magic, e.bands_shift);
        e.item_start = (uint32_t)items;
        items += (uint64_t)e.W * e.Z * e.bands * e.boxes_per_band;
        if (items >= (1ull << 31)) return false;
    }
    common.total_items = (uint32_t)items;
    return true;
}

// The TileJob view of one table entry (only the fields the kernels' address arithmetic reads).
__host__ __device__ inline void job_of_entry(const TileJob &common, const GenEntry &e, TileJob &j)
{
    j.W = e.W; j.Z = e.Z; j.Rt = e.Rt; j.Ct = e.Ct;
    j.stride_w = e.stride_w; j.stride_z = e.stride_z; j.stride_r = e.stride_r;
    j.box_tiles = common.box_tiles;
    j.boxes_per_band = e.boxes_per_band;
    j.g.grid_r = e.grid_r; j.g.grid_c = e.grid_c; j.g.mblock_m = e.mblock_m; j.g.mblock_n = e.mblock_n;
    j.g.ublock_rt = e.ublock_rt; j.g.ublock_ct = e.ublock_ct; j.g.t = e.Z; j.g.ublock_order = e.ublock_order;
    j.tile_bytes = common.tile_bytes;
    j.header_bytes = common.header_bytes;
    j.tiles_per_entry = e.tiles_per_entry;
    j.slots = e.slots; j.slot0 = e.slot0;
    j.buf_bytes = e.buf_bytes;
    j.trivial_geom = e.trivial_geom;
    j.zn1 = j.zn2 = 0;
    j.tile_h = 32;
}

// Tile (z, rt, ct) of entry w -> byte offset of its record inside the queue image.
// Restates TileLayout::map (pybuda/csrc/balancer/types.cpp:629-648): the grid core owning the
// tile, then t-major, macro-block scan in ublock order, row-major inside the ublock.
__host__ __device__ inline uint64_t tile_record_offset(const TileJob &j, uint32_t w, uint32_t z, uint32_t rt,
                                                       uint32_t ct)
{
    if (j.slots) w = (j.slot0 + w) % j.slots;
    if (j.trivial_geom) {
        uint64_t addr = ((uint64_t)z * j.Rt + rt) * j.Ct + ct;
        return ((uint64_t)w * j.tiles_per_entry + addr) * j.tile_bytes;
    }
    const buda_queue_geom &g = j.g;
    uint32_t block_rt = g.mblock_m * g.ublock_rt, block_ct = g.mblock_n * g.ublock_ct;
    uint32_t core_r = rt / block_rt, core_c = ct / block_ct;
    uint32_t u_r = rt % g.ublock_rt, u_c = ct % g.ublock_ct;
    uint32_t m = (rt / g.ublock_rt) % g.mblock_m, n = (ct / g.ublock_ct) % g.mblock_n;
    uint64_t uvol = (uint64_t)g.ublock_rt * g.ublock_ct;
    uint64_t mvol = (uint64_t)g.mblock_m * g.mblock_n * uvol;
    uint64_t mlin = (g.ublock_order == 0 ? (uint64_t)m * g.mblock_n + n : (uint64_t)n * g.mblock_m + m) * uvol;
    uint64_t addr = (uint64_t)z * mvol + mlin + (uint64_t)u_r * g.ublock_ct + u_c;
    uint64_t core = (uint64_t)core_r * g.grid_c + core_c;
    return core * j.buf_bytes + ((uint64_t)w * j.tiles_per_entry + addr) * j.tile_bytes;
}

// ------------------------------------------------------------------------------------------------
// Device status word: set by a bounded wait that gave up, read (and cleared) by
// buda_device_status().  One word per device that loads the library; kernels receive its address.
// ------------------------------------------------------------------------------------------------
#ifdef __CUDACC__
__device__ __forceinline__ void report_status(unsigned int *status, unsigned int code)
{
    atomicCAS(status, 0u, code);
}

// ------------------------------------------------------------------------------------------------
// PTX wrappers
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_fence_init()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t *bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// try_wait that lets the hardware park the thread for up to `hint_ns` (it wakes as soon as the phase
// completes), so a long wait costs no issue slots that working warps could use
// non-blocking probe of a barrier phase (try_wait may suspend the thread for a while; this never does)
__device__ __forceinline__ bool mbar_test_wait(uint64_t *bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

__device__ __forceinline__ bool mbar_try_wait_parked(uint64_t *bar, uint32_t parity, uint32_t hint_ns)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(hint_ns)
        : "memory");
    return ok != 0;
}

__device__ __forceinline__ uint64_t global_timer_ns()
{
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Longest time any single wait may take before the kernel gives up (a healthy wait is microseconds).
constexpr uint64_t kWaitLimitNs = 2000000000ull;

// Bounded wait on an mbarrier phase.  Returns false if the wait gave up (after recording `code`
// in the device status word and raising *abort_flag so every other wait in the CTA ends at once).
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t *bar, uint32_t parity, volatile int *abort_flag,
                                                  unsigned int *status, unsigned int code, uint64_t limit_ns = kWaitLimitNs)
{
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = global_timer_ns();
    while (true) {
        // parked for up to 20 us at a time: no spinning, and the abort flag / deadline are still looked at
        if (mbar_try_wait_parked(bar, parity, 20000u)) return true;
        if (*abort_flag) return false;
        if (global_timer_ns() - t0 > limit_ns) {
            *abort_flag = 1;
            report_status(status, code);
            return false;
        }
    }
}

// 1-D bulk async copy (TMA engine) global -> shared, completion counted on an mbarrier.
// Both addresses 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void *smem_dst, const void *gsrc, uint32_t bytes, uint64_t *bar)
{
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
            smem_u32(smem_dst)),
        "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}

// 1-D bulk async copy shared -> global, tracked by the issuing thread's bulk group.
__device__ __forceinline__ void bulk_s2g(void *gdst, const void *smem_src, uint32_t bytes)
{
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst),
                 "r"(smem_u32(smem_src)), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }

// all of this thread's bulk stores have finished READING shared memory
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// all but the most recent bulk group of this thread have been read out of shared memory
__device__ __forceinline__ void bulk_wait_read_but_one() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }

// all but the newest N of this thread's bulk-store groups have finished READING shared memory
template <int N>
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }

// all of this thread's bulk stores are complete
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// order this thread's generic-proxy shared-memory writes before later async-proxy (bulk copy) reads
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void named_bar_sync(int id, int threads)
{
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
// Barrier over `threads` threads that also ORs a predicate across them: every participant learns
// whether any of them gave up, so they all leave a loop together and nobody waits alone.
__device__ __forceinline__ bool named_bar_or(int id, int threads, bool pred)
{
    uint32_t r;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.u32 q, %1, 0;\n\t"
        "bar.red.or.pred p, %2, %3, q;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(r)
        : "r"((uint32_t)pred), "r"(id), "r"(threads)
        : "memory");
    return r != 0;
}
#endif  // __CUDACC__

}  // namespace buda
