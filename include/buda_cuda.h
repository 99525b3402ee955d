/*
 * buda_cuda.h -- C ABI of libbuda_cuda.so: the B200 (sm_100a) implementation of TT-Buda's
 * data-format path (tilize / untilize, Bfp8_b / Bfp4_b / Bfp2_b pack and unpack, the golden int8
 * quantise ops, and the matmul whose weights are stored as Bfp8_b tiles).
 *
 * Conventions
 *   - Every function returns a buda_status (the reference's DEVICE_STATUS_CODE values,
 *     pybuda/csrc/backend_api/backend_api.cpp:622-625) and never throws.  After a non-zero
 *     return, buda_last_error() gives the reason for the calling thread.
 *   - Pointers are DEVICE pointers unless the parameter name ends in _host.
 *   - `stream` is a cudaStream_t passed as void*; NULL is the legacy default stream.  Device
 *     entry points only enqueue work; the _host entry points return after the result is in the
 *     caller's host buffer.
 *   - Shapes are [w, z, r, c], strides are in BYTES, outermost first, exactly as in the
 *     reference's PytorchTensorDesc (pybuda/csrc/lower_to_buda/common.hpp:251-258), widened to
 *     64 bits so tensors above 4 GiB keep working.
 *   - Data formats are the integer values of the reference's DataFormat enum
 *     (pybuda/csrc/lower_to_buda/common.hpp:92-111).
 *   - There is no CPU fallback: without a CUDA device every compute entry point fails.
 */
#ifndef BUDA_CUDA_H
#define BUDA_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum buda_status {
    BUDA_SUCCESS = 0,
    BUDA_RUNTIME_ERROR = 1,
    BUDA_TIMEOUT_ERROR = 2
} buda_status;

/* DataFormat, pybuda/csrc/lower_to_buda/common.hpp:92-111 */
enum {
    BUDA_DF_Float32 = 0, BUDA_DF_Float16 = 1, BUDA_DF_Bfp8 = 2, BUDA_DF_Bfp4 = 3, BUDA_DF_Bfp2 = 11,
    BUDA_DF_Float16_b = 5, BUDA_DF_Bfp8_b = 6, BUDA_DF_Bfp4_b = 7, BUDA_DF_Bfp2_b = 15, BUDA_DF_Lf8 = 10,
    BUDA_DF_UInt16 = 12, BUDA_DF_Int8 = 14, BUDA_DF_Int32 = 8, BUDA_DF_RawUInt8 = 0xf0,
    BUDA_DF_RawUInt16 = 0xf1, BUDA_DF_RawUInt32 = 0xf2, BUDA_DF_Invalid = 0xff
};

/* Queue geometry: the DramIODesc fields that decide where a tile lands
 * (pybuda/csrc/backend_api/backend_api.cpp:409-426; tile-level order per TileLayout::map,
 * pybuda/csrc/balancer/types.cpp:629-648).  A tensor [w,z,R,C] fits when z == t,
 * R == grid_r*mblock_m*ublock_rt*32 and C == grid_c*mblock_n*ublock_ct*32.  The queue image is
 * grid_r*grid_c buffers (one per grid core, row-major over the grid); each buffer holds w entries
 * of t*mblock_m*mblock_n*ublock_rt*ublock_ct tile records. */
typedef struct buda_queue_geom {
    uint32_t grid_r, grid_c;
    uint32_t mblock_m, mblock_n;
    uint32_t ublock_rt, ublock_ct;
    uint32_t t;
    uint32_t ublock_order; /* 0 = R (row-major scan of ublocks inside the mblock), 1 = C */
    uint32_t tile_height;  /* 0 or 32: full tiles.  16, 8, 4, 2, 1: "tiny" tiles (TileDim, pybuda/csrc/lower_to_buda/
                              common.hpp:80-90): a tile covers tile_height rows x 32 columns of the tensor, so
                              R == grid_r*mblock_m*ublock_rt*tile_height; its record keeps the full size
                              (balancer_utils.hpp:24-51 has no tile-dimension term) with rows >= tile_height zero. */
} buda_queue_geom;

/* One tensor of a call that converts many tensors of different shapes (buda_*_jobs below).  `tensor` is the
 * row-major side, `image` the queue image; which one is read depends on the direction of the call.
 * band_count > 0 converts only the tile rows band_first + k * band_step, k < band_count (a tile row = 32 tensor rows
 * across the whole width): every record still lands where the full tensor's image has it, so the GPUs of a box can
 * each convert their share of one tensor's tile rows (band b -> GPU b mod g) into one image.  When the queue grid is
 * 1x1 a tile row's records are one contiguous slice of the image (TileLayout::map,
 * pybuda/csrc/balancer/types.cpp:629-648).  band_count == 0: the whole tensor. */
typedef struct buda_tensor_job {
    const void *tensor;
    void *image;
    uint64_t image_bytes;          /* capacity of the image buffer (all grid buffers) */
    uint32_t shape[4];
    uint64_t strides_bytes[4];
    buda_queue_geom geom;
    uint32_t band_first, band_step, band_count;
    uint32_t slots, first_slot;    /* image is a ring of `slots` entries per grid core (0: dense image), see the queue section */
} buda_tensor_job;

/* The choices of the block-float byte layout that the reference's published description leaves open
 * (docs/public/dataformats.rst:74-83: "Truncate bits to fit in the BFP format mantissa size, optionally round before
 * truncation"; the drawings docs/public/images/bfp{8,4,2}_blocks.png show 32-bit rows without saying which end holds
 * exponent 0 / datum 0).  The converter that fixes them is not part of the reference checkout, so each is a switch:
 * when real tile bytes of that converter become available, set the combination that reproduces them.  All zero
 * (face_order {0,1,2,3}) is this library's default and the only layout the matmul kernels read. */
enum { BUDA_BFP_ROUND_NEAREST_EVEN = 0, BUDA_BFP_ROUND_TRUNCATE = 1,
       BUDA_BFP_ROUND_HALF_THEN_TRUNCATE = 2 /* half an ulp of the kept width added before the truncation: nearest, ties away from zero */ };
enum { BUDA_BFP_OVERFLOW_SATURATE = 0, BUDA_BFP_OVERFLOW_BUMP_EXPONENT = 1 };
enum { BUDA_BFP_ORDER_LITTLE = 0, BUDA_BFP_ORDER_BIG = 1 };
typedef struct buda_bfp_policy {
    uint32_t rounding;        /* of the dropped mantissa bits */
    uint32_t overflow;        /* a magnitude that rounds up past 2^m - 1: saturate, or raise the block's shared exponent by
                                 one and encode the whole block against it */
    uint8_t face_order[4];    /* which 16x16 face is stored first, second, ... (0 = rows 0-15 x cols 0-15, 1 = rows 0-15 x
                                 cols 16-31, 2 = rows 16-31 x cols 0-15, 3 = rows 16-31 x cols 16-31); applies to every format */
    uint32_t exponent_order;  /* LITTLE: exponent of block k in byte k of the exponent section; BIG: in byte k ^ 3
                                 (first exponent in the top byte of each 32-bit word) */
    uint32_t datum_order;     /* LITTLE: datum i of a block in bits [i(m+1), (i+1)(m+1)) of the block's bytes read as
                                 little-endian words; BIG: the datum fields of each 32-bit word in reverse order */
} buda_bfp_policy;

/* Process-wide; takes effect for calls that start afterwards.  NULL restores the default.  Replaces nothing in the
 * reference (there the behaviour is fixed inside the absent converter). */
int buda_set_bfp_policy(const buda_bfp_policy *policy);
int buda_get_bfp_policy(buda_bfp_policy *policy_out);

/* ------------------------------------------------------------------ sizes (host only, no GPU) */

/* Bytes of one 32x32 tile record; with_header adds the 32-byte header/pad.
 * Replaces tile_size_bytes, pybuda/csrc/balancer/balancer_utils.hpp:24-51.  -1: unknown format. */
int64_t buda_tile_bytes(int df, int with_header);

/* Replaces data_format_byte_size, pybuda/csrc/lower_to_buda/common.cpp:167-190. */
int64_t buda_data_format_byte_size(int df, int64_t elements);

/* Replaces tt::backend::get_io_size_in_bytes (bound at backend_api.cpp:710-722; called from
 * pybuda/csrc/placer/allocator_utils.cpp:17-48).  Tilized queues are sized with the 32-byte
 * per-tile header, as the reference compiler sizes them. */
int64_t buda_io_size_bytes(int df, int untilized, uint32_t ublock_ct, uint32_t ublock_rt, uint32_t mblock_m,
                           uint32_t mblock_n, uint32_t t, uint32_t entries, uint32_t tile_height,
                           uint32_t tile_width);

/* Total bytes of the queue image of a [w,z,R,C] tensor (all grid buffers); -1 if it does not fit. */
int64_t buda_tilized_bytes(const buda_queue_geom *geom, const uint32_t shape[4], int df, int with_header);

/* Linear position of tile (t, r, c): which grid core and which tile address in its buffer.
 * Replaces TileLayout::map, pybuda/csrc/balancer/types.cpp:629-648. */
int buda_tile_map(const buda_queue_geom *geom, uint32_t t, uint32_t r, uint32_t c, uint32_t *core_r,
                  uint32_t *core_c, uint64_t *addr);

/* ------------------------------------------------------------------ tilize + pack */

/* Row-major tensor -> queue image, converting to dst_df on the way.
 * src_df Float32 or Float16_b -> dst_df Bfp8_b / Bfp4_b / Bfp2_b (block-float pack), or
 * src_df Float16 -> Bfp8 / Bfp4 / Bfp2 (5-bit shared exponent), or
 * src_df Float32 / Float16_b / Float16 -> Lf8 (one 1-5-2 float per element, docs/public/dataformats.rst:24:
 * IEEE-style with subnormals, infinities and NaNs, round to nearest even), or
 * src_df == dst_df of a plain format (Float32, Float16, Float16_b, Int8, Int32, UInt16, Lf8,
 * RawUInt8/16/32; any pair of equal element width): layout only.
 * Replaces the conversion half of tt::backend::tilize_tensor / push_input
 * (bound at backend_api.cpp:688-704). */
int buda_tilize_pack(const void *src, int src_df, const uint32_t shape[4], const uint64_t strides_bytes[4],
                     const buda_queue_geom *geom, int dst_df, int with_header, void *dst, uint64_t dst_bytes,
                     void *stream);

/* The same over n independent tensors of one shape and geometry in ONE launch (the caller loop of
 * push_to_queues / push_constants_and_parameters, pybuda/pybuda/backend.py:448-493, hoisted into
 * the kernel).  srcs_host / dsts_host are HOST arrays of n device pointers. */
int buda_tilize_pack_batch(int n, const void *const *srcs_host, int src_df, const uint32_t shape[4],
                           const uint64_t strides_bytes[4], const buda_queue_geom *geom, int dst_df,
                           int with_header, void *const *dsts_host, uint64_t dst_bytes_each, void *stream);

/* Tensors of DIFFERENT shapes, strides and queue geometries (one src_df -> dst_df conversion) in as few launches as
 * possible: the caller loop of push_constants_and_parameters / update_device_paramaters
 * (pybuda/pybuda/backend.py:458-517), which walks every constant and parameter of a graph, hoisted into the kernel.
 * Up to 192 tensors share one launch; work is still handed out in address order across them.  jobs_host is a HOST
 * array; tensor and image are device pointers. */
int buda_tilize_pack_jobs(int n, const buda_tensor_job *jobs_host, int src_df, int dst_df, int with_header, void *stream);

/* Host-buffer form: copies the tensor to the device, converts, and copies the image back to
 * dst_host (what tt::backend::tilize_tensor returns to tti/archive.py:133).  Chunked so the two
 * copy directions and the kernel overlap.  Blocks until dst_host is complete. */
int buda_tilize_pack_host(const void *src_host, int src_df, const uint32_t shape[4],
                          const uint64_t strides_bytes[4], const buda_queue_geom *geom, int dst_df,
                          int with_header, void *dst_host, uint64_t dst_bytes, void *stream);

/* buda_tilize_pack_host over n tensors of one shape (HOST arrays of n host pointers): the caller loop of
 * push_to_queues / push_constants_and_parameters / update_device_paramaters (pybuda/pybuda/backend.py:448-493),
 * hoisted into one call so that the copy-in / kernel / copy-out pipeline runs across tensor boundaries and is
 * drained once.  Returns when every image is complete. */
int buda_tilize_pack_host_batch(int n, const void *const *srcs_host, int src_df, const uint32_t shape[4],
                                const uint64_t strides_bytes[4], const buda_queue_geom *geom, int dst_df, int with_header,
                                void *const *dsts_host, uint64_t dst_bytes_each, void *stream);

/* The same for tensors of different shapes: job.tensor is a HOST pointer; job.image is a host pointer
 * (image_on_device == 0) or a device pointer, e.g. the queues the parameters live in (image_on_device != 0; slots /
 * first_slot then apply).  One pipeline over all tensors, drained once. */
int buda_tilize_pack_host_jobs(int n, const buda_tensor_job *jobs_host, int src_df, int dst_df, int with_header,
                               int image_on_device, void *stream);

/* buda_tilize_pack_host for callers that must not allocate.  It has no counterpart in the reference.
 * Same arguments and result, but the device staging for the tensor and its image is a fixed 8 MiB
 * array inside the library (held by every GPU that loads the library until the process exits)
 * instead of cudaMalloc'd buffers, and the call makes no cudaMalloc / cudaFree and creates no stream
 * or event: copies and kernel run on `stream`, and the call returns when dst_host is complete.
 * Meant for a pusher thread inside a process whose own allocator already owns the device heap, or a
 * loop that cannot take the device-wide synchronisation an allocation implies.
 * Limit: tensor bytes (rounded up to 256) + image bytes <= 8 MiB, e.g. fp32 [1,1,1024,1024] -> Bfp8_b;
 * anything larger is refused with BUDA_RUNTIME_ERROR and a message naming the limit.
 * The first call on a device also looks up the array's device address (cudaGetSymbolAddress) and
 * sets kernel attributes; make that first call before any stream capture begins.
 * `stream` must belong to the device that is current when the call is made: the array address used is that device's.
 * All calls on a device share the one array, which keeps the previous call's bytes.  The library
 * lets one host thread at a time through per device; GPU work of two calls that still overlapped
 * (e.g. issued around that lock from forked copies of a context) would race on the array.
 * Nothing needs clearing between calls: the kernel overwrites every byte it later copies out. */
int buda_tilize_pack_host_noalloc(const void *src_host, int src_df, const uint32_t shape[4],
                                  const uint64_t strides_bytes[4], const buda_queue_geom *geom, int dst_df,
                                  int with_header, void *dst_host, uint64_t dst_bytes, void *stream);

/* ------------------------------------------------------------------ unpack + untilize */

/* Queue image -> row-major tensor.  Bfp*_b sources decode to Float32 or Float16_b; plain sources
 * keep their format.  Replaces the conversion half of tt::backend::get_output
 * (bound at backend_api.cpp:701). */
int buda_unpack_untilize(const void *src, int src_df, int with_header, const buda_queue_geom *geom, void *dst,
                         int dst_df, const uint32_t shape[4], const uint64_t strides_bytes[4], void *stream);

int buda_unpack_untilize_batch(int n, const void *const *srcs_host, int src_df, int with_header,
                               const buda_queue_geom *geom, void *const *dsts_host, int dst_df,
                               const uint32_t shape[4], const uint64_t strides_bytes[4], void *stream);

/* Inverse of buda_tilize_pack_jobs: job.image is read, job.tensor written. */
int buda_unpack_untilize_jobs(int n, const buda_tensor_job *jobs_host, int src_df, int with_header, int dst_df, void *stream);

int buda_unpack_untilize_host(const void *src_host, int src_df, int with_header, const buda_queue_geom *geom,
                              void *dst_host, int dst_df, const uint32_t shape[4],
                              const uint64_t strides_bytes[4], void *stream);

int buda_unpack_untilize_host_jobs(int n, const buda_tensor_job *jobs_host, int src_df, int with_header, int dst_df,
                                   int image_on_device, void *stream);

/* ------------------------------------------------------------------ device-resident queues
 * A queue is a ring of `slots` entries per grid core in device memory: core buffers of
 * slots * t*mblock_m*mblock_n*ublock_rt*ublock_ct tile records, laid out core after core (the
 * bufq_num_slots / bufq_entry_size of the reference's DramIODesc, backend_api.cpp:428-447).
 * Entry w of the tensor goes to slot (first_slot + w) % slots.  These are the device halves of
 * tt::backend::push_input and get_output (backend_api.cpp:688-701): the host layer keeps the
 * read / write pointers, this library moves and converts the data.  With a host tensor
 * (src_is_host / dst_is_host != 0) the call copies in slices overlapped with the kernel and blocks
 * until done; with a device tensor it only enqueues on `stream`. */
int64_t buda_queue_bytes(const buda_queue_geom *geom, int df, int with_header, uint32_t slots);

int buda_queue_write(const void *src, int src_is_host, int src_df, const uint32_t shape[4],
                     const uint64_t strides_bytes[4], const buda_queue_geom *geom, int dst_df, int with_header,
                     void *queue_base, uint32_t slots, uint32_t first_slot, void *stream);

int buda_queue_read(const void *queue_base, int src_df, int with_header, const buda_queue_geom *geom, uint32_t slots,
                    uint32_t first_slot, void *dst, int dst_is_host, int dst_df, const uint32_t shape[4],
                    const uint64_t strides_bytes[4], void *stream);

/* A tensor pushed through one of the reference's runtime tensor transforms, converted in ONE kernel: the kernel's
 * index arithmetic reads the source the way the transform would have rewritten it, so no padded / gathered copy of
 * the tensor is ever made.  `shape` is the tile-aligned [w, t, R, C] the queue covers; the view says where element
 * (w, z, r, c) of that shape comes from:
 *   BUDA_SRC_PADDED           the tensor [w, t, valid_r, valid_c] (its own strides in strides_bytes), zero outside:
 *                             the tile padding of pad_pytorch_tensor_to_buda (pybuda/pybuda/tensor.py:805-877; a
 *                             tile-broadcast dim, of size 1, stands for its whole tile: bcast_r / bcast_c) applied to a
 *                             ReinterpretShape view (tensor.py:1407-1413)
 *   BUDA_SRC_EMBEDDING_INDEX  a vector of `emb_count` row indices per entry (entry stride strides_bytes[0]) laid out
 *                             for an embedding op (_embedding_index, pybuda/pybuda/tensor.py:1382-1405): each 32x32
 *                             tile is 1024 consecutive indices, emb_group indices per queue tile row, all ones past
 *                             the last index, zero past the group; t == 1
 *   BUDA_SRC_PRESTRIDE        a convolution activation [w, ps_z, ps_h, ps_w] (strides_bytes) cut into its stride phases:
 *                             row k * ps_z + zc, column hr * ceil(ps_w / s) + wc  <-  act[w, zc, hr * s + y_k, wc * s + x_k]
 *                             (pybuda/pybuda/tensor.py:1415-1422, golden pybuda/pybuda/op/eval/pybuda/tm.py:316-335); t == 1
 * src is a DEVICE pointer.  queue_base / slots / first_slot as in buda_queue_write (slots == 0: a dense image). */
enum { BUDA_SRC_DENSE = 0, BUDA_SRC_PADDED = 1, BUDA_SRC_EMBEDDING_INDEX = 2, BUDA_SRC_PRESTRIDE = 3 };
typedef struct buda_source_view {
    uint32_t mode;
    uint32_t valid_r, valid_c;
    uint32_t bcast_r, bcast_c;      /* BUDA_SRC_PADDED: rows / columns all read row 0 / column 0 (valid_r / valid_c == 1) */
    uint64_t emb_count, emb_group;
    uint32_t ps_stride, ps_z, ps_h, ps_w;
    uint32_t ps_n_offsets;          /* 1..64 */
    int32_t ps_xy[128];             /* (x, y) pairs, each inside the stride window */
} buda_source_view;

int buda_queue_write_view(const void *src, int src_df, const uint32_t shape[4], const uint64_t strides_bytes[4],
                          const buda_source_view *view, const buda_queue_geom *geom, int dst_df, int with_header,
                          void *queue_base, uint64_t queue_bytes, uint32_t slots, uint32_t first_slot, void *stream);

/* Read `entries` entries and apply the output host transforms on the way: the t slices of an
 * entry are laid side by side, hstack across (columns) and vstack down (rows), giving a dense
 * [entries, t/(hstack*vstack), R*vstack, C*hstack] device tensor.  stack_row_major != 0: slice z sits
 * at row (z / hstack) % vstack, column z % hstack; otherwise at column (z / vstack) % hstack, row
 * z % vstack.  Same result as the golden hstack / vstack (pybuda/pybuda/op/eval/buda/tm.py:114-137)
 * applied to the untilized tensor; this is what tt::backend::get_output does for descriptors whose
 * hstack_factor / vstack_factor / stack_row_major are set (pybuda/pybuda/backend.py:294-302). */
int buda_queue_read_stacked(const void *queue_base, int src_df, int with_header, const buda_queue_geom *geom,
                            uint32_t slots, uint32_t first_slot, uint32_t entries, uint32_t hstack, uint32_t vstack,
                            int stack_row_major, void *dst, int dst_df, void *stream);

/* ------------------------------------------------------------------ memory and device plumbing
 * What the host layer needs so that it links against this library only and never against the
 * CUDA runtime itself.  No counterpart in the reference (its backend owns device memory). */
int buda_malloc(void **ptr, uint64_t bytes);
int buda_free(void *ptr);
int buda_host_alloc(void **ptr, uint64_t bytes);  /* pinned host memory */
int buda_host_free(void *ptr);
/* kind 0 host->device, 1 device->host, 2 device->device; returns after the copy is complete */
int buda_memcpy(void *dst, const void *src, uint64_t bytes, int kind, void *stream);
int buda_stream_synchronize(void *stream);
int buda_pointer_is_device(const void *ptr, int *is_device, int *device_ordinal);
int buda_get_device(int *ordinal);
int buda_set_device(int ordinal);
int buda_device_count(int *count);

/* ------------------------------------------------------------------ golden int8 quantise ops
 * The scale used for element i is scale[(i / inner) % scale_len]; scale_len == 1 is a per-tensor
 * scale, otherwise inner is the product of the dims after the quantisation axis
 * (reshape_to_match_input, pybuda/pybuda/op/eval/pybuda/quantize.py:38-52).  Results are
 * bit-identical to the reference's torch expressions. */

/* mode 0 Quantize      clamp(round(x / scale) + zp, lo, hi)   quantize.py:56-66
 * mode 1 BudaQuantize  clamp(round(x * scale) + zp, lo, hi)   quantize.py:68-77, buda/quantize.py:24-33 */
int buda_quantize(const float *x, int64_t n, const float *scale, int64_t scale_len, int64_t inner, float zero_point,
                  int mode, float lo, float hi, int8_t *out, void *stream);

/* Dequantize  (float(x) - zp) * scale   quantize.py:79-93, buda/quantize.py:35-40 */
int buda_dequantize(const int8_t *x, int64_t n, const float *scale, int64_t scale_len, int64_t inner,
                    float zero_point, float *out, void *stream);

/* mode 0 Requantize      round((inp_scale / out_scale) * float(x) + zp)   quantize.py:95-110
 * mode 1 BudaRequantize  round(float(x) * scale + zp)   quantize.py:112-122, buda/quantize.py:42-53
 * (mode 1 ignores out_scale) */
int buda_requantize(const int32_t *x, int64_t n, const float *inp_scale, const float *out_scale, int64_t scale_len,
                    int64_t inner, float zero_point, int mode, float lo, float hi, int8_t *out, void *stream);

/* ------------------------------------------------------------------ matmul with Bfp8_b weights
 * C[M,N] (bfloat16, row stride ldc elements) = A[M,K] (bfloat16, row stride lda elements) @ W,
 * W a [K,N] tensor stored as the Bfp8_b queue image of geometry grid 1x1, ublock 1x1, order R,
 * no tile header (tile (kt,nt) at record kt*(N/32)+nt).  binary32 accumulation on tcgen05 tensor
 * cores; weights are decoded in registers inside the kernel.  The device counterpart of the golden
 * matmul (pybuda/pybuda/op/eval/pybuda/matmul.py:20-33) for a weight queue whose df is Bfp8_b
 * (pybuda/csrc/passes/amp.cpp:457-500).  M % 128 == 0, N % 128 == 0, K % 64 == 0. */
int buda_bfp8b_gemm(const void *A, int64_t M, int64_t K, int64_t lda, const void *W_tiles, int64_t N, void *C,
                    int64_t ldc, void *stream);

/* The same product written to n_dst (1..8) destinations: C_dsts[0] in this device's memory, the others
 * typically the same matrix in peer devices' memory (buda_ipc_open), each already pointing at the
 * column block this device owns.  The epilogue stores every output tile to all destinations, so a
 * column-parallel matmul (pybuda/csrc/passes/dataformat.cpp:409-418 fixes the weight format; the
 * split of the weight columns over devices follows the reference's grid-column split of a matmul,
 * pybuda/csrc/balancer/types.cpp:629-648) leaves the gathered result on every device with no
 * separate all-gather.  Nothing is read from a peer.  Peers' stores are complete when the kernel is;
 * the caller synchronises the devices (a barrier) before reading. */
int buda_bfp8b_gemm_scatter(const void *A, int64_t M, int64_t K, int64_t lda, const void *W_tiles, int64_t N,
                            void *const *C_dsts, int n_dst, int64_t ldc, void *stream);

/* The same exchange through the NVSwitch: C_multicast is the multicast address of the [M, N] matrix that every device of
 * the group has bound to one multicast object (cuMulticast*; torch's symmetric memory hands it out), already pointing at
 * the column block this device owns, as C_local does in this device's own copy.  The epilogue writes the tile to
 * C_local and then issues ONE multimem store per 16 bytes, which the switch replicates to every device: a device sends
 * its block once instead of once per peer.  Same completion rule as above.  M > 256. */
int buda_bfp8b_gemm_multicast(const void *A, int64_t M, int64_t K, int64_t lda, const void *W_tiles, int64_t N, void *C_local,
                              void *C_multicast, int64_t ldc, void *stream);

/* Prestride transform of a convolution activation (device pointers): the [w, z, H, W] tensor, padded with
 * zeros to multiples of `stride`, becomes [w, 1, n_offsets*z, ceil(H/stride)*ceil(W/stride)]:
 *   dst[w, k*z + zc, hr*Ws + wc] = src[w, zc, hr*stride + y_k, wc*stride + x_k],  (x_k, y_k) = xy_offsets[2k], [2k+1]
 * written dense into [w, dst_rows, dst_cols] with zeros outside.  It is what a queue whose descriptor carries
 * a StrideDescriptor does to a pushed tensor before tilizing (pybuda/pybuda/tensor.py:1415-1422; golden
 * pybuda/pybuda/op/eval/pybuda/tm.py:316-335).  xy_offsets is a HOST array of n_offsets (x, y) pairs. */
int buda_prestride(const void *src, int elem_bytes, const uint32_t shape[4], const uint64_t strides_bytes[4], int stride,
                   const int *xy_offsets, int n_offsets, void *dst, uint32_t dst_rows, uint32_t dst_cols, void *stream);

/* acc[M,N] (int32) = A[M,K] (int8, row-major, row stride lda bytes) @ W[K,N], W the tilized image of an
 * Int8 queue (default geometry: 32x32 tiles row-major over [K/32][N/32], four 16x16 faces of 16-byte
 * rows, 1024 bytes per tile, no header) -- what buda_tilize_pack writes for a [1,1,K,N] int8 tensor.
 * The epilogue finishes the reference's matmul -> requantization chain in the same kernel
 * (pybuda/csrc/graph_lib/python_bindings.cpp:655-676; an int8 matmul yields int32,
 * pybuda/pybuda/op/eval/common.py:50-65):
 *   BUDA_I8_OUT_INT32        C int32  = acc
 *   BUDA_I8_OUT_REQUANT_I8   C int8   = clamp(round(float(acc) * scale + zero_point), -128, 127)
 *                                        (pybuda/pybuda/op/eval/buda/quantize.py:42-53)
 *   BUDA_I8_OUT_DEQUANT_F32  C float32 = (float(acc) - zero_point) * scale   (quantize.py:35-40)
 * scale: device pointer, scale_len == 1 (per tensor) or == N (per output column).  ldc in elements of
 * the output type.  Needs K % 128 == 0, N % 256 == 0, 16-byte aligned pointers and rows; any M. */
#define BUDA_I8_OUT_INT32 0
#define BUDA_I8_OUT_REQUANT_I8 1
#define BUDA_I8_OUT_DEQUANT_F32 2
int buda_i8_gemm(const void *A, int64_t M, int64_t K, int64_t lda, const void *W_tiles, int64_t N, const float *scale,
                 int64_t scale_len, float zero_point, int out_mode, void *C, int64_t ldc, void *stream);

/* Inter-process handles for device memory from buda_malloc, so that one process per GPU can hand its
 * output matrix to its peers.  export: 64-byte handle of an allocation's base pointer.  open: maps a
 * peer's allocation into this process (peer access is enabled on demand).  close: unmaps it. */
int buda_ipc_export(const void *dev_ptr, unsigned char handle_out[64]);
int buda_ipc_open(const unsigned char handle[64], void **dev_ptr_out);
int buda_ipc_close(void *dev_ptr);

/* ------------------------------------------------------------------ errors and status */

/* Copies the calling thread's last error text (NUL terminated) into buf; returns its length. */
size_t buda_last_error(char *buf, size_t buf_len);

/* Synchronises the current device, reads and clears the device status word.  *status_out gets 0 if every
 * kernel since the last call completed normally, otherwise a code naming the bounded wait that
 * gave up (see BUDA_DEVSTAT_*); the function then returns BUDA_TIMEOUT_ERROR. */
int buda_device_status(int *status_out);

enum {
    BUDA_DEVSTAT_OK = 0,
    BUDA_DEVSTAT_PACK_FULL_WAIT = 1,   /* pack: consumer waited too long for a staged band     */
    BUDA_DEVSTAT_PACK_EMPTY_WAIT = 2,  /* pack: producer waited too long for a free stage      */
    BUDA_DEVSTAT_UNPACK_FULL_WAIT = 3,
    BUDA_DEVSTAT_UNPACK_EMPTY_WAIT = 4,
    BUDA_DEVSTAT_GEMM_WAIT = 5,
    BUDA_DEVSTAT_SELFTEST_WAIT = 6     /* buda_selftest_bounded_wait (buda_cuda_testing.h): the wait that nothing completes ran out */
};

/* Number of kernels this library has launched in this process (for launch accounting). */
uint64_t buda_launch_count(void);

/* Library / build identification, e.g. "buda_cuda sm_100a". */
const char *buda_version(void);

#ifdef __cplusplus
}
#endif
#endif /* BUDA_CUDA_H */
