// C ABI of libbuda_cuda.so (declared in include/buda_cuda.h): argument checking, job set-up,
// kernel selection, the host-buffer pipelines, error text and the device status word.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <vector>

#include "buda_common.cuh"

namespace buda {
cudaError_t launch_tilize(const TileJob &job, const PtrTable &ptrs, int batch, int mant_bits, int es, int a_format, int path,
                          int vec_ok, int sm_count, cudaStream_t stream, unsigned int *status);
cudaError_t launch_untilize(const TileJob &job, const PtrTable &ptrs, int batch, int mant_bits, int es, int a_format, int path,
                            int vec_ok, int sm_count, cudaStream_t stream, unsigned int *status);
cudaError_t launch_tilize_table(const TileJob &job, const GenTable &table, int mant_bits, int es, int a_format, int sm_count,
                                cudaStream_t stream, unsigned int *status);
cudaError_t launch_tilize_direct_policy(const TileJob &job, const PtrTable &ptrs, int batch, int mant_bits, int es, int a_format,
                                        int vec_ok, int sm_count, cudaStream_t stream);
cudaError_t launch_untilize_table(const TileJob &job, const GenTable &table, int mant_bits, int es, int a_format, int sm_count,
                                  cudaStream_t stream, unsigned int *status);
cudaError_t launch_untilize_direct_policy(const TileJob &job, const PtrTable &ptrs, int batch, int mant_bits, int es, int a_format,
                                          int vec_ok, int sm_count, cudaStream_t stream);
cudaError_t launch_quantize(const float *x, int64_t n, const float *scale, int64_t scale_len, int64_t inner, float zp,
                            int mode, float lo, float hi, int8_t *out, int sm_count, cudaStream_t stream);
cudaError_t launch_dequantize(const int8_t *x, int64_t n, const float *scale, int64_t scale_len, int64_t inner, float zp,
                              float *out, int sm_count, cudaStream_t stream);
cudaError_t launch_requantize(const int32_t *x, int64_t n, const float *scale_a, const float *scale_b, int64_t scale_len,
                              int64_t inner, float zp, int mode, float lo, float hi, int8_t *out, int sm_count,
                              cudaStream_t stream);
cudaError_t launch_bfp8b_gemm(const void *A, int64_t M, int64_t K, int64_t lda, const void *W, int64_t N, void *const *C,
                              int n_dst, void *C_mc, int64_t ldc, int sm_count, cudaStream_t stream, unsigned int *status, char *err,
                              size_t err_len);

int gemm_kernel_choice(int which);
cudaError_t launch_prestride(const void *src, int elem_bytes, const uint32_t shape[4], const uint64_t strides[4], int stride,
                             const int *xy_offsets, int n_offsets, void *dst, uint32_t dst_rows, uint32_t dst_cols, int sm_count,
                             cudaStream_t stream);
cudaError_t launch_i8_gemm(const void *A, int64_t M, int64_t K, int64_t lda, const void *W, int64_t N, const float *scale,
                           int64_t scale_len, float zero_point, int out_mode, void *C, int64_t ldc, int sm_count, cudaStream_t stream,
                           unsigned int *status, char *err, size_t err_len);

// One CTA, one thread waiting: the barrier expects one arrival that never comes.  The other 31 lanes only take part in
// the final warp convergence.  The wait is the product kernels' own mbar_wait_bounded with a caller-given limit.
__global__ void selftest_wait_kernel(unsigned int *status, uint64_t limit_ns)
{
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        abort_flag = 0;
        mbar_fence_init();
    }
    __syncwarp();
    if (threadIdx.x == 0)
        (void)mbar_wait_bounded(&bar, 0u, &abort_flag, status, BUDA_DEVSTAT_SELFTEST_WAIT, limit_ns);
    __syncwarp();
}

// One status word per device that loads the library; kernels get its device address.
__device__ unsigned int g_device_status = 0;
}  // namespace buda

using namespace buda;

namespace {

thread_local char t_err[512] = "";
std::atomic<uint64_t> g_launches{0};

int fail(int code, const char *fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(t_err, sizeof(t_err), fmt, ap);
    va_end(ap);
    return code;
}

int cuda_fail(cudaError_t e, const char *what)
{
    return fail(BUDA_RUNTIME_ERROR, "%s: %s", what, cudaGetErrorString(e));
}

constexpr int kMaxDevices = 64;
constexpr int kPipeDepth = 4;

// The process-wide byte-layout policy (buda_set_bfp_policy).  Read once per call.
std::mutex g_policy_mu;
BfpPolicy g_policy = default_policy();
buda_bfp_policy g_policy_public = {0, 0, {0, 1, 2, 3}, 0, 0};

BfpPolicy current_policy()
{
    std::lock_guard<std::mutex> lock(g_policy_mu);
    return g_policy;
}

struct DevCtx {
    std::once_flag once;
    cudaError_t init_err = cudaSuccess;
    int sm_count = 0;
    unsigned int *status = nullptr;
    // host-buffer pipeline resources (guarded by host_mu)
    std::mutex host_mu;
    cudaStream_t s_in = nullptr, s_out = nullptr, s_comp = nullptr;
    cudaEvent_t ev_in[kPipeDepth] = {}, ev_comp[kPipeDepth] = {}, ev_out[kPipeDepth] = {};
    uint8_t *stage_a[kPipeDepth] = {};  // row-major side
    uint8_t *stage_b[kPipeDepth] = {};  // queue-image side
    size_t cap_a = 0, cap_b = 0;
    bool pipe_ready = false;
};

DevCtx g_ctx[kMaxDevices];

int get_ctx(DevCtx **out)
{
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail(e, "no usable CUDA device (this library has no CPU path)");
    if (dev < 0 || dev >= kMaxDevices) return fail(BUDA_RUNTIME_ERROR, "device ordinal %d out of range", dev);
    DevCtx &c = g_ctx[dev];
    std::call_once(c.once, [&]() {
        cudaError_t r = cudaDeviceGetAttribute(&c.sm_count, cudaDevAttrMultiProcessorCount, dev);
        if (r == cudaSuccess) r = cudaGetSymbolAddress((void **)&c.status, g_device_status);
        c.init_err = r;
    });
    if (c.init_err != cudaSuccess) return cuda_fail(c.init_err, "device set-up failed");
    *out = &c;
    return BUDA_SUCCESS;
}

bool is_bfp_b(int df) { return df == BUDA_DF_Bfp8_b || df == BUDA_DF_Bfp4_b || df == BUDA_DF_Bfp2_b; }
bool is_bfp_a(int df) { return df == BUDA_DF_Bfp8 || df == BUDA_DF_Bfp4 || df == BUDA_DF_Bfp2; }

// Fills the job for a [w,z,R,C] tensor in a queue of geometry g holding format qdf.
int make_job(const uint32_t shape[4], const uint64_t strides[4], const buda_queue_geom *g, int qdf, int with_header,
             int batch, TileJob &j, uint32_t slots = 0, uint32_t slot0 = 0)
{
    if (!shape || !strides || !g) return fail(BUDA_RUNTIME_ERROR, "null shape / strides / geometry");
    const int64_t tb = buda_tile_bytes(qdf, with_header);
    if (tb < 0) return fail(BUDA_RUNTIME_ERROR, "unsupported queue data format %d", qdf);
    if (shape[2] == 0 || shape[3] == 0 || shape[0] == 0 || shape[1] == 0)
        return fail(BUDA_RUNTIME_ERROR, "empty tensor [%u,%u,%u,%u]", shape[0], shape[1], shape[2], shape[3]);
    const uint32_t th = g->tile_height ? g->tile_height : 32u;
    if (th > 32u || (th & (th - 1u)))
        return fail(BUDA_RUNTIME_ERROR, "tile height %u is not one of 32, 16, 8, 4, 2, 1", th);
    if (shape[2] % th || shape[3] % 32)
        return fail(BUDA_RUNTIME_ERROR, "rows and columns must be multiples of the %ux32 tile, got [%u,%u]", th, shape[2],
                    shape[3]);
    if (!g->grid_r || !g->grid_c || !g->mblock_m || !g->mblock_n || !g->ublock_rt || !g->ublock_ct || !g->t ||
        g->ublock_order > 1)
        return fail(BUDA_RUNTIME_ERROR, "invalid queue geometry");
    if (g->t != shape[1]) return fail(BUDA_RUNTIME_ERROR, "queue t=%u does not match tensor z=%u", g->t, shape[1]);
    if ((uint64_t)g->grid_r * g->mblock_m * g->ublock_rt * th != shape[2] ||
        (uint64_t)g->grid_c * g->mblock_n * g->ublock_ct * 32u != shape[3])
        return fail(BUDA_RUNTIME_ERROR, "queue geometry covers %llux%llu, tensor is %ux%u",
                    (unsigned long long)g->grid_r * g->mblock_m * g->ublock_rt * th,
                    (unsigned long long)g->grid_c * g->mblock_n * g->ublock_ct * 32u, shape[2], shape[3]);
    j.W = shape[0]; j.Z = shape[1]; j.Rt = shape[2] / th; j.Ct = shape[3] / 32;
    j.tile_h = th;
    j.pol = default_policy();           // the callers that honour a policy overwrite it
    memset(&j.view, 0, sizeof(j.view)); // dense source unless buda_queue_write_view says otherwise
    j.work_slot = 0;                    // set per launch by the staged launchers
    j.stride_w = strides[0]; j.stride_z = strides[1]; j.stride_r = strides[2];
    j.box_tiles = (uint32_t)box_tiles_for((int)strides[3], bfp_mant_bits(qdf) != 0);
    j.boxes_per_band = (j.Ct + j.box_tiles - 1) / j.box_tiles;
    const uint64_t items_per_tensor = (uint64_t)j.W * j.Z * j.Rt * j.boxes_per_band;
    if (items_per_tensor * (uint64_t)batch >= (1ull << 31))
        return fail(BUDA_RUNTIME_ERROR, "too many tile bands in one launch (%llu); split the batch",
                    (unsigned long long)(items_per_tensor * batch));
    j.items_per_tensor = (uint32_t)items_per_tensor;
    j.total_items = (uint32_t)(items_per_tensor * batch);
    j.g = *g;
    j.tile_bytes = (uint32_t)tb;
    j.header_bytes = with_header ? 32u : 0u;
    j.tiles_per_entry = (uint64_t)g->t * g->mblock_m * g->mblock_n * g->ublock_rt * g->ublock_ct;
    if (slots && (slot0 >= slots || j.W > slots))
        return fail(BUDA_RUNTIME_ERROR, "ring of %u slots cannot take %u entries at slot %u", slots, j.W, slot0);
    j.slots = slots;
    j.slot0 = slot0;
    j.zn1 = j.zn2 = 0;
    j.stride_z_mid = j.stride_z_out = 0;
    j.buf_bytes = (uint64_t)(slots ? slots : j.W) * j.tiles_per_entry * j.tile_bytes;
    j.trivial_geom = (g->grid_r == 1 && g->grid_c == 1 && g->ublock_rt == 1 && g->ublock_ct == 1 && g->ublock_order == 0);
    return BUDA_SUCCESS;
}

// Which conversion a (row-major format, queue format) pair asks for.  mant = 7/3/1 for a Bfp
// pack/unpack, 0 for a plain relayout; es = element bytes on the row-major side.
int classify(int rm_df, int q_df, int &mant, int &es, bool unpacking = false)
{
    if (is_bfp_b(q_df)) {
        if (rm_df != BUDA_DF_Float32 && rm_df != BUDA_DF_Float16_b)
            return fail(BUDA_RUNTIME_ERROR, "Bfp*_b queues convert from/to Float32 or Float16_b, not format %d", rm_df);
        mant = bfp_mant_bits(q_df);
        es = rm_df == BUDA_DF_Float32 ? 4 : 2;
        return BUDA_SUCCESS;
    }
    if (is_bfp_a(q_df)) {
        // 5-bit shared exponent: packs from Float16 (the torch dtype these formats travel as); unpacks to
        // Float16 or Float32
        if (rm_df != BUDA_DF_Float16 && !(unpacking && rm_df == BUDA_DF_Float32))
            return fail(BUDA_RUNTIME_ERROR, "Bfp8 / Bfp4 / Bfp2 queues pack from Float16 and unpack to Float16 or Float32, not format %d",
                        rm_df);
        mant = bfp_mant_bits(q_df);
        es = rm_df == BUDA_DF_Float32 ? 4 : 2;
        return BUDA_SUCCESS;
    }
    if (q_df == BUDA_DF_Lf8 && (rm_df == BUDA_DF_Float32 || rm_df == BUDA_DF_Float16_b || rm_df == BUDA_DF_Float16)) {
        // element-wise conversion to / from the 1-5-2 float (direct kernels only); an Lf8 row-major side is a relayout
        mant = kLf8;
        es = rm_df == BUDA_DF_Float32 ? 4 : 2;
        return BUDA_SUCCESS;
    }
    es = plain_elem_bytes(q_df);
    if (es == 0) return fail(BUDA_RUNTIME_ERROR, "unsupported queue data format %d", q_df);
    if (plain_elem_bytes(rm_df) != es)
        return fail(BUDA_RUNTIME_ERROR, "plain tilize keeps the element width: format %d vs queue format %d", rm_df, q_df);
    mant = 0;
    return BUDA_SUCCESS;
}

// The kernels' flag for a binary16 row-major side: the "a" block-float formats travel as binary16, and Lf8 converts
// from / to it as well as from / to the 8-bit-exponent floats.
inline int half_side(int rm_df, int q_df) { return (is_bfp_a(q_df) || (q_df == BUDA_DF_Lf8 && rm_df == BUDA_DF_Float16)) ? 1 : 0; }

inline bool aligned16(uint64_t v) { return (v & 15u) == 0; }

// The staged (bulk-copy) kernels need every row start 16-byte aligned on both sides; the direct
// kernels use 4-element vector accesses when rows are aligned to 4 elements.
void pick_path(const TileJob &j, const PtrTable &p, int batch, int es, int &path, int &vec_ok, int mant = 0)
{
    const uint64_t valign = 4u * (uint64_t)es - 1u;
    uint64_t bits = j.stride_w | j.stride_z | j.stride_r;
    for (int b = 0; b < batch; b++) bits |= (uint64_t)p.src[b] | (uint64_t)p.dst[b];
    path = ((bits & 15u) == 0 && j.tile_h == 32u && mant != kLf8) ? 0 : 1;   // tiny tiles and Lf8 conversions: direct kernels only
    vec_ok = (bits & valign) == 0 ? 1 : 0;
}

int check_queue_ptrs_aligned(const void *const *q, int n)
{
    for (int b = 0; b < n; b++)
        if (!aligned16((uint64_t)q[b])) return fail(BUDA_RUNTIME_ERROR, "queue image pointers must be 16-byte aligned");
    return BUDA_SUCCESS;
}

// Table entry of the general kernel flavour for one tensor whose job has been validated by make_job.
// band_count == 0 takes every tile row.
int fill_entry(const TileJob &j, const void *rm, void *q, uint32_t band_first, uint32_t band_step, uint32_t band_count, GenEntry &e)
{
    const buda_queue_geom &g = j.g;
    if ((g.grid_r | g.grid_c | g.mblock_m | g.mblock_n | g.ublock_rt | g.ublock_ct) > 0xffffu)
        return fail(BUDA_RUNTIME_ERROR, "queue geometry terms above 65535 are not supported in a job table");
    if (band_count == 0) {
        band_first = 0; band_step = 1; band_count = j.Rt;
    }
    if (band_step == 0 || (uint64_t)band_first + (uint64_t)(band_count - 1) * band_step >= j.Rt)
        return fail(BUDA_RUNTIME_ERROR, "tile rows %u + k*%u, k < %u, reach past the tensor's %u tile rows", band_first, band_step,
                    band_count, j.Rt);
    memset(&e, 0, sizeof(e));
    e.rm = (const uint8_t *)rm;
    e.q = (uint8_t *)q;
    e.stride_w = j.stride_w; e.stride_z = j.stride_z; e.stride_r = j.stride_r;
    e.W = j.W; e.Z = j.Z; e.Rt = j.Rt; e.Ct = j.Ct;
    e.band_first = band_first; e.band_step = band_step; e.bands = band_count;
    e.slots = j.slots; e.slot0 = j.slot0;
    e.tiles_per_entry = j.tiles_per_entry;
    e.buf_bytes = j.buf_bytes;
    e.grid_r = (uint16_t)g.grid_r; e.grid_c = (uint16_t)g.grid_c; e.mblock_m = (uint16_t)g.mblock_m; e.mblock_n = (uint16_t)g.mblock_n;
    e.ublock_rt = (uint16_t)g.ublock_rt; e.ublock_ct = (uint16_t)g.ublock_ct;
    e.ublock_order = (uint8_t)g.ublock_order;
    e.trivial_geom = (uint8_t)j.trivial_geom;
    return BUDA_SUCCESS;
}

// One launch of a uniform batch through the kernel the alignment allows, in the flavour the policy asks for.
// direction 0 = tilize + pack (pt.src row-major, pt.dst image), 1 = unpack + untilize (pt.src image, pt.dst row-major).
int launch_uniform(int direction, DevCtx *ctx, TileJob &job, const PtrTable &pt, int nb, int mant, int es, int a_format, int path,
                   int vec_ok, cudaStream_t stream)
{
    BfpPolicy pol = current_policy();
    if (direction == 1) pol.rmode = pol.bump = 0;   // a reader does not care how the writer rounded: keeps the plain flavour where only those differ
    if (mant == 0 || mant == kLf8) pol.rmode = pol.bump = pol.exp_be = pol.datum_be = 0;   // formats without a shared exponent: only the face order applies
    cudaError_t e;
    if (policy_is_default(pol)) {
        e = direction == 0 ? launch_tilize(job, pt, nb, mant, es, a_format, path, vec_ok, ctx->sm_count, stream, ctx->status)
                           : launch_untilize(job, pt, nb, mant, es, a_format, path, vec_ok, ctx->sm_count, stream, ctx->status);
    } else {
        job.pol = pol;
        if (path == 0 && job.zn1 == 0) {
            GenTable *tab = new GenTable;   // ~20 KB: kept off the stack of whatever thread calls in
            tab->n = (uint32_t)nb;
            tab->pad = 0;
            int rc = BUDA_SUCCESS;
            for (int b = 0; b < nb && rc == BUDA_SUCCESS; b++)
                rc = direction == 0 ? fill_entry(job, pt.src[b], pt.dst[b], 0, 1, 0, tab->e[b])
                                    : fill_entry(job, pt.dst[b], const_cast<uint8_t *>(pt.src[b]), 0, 1, 0, tab->e[b]);
            if (rc != BUDA_SUCCESS) {
                delete tab;
                return rc;
            }
            e = direction == 0 ? launch_tilize_table(job, *tab, mant, es, a_format, ctx->sm_count, stream, ctx->status)
                               : launch_untilize_table(job, *tab, mant, es, a_format, ctx->sm_count, stream, ctx->status);
            delete tab;
        } else {
            e = direction == 0 ? launch_tilize_direct_policy(job, pt, nb, mant, es, a_format, vec_ok, ctx->sm_count, stream)
                               : launch_untilize_direct_policy(job, pt, nb, mant, es, a_format, vec_ok, ctx->sm_count, stream);
        }
    }
    if (e != cudaSuccess) return cuda_fail(e, direction == 0 ? "tilize launch failed" : "untilize launch failed");
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return BUDA_SUCCESS;
}

int tilize_device(int n, const void *const *srcs, int src_df, const uint32_t shape[4], const uint64_t strides[4],
                  const buda_queue_geom *geom, int dst_df, int with_header, void *const *dsts, uint64_t dst_bytes_each,
                  cudaStream_t stream, int force_path, uint32_t slots = 0, uint32_t slot0 = 0)
{
    DevCtx *ctx;
    if (int rc = get_ctx(&ctx)) return rc;
    if (n <= 0) return BUDA_SUCCESS;
    if (!srcs || !dsts) return fail(BUDA_RUNTIME_ERROR, "null pointer table");
    int mant, es;
    if (int rc = classify(src_df, dst_df, mant, es)) return rc;
    if (strides && strides[3] != (uint64_t)es)
        return fail(BUDA_RUNTIME_ERROR, "innermost stride must equal the element size (%d), got %llu", es,
                    (unsigned long long)strides[3]);
    if (int rc = check_queue_ptrs_aligned(dsts, n)) return rc;
    for (int b0 = 0; b0 < n; b0 += kMaxBatch) {
        const int nb = (n - b0 < kMaxBatch) ? (n - b0) : kMaxBatch;
        TileJob job;
        if (int rc = make_job(shape, strides, geom, dst_df, with_header, nb, job, slots, slot0)) return rc;
        const uint64_t need = job.buf_bytes * geom->grid_r * geom->grid_c;
        if (dst_bytes_each < need)
            return fail(BUDA_RUNTIME_ERROR, "destination holds %llu bytes, the queue image needs %llu",
                        (unsigned long long)dst_bytes_each, (unsigned long long)need);
        PtrTable pt;
        memset(&pt, 0, sizeof(pt));
        for (int b = 0; b < nb; b++) {
            if (!srcs[b0 + b] || !dsts[b0 + b]) return fail(BUDA_RUNTIME_ERROR, "null tensor pointer in batch");
            pt.src[b] = (const uint8_t *)srcs[b0 + b];
            pt.dst[b] = (uint8_t *)dsts[b0 + b];
        }
        int path, vec_ok;
        pick_path(job, pt, nb, es, path, vec_ok, mant);
        if (force_path >= 0) {
            if (force_path == 0 && path != 0) return fail(BUDA_RUNTIME_ERROR, "staged path needs 16-byte aligned rows and 32-row tiles");
            path = force_path;
        }
        if (int rc = launch_uniform(0, ctx, job, pt, nb, mant, es, half_side(src_df, dst_df), path, vec_ok, stream)) return rc;
    }
    return BUDA_SUCCESS;
}

int untilize_device(int n, const void *const *srcs, int src_df, int with_header, const buda_queue_geom *geom,
                    void *const *dsts, int dst_df, const uint32_t shape[4], const uint64_t strides[4], cudaStream_t stream,
                    int force_path, uint32_t slots = 0, uint32_t slot0 = 0)
{
    DevCtx *ctx;
    if (int rc = get_ctx(&ctx)) return rc;
    if (n <= 0) return BUDA_SUCCESS;
    if (!srcs || !dsts) return fail(BUDA_RUNTIME_ERROR, "null pointer table");
    int mant, es;
    if (int rc = classify(dst_df, src_df, mant, es, true)) return rc;
    if (strides && strides[3] != (uint64_t)es)
        return fail(BUDA_RUNTIME_ERROR, "innermost stride must equal the element size (%d), got %llu", es,
                    (unsigned long long)strides[3]);
    if (int rc = check_queue_ptrs_aligned(srcs, n)) return rc;
    for (int b0 = 0; b0 < n; b0 += kMaxBatch) {
        const int nb = (n - b0 < kMaxBatch) ? (n - b0) : kMaxBatch;
        TileJob job;
        if (int rc = make_job(shape, strides, geom, src_df, with_header, nb, job, slots, slot0)) return rc;
        PtrTable pt;
        memset(&pt, 0, sizeof(pt));
        for (int b = 0; b < nb; b++) {
            if (!srcs[b0 + b] || !dsts[b0 + b]) return fail(BUDA_RUNTIME_ERROR, "null tensor pointer in batch");
            pt.src[b] = (const uint8_t *)srcs[b0 + b];
            pt.dst[b] = (uint8_t *)dsts[b0 + b];
        }
        int path, vec_ok;
        pick_path(job, pt, nb, es, path, vec_ok, mant);
        if (force_path >= 0) {
            if (force_path == 0 && path != 0) return fail(BUDA_RUNTIME_ERROR, "staged path needs 16-byte aligned rows and 32-row tiles");
            path = force_path;
        }
        if (int rc = launch_uniform(1, ctx, job, pt, nb, mant, es, half_side(dst_df, src_df), path, vec_ok, stream)) return rc;
    }
    return BUDA_SUCCESS;
}

// ------------------------------------------------------------------------------------------------
// host-buffer pipeline: the tensor moves in slices of whole tile-row bands through kPipeDepth
// staging slots; copy-in, kernel and copy-out of different slices run on three streams.
// ------------------------------------------------------------------------------------------------
int ensure_pipe(DevCtx *c, size_t need_a, size_t need_b)
{
    if (!c->pipe_ready) {
        cudaError_t e;
        if ((e = cudaStreamCreateWithFlags(&c->s_in, cudaStreamNonBlocking)) != cudaSuccess) return cuda_fail(e, "stream");
        if ((e = cudaStreamCreateWithFlags(&c->s_out, cudaStreamNonBlocking)) != cudaSuccess) return cuda_fail(e, "stream");
        if ((e = cudaStreamCreateWithFlags(&c->s_comp, cudaStreamNonBlocking)) != cudaSuccess) return cuda_fail(e, "stream");
        for (int i = 0; i < kPipeDepth; i++) {
            if ((e = cudaEventCreateWithFlags(&c->ev_in[i], cudaEventDisableTiming)) != cudaSuccess) return cuda_fail(e, "event");
            if ((e = cudaEventCreateWithFlags(&c->ev_comp[i], cudaEventDisableTiming)) != cudaSuccess) return cuda_fail(e, "event");
            if ((e = cudaEventCreateWithFlags(&c->ev_out[i], cudaEventDisableTiming)) != cudaSuccess) return cuda_fail(e, "event");
        }
        c->pipe_ready = true;
    }
    if (need_a > c->cap_a) {
        for (int i = 0; i < kPipeDepth; i++) {
            if (c->stage_a[i]) cudaFree(c->stage_a[i]);
            c->stage_a[i] = nullptr;
            cudaError_t e = cudaMalloc((void **)&c->stage_a[i], need_a);
            if (e != cudaSuccess) { c->cap_a = 0; return cuda_fail(e, "staging allocation"); }
        }
        c->cap_a = need_a;
    }
    if (need_b > c->cap_b && need_b > 0) {
        for (int i = 0; i < kPipeDepth; i++) {
            if (c->stage_b[i]) cudaFree(c->stage_b[i]);
            c->stage_b[i] = nullptr;
            cudaError_t e = cudaMalloc((void **)&c->stage_b[i], need_b);
            if (e != cudaSuccess) { c->cap_b = 0; return cuda_fail(e, "staging allocation"); }
        }
        c->cap_b = need_b;
    }
    return BUDA_SUCCESS;
}

constexpr uint64_t kSliceTargetBytes = 8ull << 20;  // row-major bytes per pipeline slice

struct SlicePlan {
    bool sliced;          // true: slices of whole tile-row bands of one (w,z) plane
    uint32_t bands_per_slice, slices_per_plane;
};

// Slicing needs the bands of a plane to be contiguous in the queue image (trivial geometry) and
// the plane's rows to be evenly pitched.
SlicePlan plan_slices(const TileJob &j, uint64_t row_bytes)
{
    SlicePlan p{false, j.Rt, 1};
    if (!j.trivial_geom) return p;
    const uint64_t band_bytes = (uint64_t)j.tile_h * row_bytes;
    uint64_t bps = kSliceTargetBytes / (band_bytes ? band_bytes : 1);
    if (bps < 1) bps = 1;
    if (bps > j.Rt) bps = j.Rt;
    p.sliced = true;
    p.bands_per_slice = (uint32_t)bps;
    p.slices_per_plane = (uint32_t)((j.Rt + bps - 1) / bps);
    return p;
}

int status_after_sync(DevCtx *ctx)
{
    unsigned int st = 0;
    cudaError_t e = cudaMemcpy(&st, ctx->status, sizeof(st), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return cuda_fail(e, "reading the device status word");
    if (st != 0) {
        unsigned int zero = 0;
        cudaMemcpy(ctx->status, &zero, sizeof(zero), cudaMemcpyHostToDevice);
        return fail(BUDA_TIMEOUT_ERROR, "a kernel gave up waiting (device status %u)", st);
    }
    return BUDA_SUCCESS;
}

// One tensor of a host-buffer conversion: the row-major tensor is in HOST memory; the queue image is in host
// memory or already in device memory (possibly a ring of `slots` entries), the same for every item of a call.
struct HostItem {
    const void *rm_host;
    const void *q_ptr;
    const uint32_t *shape;
    const uint64_t *strides;
    const buda_queue_geom *geom;
    uint64_t q_bytes;
    uint32_t slots, slot0;
};

// direction 0: row-major -> queue image; 1: queue image -> row-major.
// The copy-in / kernel / copy-out pipeline keeps running across tensor boundaries and is drained once, at the end.
// Whatever the outcome, nothing of this call is still in flight on the staging slots when the lock is released.
int host_pipeline_items(int direction, int n, const HostItem *items, int rm_df, int q_df, int with_header, int q_on_device)
{
    DevCtx *ctx;
    if (int rc = get_ctx(&ctx)) return rc;
    if (n <= 0) return BUDA_SUCCESS;
    if (!items) return fail(BUDA_RUNTIME_ERROR, "null buffer table");
    int mant, es;
    if (int rc = classify(rm_df, q_df, mant, es, direction == 1)) return rc;

    // validate everything and size the staging slots before anything is enqueued
    struct Plan {
        TileJob full;
        SlicePlan plan;
        uint64_t row_bytes, image_bytes;
    };
    std::vector<Plan> plans((size_t)n);
    uint64_t need_a = 0, need_b = 0;
    for (int i = 0; i < n; i++) {
        const HostItem &it = items[i];
        if (!it.rm_host || !it.q_ptr) return fail(BUDA_RUNTIME_ERROR, "null buffer");
        Plan &pl = plans[(size_t)i];
        if (int rc = make_job(it.shape, it.strides, it.geom, q_df, with_header, 1, pl.full, it.slots, it.slot0)) return rc;
        if (it.strides[3] != (uint64_t)es) return fail(BUDA_RUNTIME_ERROR, "innermost stride must equal the element size");
        pl.image_bytes = pl.full.buf_bytes * it.geom->grid_r * it.geom->grid_c;
        if (it.q_bytes < pl.image_bytes)
            return fail(BUDA_RUNTIME_ERROR, "queue image buffer holds %llu bytes, needs %llu", (unsigned long long)it.q_bytes,
                        (unsigned long long)pl.image_bytes);
        pl.row_bytes = (uint64_t)it.shape[3] * es;
        if (it.strides[2] < pl.row_bytes) return fail(BUDA_RUNTIME_ERROR, "row stride smaller than a row");
        pl.plan = plan_slices(pl.full, pl.row_bytes);
        const uint64_t slice_a = pl.plan.sliced ? (uint64_t)pl.plan.bands_per_slice * pl.full.tile_h * pl.row_bytes
                                                : (uint64_t)it.shape[0] * it.shape[1] * it.shape[2] * pl.row_bytes;
        const uint64_t slice_b = q_on_device ? 0
                                             : (pl.plan.sliced ? (uint64_t)pl.plan.bands_per_slice * pl.full.Ct * pl.full.tile_bytes
                                                               : pl.image_bytes);
        if (slice_a > need_a) need_a = slice_a;
        if (slice_b > need_b) need_b = slice_b;
    }

    std::lock_guard<std::mutex> lock(ctx->host_mu);
    if (int rc = ensure_pipe(ctx, need_a, need_b)) return rc;

    auto drain = [&]() -> cudaError_t {
        cudaError_t first = cudaSuccess, e;
        if ((e = cudaStreamSynchronize(ctx->s_in)) != cudaSuccess && first == cudaSuccess) first = e;
        if ((e = cudaStreamSynchronize(ctx->s_comp)) != cudaSuccess && first == cudaSuccess) first = e;
        if ((e = cudaStreamSynchronize(ctx->s_out)) != cudaSuccess && first == cudaSuccess) first = e;
        return first;
    };
    // leaves with the pipeline drained (best effort) so that the next caller never meets this call's work
    auto bail = [&](int rc) -> int {
        (void)drain();
        return rc;
    };

    uint64_t k = 0;   // slices issued so far
    for (int bi = 0; bi < n; bi++) {
        const HostItem &it = items[bi];
        const Plan &pl = plans[(size_t)bi];
        const TileJob &full = pl.full;
        const uint32_t *shape = it.shape;
        const uint64_t *strides = it.strides;
        const uint64_t row_bytes = pl.row_bytes;
        uint8_t *rm_host = (uint8_t *)it.rm_host;
        uint8_t *q_mem = (uint8_t *)it.q_ptr;
        cudaError_t e = cudaSuccess;
        auto copy_rows = [&](uint8_t *dev, uint8_t *host, uint64_t rows, cudaStream_t s, bool to_dev) -> cudaError_t {
            // rows of `row_bytes` at pitch strides[2] on the host, dense on the device
            if (strides[2] == row_bytes)
                return cudaMemcpyAsync(to_dev ? (void *)dev : (void *)host, to_dev ? (void *)host : (void *)dev,
                                       rows * row_bytes, to_dev ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToHost, s);
            return to_dev ? cudaMemcpy2DAsync(dev, row_bytes, host, strides[2], row_bytes, rows, cudaMemcpyHostToDevice, s)
                          : cudaMemcpy2DAsync(host, strides[2], dev, row_bytes, row_bytes, rows, cudaMemcpyDeviceToHost, s);
        };

        if (!pl.plan.sliced) {
            // one shot: the whole tensor goes through slot 0, after everything issued so far has left the slots
            if (k > 0) {
                if ((e = drain()) != cudaSuccess) return cuda_fail(e, "synchronize");
                k = 0;
            }
            uint8_t *a = ctx->stage_a[0];
            uint8_t *b = q_on_device ? q_mem : ctx->stage_b[0];
            const uint64_t dense[4] = {(uint64_t)shape[1] * shape[2] * row_bytes, (uint64_t)shape[2] * row_bytes, row_bytes,
                                       (uint64_t)es};
            const void *srcs[1];
            void *dsts[1];
            if (direction == 0) {
                for (uint32_t w = 0; w < shape[0] && e == cudaSuccess; w++)
                    for (uint32_t z = 0; z < shape[1] && e == cudaSuccess; z++)
                        e = copy_rows(a + w * dense[0] + z * dense[1], rm_host + w * strides[0] + z * strides[1], shape[2],
                                      ctx->s_comp, true);
                if (e != cudaSuccess) return bail(cuda_fail(e, "host to device copy"));
                srcs[0] = a; dsts[0] = b;
                if (int rc = tilize_device(1, srcs, rm_df, shape, dense, it.geom, q_df, with_header, dsts, pl.image_bytes, ctx->s_comp, -1,
                                           q_on_device ? it.slots : 0, q_on_device ? it.slot0 : 0))
                    return bail(rc);
                if (!q_on_device) e = cudaMemcpyAsync(q_mem, b, pl.image_bytes, cudaMemcpyDeviceToHost, ctx->s_comp);
            } else {
                if (!q_on_device) e = cudaMemcpyAsync(b, q_mem, pl.image_bytes, cudaMemcpyHostToDevice, ctx->s_comp);
                if (e != cudaSuccess) return bail(cuda_fail(e, "host to device copy"));
                srcs[0] = b; dsts[0] = a;
                if (int rc = untilize_device(1, srcs, q_df, with_header, it.geom, dsts, rm_df, shape, dense, ctx->s_comp, -1,
                                             q_on_device ? it.slots : 0, q_on_device ? it.slot0 : 0))
                    return bail(rc);
                for (uint32_t w = 0; w < shape[0] && e == cudaSuccess; w++)
                    for (uint32_t z = 0; z < shape[1] && e == cudaSuccess; z++)
                        e = copy_rows(a + w * dense[0] + z * dense[1], rm_host + w * strides[0] + z * strides[1], shape[2],
                                      ctx->s_comp, false);
            }
            if (e != cudaSuccess) return bail(cuda_fail(e, "copy"));
            if ((e = cudaStreamSynchronize(ctx->s_comp)) != cudaSuccess) return bail(cuda_fail(e, "synchronize"));
            continue;
        }

        // sliced: each slice is a [1,1,bands*32,C] tensor whose records are one contiguous run of the image
        const SlicePlan &plan = pl.plan;
        for (uint32_t w = 0; w < shape[0]; w++) {
            for (uint32_t z = 0; z < shape[1]; z++) {
                for (uint32_t sl = 0; sl < plan.slices_per_plane; sl++, k++) {
                    const int slot = (int)(k % kPipeDepth);
                    const uint32_t band0 = sl * plan.bands_per_slice;
                    const uint32_t nb = (full.Rt - band0 < plan.bands_per_slice) ? (full.Rt - band0) : plan.bands_per_slice;
                    const uint32_t sshape[4] = {1, 1, nb * full.tile_h, shape[3]};
                    const uint64_t sstr[4] = {(uint64_t)nb * full.tile_h * row_bytes, (uint64_t)nb * full.tile_h * row_bytes, row_bytes,
                                              (uint64_t)es};
                    buda_queue_geom sg = *it.geom;
                    sg.t = 1;
                    sg.mblock_m = nb;
                    uint8_t *a = ctx->stage_a[slot];
                    uint8_t *rm_ptr = rm_host + w * strides[0] + z * strides[1] + (uint64_t)band0 * full.tile_h * strides[2];
                    uint8_t *q_ptr = q_mem + tile_record_offset(full, w, z, band0, 0);
                    uint8_t *b = q_on_device ? q_ptr : ctx->stage_b[slot];
                    const uint64_t q_len = (uint64_t)nb * full.Ct * full.tile_bytes;
                    const void *srcs[1];
                    void *dsts[1];
                    // the staging slot is free once the last stream that used it has passed ev_out
                    if (k >= (uint64_t)kPipeDepth) {
                        if ((e = cudaStreamWaitEvent(ctx->s_in, ctx->ev_out[slot], 0)) != cudaSuccess) return bail(cuda_fail(e, "wait"));
                    }
                    if (direction == 0) {
                        if ((e = copy_rows(a, rm_ptr, (uint64_t)nb * full.tile_h, ctx->s_in, true)) != cudaSuccess)
                            return bail(cuda_fail(e, "host to device copy"));
                    } else if (!q_on_device) {
                        if ((e = cudaMemcpyAsync(b, q_ptr, q_len, cudaMemcpyHostToDevice, ctx->s_in)) != cudaSuccess)
                            return bail(cuda_fail(e, "host to device copy"));
                    }
                    cudaEventRecord(ctx->ev_in[slot], ctx->s_in);
                    cudaStreamWaitEvent(ctx->s_comp, ctx->ev_in[slot], 0);
                    if (direction == 0) {
                        srcs[0] = a; dsts[0] = b;
                        if (int rc = tilize_device(1, srcs, rm_df, sshape, sstr, &sg, q_df, with_header, dsts, q_len, ctx->s_comp, -1))
                            return bail(rc);
                    } else {
                        srcs[0] = b; dsts[0] = a;
                        if (int rc = untilize_device(1, srcs, q_df, with_header, &sg, dsts, rm_df, sshape, sstr, ctx->s_comp, -1))
                            return bail(rc);
                    }
                    cudaEventRecord(ctx->ev_comp[slot], ctx->s_comp);
                    cudaStreamWaitEvent(ctx->s_out, ctx->ev_comp[slot], 0);
                    if (direction == 0) {
                        if (!q_on_device && (e = cudaMemcpyAsync(q_ptr, b, q_len, cudaMemcpyDeviceToHost, ctx->s_out)) != cudaSuccess)
                            return bail(cuda_fail(e, "device to host copy"));
                    } else {
                        if ((e = copy_rows(a, rm_ptr, (uint64_t)nb * full.tile_h, ctx->s_out, false)) != cudaSuccess)
                            return bail(cuda_fail(e, "device to host copy"));
                    }
                    cudaEventRecord(ctx->ev_out[slot], ctx->s_out);
                }
            }
        }
    }
    if (cudaError_t e = drain()) return cuda_fail(e, "synchronize");
    return status_after_sync(ctx);
}

// n tensors of one shape and geometry (rm_hosts[i] <-> q_ptrs[i])
int host_pipeline_n(int direction, int n, const void *const *rm_hosts, int rm_df, const uint32_t shape[4], const uint64_t strides[4],
                    const buda_queue_geom *geom, int q_df, int with_header, const void *const *q_ptrs, uint64_t q_bytes,
                    int q_on_device, uint32_t slots, uint32_t slot0)
{
    if (n <= 0) return BUDA_SUCCESS;
    if (!rm_hosts || !q_ptrs) return fail(BUDA_RUNTIME_ERROR, "null buffer table");
    if (!shape || !strides || !geom) return fail(BUDA_RUNTIME_ERROR, "null shape / strides / geometry");
    std::vector<HostItem> items((size_t)n);
    for (int i = 0; i < n; i++) items[(size_t)i] = HostItem{rm_hosts[i], q_ptrs[i], shape, strides, geom, q_bytes, slots, slot0};
    return host_pipeline_items(direction, n, items.data(), rm_df, q_df, with_header, q_on_device);
}

int host_pipeline(int direction, const void *rm_host, int rm_df, const uint32_t shape[4], const uint64_t strides[4],
                  const buda_queue_geom *geom, int q_df, int with_header, const void *q, uint64_t q_bytes, int q_on_device,
                  uint32_t slots, uint32_t slot0)
{
    if (!rm_host || !q) return fail(BUDA_RUNTIME_ERROR, "null buffer");
    const void *rms[1] = {rm_host};
    const void *qs[1] = {q};
    return host_pipeline_n(direction, 1, rms, rm_df, shape, strides, geom, q_df, with_header, qs, q_bytes, q_on_device, slots, slot0);
}

// n tensors with their own shapes through the general kernel flavour: aligned ones share launches of up to kMaxGen
// table entries; a tensor whose rows are not 16-byte aligned (or that has tiny tiles) gets a launch of the direct kernel.
int jobs_device(int direction, int n, const buda_tensor_job *jobs, int rm_df, int q_df, int with_header, cudaStream_t stream)
{
    DevCtx *ctx;
    if (int rc = get_ctx(&ctx)) return rc;
    if (n <= 0) return BUDA_SUCCESS;
    if (!jobs) return fail(BUDA_RUNTIME_ERROR, "null job table");
    int mant, es;
    if (int rc = classify(rm_df, q_df, mant, es, direction == 1)) return rc;
    const int a_format = half_side(rm_df, q_df);
    BfpPolicy pol = current_policy();
    if (direction == 1) pol.rmode = pol.bump = 0;   // a reader does not care how the writer rounded: keeps the plain flavour where only those differ
    if (mant == 0 || mant == kLf8) pol.rmode = pol.bump = pol.exp_be = pol.datum_be = 0;   // formats without a shared exponent: only the face order applies
    GenTable *tab = new GenTable;
    tab->n = 0;
    tab->pad = 0;
    TileJob common;
    memset(&common, 0, sizeof(common));
    int rc = BUDA_SUCCESS;
    auto flush = [&]() -> int {
        if (tab->n == 0) return BUDA_SUCCESS;
        cudaError_t e = direction == 0 ? launch_tilize_table(common, *tab, mant, es, a_format, ctx->sm_count, stream, ctx->status)
                                       : launch_untilize_table(common, *tab, mant, es, a_format, ctx->sm_count, stream, ctx->status);
        tab->n = 0;
        if (e != cudaSuccess) return cuda_fail(e, "job table launch failed");
        g_launches.fetch_add(1, std::memory_order_relaxed);
        return BUDA_SUCCESS;
    };
    for (int i = 0; i < n && rc == BUDA_SUCCESS; i++) {
        const buda_tensor_job &jb = jobs[i];
        if (!jb.tensor || !jb.image) { rc = fail(BUDA_RUNTIME_ERROR, "null tensor pointer in job %d", i); break; }
        TileJob j;
        if ((rc = make_job(jb.shape, jb.strides_bytes, &jb.geom, q_df, with_header, 1, j, jb.slots, jb.first_slot))) break;
        if (jb.strides_bytes[3] != (uint64_t)es) { rc = fail(BUDA_RUNTIME_ERROR, "innermost stride must equal the element size (%d)", es); break; }
        const uint64_t need = j.buf_bytes * jb.geom.grid_r * jb.geom.grid_c;
        if (jb.image_bytes < need) {
            rc = fail(BUDA_RUNTIME_ERROR, "job %d: image buffer holds %llu bytes, the queue image needs %llu", i,
                      (unsigned long long)jb.image_bytes, (unsigned long long)need);
            break;
        }
        if (!aligned16((uint64_t)jb.image)) { rc = fail(BUDA_RUNTIME_ERROR, "queue image pointers must be 16-byte aligned"); break; }
        PtrTable pt;
        memset(&pt, 0, sizeof(pt));
        pt.src[0] = (const uint8_t *)(direction == 0 ? jb.tensor : jb.image);
        pt.dst[0] = (uint8_t *)(direction == 0 ? jb.image : const_cast<void *>(jb.tensor));
        int path, vec_ok;
        pick_path(j, pt, 1, es, path, vec_ok, mant);
        if (path == 0) {
            common = j;
            common.pol = pol;
            if ((rc = fill_entry(j, jb.tensor, jb.image, jb.band_first, jb.band_step, jb.band_count, tab->e[tab->n]))) break;
            if (++tab->n == (uint32_t)kMaxGen) rc = flush();
        } else {
            if (jb.band_count != 0) { rc = fail(BUDA_RUNTIME_ERROR, "job %d: a selection of tile rows needs 16-byte aligned rows and 32-row tiles", i); break; }
            rc = launch_uniform(direction, ctx, j, pt, 1, mant, es, a_format, 1, vec_ok, stream);
        }
    }
    if (rc == BUDA_SUCCESS) rc = flush();
    delete tab;
    return rc;
}

}  // namespace

// ================================================================================================
// exported functions
// ================================================================================================
extern "C" {

int64_t buda_tile_bytes(int df, int with_header)
{
    const int64_t h = with_header ? 32 : 0;
    switch (df) {
        case BUDA_DF_Float32: case BUDA_DF_Int32: case BUDA_DF_RawUInt32: return 4096 + h;
        case BUDA_DF_Float16: case BUDA_DF_Float16_b: case BUDA_DF_UInt16: case BUDA_DF_RawUInt16: return 2048 + h;
        case BUDA_DF_Bfp8: case BUDA_DF_Bfp8_b: return 1024 + 64 + h;
        case BUDA_DF_Bfp4: case BUDA_DF_Bfp4_b: return 512 + 64 + h;
        case BUDA_DF_Bfp2: case BUDA_DF_Bfp2_b: return 256 + 64 + h;
        case BUDA_DF_Lf8: case BUDA_DF_Int8: case BUDA_DF_RawUInt8: return 1024 + h;
        default: return -1;
    }
}

int64_t buda_data_format_byte_size(int df, int64_t elements)
{
    switch (df) {
        case BUDA_DF_Float32: case BUDA_DF_Int32: case BUDA_DF_RawUInt32: return 4 * elements;
        case BUDA_DF_UInt16: case BUDA_DF_Float16_b: case BUDA_DF_Float16: case BUDA_DF_RawUInt16: return 2 * elements;
        case BUDA_DF_Bfp8_b: case BUDA_DF_Bfp8: return elements + elements / 16;
        case BUDA_DF_Bfp4_b: case BUDA_DF_Bfp4: return elements / 2 + elements / 16;
        case BUDA_DF_Bfp2_b: case BUDA_DF_Bfp2: return elements / 4 + elements / 16;
        case BUDA_DF_Lf8: case BUDA_DF_Int8: case BUDA_DF_RawUInt8: return elements;
        case BUDA_DF_Invalid: return 0;
        default: return -1;
    }
}

int64_t buda_io_size_bytes(int df, int untilized, uint32_t ublock_ct, uint32_t ublock_rt, uint32_t mblock_m,
                           uint32_t mblock_n, uint32_t t, uint32_t entries, uint32_t tile_height, uint32_t tile_width)
{
    const int64_t tiles = (int64_t)ublock_ct * ublock_rt * mblock_m * mblock_n * t * entries;
    if (untilized) {
        // a flat queue holds plain elements; block-float formats are read back as 16-bit floats
        int64_t es = plain_elem_bytes(df);
        if (es == 0) es = bfp_mant_bits(df) ? 2 : 0;
        if (es == 0) return -1;
        return tiles * tile_height * tile_width * es;
    }
    const int64_t tb = buda_tile_bytes(df, 1);
    if (tb < 0) return -1;
    // Tiny tiles keep full-size records: the reference's tile size has no tile-dimension term
    // (balancer_utils.hpp:24-51) and its allocator sizes every queue with the default tile dims
    // (placer/allocator_utils.cpp:33-43), which is also what the pack kernels write.
    return tiles * tb;
}

int64_t buda_tilized_bytes(const buda_queue_geom *geom, const uint32_t shape[4], int df, int with_header)
{
    TileJob j;
    const uint64_t st[4] = {0, 0, 0, 0};
    if (make_job(shape, st, geom, df, with_header, 1, j)) return -1;
    return (int64_t)(j.buf_bytes * geom->grid_r * geom->grid_c);
}

int buda_tile_map(const buda_queue_geom *g, uint32_t t, uint32_t r, uint32_t c, uint32_t *core_r, uint32_t *core_c,
                  uint64_t *addr)
{
    if (!g || !core_r || !core_c || !addr) return fail(BUDA_RUNTIME_ERROR, "null argument");
    if (!g->grid_r || !g->grid_c || !g->mblock_m || !g->mblock_n || !g->ublock_rt || !g->ublock_ct || g->ublock_order > 1)
        return fail(BUDA_RUNTIME_ERROR, "invalid queue geometry");
    if (t >= g->t || r >= g->grid_r * g->mblock_m * g->ublock_rt || c >= g->grid_c * g->mblock_n * g->ublock_ct)
        return fail(BUDA_RUNTIME_ERROR, "tile coordinate (%u,%u,%u) outside the queue", t, r, c);
    TileJob j;
    memset(&j, 0, sizeof(j));
    j.g = *g;
    j.tile_bytes = 1;
    j.tiles_per_entry = (uint64_t)g->t * g->mblock_m * g->mblock_n * g->ublock_rt * g->ublock_ct;
    j.buf_bytes = 1ull << 40;  // splits the offset into (core, address)
    j.trivial_geom = 0;
    const uint64_t off = tile_record_offset(j, 0, t, r, c);
    const uint64_t core = off >> 40;
    *core_r = (uint32_t)(core / g->grid_c);
    *core_c = (uint32_t)(core % g->grid_c);
    *addr = off & ((1ull << 40) - 1);
    return BUDA_SUCCESS;
}

int buda_tilize_pack(const void *src, int src_df, const uint32_t shape[4], const uint64_t strides_bytes[4],
                     const buda_queue_geom *geom, int dst_df, int with_header, void *dst, uint64_t dst_bytes, void *stream)
{
    const void *srcs[1] = {src};
    void *dsts[1] = {dst};
    return tilize_device(1, srcs, src_df, shape, strides_bytes, geom, dst_df, with_header, dsts, dst_bytes,
                         (cudaStream_t)stream, -1);
}

int buda_tilize_pack_batch(int n, const void *const *srcs_host, int src_df, const uint32_t shape[4],
                           const uint64_t strides_bytes[4], const buda_queue_geom *geom, int dst_df, int with_header,
                           void *const *dsts_host, uint64_t dst_bytes_each, void *stream)
{
    return tilize_device(n, srcs_host, src_df, shape, strides_bytes, geom, dst_df, with_header, dsts_host, dst_bytes_each,
                         (cudaStream_t)stream, -1);
}

// Same as buda_tilize_pack_batch with the kernel chosen by the caller: 0 staged, 1 direct.
// For tests and measurements of the two kernels on the same input.
int buda_tilize_pack_batch_path(int n, const void *const *srcs_host, int src_df, const uint32_t shape[4],
                                const uint64_t strides_bytes[4], const buda_queue_geom *geom, int dst_df, int with_header,
                                void *const *dsts_host, uint64_t dst_bytes_each, void *stream, int path)
{
    return tilize_device(n, srcs_host, src_df, shape, strides_bytes, geom, dst_df, with_header, dsts_host, dst_bytes_each,
                         (cudaStream_t)stream, path);
}

int buda_tilize_pack_host(const void *src_host, int src_df, const uint32_t shape[4], const uint64_t strides_bytes[4],
                          const buda_queue_geom *geom, int dst_df, int with_header, void *dst_host, uint64_t dst_bytes,
                          void *stream)
{
    (void)stream;
    return host_pipeline(0, src_host, src_df, shape, strides_bytes, geom, dst_df, with_header, dst_host, dst_bytes, 0, 0, 0);
}

int buda_tilize_pack_host_batch(int n, const void *const *srcs_host, int src_df, const uint32_t shape[4],
                                const uint64_t strides_bytes[4], const buda_queue_geom *geom, int dst_df, int with_header,
                                void *const *dsts_host, uint64_t dst_bytes_each, void *stream)
{
    (void)stream;
    return host_pipeline_n(0, n, srcs_host, src_df, shape, strides_bytes, geom, dst_df, with_header, dsts_host, dst_bytes_each, 0, 0, 0);
}

int buda_unpack_untilize(const void *src, int src_df, int with_header, const buda_queue_geom *geom, void *dst, int dst_df,
                         const uint32_t shape[4], const uint64_t strides_bytes[4], void *stream)
{
    const void *srcs[1] = {src};
    void *dsts[1] = {dst};
    return untilize_device(1, srcs, src_df, with_header, geom, dsts, dst_df, shape, strides_bytes, (cudaStream_t)stream, -1);
}

int buda_unpack_untilize_batch(int n, const void *const *srcs_host, int src_df, int with_header,
                               const buda_queue_geom *geom, void *const *dsts_host, int dst_df, const uint32_t shape[4],
                               const uint64_t strides_bytes[4], void *stream)
{
    return untilize_device(n, srcs_host, src_df, with_header, geom, dsts_host, dst_df, shape, strides_bytes,
                           (cudaStream_t)stream, -1);
}

int buda_unpack_untilize_batch_path(int n, const void *const *srcs_host, int src_df, int with_header,
                                    const buda_queue_geom *geom, void *const *dsts_host, int dst_df,
                                    const uint32_t shape[4], const uint64_t strides_bytes[4], void *stream, int path)
{
    return untilize_device(n, srcs_host, src_df, with_header, geom, dsts_host, dst_df, shape, strides_bytes,
                           (cudaStream_t)stream, path);
}

int buda_unpack_untilize_host(const void *src_host, int src_df, int with_header, const buda_queue_geom *geom,
                              void *dst_host, int dst_df, const uint32_t shape[4], const uint64_t strides_bytes[4],
                              void *stream)
{
    (void)stream;
    int64_t need = buda_tilized_bytes(geom, shape, src_df, with_header);
    if (need < 0) return fail(BUDA_RUNTIME_ERROR, "tensor does not fit the queue geometry");
    return host_pipeline(1, dst_host, dst_df, shape, strides_bytes, geom, src_df, with_header, src_host, (uint64_t)need, 0, 0, 0);
}

int64_t buda_queue_bytes(const buda_queue_geom *geom, int df, int with_header, uint32_t slots)
{
    if (!geom) return -1;
    const int64_t tb = buda_tile_bytes(df, with_header);
    if (tb < 0 || slots == 0) return -1;
    return (int64_t)geom->grid_r * geom->grid_c * slots * geom->t * geom->mblock_m * geom->mblock_n * geom->ublock_rt *
           geom->ublock_ct * tb;
}

int buda_queue_write(const void *src, int src_is_host, int src_df, const uint32_t shape[4], const uint64_t strides_bytes[4],
                     const buda_queue_geom *geom, int dst_df, int with_header, void *queue_base, uint32_t slots,
                     uint32_t first_slot, void *stream)
{
    if (slots == 0) return fail(BUDA_RUNTIME_ERROR, "a queue has at least one slot");
    const int64_t qb = buda_queue_bytes(geom, dst_df, with_header, slots);
    if (qb < 0) return fail(BUDA_RUNTIME_ERROR, "invalid queue geometry or format");
    if (src_is_host)
        return host_pipeline(0, src, src_df, shape, strides_bytes, geom, dst_df, with_header, queue_base, (uint64_t)qb, 1, slots,
                             first_slot);
    const void *srcs[1] = {src};
    void *dsts[1] = {queue_base};
    return tilize_device(1, srcs, src_df, shape, strides_bytes, geom, dst_df, with_header, dsts, (uint64_t)qb,
                         (cudaStream_t)stream, -1, slots, first_slot);
}

int buda_queue_write_view(const void *src, int src_df, const uint32_t shape[4], const uint64_t strides_bytes[4],
                          const buda_source_view *view, const buda_queue_geom *geom, int dst_df, int with_header, void *queue_base,
                          uint64_t queue_bytes, uint32_t slots, uint32_t first_slot, void *stream)
{
    DevCtx *ctx;
    if (int rc = get_ctx(&ctx)) return rc;
    if (!src || !queue_base || !view || !geom || !shape || !strides_bytes) return fail(BUDA_RUNTIME_ERROR, "null argument");
    int mant, es;
    if (int rc = classify(src_df, dst_df, mant, es)) return rc;
    if (strides_bytes[3] != (uint64_t)es) return fail(BUDA_RUNTIME_ERROR, "innermost stride must equal the element size (%d)", es);
    if (geom->tile_height != 0 && geom->tile_height != 32) return fail(BUDA_RUNTIME_ERROR, "source views need 32-row tiles");
    TileJob job;
    if (int rc = make_job(shape, strides_bytes, geom, dst_df, with_header, 1, job, slots, first_slot)) return rc;
    const uint64_t need = job.buf_bytes * geom->grid_r * geom->grid_c;
    if (queue_bytes < need)
        return fail(BUDA_RUNTIME_ERROR, "destination holds %llu bytes, the queue image needs %llu", (unsigned long long)queue_bytes,
                    (unsigned long long)need);
    if (!aligned16((uint64_t)queue_base)) return fail(BUDA_RUNTIME_ERROR, "queue image pointers must be 16-byte aligned");
    SourceView &v = job.view;
    memset(&v, 0, sizeof(v));
    switch (view->mode) {
        case BUDA_SRC_PADDED:
            if (view->valid_r == 0 || view->valid_c == 0 || view->valid_r > shape[2] || view->valid_c > shape[3])
                return fail(BUDA_RUNTIME_ERROR, "padded view: valid extent %ux%u outside the %ux%u the queue covers", view->valid_r,
                            view->valid_c, shape[2], shape[3]);
            if ((view->bcast_r && view->valid_r != 1) || (view->bcast_c && view->valid_c != 1))
                return fail(BUDA_RUNTIME_ERROR, "padded view: only a dimension of size 1 is broadcast across its tile");
            v.mode = kSrcPadded;
            v.valid_r = view->valid_r;
            v.valid_c = view->valid_c;
            v.bcast_r = view->bcast_r ? 1u : 0u;
            v.bcast_c = view->bcast_c ? 1u : 0u;
            break;
        case BUDA_SRC_EMBEDDING_INDEX:
            if (shape[1] != 1) return fail(BUDA_RUNTIME_ERROR, "embedding-index view: t must be 1");
            if (mant != 0) return fail(BUDA_RUNTIME_ERROR, "embedding-index view: indices go to a raw / integer queue");
            if (view->emb_group == 0 || view->emb_group % 32 || view->emb_group > (uint64_t)shape[3] * 32u)
                return fail(BUDA_RUNTIME_ERROR, "embedding-index view: %llu indices per tile row do not fit %u columns",
                            (unsigned long long)view->emb_group, shape[3]);
            if (view->emb_count > (uint64_t)(shape[2] / 32u) * view->emb_group)
                return fail(BUDA_RUNTIME_ERROR, "embedding-index view: %llu indices do not fit the queue", (unsigned long long)view->emb_count);
            v.mode = kSrcEmbedding;
            v.emb_count = view->emb_count;
            v.emb_group = view->emb_group;
            break;
        case BUDA_SRC_PRESTRIDE: {
            if (shape[1] != 1) return fail(BUDA_RUNTIME_ERROR, "prestride view: t must be 1");
            const uint32_t sdv = view->ps_stride;
            if (sdv < 1 || sdv > 127 || view->ps_n_offsets < 1 || view->ps_n_offsets > 64 || !view->ps_z || !view->ps_h || !view->ps_w)
                return fail(BUDA_RUNTIME_ERROR, "prestride view: stride %u with %u offsets is not supported", sdv, view->ps_n_offsets);
            v.mode = kSrcPrestride;
            v.ps_stride = sdv;
            v.ps_noff = view->ps_n_offsets;
            v.ps_z = view->ps_z; v.ps_h = view->ps_h; v.ps_w = view->ps_w;
            v.ps_hs = (view->ps_h + sdv - 1) / sdv;
            v.ps_ws = (view->ps_w + sdv - 1) / sdv;
            for (uint32_t k = 0; k < view->ps_n_offsets; k++) {
                const int32_t x = view->ps_xy[2 * k], y = view->ps_xy[2 * k + 1];
                if (x < 0 || y < 0 || x >= (int32_t)sdv || y >= (int32_t)sdv)
                    return fail(BUDA_RUNTIME_ERROR, "prestride view: offset %u = (%d, %d) lies outside the %ux%u stride window", k, x, y, sdv, sdv);
                v.ps_x[k] = (int8_t)x;
                v.ps_y[k] = (int8_t)y;
            }
            if ((uint64_t)v.ps_noff * v.ps_z > shape[2] || (uint64_t)v.ps_hs * v.ps_ws > shape[3])
                return fail(BUDA_RUNTIME_ERROR, "prestride view: [%llu x %llu] does not fit the queue's %ux%u",
                            (unsigned long long)v.ps_noff * v.ps_z, (unsigned long long)v.ps_hs * v.ps_ws, shape[2], shape[3]);
            break;
        }
        default:
            return fail(BUDA_RUNTIME_ERROR, "unknown source view mode %u", view->mode);
    }
    job.pol = current_policy();
    PtrTable pt;
    memset(&pt, 0, sizeof(pt));
    pt.src[0] = (const uint8_t *)src;
    pt.dst[0] = (uint8_t *)queue_base;
    cudaError_t e = launch_tilize_direct_policy(job, pt, 1, mant, es, half_side(src_df, dst_df), 0, ctx->sm_count, (cudaStream_t)stream);
    if (e != cudaSuccess) return cuda_fail(e, "tilize launch failed");
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return BUDA_SUCCESS;
}

int buda_queue_read(const void *queue_base, int src_df, int with_header, const buda_queue_geom *geom, uint32_t slots,
                    uint32_t first_slot, void *dst, int dst_is_host, int dst_df, const uint32_t shape[4],
                    const uint64_t strides_bytes[4], void *stream)
{
    if (slots == 0) return fail(BUDA_RUNTIME_ERROR, "a queue has at least one slot");
    const int64_t qb = buda_queue_bytes(geom, src_df, with_header, slots);
    if (qb < 0) return fail(BUDA_RUNTIME_ERROR, "invalid queue geometry or format");
    if (dst_is_host)
        return host_pipeline(1, dst, dst_df, shape, strides_bytes, geom, src_df, with_header, queue_base, (uint64_t)qb, 1, slots,
                             first_slot);
    const void *srcs[1] = {queue_base};
    void *dsts[1] = {dst};
    return untilize_device(1, srcs, src_df, with_header, geom, dsts, dst_df, shape, strides_bytes, (cudaStream_t)stream, -1,
                           slots, first_slot);
}

int buda_queue_read_stacked(const void *queue_base, int src_df, int with_header, const buda_queue_geom *geom, uint32_t slots,
                            uint32_t first_slot, uint32_t entries, uint32_t hstack, uint32_t vstack, int stack_row_major, void *dst,
                            int dst_df, void *stream)
{
    DevCtx *ctx;
    if (int rc = get_ctx(&ctx)) return rc;
    if (!queue_base || !dst || !geom) return fail(BUDA_RUNTIME_ERROR, "null argument");
    if (slots == 0 || entries == 0) return fail(BUDA_RUNTIME_ERROR, "a queue has at least one slot and a read at least one entry");
    if (hstack == 0 || vstack == 0 || geom->t % (hstack * vstack))
        return fail(BUDA_RUNTIME_ERROR, "t = %u is not a multiple of hstack %u x vstack %u", geom->t, hstack, vstack);
    int mant, es;
    if (int rc = classify(dst_df, src_df, mant, es, true)) return rc;
    const uint32_t R = geom->grid_r * geom->mblock_m * geom->ublock_rt * 32u, C = geom->grid_c * geom->mblock_n * geom->ublock_ct * 32u;
    const uint64_t out_row = (uint64_t)C * hstack * es;                 // bytes of one row of the stacked result
    const uint64_t out_plane = (uint64_t)R * vstack * out_row;          // one [R*v, C*h] slice
    const uint32_t shape[4] = {entries, geom->t, R, C};
    const uint64_t strides[4] = {(uint64_t)(geom->t / (hstack * vstack)) * out_plane, 0, out_row, (uint64_t)es};
    TileJob job;
    if (int rc = make_job(shape, strides, geom, src_df, with_header, 1, job, slots, first_slot)) return rc;
    // slice z of an entry sits at grid position (vv, hh) of output slice zo
    if (stack_row_major) {  // z = (zo * v + vv) * h + hh
        job.zn1 = hstack; job.stride_z = (uint64_t)C * es;
        job.zn2 = vstack; job.stride_z_mid = (uint64_t)R * out_row;
    } else {                // z = (zo * h + hh) * v + vv
        job.zn1 = vstack; job.stride_z = (uint64_t)R * out_row;
        job.zn2 = hstack; job.stride_z_mid = (uint64_t)C * es;
    }
    job.stride_z_out = out_plane;
    if (!aligned16((uint64_t)queue_base)) return fail(BUDA_RUNTIME_ERROR, "queue image pointers must be 16-byte aligned");
    PtrTable pt;
    memset(&pt, 0, sizeof(pt));
    pt.src[0] = (const uint8_t *)queue_base;
    pt.dst[0] = (uint8_t *)dst;
    int path, vec_ok;
    pick_path(job, pt, 1, es, path, vec_ok, mant);
    if (((job.stride_z | job.stride_z_mid | job.stride_z_out) & 15u) != 0) path = 1, vec_ok = 0;
    return launch_uniform(1, ctx, job, pt, 1, mant, es, half_side(dst_df, src_df), path, vec_ok, (cudaStream_t)stream);
}

int buda_tilize_pack_jobs(int n, const buda_tensor_job *jobs_host, int src_df, int dst_df, int with_header, void *stream)
{
    return jobs_device(0, n, jobs_host, src_df, dst_df, with_header, (cudaStream_t)stream);
}

int buda_unpack_untilize_jobs(int n, const buda_tensor_job *jobs_host, int src_df, int with_header, int dst_df, void *stream)
{
    return jobs_device(1, n, jobs_host, dst_df, src_df, with_header, (cudaStream_t)stream);
}

static int host_jobs(int direction, int n, const buda_tensor_job *jobs, int rm_df, int q_df, int with_header, int image_on_device)
{
    if (n <= 0) return BUDA_SUCCESS;
    if (!jobs) return fail(BUDA_RUNTIME_ERROR, "null job table");
    std::vector<HostItem> items((size_t)n);
    for (int i = 0; i < n; i++) {
        if (jobs[i].band_count != 0) return fail(BUDA_RUNTIME_ERROR, "job %d: the host-buffer entry points convert whole tensors", i);
        items[(size_t)i] = HostItem{jobs[i].tensor, jobs[i].image, jobs[i].shape, jobs[i].strides_bytes, &jobs[i].geom,
                                    jobs[i].image_bytes, image_on_device ? jobs[i].slots : 0u, image_on_device ? jobs[i].first_slot : 0u};
    }
    return host_pipeline_items(direction, n, items.data(), rm_df, q_df, with_header, image_on_device ? 1 : 0);
}

int buda_tilize_pack_host_jobs(int n, const buda_tensor_job *jobs_host, int src_df, int dst_df, int with_header, int image_on_device,
                               void *stream)
{
    (void)stream;
    return host_jobs(0, n, jobs_host, src_df, dst_df, with_header, image_on_device);
}

int buda_unpack_untilize_host_jobs(int n, const buda_tensor_job *jobs_host, int src_df, int with_header, int dst_df,
                                   int image_on_device, void *stream)
{
    (void)stream;
    return host_jobs(1, n, jobs_host, dst_df, src_df, with_header, image_on_device);
}

int buda_set_bfp_policy(const buda_bfp_policy *policy)
{
    buda_bfp_policy pub = {0, 0, {0, 1, 2, 3}, 0, 0};
    if (policy) pub = *policy;
    if (pub.rounding > 2 || pub.overflow > 1 || pub.exponent_order > 1 || pub.datum_order > 1)
        return fail(BUDA_RUNTIME_ERROR, "unknown block-float policy value");
    BfpPolicy p = default_policy();
    bool seen[4] = {false, false, false, false};
    for (int pos = 0; pos < 4; pos++) {
        const unsigned f = pub.face_order[pos];
        if (f > 3 || seen[f]) return fail(BUDA_RUNTIME_ERROR, "face_order must be a permutation of 0, 1, 2, 3");
        seen[f] = true;
        p.face_at[pos] = (uint8_t)f;
        p.face_pos[f] = (uint8_t)pos;
    }
    p.rmode = (uint8_t)pub.rounding;
    p.bump = (uint8_t)pub.overflow;
    p.exp_be = (uint8_t)pub.exponent_order;
    p.datum_be = (uint8_t)pub.datum_order;
    std::lock_guard<std::mutex> lock(g_policy_mu);
    g_policy = p;
    g_policy_public = pub;
    return BUDA_SUCCESS;
}

int buda_get_bfp_policy(buda_bfp_policy *policy_out)
{
    if (!policy_out) return fail(BUDA_RUNTIME_ERROR, "null argument");
    std::lock_guard<std::mutex> lock(g_policy_mu);
    *policy_out = g_policy_public;
    return BUDA_SUCCESS;
}

int buda_malloc(void **ptr, uint64_t bytes)
{
    DevCtx *ctx;
    if (int rc = get_ctx(&ctx)) return rc;
    if (!ptr) return fail(BUDA_RUNTIME_ERROR, "null argument");
    cudaError_t e = cudaMalloc(ptr, bytes ? bytes : 1);
    return e == cudaSuccess ? BUDA_SUCCESS : cuda_fail(e, "device allocation");
}

int buda_free(void *ptr)
{
    cudaError_t e = cudaFree(ptr);
    return e == cudaSuccess ? BUDA_SUCCESS : cuda_fail(e, "device free");
}

int buda_host_alloc(void **ptr, uint64_t bytes)
{
    DevCtx *ctx;
    if (int rc = get_ctx(&ctx)) return rc;
    if (!ptr) return fail(BUDA_RUNTIME_ERROR, "null argument");
    cudaError_t e = cudaMallocHost(ptr, bytes ? bytes : 1);
    return e == cudaSuccess ? BUDA_SUCCESS : cuda_fail(e, "pinned host allocation");
}

int buda_host_free(void *ptr)
{
    cudaError_t e = cudaFreeHost(ptr);
    return e == cudaSuccess ? BUDA_SUCCESS : cuda_fail(e, "pinned host free");
}

int buda_memcpy(void *dst, const void *src, uint64_t bytes, int kind, void *stream)
{
    DevCtx *ctx;
    if (int rc = get_ctx(&ctx)) return rc;
    cudaMemcpyKind k = kind == 0 ? cudaMemcpyHostToDevice : kind == 1 ? cudaMemcpyDeviceToHost : cudaMemcpyDeviceToDevice;
    cudaError_t e = cudaMemcpyAsync(dst, src, bytes, k, (cudaStream_t)stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize((cudaStream_t)stream);
    return e == cudaSuccess ? BUDA_SUCCESS : cuda_fail(e, "memcpy");
}

int buda_stream_synchronize(void *stream)
{
    cudaError_t e = cudaStreamSynchronize((cudaStream_t)stream);
    return e == cudaSuccess ? BUDA_SUCCESS : cuda_fail(e, "stream synchronize");
}

int buda_pointer_is_device(const void *ptr, int *is_device, int *device_ordinal)
{
    cudaPointerAttributes a;
    cudaError_t e = cudaPointerGetAttributes(&a, ptr);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return cuda_fail(e, "pointer query");
    }
    if (is_device) *is_device = (a.type == cudaMemoryTypeDevice || a.type == cudaMemoryTypeManaged) ? 1 : 0;
    if (device_ordinal) *device_ordinal = a.device;
    return BUDA_SUCCESS;
}

int buda_get_device(int *ordinal)
{
    cudaError_t e = cudaGetDevice(ordinal);
    return e == cudaSuccess ? BUDA_SUCCESS : cuda_fail(e, "no usable CUDA device (this library has no CPU path)");
}

int buda_set_device(int ordinal)
{
    cudaError_t e = cudaSetDevice(ordinal);
    return e == cudaSuccess ? BUDA_SUCCESS : cuda_fail(e, "set device");
}

int buda_device_count(int *count)
{
    cudaError_t e = cudaGetDeviceCount(count);
    if (e != cudaSuccess) {
        if (count) *count = 0;
        cudaGetLastError();
        return cuda_fail(e, "no usable CUDA device (this library has no CPU path)");
    }
    return BUDA_SUCCESS;
}

static int check_quant_args(const void *x, int64_t n, const void *scale, int64_t scale_len, int64_t inner, const void *out)
{
    if (n < 0) return fail(BUDA_RUNTIME_ERROR, "negative element count");
    if (n == 0) return BUDA_SUCCESS;
    if (!x || !scale || !out) return fail(BUDA_RUNTIME_ERROR, "null tensor pointer");
    if (scale_len < 1 || inner < 1) return fail(BUDA_RUNTIME_ERROR, "scale_len and inner must be >= 1");
    return BUDA_SUCCESS;
}

int buda_quantize(const float *x, int64_t n, const float *scale, int64_t scale_len, int64_t inner, float zero_point,
                  int mode, float lo, float hi, int8_t *out, void *stream)
{
    DevCtx *ctx;
    if (int rc = get_ctx(&ctx)) return rc;
    if (int rc = check_quant_args(x, n, scale, scale_len, inner, out)) return rc;
    if (n == 0) return BUDA_SUCCESS;
    if (mode != 0 && mode != 1) return fail(BUDA_RUNTIME_ERROR, "quantize mode must be 0 or 1");
    cudaError_t e = launch_quantize(x, n, scale, scale_len, inner, zero_point, mode, lo, hi, out, ctx->sm_count,
                                    (cudaStream_t)stream);
    if (e != cudaSuccess) return cuda_fail(e, "quantize launch failed");
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return BUDA_SUCCESS;
}

int buda_dequantize(const int8_t *x, int64_t n, const float *scale, int64_t scale_len, int64_t inner, float zero_point,
                    float *out, void *stream)
{
    DevCtx *ctx;
    if (int rc = get_ctx(&ctx)) return rc;
    if (int rc = check_quant_args(x, n, scale, scale_len, inner, out)) return rc;
    if (n == 0) return BUDA_SUCCESS;
    cudaError_t e = launch_dequantize(x, n, scale, scale_len, inner, zero_point, out, ctx->sm_count, (cudaStream_t)stream);
    if (e != cudaSuccess) return cuda_fail(e, "dequantize launch failed");
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return BUDA_SUCCESS;
}

int buda_requantize(const int32_t *x, int64_t n, const float *inp_scale, const float *out_scale, int64_t scale_len,
                    int64_t inner, float zero_point, int mode, float lo, float hi, int8_t *out, void *stream)
{
    DevCtx *ctx;
    if (int rc = get_ctx(&ctx)) return rc;
    if (int rc = check_quant_args(x, n, inp_scale, scale_len, inner, out)) return rc;
    if (n == 0) return BUDA_SUCCESS;
    if (mode != 0 && mode != 1) return fail(BUDA_RUNTIME_ERROR, "requantize mode must be 0 or 1");
    if (mode == 0 && !out_scale) return fail(BUDA_RUNTIME_ERROR, "Requantize needs out_scale");
    cudaError_t e = launch_requantize(x, n, inp_scale, out_scale, scale_len, inner, zero_point, mode, lo, hi, out,
                                      ctx->sm_count, (cudaStream_t)stream);
    if (e != cudaSuccess) return cuda_fail(e, "requantize launch failed");
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return BUDA_SUCCESS;
}

static int gemm_scatter_impl(const void *A, int64_t M, int64_t K, int64_t lda, const void *W_tiles, int64_t N, void *const *C_dsts,
                             int n_dst, void *C_mc, int64_t ldc, void *stream);

int buda_bfp8b_gemm_scatter(const void *A, int64_t M, int64_t K, int64_t lda, const void *W_tiles, int64_t N, void *const *C_dsts,
                            int n_dst, int64_t ldc, void *stream)
{
    return gemm_scatter_impl(A, M, K, lda, W_tiles, N, C_dsts, n_dst, nullptr, ldc, stream);
}

int buda_bfp8b_gemm_multicast(const void *A, int64_t M, int64_t K, int64_t lda, const void *W_tiles, int64_t N, void *C_local,
                              void *C_multicast, int64_t ldc, void *stream)
{
    if (!C_local || !C_multicast) return fail(BUDA_RUNTIME_ERROR, "null matrix pointer");
    void *dst[1] = {C_local};
    return gemm_scatter_impl(A, M, K, lda, W_tiles, N, dst, 1, C_multicast, ldc, stream);
}

static int gemm_scatter_impl(const void *A, int64_t M, int64_t K, int64_t lda, const void *W_tiles, int64_t N, void *const *C_dsts,
                             int n_dst, void *C_mc, int64_t ldc, void *stream)
{
    DevCtx *ctx;
    if (int rc = get_ctx(&ctx)) return rc;
    if (!A || !W_tiles || !C_dsts) return fail(BUDA_RUNTIME_ERROR, "null matrix pointer");
    {
        const BfpPolicy pol = current_policy();
        BfpPolicy layout = pol;
        layout.rmode = layout.bump = 0;   // rounding and overflow do not change how bytes are read back
        if (!policy_is_default(layout))
            return fail(BUDA_RUNTIME_ERROR, "the matmul reads weight images in the default byte layout; the current block-float policy changes it");
    }
    for (int d = 0; d < n_dst && d < 8; d++)
        if (!C_dsts[d]) return fail(BUDA_RUNTIME_ERROR, "null destination %d", d);
    char msg[256] = "";
    cudaError_t e = launch_bfp8b_gemm(A, M, K, lda, W_tiles, N, C_dsts, n_dst, C_mc, ldc, ctx->sm_count, (cudaStream_t)stream,
                                      ctx->status, msg, sizeof(msg));
    if (e != cudaSuccess) return msg[0] ? fail(BUDA_RUNTIME_ERROR, "%s", msg) : cuda_fail(e, "gemm launch failed");
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return BUDA_SUCCESS;
}

int buda_bfp8b_gemm(const void *A, int64_t M, int64_t K, int64_t lda, const void *W_tiles, int64_t N, void *C, int64_t ldc,
                    void *stream)
{
    if (!C) return fail(BUDA_RUNTIME_ERROR, "null matrix pointer");
    void *dst[1] = {C};
    return buda_bfp8b_gemm_scatter(A, M, K, lda, W_tiles, N, dst, 1, ldc, stream);
}

int buda_i8_gemm(const void *A, int64_t M, int64_t K, int64_t lda, const void *W_tiles, int64_t N, const float *scale,
                 int64_t scale_len, float zero_point, int out_mode, void *C, int64_t ldc, void *stream)
{
    DevCtx *ctx;
    if (int rc = get_ctx(&ctx)) return rc;
    if (!A || !W_tiles || !C) return fail(BUDA_RUNTIME_ERROR, "null matrix pointer");
    if (current_policy().face_pos[1] != 1 || current_policy().face_pos[2] != 2)
        return fail(BUDA_RUNTIME_ERROR, "the matmul reads weight images in the default face order; the current policy changes it");
    char msg[256] = "";
    cudaError_t e = launch_i8_gemm(A, M, K, lda, W_tiles, N, scale, scale_len, zero_point, out_mode, C, ldc, ctx->sm_count,
                                   (cudaStream_t)stream, ctx->status, msg, sizeof(msg));
    if (e != cudaSuccess) return msg[0] ? fail(BUDA_RUNTIME_ERROR, "%s", msg) : cuda_fail(e, "int8 gemm launch failed");
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return BUDA_SUCCESS;
}

int buda_prestride(const void *src, int elem_bytes, const uint32_t shape[4], const uint64_t strides_bytes[4], int stride,
                   const int *xy_offsets, int n_offsets, void *dst, uint32_t dst_rows, uint32_t dst_cols, void *stream)
{
    DevCtx *ctx;
    if (int rc = get_ctx(&ctx)) return rc;
    if (!src || !dst || !shape || !strides_bytes || !xy_offsets) return fail(BUDA_RUNTIME_ERROR, "null argument");
    if (elem_bytes != 1 && elem_bytes != 2 && elem_bytes != 4) return fail(BUDA_RUNTIME_ERROR, "element size %d is not 1, 2 or 4", elem_bytes);
    if (stride < 1 || n_offsets < 1 || n_offsets > 64) return fail(BUDA_RUNTIME_ERROR, "stride %d with %d offsets is not supported", stride, n_offsets);
    for (int k = 0; k < n_offsets; k++)
        if (xy_offsets[2 * k] < 0 || xy_offsets[2 * k] >= stride || xy_offsets[2 * k + 1] < 0 || xy_offsets[2 * k + 1] >= stride)
            return fail(BUDA_RUNTIME_ERROR, "offset %d = (%d, %d) lies outside the %dx%d stride window", k, xy_offsets[2 * k],
                        xy_offsets[2 * k + 1], stride, stride);
    if (strides_bytes[3] != (uint64_t)elem_bytes) return fail(BUDA_RUNTIME_ERROR, "innermost stride must equal the element size");
    const uint64_t hs = (shape[2] + (uint32_t)stride - 1) / (uint32_t)stride, ws = (shape[3] + (uint32_t)stride - 1) / (uint32_t)stride;
    if ((uint64_t)n_offsets * shape[1] > dst_rows || hs * ws > dst_cols)
        return fail(BUDA_RUNTIME_ERROR, "prestrided tensor [%llu x %llu] does not fit the destination [%u x %u]",
                    (unsigned long long)n_offsets * shape[1], (unsigned long long)(hs * ws), dst_rows, dst_cols);
    cudaError_t e = launch_prestride(src, elem_bytes, shape, strides_bytes, stride, xy_offsets, n_offsets, dst, dst_rows, dst_cols,
                                     ctx->sm_count, (cudaStream_t)stream);
    if (e != cudaSuccess) return cuda_fail(e, "prestride launch failed");
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return BUDA_SUCCESS;
}

int buda_selftest_bounded_wait(uint32_t limit_ms, void *stream)
{
    DevCtx *ctx;
    if (int rc = get_ctx(&ctx)) return rc;
    if (limit_ms < 1 || limit_ms > 1000) return fail(BUDA_RUNTIME_ERROR, "limit of %u ms is outside 1..1000", limit_ms);
    selftest_wait_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(ctx->status, (uint64_t)limit_ms * 1000000ull);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "self-test launch failed");
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return BUDA_SUCCESS;
}

int buda_gemm_select_kernel(int which) { return gemm_kernel_choice(which); }

int buda_ipc_export(const void *dev_ptr, unsigned char handle_out[64])
{
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    if (!dev_ptr || !handle_out) return fail(BUDA_RUNTIME_ERROR, "null argument");
    cudaIpcMemHandle_t h;
    cudaError_t e = cudaIpcGetMemHandle(&h, const_cast<void *>(dev_ptr));
    if (e != cudaSuccess) return cuda_fail(e, "cudaIpcGetMemHandle failed");
    memcpy(handle_out, &h, 64);
    return BUDA_SUCCESS;
}

int buda_ipc_open(const unsigned char handle[64], void **dev_ptr_out)
{
    if (!handle || !dev_ptr_out) return fail(BUDA_RUNTIME_ERROR, "null argument");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, 64);
    void *ptr = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) return cuda_fail(e, "cudaIpcOpenMemHandle failed");
    *dev_ptr_out = ptr;
    return BUDA_SUCCESS;
}

int buda_ipc_close(void *dev_ptr)
{
    if (!dev_ptr) return BUDA_SUCCESS;
    cudaError_t e = cudaIpcCloseMemHandle(dev_ptr);
    if (e != cudaSuccess) return cuda_fail(e, "cudaIpcCloseMemHandle failed");
    return BUDA_SUCCESS;
}

size_t buda_last_error(char *buf, size_t buf_len)
{
    const size_t n = strlen(t_err);
    if (buf && buf_len) {
        const size_t c = n < buf_len - 1 ? n : buf_len - 1;
        memcpy(buf, t_err, c);
        buf[c] = 0;
    }
    return n;
}

int buda_device_status(int *status_out)
{
    DevCtx *ctx;
    if (int rc = get_ctx(&ctx)) return rc;
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return cuda_fail(e, "device synchronize");
    unsigned int st = 0;
    e = cudaMemcpy(&st, ctx->status, sizeof(st), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return cuda_fail(e, "reading the device status word");
    if (status_out) *status_out = (int)st;
    if (st != 0) {
        unsigned int zero = 0;
        cudaMemcpy(ctx->status, &zero, sizeof(zero), cudaMemcpyHostToDevice);
        return fail(BUDA_TIMEOUT_ERROR, "a kernel gave up waiting (device status %u)", st);
    }
    return BUDA_SUCCESS;
}

uint64_t buda_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

const char *buda_version(void) { return "buda_cuda 0.1 sm_100a"; }

}  // extern "C"

// ------------------------------------------------------------------------------------------------
// Tilize + pack for callers that must not allocate.
//
// The host-buffer entry point above stages the tensor and its image in device buffers it gets from
// cudaMalloc.  Some hosts of this library cannot do that: a pusher thread that lives inside a
// training process whose own allocator has already claimed the device heap (a fresh cudaMalloc there
// fails or fragments the pool), or a feeder loop that cannot afford the device-wide synchronisation a
// cudaMalloc / cudaFree implies.  For them the staging area is a fixed array that is part of the
// library image: every GPU that loads the library carries these 8 MiB until the process exits.
// ------------------------------------------------------------------------------------------------
namespace {

constexpr uint64_t kNoAllocScratchBytes = 8ull << 20;

// File-scope device array.  In host code this name is only a stand-in for the symbol, never a device
// address: the address each device gives it is looked up with cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

struct NoAllocDev {
    std::once_flag once;
    cudaError_t err = cudaSuccess;
    unsigned char *base = nullptr;  // device address of g_noalloc_scratch on this device
    std::mutex mu;                  // one call at a time per device: the array is shared
};
NoAllocDev g_noalloc[kMaxDevices];

}  // namespace

extern "C" int buda_tilize_pack_host_noalloc(const void *src_host, int src_df, const uint32_t shape[4],
                                             const uint64_t strides_bytes[4], const buda_queue_geom *geom, int dst_df,
                                             int with_header, void *dst_host, uint64_t dst_bytes, void *stream)
{
    DevCtx *ctx;
    if (int rc = get_ctx(&ctx)) return rc;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return fail(BUDA_RUNTIME_ERROR, "no current device");
    NoAllocDev &na = g_noalloc[dev];
    // set-up, once per device, with that device current (this is the first call's extra work)
    std::call_once(na.once, [&]() { na.err = cudaGetSymbolAddress((void **)&na.base, g_noalloc_scratch); });
    if (na.err != cudaSuccess || na.base == nullptr) return cuda_fail(na.err, "looking up the static scratch array");

    if (!src_host || !dst_host || !shape || !strides_bytes || !geom) return fail(BUDA_RUNTIME_ERROR, "null argument");
    int mant, es;
    if (int rc = classify(src_df, dst_df, mant, es)) return rc;
    TileJob job;
    if (int rc = make_job(shape, strides_bytes, geom, dst_df, with_header, 1, job)) return rc;
    if (strides_bytes[3] != (uint64_t)es) return fail(BUDA_RUNTIME_ERROR, "innermost stride must equal the element size");
    const uint64_t row_bytes = (uint64_t)shape[3] * es;
    if (strides_bytes[2] < row_bytes) return fail(BUDA_RUNTIME_ERROR, "row stride smaller than a row");
    const uint64_t src_bytes = (uint64_t)shape[0] * shape[1] * shape[2] * row_bytes;
    const uint64_t image_bytes = job.buf_bytes * geom->grid_r * geom->grid_c;
    const uint64_t image_off = (src_bytes + 255u) & ~255ull;
    if (image_off + image_bytes > kNoAllocScratchBytes)
        return fail(BUDA_RUNTIME_ERROR,
                    "tensor (%llu bytes) plus its image (%llu bytes) exceed the %llu-byte static scratch of the no-allocation "
                    "entry point; use buda_tilize_pack_host",
                    (unsigned long long)src_bytes, (unsigned long long)image_bytes, (unsigned long long)kNoAllocScratchBytes);
    if (dst_bytes < image_bytes)
        return fail(BUDA_RUNTIME_ERROR, "destination holds %llu bytes, the queue image needs %llu", (unsigned long long)dst_bytes,
                    (unsigned long long)image_bytes);

    std::lock_guard<std::mutex> lock(na.mu);
    cudaStream_t s = (cudaStream_t)stream;
    unsigned char *d_src = na.base, *d_img = na.base + image_off;
    const uint64_t dense[4] = {(uint64_t)shape[1] * shape[2] * row_bytes, (uint64_t)shape[2] * row_bytes, row_bytes, (uint64_t)es};
    cudaError_t e = cudaSuccess;
    for (uint32_t w = 0; w < shape[0] && e == cudaSuccess; w++) {
        for (uint32_t z = 0; z < shape[1] && e == cudaSuccess; z++) {
            const uint8_t *h = (const uint8_t *)src_host + w * strides_bytes[0] + z * strides_bytes[1];
            unsigned char *d = d_src + w * dense[0] + z * dense[1];
            e = (strides_bytes[2] == row_bytes)
                    ? cudaMemcpyAsync(d, h, (uint64_t)shape[2] * row_bytes, cudaMemcpyHostToDevice, s)
                    : cudaMemcpy2DAsync(d, row_bytes, h, strides_bytes[2], row_bytes, shape[2], cudaMemcpyHostToDevice, s);
        }
    }
    // From here on work may be in flight on the shared array: every way out waits for the stream first, so the next
    // caller (possibly on another stream) never meets it.
    if (e != cudaSuccess) {
        (void)cudaStreamSynchronize(s);
        return cuda_fail(e, "host to device copy");
    }
    // the kernel writes every byte of every tile record (header included), so nothing left in the
    // array by an earlier call can show through and nothing has to be cleared first
    const void *srcs[1] = {d_src};
    void *dsts[1] = {d_img};
    if (int rc = tilize_device(1, srcs, src_df, shape, dense, geom, dst_df, with_header, dsts, image_bytes, s, -1)) {
        (void)cudaStreamSynchronize(s);
        return rc;
    }
    e = cudaMemcpyAsync(dst_host, d_img, image_bytes, cudaMemcpyDeviceToHost, s);
    const cudaError_t es2 = cudaStreamSynchronize(s);
    if (e != cudaSuccess) return cuda_fail(e, "device to host copy");
    if (es2 != cudaSuccess) return cuda_fail(es2, "synchronize");
    return status_after_sync(ctx);
}
