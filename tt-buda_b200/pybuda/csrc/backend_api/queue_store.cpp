// Device-resident queues behind the converter entry points (see backend.hpp).
#include <algorithm>
#include <chrono>
#include <condition_variable>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <map>
#include <memory>
#include <mutex>
#include <stdexcept>
#include <unordered_map>

#include "backend_api/backend.hpp"
#include "buda_cuda.h"

namespace tt::backend
{

namespace
{

thread_local std::string t_last_error;

DEVICE_STATUS_CODE fail(DEVICE_STATUS_CODE code, const std::string &msg)
{
    t_last_error = msg;
    return code;
}

std::string cabi_error()
{
    char buf[512];
    buda_last_error(buf, sizeof(buf));
    return buf;
}

DEVICE_STATUS_CODE from_cabi(int rc, const char *what)
{
    if (rc == BUDA_SUCCESS)
        return DEVICE_STATUS_CODE::Success;
    return fail(rc == BUDA_TIMEOUT_ERROR ? DEVICE_STATUS_CODE::TimeoutError : DEVICE_STATUS_CODE::RuntimeError,
                std::string(what) + ": " + cabi_error());
}

buda_queue_geom geom_of(const tt_dram_io_desc &q)
{
    buda_queue_geom g = {};
    g.grid_r = q.bufq_grid_dim_r;
    g.grid_c = q.bufq_grid_dim_c;
    g.mblock_m = q.mblock_m;
    g.mblock_n = q.mblock_n;
    g.ublock_rt = q.ublock_rt;
    g.ublock_ct = q.ublock_ct;
    g.t = q.t;
    g.ublock_order = q.ublock_order;
    g.tile_height = q.tile_height;
    return g;
}

bool on_device(const void *p)
{
    int is_dev = 0, ord = 0;
    if (buda_pointer_is_device(p, &is_dev, &ord) != BUDA_SUCCESS)
        return false;  // plain host memory the driver does not know
    return is_dev != 0;
}

std::array<std::uint64_t, 4> strides64(const tt_PytorchTensorDesc &d)
{
    return {d.strides[0], d.strides[1], d.strides[2], d.strides[3]};
}

// A tensor covers the queue when its last two dims are the queue's rows and columns and its z is t.
std::string check_tensor_fits(const tt_dram_io_desc &q, const tt_PytorchTensorDesc &d)
{
    if (q.tile_width != 32 || q.tile_height == 0 || q.tile_height > 32 || (q.tile_height & (q.tile_height - 1)))
        return "tiles are 32 columns wide and 32, 16, 8, 4, 2 or 1 rows high";
    if (q.layout != IO_LAYOUT::Tilized)
        return "only tilized queues are supported";
    if (q.hstack_factor != 1 || q.vstack_factor != 1)
        return "hstack / vstack host transforms are not supported";
    if (d.ptr == nullptr)
        return "tensor descriptor has a null pointer";
    if (d.shape[1] != q.t || d.shape[2] != q.rows() || d.shape[3] != q.cols())
    {
        char b[256];
        snprintf(b, sizeof(b), "tensor [%u,%u,%u,%u] does not match queue '%s' entries [t=%u, %u x %u]", d.shape[0],
                 d.shape[1], d.shape[2], d.shape[3], q.queue_name.c_str(), q.t, q.rows(), q.cols());
        return b;
    }
    return "";
}

// ------------------------------------------------------------------------------------------------
// queue registry
// ------------------------------------------------------------------------------------------------
struct QueueState
{
    std::mutex mu;
    std::condition_variable cv;
    int device = 0;
    void *base = nullptr;
    std::uint64_t bytes = 0;
    std::uint32_t slots = 0;
    std::uint32_t wr = 0, rd = 0, occupancy = 0;
    tt_dram_io_desc desc;
};

std::mutex g_registry_mu;
std::unordered_map<std::string, std::shared_ptr<QueueState>> g_queues;

bool same_geometry(const tt_dram_io_desc &a, const tt_dram_io_desc &b)
{
    return a.bufq_grid_dim_r == b.bufq_grid_dim_r && a.bufq_grid_dim_c == b.bufq_grid_dim_c && a.mblock_m == b.mblock_m &&
           a.mblock_n == b.mblock_n && a.ublock_rt == b.ublock_rt && a.ublock_ct == b.ublock_ct && a.t == b.t &&
           a.ublock_order == b.ublock_order && a.bufq_target_format == b.bufq_target_format && a.tile_header == b.tile_header &&
           a.tile_height == b.tile_height &&
           a.bufq_num_slots == b.bufq_num_slots;
}

// Finds the queue, creating its device memory on first use (create == true).
DEVICE_STATUS_CODE get_queue(const tt_dram_io_desc &q, bool create, std::shared_ptr<QueueState> &out)
{
    std::lock_guard<std::mutex> lock(g_registry_mu);
    auto it = g_queues.find(q.key());
    if (it != g_queues.end())
    {
        if (!same_geometry(it->second->desc, q))
            return fail(DEVICE_STATUS_CODE::RuntimeError,
                        "queue '" + q.queue_name + "' already exists with a different geometry or format");
        out = it->second;
        return DEVICE_STATUS_CODE::Success;
    }
    if (!create)
        return fail(DEVICE_STATUS_CODE::RuntimeError, "queue '" + q.queue_name + "' has never been written");
    auto st = std::make_shared<QueueState>();
    const buda_queue_geom g = geom_of(q);
    st->slots = std::max<std::uint32_t>(1, q.bufq_num_slots);
    const std::int64_t bytes = buda_queue_bytes(&g, (int)q.bufq_target_format, q.tile_header ? 1 : 0, st->slots);
    if (bytes <= 0)
        return fail(DEVICE_STATUS_CODE::RuntimeError, "queue '" + q.queue_name + "': invalid geometry or data format");
    if (buda_get_device(&st->device) != BUDA_SUCCESS)
        return fail(DEVICE_STATUS_CODE::RuntimeError, cabi_error());
    if (buda_malloc(&st->base, (std::uint64_t)bytes) != BUDA_SUCCESS)
        return fail(DEVICE_STATUS_CODE::RuntimeError, "queue '" + q.queue_name + "': " + cabi_error());
    st->bytes = (std::uint64_t)bytes;
    st->desc = q;
    g_queues[q.key()] = st;
    out = st;
    return DEVICE_STATUS_CODE::Success;
}

// ------------------------------------------------------------------------------------------------
// backend-owned host memory (results of get_output / tilize_tensor / debinarize_tensor)
// ------------------------------------------------------------------------------------------------
std::mutex g_host_mu;
std::unordered_map<const void *, std::uint64_t> g_host_live;           // ptr -> capacity
std::multimap<std::uint64_t, void *> g_host_pool;                      // capacity -> free pinned block
std::uint64_t g_host_pool_bytes = 0;
constexpr std::uint64_t kHostPoolCap = 1ull << 30;

void *host_acquire(std::uint64_t bytes)
{
    {
        std::lock_guard<std::mutex> lock(g_host_mu);
        auto it = g_host_pool.lower_bound(bytes);
        if (it != g_host_pool.end() && it->first <= bytes + bytes / 4 + 4096)
        {
            void *p = it->second;
            g_host_live[p] = it->first;
            g_host_pool_bytes -= it->first;
            g_host_pool.erase(it);
            return p;
        }
    }
    void *p = nullptr;
    if (buda_host_alloc(&p, bytes) != BUDA_SUCCESS)
        return nullptr;
    std::lock_guard<std::mutex> lock(g_host_mu);
    g_host_live[p] = bytes;
    return p;
}

bool host_release(const void *p)
{
    std::uint64_t cap = 0;
    {
        std::lock_guard<std::mutex> lock(g_host_mu);
        auto it = g_host_live.find(p);
        if (it == g_host_live.end())
            return false;
        cap = it->second;
        g_host_live.erase(it);
        if (g_host_pool_bytes + cap <= kHostPoolCap)
        {
            g_host_pool.emplace(cap, const_cast<void *>(p));
            g_host_pool_bytes += cap;
            return true;
        }
    }
    buda_host_free(const_cast<void *>(p));
    return true;
}

DataFormat default_output_format(DataFormat queue_df)
{
    switch (queue_df)
    {
        case DataFormat::Bfp8_b:
        case DataFormat::Bfp4_b:
        case DataFormat::Bfp2_b: return DataFormat::Float16_b;  // what the Python side maps these queues to
        case DataFormat::Int32: return DataFormat::RawUInt32;
        default: return queue_df;
    }
}

}  // namespace

std::string last_error() { return t_last_error; }

tt_dram_io_desc make_queue_desc(const std::string &name, std::array<std::uint32_t, 4> shape, DataFormat df,
                                std::pair<std::uint32_t, std::uint32_t> grid, std::pair<std::uint32_t, std::uint32_t> ublock,
                                std::uint32_t ublock_order, std::uint32_t num_slots, IO_TYPE io_type, bool tile_header,
                                std::uint32_t tile_height)
{
    if (tile_height == 0 || tile_height > 32 || (tile_height & (tile_height - 1)))
        throw std::runtime_error("tile_height must be 32, 16, 8, 4, 2 or 1");
    if (shape[2] % tile_height || shape[3] % 32)
        throw std::runtime_error("queue rows and columns must be multiples of the tile (tile_height x 32)");
    const std::uint32_t rt = shape[2] / tile_height, ct = shape[3] / 32;
    if (!grid.first || !grid.second || !ublock.first || !ublock.second || rt % (grid.first * ublock.first) ||
        ct % (grid.second * ublock.second))
        throw std::runtime_error("grid x ublock does not divide the tensor's tile counts");
    if (tile_size_bytes(df, tile_header) == 0xbadface)
        throw std::runtime_error("invalid data format for a queue");
    tt_dram_io_desc q;
    q.queue_name = name;
    q.bufq_grid_dim_r = grid.first;
    q.bufq_grid_dim_c = grid.second;
    q.ublock_rt = ublock.first;
    q.ublock_ct = ublock.second;
    q.mblock_m = rt / (grid.first * ublock.first);
    q.mblock_n = ct / (grid.second * ublock.second);
    q.t = shape[1];
    q.input_count = shape[0];
    q.bufq_num_slots = num_slots ? num_slots : std::max<std::uint32_t>(1, 2 * shape[0]);
    q.bufq_target_format = df;
    q.ublock_order = ublock_order;
    q.tile_header = tile_header;
    q.tile_height = tile_height;
    q.io_type = io_type;
    q.bufq_entry_size = (std::uint32_t)(q.tiles_per_entry() * tile_size_bytes(df, tile_header));
    return q;
}

// ------------------------------------------------------------------------------------------------
// push
// ------------------------------------------------------------------------------------------------
namespace
{
// Device memory freed when the scope ends.
struct DeviceScratch
{
    void *p = nullptr;
    ~DeviceScratch()
    {
        if (p)
            buda_free(p);
    }
};

// Slots of a queue held for one push: taken under the queue's lock (a ring queue waits, up to its timeout, until the
// entries fit; a RandomAccess queue writes where ram_ptr says), released by commit() once the data is in place.
struct SlotClaim
{
    std::shared_ptr<QueueState> st;
    std::unique_lock<std::mutex> lock;
    std::uint32_t first_slot = 0, entries = 0;
    bool ring = false;

    DEVICE_STATUS_CODE take(const tt_dram_io_desc &q, std::uint32_t n, int timeout_in_seconds, int ram_ptr)
    {
        if (auto rc = get_queue(q, true, st); rc != DEVICE_STATUS_CODE::Success)
            return rc;
        if (n > st->slots)
            return fail(DEVICE_STATUS_CODE::RuntimeError, "push_input: more entries than the queue has slots");
        entries = n;
        ring = q.io_type != IO_TYPE::RandomAccess;
        lock = std::unique_lock<std::mutex>(st->mu);
        if (!ring)
        {
            if (ram_ptr < 0 || (std::uint32_t)ram_ptr + n > st->slots)
                return fail(DEVICE_STATUS_CODE::RuntimeError, "push_input: ram_ptr outside the queue");
            first_slot = (std::uint32_t)ram_ptr;
            return DEVICE_STATUS_CODE::Success;
        }
        const auto deadline = std::chrono::steady_clock::now() + std::chrono::seconds(std::max(0, timeout_in_seconds));
        if (!st->cv.wait_until(lock, deadline, [&] { return st->occupancy + n <= st->slots; }))
            return fail(DEVICE_STATUS_CODE::TimeoutError, "push_input: queue '" + q.queue_name + "' stayed full");
        first_slot = st->wr;
        return DEVICE_STATUS_CODE::Success;
    }

    void commit()
    {
        if (ring)
        {
            st->wr = (st->wr + entries) % st->slots;
            st->occupancy += entries;
        }
        else
        {
            st->occupancy = std::max(st->occupancy, first_slot + entries);
        }
        lock.unlock();
        st->cv.notify_all();
    }
};

std::string check_queue_tiles(const tt_dram_io_desc &q)
{
    if (q.tile_width != 32 || q.tile_height == 0 || q.tile_height > 32 || (q.tile_height & (q.tile_height - 1)))
        return "tiles are 32 columns wide and 32, 16, 8, 4, 2 or 1 rows high";
    if (q.layout != IO_LAYOUT::Tilized)
        return "only tilized queues are supported";
    if (q.hstack_factor != 1 || q.vstack_factor != 1)
        return "hstack / vstack host transforms are not supported";
    return "";
}

// The tensor on the device: itself when it already lives there, otherwise a scratch copy of its `bytes` bytes.
DEVICE_STATUS_CODE device_copy_of(const void *ptr, std::uint64_t bytes, DeviceScratch &scratch, const void *&dev)
{
    dev = ptr;
    if (on_device(ptr))
        return DEVICE_STATUS_CODE::Success;
    if (buda_malloc(&scratch.p, bytes) != BUDA_SUCCESS || buda_memcpy(scratch.p, ptr, bytes, 0, nullptr) != BUDA_SUCCESS)
        return fail(DEVICE_STATUS_CODE::RuntimeError, "push_input: " + cabi_error());
    dev = scratch.p;
    return DEVICE_STATUS_CODE::Success;
}

// bytes a strided [w,z,r,c] tensor spans from its first to its last element
std::uint64_t span_bytes(const tt_PytorchTensorDesc &t)
{
    std::uint64_t last = 0;
    for (int i = 0; i < 4; i++)
        last += (std::uint64_t)(t.shape[i] ? t.shape[i] - 1 : 0) * t.strides[i];
    return last + t.itemsize;
}
}  // namespace

// A tensor pushed through a source view (see buda_source_view): one kernel reads it the way the runtime transform
// would have rewritten it and writes the queue's tiles.  `tensor` describes the SOURCE (its own shape and strides).
DEVICE_STATUS_CODE push_input_view(const tt_dram_io_desc &q, const tt_PytorchTensorDesc &tensor, const tt_SourceView &view,
                                   const bool push_one, const int timeout_in_seconds, const int ram_ptr)
{
    if (const std::string why = check_queue_tiles(q); !why.empty())
        return fail(DEVICE_STATUS_CODE::RuntimeError, "push_input: " + why);
    if (q.tile_height != 32)
        return fail(DEVICE_STATUS_CODE::RuntimeError, "push_input: a transformed push needs 32-row tiles");
    if (tensor.ptr == nullptr)
        return fail(DEVICE_STATUS_CODE::RuntimeError, "push_input: tensor descriptor has a null pointer");
    const std::uint32_t entries = tensor.shape[0];
    if (push_one && entries != 1)
        return fail(DEVICE_STATUS_CODE::RuntimeError, "push_input: a single-entry push needs a tensor with w == 1");
    buda_source_view v = {};
    v.mode = (std::uint32_t)view.mode;
    const std::uint32_t es = tensor.itemsize;
    std::uint64_t strides[4] = {tensor.strides[0], tensor.strides[1], tensor.strides[2], es};
    switch (view.mode)
    {
        case SOURCE_VIEW::Padded:
            if (tensor.shape[1] != q.t || tensor.shape[2] > q.rows() || tensor.shape[3] > q.cols())
                return fail(DEVICE_STATUS_CODE::RuntimeError, "push_input: the tensor is larger than the queue's entries");
            if ((view.broadcast_rows && tensor.shape[2] != 1) || (view.broadcast_cols && tensor.shape[3] != 1))
                return fail(DEVICE_STATUS_CODE::RuntimeError, "push_input: only a dimension of size 1 is broadcast across its tile");
            v.valid_r = tensor.shape[2];
            v.valid_c = tensor.shape[3];
            v.bcast_r = view.broadcast_rows ? 1 : 0;
            v.bcast_c = view.broadcast_cols ? 1 : 0;
            break;
        case SOURCE_VIEW::EmbeddingIndex:
            v.emb_count = view.count;
            v.emb_group = view.group;
            strides[1] = strides[2] = 0;
            break;
        case SOURCE_VIEW::Prestride:
        {
            const Stride &sd = view.stride;
            if (sd.xy_offsets.empty() || sd.xy_offsets.size() > 64)
                return fail(DEVICE_STATUS_CODE::RuntimeError, "push_input: stride descriptor needs 1..64 xy offsets");
            v.ps_stride = (std::uint32_t)sd.stride;
            v.ps_z = tensor.shape[1];
            v.ps_h = tensor.shape[2];
            v.ps_w = tensor.shape[3];
            v.ps_n_offsets = (std::uint32_t)sd.xy_offsets.size();
            for (std::size_t k = 0; k < sd.xy_offsets.size(); k++)
            {
                v.ps_xy[2 * k] = sd.xy_offsets[k].first;
                v.ps_xy[2 * k + 1] = sd.xy_offsets[k].second;
            }
            break;
        }
        default: return fail(DEVICE_STATUS_CODE::RuntimeError, "push_input: unknown source view");
    }
    if (tensor.strides[3] != es)
        return fail(DEVICE_STATUS_CODE::RuntimeError, "push_input: a transformed push needs unit-stride rows");
    DeviceScratch staged;
    const void *src = nullptr;
    if (auto rc = device_copy_of(tensor.ptr, span_bytes(tensor), staged, src); rc != DEVICE_STATUS_CODE::Success)
        return rc;
    SlotClaim claim;
    if (auto rc = claim.take(q, entries, timeout_in_seconds, ram_ptr); rc != DEVICE_STATUS_CODE::Success)
        return rc;
    const buda_queue_geom g = geom_of(q);
    const std::uint32_t qshape[4] = {entries, q.t, q.rows(), q.cols()};
    int rc = buda_queue_write_view(src, (int)tensor.format, qshape, strides, &v, &g, (int)q.bufq_target_format, q.tile_header ? 1 : 0,
                                   claim.st->base, claim.st->bytes, claim.st->slots, claim.first_slot, nullptr);
    if (rc == BUDA_SUCCESS)
        rc = buda_stream_synchronize(nullptr);  // the caller (or the scratch copy) may go away as soon as we return
    if (rc != BUDA_SUCCESS)
        return from_cabi(rc, "push_input");
    claim.commit();
    return DEVICE_STATUS_CODE::Success;
}

DEVICE_STATUS_CODE push_input(const tt_dram_io_desc &q, const tt_PytorchTensorDesc &tensor, const bool push_one,
                              const int timeout_in_seconds, const int ram_ptr)
{
    if (q.s_descriptor.stride > 1)
    {
        // A queue whose descriptor carries a StrideDescriptor takes the ORIGINAL [w, z, H, W] activation and stores its
        // prestrided form (the reference's backend applies the descriptor inside push_input,
        // pybuda/pybuda/tensor.py:1415-1422): here the pack kernel gathers it while it tilizes.
        if (q.t != 1)
            return fail(DEVICE_STATUS_CODE::RuntimeError, "push_input: a prestriding queue has t == 1");
        tt_SourceView view;
        view.mode = SOURCE_VIEW::Prestride;
        view.stride = q.s_descriptor;
        return push_input_view(q, tensor, view, push_one, timeout_in_seconds, ram_ptr);
    }
    const std::string why = check_tensor_fits(q, tensor);
    if (!why.empty())
        return fail(DEVICE_STATUS_CODE::RuntimeError, "push_input: " + why);
    if (push_one && tensor.shape[0] != 1)
        return fail(DEVICE_STATUS_CODE::RuntimeError, "push_input: a single-entry push needs a tensor with w == 1");
    SlotClaim claim;
    if (auto rc = claim.take(q, tensor.shape[0], timeout_in_seconds, ram_ptr); rc != DEVICE_STATUS_CODE::Success)
        return rc;
    const buda_queue_geom g = geom_of(q);
    const bool host = !on_device(tensor.ptr);
    const auto st64 = strides64(tensor);
    int rc = buda_queue_write(tensor.ptr, host ? 1 : 0, (int)tensor.format, tensor.shape.data(), st64.data(), &g,
                              (int)q.bufq_target_format, q.tile_header ? 1 : 0, claim.st->base, claim.st->slots, claim.first_slot,
                              nullptr);
    if (rc == BUDA_SUCCESS && !host)
        rc = buda_stream_synchronize(nullptr);  // the caller may free the source as soon as we return
    if (rc != BUDA_SUCCESS)
        return from_cabi(rc, "push_input");
    claim.commit();
    return DEVICE_STATUS_CODE::Success;
}

// Many tensors to many queues in one go: what the reference's parameter loop does one push_input at a time
// (pybuda/pybuda/backend.py:458-517).  Slots are claimed in every queue first, then all conversions that share a
// (source format, queue format, header) combination run as ONE job table -- one launch for up to 192 device-resident
// tensors, or one copy / convert pipeline over all host tensors -- and the queues' pointers move when everything is in.
DEVICE_STATUS_CODE push_input_batch(const std::vector<tt_dram_io_desc> &queues, const std::vector<tt_PytorchTensorDesc> &tensors,
                                    const bool push_one, const int timeout_in_seconds, const std::vector<int> &ram_ptrs)
{
    const std::size_t n = queues.size();
    if (tensors.size() != n || (!ram_ptrs.empty() && ram_ptrs.size() != n))
        return fail(DEVICE_STATUS_CODE::RuntimeError, "push_input_batch: queues, tensors and ram pointers differ in number");
    std::vector<SlotClaim> claims(n);
    std::vector<buda_tensor_job> jobs(n);
    std::vector<bool> host(n);
    for (std::size_t i = 0; i < n; i++)
    {
        const tt_dram_io_desc &q = queues[i];
        const tt_PytorchTensorDesc &t = tensors[i];
        if (q.s_descriptor.stride > 1)
            return fail(DEVICE_STATUS_CODE::RuntimeError, "push_input_batch: prestriding queues take push_input");
        if (const std::string why = check_tensor_fits(q, t); !why.empty())
            return fail(DEVICE_STATUS_CODE::RuntimeError, "push_input_batch: " + why);
        if (push_one && t.shape[0] != 1)
            return fail(DEVICE_STATUS_CODE::RuntimeError, "push_input_batch: a single-entry push needs tensors with w == 1");
        for (std::size_t k = 0; k < i; k++)
            if (queues[k].key() == q.key())
                return fail(DEVICE_STATUS_CODE::RuntimeError, "push_input_batch: queue '" + q.queue_name + "' appears twice");
        if (auto rc = claims[i].take(q, t.shape[0], timeout_in_seconds, ram_ptrs.empty() ? -1 : ram_ptrs[i]);
            rc != DEVICE_STATUS_CODE::Success)
            return rc;   // claims taken so far release their locks as they go out of scope; nothing was written
        buda_tensor_job &j = jobs[i];
        memset(&j, 0, sizeof(j));
        j.tensor = t.ptr;
        j.image = claims[i].st->base;
        j.image_bytes = claims[i].st->bytes;
        for (int d = 0; d < 4; d++)
        {
            j.shape[d] = t.shape[d];
            j.strides_bytes[d] = t.strides[d];
        }
        j.geom = geom_of(q);
        j.slots = claims[i].st->slots;
        j.first_slot = claims[i].first_slot;
        host[i] = !on_device(t.ptr);
    }
    // one call per (source format, queue format, header, host / device) combination
    std::vector<bool> done(n, false);
    for (std::size_t i = 0; i < n; i++)
    {
        if (done[i])
            continue;
        std::vector<buda_tensor_job> group;
        for (std::size_t k = i; k < n; k++)
        {
            if (!done[k] && tensors[k].format == tensors[i].format && queues[k].bufq_target_format == queues[i].bufq_target_format &&
                queues[k].tile_header == queues[i].tile_header && host[k] == host[i])
            {
                group.push_back(jobs[k]);
                done[k] = true;
            }
        }
        const int src_df = (int)tensors[i].format, dst_df = (int)queues[i].bufq_target_format, hdr = queues[i].tile_header ? 1 : 0;
        int rc = host[i] ? buda_tilize_pack_host_jobs((int)group.size(), group.data(), src_df, dst_df, hdr, 1, nullptr)
                         : buda_tilize_pack_jobs((int)group.size(), group.data(), src_df, dst_df, hdr, nullptr);
        if (rc != BUDA_SUCCESS)
            return from_cabi(rc, "push_input_batch");
    }
    if (int rc = buda_stream_synchronize(nullptr); rc != BUDA_SUCCESS)   // the callers may free their tensors once we return
        return from_cabi(rc, "push_input_batch");
    for (auto &c : claims)
        c.commit();
    return DEVICE_STATUS_CODE::Success;
}

DEVICE_STATUS_CODE push_input(const tt_dram_io_desc &q, const tt_TilizedTensorDesc &tensor, const int timeout_in_seconds,
                              const int ram_ptr)
{
    if (tensor.ptr == nullptr)
        return fail(DEVICE_STATUS_CODE::RuntimeError, "push_input: tilized descriptor has a null pointer");
    if (tensor.format != q.bufq_target_format)
        return fail(DEVICE_STATUS_CODE::RuntimeError, "push_input: tilized tensor format differs from the queue's");
    const std::uint32_t cores = q.bufq_grid_dim_r * q.bufq_grid_dim_c;
    if (tensor.num_buffers != cores || q.bufq_entry_size == 0 || tensor.buf_size_bytes % q.bufq_entry_size)
        return fail(DEVICE_STATUS_CODE::RuntimeError, "push_input: tilized tensor does not match the queue's buffers");
    const std::uint32_t entries = tensor.buf_size_bytes / q.bufq_entry_size;
    SlotClaim claim;
    if (auto rc = claim.take(q, entries, timeout_in_seconds, ram_ptr); rc != DEVICE_STATUS_CODE::Success)
        return rc;
    QueueState *st = claim.st.get();
    const std::uint32_t first_slot = claim.first_slot;
    // the image is already in queue order: copy entry by entry into the ring of each grid buffer
    const std::uint64_t entry = q.bufq_entry_size;
    const std::uint64_t core_stride = (std::uint64_t)st->slots * entry;
    const int kind = on_device(tensor.ptr) ? 2 : 0;
    for (std::uint32_t c = 0; c < cores; c++)
    {
        std::uint32_t done = 0;
        while (done < entries)
        {
            const std::uint32_t slot = (first_slot + done) % st->slots;
            const std::uint32_t run = std::min(entries - done, st->slots - slot);
            int rc = buda_memcpy((std::uint8_t *)st->base + c * core_stride + slot * entry,
                                 (const std::uint8_t *)tensor.ptr + (std::uint64_t)c * tensor.buf_size_bytes + done * entry,
                                 run * entry, kind, nullptr);
            if (rc != BUDA_SUCCESS)
                return from_cabi(rc, "push_input");
            done += run;
        }
    }
    claim.commit();
    return DEVICE_STATUS_CODE::Success;
}

// ------------------------------------------------------------------------------------------------
// read / pop
// ------------------------------------------------------------------------------------------------
DEVICE_STATUS_CODE get_output(const tt_dram_io_desc &q, tt_PytorchTensorDesc &out, const bool pop_one,
                              const int timeout_in_seconds, const int rd_ptr)
{
    if (q.tile_width != 32 || q.tile_height == 0 || q.tile_height > 32 || (q.tile_height & (q.tile_height - 1)) ||
        q.layout != IO_LAYOUT::Tilized)
        return fail(DEVICE_STATUS_CODE::RuntimeError, "get_output: only tilized queues of 32x32 tiles are supported");
    const std::uint32_t hs = std::max<std::uint32_t>(1, q.hstack_factor), vs = std::max<std::uint32_t>(1, q.vstack_factor);
    if (q.t % (hs * vs))
        return fail(DEVICE_STATUS_CODE::RuntimeError, "get_output: t is not a multiple of hstack_factor x vstack_factor");
    std::shared_ptr<QueueState> st;
    if (auto rc = get_queue(q, false, st); rc != DEVICE_STATUS_CODE::Success)
        return rc;
    const std::uint32_t entries = pop_one ? 1 : std::max<std::uint32_t>(1, q.input_count);
    if (entries > st->slots)
        return fail(DEVICE_STATUS_CODE::RuntimeError, "get_output: more entries than the queue has slots");

    std::unique_lock<std::mutex> lock(st->mu);
    std::uint32_t first_slot;
    if (q.io_type == IO_TYPE::RandomAccess)
    {
        if (rd_ptr < 0 || (std::uint32_t)rd_ptr + entries > st->slots)
            return fail(DEVICE_STATUS_CODE::RuntimeError, "get_output: rd_ptr outside the queue");
        first_slot = (std::uint32_t)rd_ptr;
    }
    else
    {
        const auto deadline = std::chrono::steady_clock::now() + std::chrono::seconds(std::max(0, timeout_in_seconds));
        if (!st->cv.wait_until(lock, deadline, [&] { return st->occupancy >= entries; }))
            return fail(DEVICE_STATUS_CODE::TimeoutError, "get_output: queue '" + q.queue_name + "' stayed empty");
        first_slot = rd_ptr >= 0 ? ((std::uint32_t)rd_ptr % st->slots) : st->rd;
    }
    // the caller may ask for Float32 / Float16_b by presetting out.format; otherwise the queue decides
    DataFormat fmt = out.format;
    const bool bfp = is_bfp_data_format(q.bufq_target_format);
    if (bfp)
    {
        if (fmt != DataFormat::Float32 && fmt != DataFormat::Float16_b)
            fmt = default_output_format(q.bufq_target_format);
    }
    else if (q.bufq_target_format == DataFormat::Lf8 &&
             (fmt == DataFormat::Float32 || fmt == DataFormat::Float16_b || fmt == DataFormat::Float16))
    {
        // an Lf8 queue decodes to the float the caller names; with no request its bytes come back as they are
    }
    else
    {
        fmt = q.bufq_target_format;
    }
    const std::uint32_t itemsize = data_format_byte_size(fmt, 1);
    // output host transforms: the t slices are stacked hs across and vs down
    const std::array<std::uint32_t, 4> shape = {entries, q.t / (hs * vs), q.rows() * vs, q.cols() * hs};
    const std::uint64_t bytes = (std::uint64_t)entries * q.t * q.rows() * q.cols() * itemsize;
    if ((std::uint64_t)q.t * q.rows() * q.cols() * itemsize > 0xffffffffull)
        return fail(DEVICE_STATUS_CODE::RuntimeError, "get_output: an entry above 4 GiB does not fit 32-bit byte strides");
    void *host = host_acquire(bytes);
    if (!host)
        return fail(DEVICE_STATUS_CODE::RuntimeError, "get_output: " + cabi_error());
    const std::array<std::uint64_t, 4> st64 = {(std::uint64_t)shape[1] * shape[2] * shape[3] * itemsize,
                                               (std::uint64_t)shape[2] * shape[3] * itemsize, (std::uint64_t)shape[3] * itemsize,
                                               itemsize};
    const buda_queue_geom g = geom_of(q);
    int rc;
    if (hs * vs == 1)
    {
        rc = buda_queue_read(st->base, (int)q.bufq_target_format, q.tile_header ? 1 : 0, &g, st->slots, first_slot, host, 1, (int)fmt,
                             shape.data(), st64.data(), nullptr);
    }
    else
    {
        // untilize into the stacked layout on the device, then one copy to the host
        void *dev = nullptr;
        rc = buda_malloc(&dev, bytes);
        if (rc == BUDA_SUCCESS)
        {
            rc = buda_queue_read_stacked(st->base, (int)q.bufq_target_format, q.tile_header ? 1 : 0, &g, st->slots, first_slot, entries,
                                         hs, vs, q.stack_row_major ? 1 : 0, dev, (int)fmt, nullptr);
            if (rc == BUDA_SUCCESS)
                rc = buda_memcpy(host, dev, bytes, 1, nullptr);
            buda_free(dev);
        }
    }
    if (rc != BUDA_SUCCESS)
    {
        host_release(host);
        return from_cabi(rc, "get_output");
    }
    tt_PytorchTensorDesc result(host, itemsize, fmt == DataFormat::Int32 ? DataFormat::RawUInt32 : fmt, shape,
                                {(std::uint32_t)st64[0], (std::uint32_t)st64[1], (std::uint32_t)st64[2], itemsize}, 4);
    result.backend_owned = true;
    out = std::move(result);
    return DEVICE_STATUS_CODE::Success;
}

DEVICE_STATUS_CODE pop_output(const tt_dram_io_desc &q, const bool pop_one, const int timeout_in_seconds)
{
    std::shared_ptr<QueueState> st;
    if (auto rc = get_queue(q, false, st); rc != DEVICE_STATUS_CODE::Success)
        return rc;
    if (q.io_type == IO_TYPE::RandomAccess)
        return DEVICE_STATUS_CODE::Success;  // nothing to advance
    const std::uint32_t entries = pop_one ? 1 : std::max<std::uint32_t>(1, q.input_count);
    std::unique_lock<std::mutex> lock(st->mu);
    const auto deadline = std::chrono::steady_clock::now() + std::chrono::seconds(std::max(0, timeout_in_seconds));
    if (!st->cv.wait_until(lock, deadline, [&] { return st->occupancy >= entries; }))
        return fail(DEVICE_STATUS_CODE::TimeoutError, "pop_output: queue '" + q.queue_name + "' stayed empty");
    st->rd = (st->rd + entries) % st->slots;
    st->occupancy -= entries;
    lock.unlock();
    st->cv.notify_all();
    return DEVICE_STATUS_CODE::Success;
}

// ------------------------------------------------------------------------------------------------
// offline tilize
// ------------------------------------------------------------------------------------------------
tt_TilizedTensorDesc tilize_tensor(const tt_dram_io_desc &q, const tt_PytorchTensorDesc &tensor)
{
    const std::string why = check_tensor_fits(q, tensor);
    if (!why.empty())
        throw std::runtime_error("tilize_tensor: " + why);
    const buda_queue_geom g = geom_of(q);
    const std::int64_t total = buda_tilized_bytes(&g, tensor.shape.data(), (int)q.bufq_target_format, q.tile_header ? 1 : 0);
    if (total < 0)
        throw std::runtime_error("tilize_tensor: " + cabi_error());
    const std::uint32_t cores = q.bufq_grid_dim_r * q.bufq_grid_dim_c;
    if ((std::uint64_t)total / cores > 0xffffffffull)
        throw std::runtime_error("tilize_tensor: a grid buffer above 4 GiB does not fit buf_size_bytes");
    void *host = host_acquire((std::uint64_t)total);
    if (!host)
        throw std::runtime_error("tilize_tensor: " + cabi_error());
    const auto st64 = strides64(tensor);
    int rc;
    if (!on_device(tensor.ptr))
    {
        rc = buda_tilize_pack_host(tensor.ptr, (int)tensor.format, tensor.shape.data(), st64.data(), &g,
                                   (int)q.bufq_target_format, q.tile_header ? 1 : 0, host, (std::uint64_t)total, nullptr);
    }
    else
    {
        void *dev = nullptr;
        rc = buda_malloc(&dev, (std::uint64_t)total);
        if (rc == BUDA_SUCCESS)
        {
            rc = buda_tilize_pack(tensor.ptr, (int)tensor.format, tensor.shape.data(), st64.data(), &g,
                                  (int)q.bufq_target_format, q.tile_header ? 1 : 0, dev, (std::uint64_t)total, nullptr);
            if (rc == BUDA_SUCCESS)
                rc = buda_memcpy(host, dev, (std::uint64_t)total, 1, nullptr);
            buda_free(dev);
        }
    }
    if (rc != BUDA_SUCCESS)
    {
        host_release(host);
        throw std::runtime_error("tilize_tensor: " + cabi_error());
    }
    tt_TilizedTensorDesc d;
    d.ptr = host;
    d.num_buffers = cores;
    d.buf_size_bytes = (std::uint32_t)((std::uint64_t)total / cores);
    d.format = q.bufq_target_format;
    return d;
}

DEVICE_STATUS_CODE free_tensor(tt_PytorchTensorDesc &desc)
{
    if (desc.ptr && host_release(desc.ptr))
    {
        desc.ptr = nullptr;
        desc.backend_owned = false;
        return DEVICE_STATUS_CODE::Success;
    }
    // not ours: a borrowed tensor; dropping the descriptor's reference is all there is to do
    return DEVICE_STATUS_CODE::Success;
}

DEVICE_STATUS_CODE free_tensor(tt_TilizedTensorDesc &desc)
{
    if (desc.ptr && host_release(desc.ptr))
        desc.ptr = nullptr;
    return DEVICE_STATUS_CODE::Success;
}

// ------------------------------------------------------------------------------------------------
// raw dump / load (reference: binarize_tensor / debinarize_tensor, backend_api.cpp:705-708)
// ------------------------------------------------------------------------------------------------
namespace
{
DEVICE_STATUS_CODE write_file(const void *p, std::uint64_t bytes, const std::string &path)
{
    std::vector<char> bounce;
    if (on_device(p))
    {
        bounce.resize(bytes);
        if (int rc = buda_memcpy(bounce.data(), p, bytes, 1, nullptr); rc != BUDA_SUCCESS)
            return from_cabi(rc, "binarize_tensor");
        p = bounce.data();
    }
    std::ofstream f(path, std::ios::binary | std::ios::trunc);
    if (!f)
        return fail(DEVICE_STATUS_CODE::RuntimeError, "binarize_tensor: cannot open " + path);
    f.write((const char *)p, (std::streamsize)bytes);
    return f ? DEVICE_STATUS_CODE::Success : fail(DEVICE_STATUS_CODE::RuntimeError, "binarize_tensor: short write to " + path);
}

DEVICE_STATUS_CODE read_file(void *&out, std::uint64_t bytes, const std::string &path)
{
    std::ifstream f(path, std::ios::binary | std::ios::ate);
    if (!f)
        return fail(DEVICE_STATUS_CODE::RuntimeError, "debinarize_tensor: cannot open " + path);
    const std::uint64_t have = (std::uint64_t)f.tellg();
    if (have != bytes)
        return fail(DEVICE_STATUS_CODE::RuntimeError, "debinarize_tensor: " + path + " holds " + std::to_string(have) +
                                                          " bytes, the descriptor needs " + std::to_string(bytes));
    void *host = host_acquire(bytes);
    if (!host)
        return fail(DEVICE_STATUS_CODE::RuntimeError, "debinarize_tensor: " + cabi_error());
    f.seekg(0);
    f.read((char *)host, (std::streamsize)bytes);
    if (!f)
    {
        host_release(host);
        return fail(DEVICE_STATUS_CODE::RuntimeError, "debinarize_tensor: short read from " + path);
    }
    out = host;
    return DEVICE_STATUS_CODE::Success;
}
}  // namespace

DEVICE_STATUS_CODE binarize_tensor(const tt_PytorchTensorDesc &desc, const std::string &path)
{
    if (!desc.ptr)
        return fail(DEVICE_STATUS_CODE::RuntimeError, "binarize_tensor: null pointer");
    // dense tensors only: the file is the tensor's bytes in row-major order
    std::uint64_t expect = desc.itemsize;
    for (int i = 3; i >= 0; i--)
    {
        if (desc.shape[i] != 1 && desc.strides[i] != expect)
            return fail(DEVICE_STATUS_CODE::RuntimeError, "binarize_tensor: tensor is not dense row-major");
        expect *= desc.shape[i];
    }
    return write_file(desc.ptr, desc.numel() * desc.itemsize, path);
}

DEVICE_STATUS_CODE binarize_tensor(const tt_TilizedTensorDesc &desc, const std::string &path)
{
    if (!desc.ptr)
        return fail(DEVICE_STATUS_CODE::RuntimeError, "binarize_tensor: null pointer");
    return write_file(desc.ptr, desc.total_bytes(), path);
}

DEVICE_STATUS_CODE debinarize_tensor(tt_PytorchTensorDesc &desc, const std::string &path)
{
    void *host = nullptr;
    if (auto rc = read_file(host, desc.numel() * desc.itemsize, path); rc != DEVICE_STATUS_CODE::Success)
        return rc;
    desc.ptr = host;
    desc.backend_owned = true;
    std::uint32_t s = desc.itemsize;
    for (int i = 3; i >= 0; i--)
    {
        desc.strides[i] = s;
        s *= desc.shape[i];
    }
    return DEVICE_STATUS_CODE::Success;
}

DEVICE_STATUS_CODE debinarize_tensor(tt_TilizedTensorDesc &desc, const std::string &path)
{
    void *host = nullptr;
    if (auto rc = read_file(host, desc.total_bytes(), path); rc != DEVICE_STATUS_CODE::Success)
        return rc;
    desc.ptr = host;
    return DEVICE_STATUS_CODE::Success;
}

// ------------------------------------------------------------------------------------------------
// sizes and addresses
// ------------------------------------------------------------------------------------------------
int get_io_size_in_bytes(DataFormat df, bool is_untilized, int ublock_ct, int ublock_rt, int mblock_m, int mblock_n, int t,
                         int entries, int tile_height, int tile_width)
{
    const std::int64_t n = buda_io_size_bytes((int)df, is_untilized ? 1 : 0, ublock_ct, ublock_rt, mblock_m, mblock_n, t, entries,
                                              tile_height, tile_width);
    if (n < 0)
        throw std::runtime_error("get_io_size_in_bytes: invalid data format");
    if (n > 0x7fffffff)
        throw std::runtime_error("get_io_size_in_bytes: size does not fit the 32-bit return type");
    return (int)n;
}

// Queue entries start on 32-byte boundaries (a multiple of the 16 bytes the bulk-copy engine needs).
std::uint32_t get_next_aligned_address(std::uint32_t address) { return (address + 31u) & ~31u; }

// Queues live in this process's device memory: there is no channel / sub-channel to translate.
DEVICE_STATUS_CODE translate_addresses(tt_dram_io_desc &) { return DEVICE_STATUS_CODE::Success; }

std::uint64_t queue_device_address(const tt_dram_io_desc &q)
{
    std::lock_guard<std::mutex> lock(g_registry_mu);
    auto it = g_queues.find(q.key());
    return it == g_queues.end() ? 0 : (std::uint64_t)it->second->base;
}

std::uint32_t queue_occupancy(const tt_dram_io_desc &q)
{
    std::lock_guard<std::mutex> lock(g_registry_mu);
    auto it = g_queues.find(q.key());
    if (it == g_queues.end())
        return 0;
    std::lock_guard<std::mutex> l2(it->second->mu);
    return it->second->occupancy;
}

DEVICE_STATUS_CODE release_queue(const tt_dram_io_desc &q)
{
    std::shared_ptr<QueueState> st;
    {
        std::lock_guard<std::mutex> lock(g_registry_mu);
        auto it = g_queues.find(q.key());
        if (it == g_queues.end())
            return DEVICE_STATUS_CODE::Success;
        st = it->second;
        g_queues.erase(it);
    }
    std::lock_guard<std::mutex> lock(st->mu);
    if (st->base)
        buda_free(st->base);
    st->base = nullptr;
    return DEVICE_STATUS_CODE::Success;
}

void release_all_queues()
{
    std::unordered_map<std::string, std::shared_ptr<QueueState>> all;
    {
        std::lock_guard<std::mutex> lock(g_registry_mu);
        all.swap(g_queues);
    }
    for (auto &kv : all)
    {
        std::lock_guard<std::mutex> lock(kv.second->mu);
        if (kv.second->base)
            buda_free(kv.second->base);
        kv.second->base = nullptr;
    }
}

// ------------------------------------------------------------------------------------------------
// matmul against a Bfp8_b parameter queue
// ------------------------------------------------------------------------------------------------
DEVICE_STATUS_CODE matmul_bfp8b(const tt_PytorchTensorDesc &act, const tt_dram_io_desc &wq, tt_PytorchTensorDesc &out)
{
    if (wq.bufq_target_format != DataFormat::Bfp8_b || wq.tile_header || wq.bufq_grid_dim_r != 1 || wq.bufq_grid_dim_c != 1 ||
        wq.ublock_rt != 1 || wq.ublock_ct != 1 || wq.ublock_order != 0 || wq.t != 1)
        return fail(DEVICE_STATUS_CODE::RuntimeError,
                    "matmul_bfp8b: the weight queue must be Bfp8_b, grid 1x1, ublock 1x1, order r, t = 1, no tile header");
    if (act.format != DataFormat::Float16_b || out.format != DataFormat::Float16_b)
        return fail(DEVICE_STATUS_CODE::RuntimeError, "matmul_bfp8b: activations and output must be Float16_b");
    std::shared_ptr<QueueState> st;
    if (auto rc = get_queue(wq, false, st); rc != DEVICE_STATUS_CODE::Success)
        return rc;
    const std::uint64_t K = wq.rows(), N = wq.cols();
    const std::uint64_t M = (std::uint64_t)act.shape[0] * act.shape[1] * act.shape[2];
    if (act.shape[3] != K || out.shape[3] != N || (std::uint64_t)out.shape[0] * out.shape[1] * out.shape[2] != M)
        return fail(DEVICE_STATUS_CODE::RuntimeError, "matmul_bfp8b: shapes do not match [M,K] x [K,N] -> [M,N]");
    if (act.strides[3] != 2 || out.strides[3] != 2 || act.strides[2] % 2 || out.strides[2] % 2)
        return fail(DEVICE_STATUS_CODE::RuntimeError, "matmul_bfp8b: rows must be dense bfloat16");
    if (!on_device(out.ptr) && out.strides[2] / 2 != N)
        return fail(DEVICE_STATUS_CODE::RuntimeError, "matmul_bfp8b: host output must be dense");
    std::unique_lock<std::mutex> lock(st->mu);
    const std::uint32_t slot = wq.io_type == IO_TYPE::RandomAccess ? 0 : (st->wr + st->slots - 1) % st->slots;
    const std::uint8_t *w = (const std::uint8_t *)st->base + (std::uint64_t)slot * wq.bufq_entry_size;
    const bool a_host = !on_device(act.ptr), c_host = !on_device(out.ptr);
    void *a_dev = const_cast<void *>(act.ptr), *c_dev = const_cast<void *>(out.ptr);
    std::uint64_t lda = act.strides[2] / 2, ldc = out.strides[2] / 2;
    int rc = BUDA_SUCCESS;
    if (a_host)
    {
        if (lda != K)
            return fail(DEVICE_STATUS_CODE::RuntimeError, "matmul_bfp8b: host activations must be dense");
        rc = buda_malloc(&a_dev, M * K * 2);
        if (rc == BUDA_SUCCESS)
            rc = buda_memcpy(a_dev, act.ptr, M * K * 2, 0, nullptr);
    }
    if (rc == BUDA_SUCCESS && c_host)
        rc = buda_malloc(&c_dev, M * N * 2);
    if (rc == BUDA_SUCCESS)
        rc = buda_bfp8b_gemm(a_dev, (std::int64_t)M, (std::int64_t)K, (std::int64_t)lda, w, (std::int64_t)N, c_dev,
                             (std::int64_t)ldc, nullptr);
    if (rc == BUDA_SUCCESS)
        rc = c_host ? buda_memcpy(const_cast<void *>(out.ptr), c_dev, M * N * 2, 1, nullptr) : buda_stream_synchronize(nullptr);
    if (a_host && a_dev)
        buda_free(a_dev);
    if (c_host && c_dev)
        buda_free(c_dev);
    return from_cabi(rc, "matmul_bfp8b");
}

}  // namespace tt::backend
