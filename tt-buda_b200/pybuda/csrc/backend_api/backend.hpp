// The converter entry points of the reference's backend (tt::backend::*, bound at
// pybuda/csrc/backend_api/backend_api.cpp:688-726) re-implemented for device-resident queues on a
// CUDA GPU.  All data movement and arithmetic happens behind the C ABI of libbuda_cuda.so; this
// layer keeps descriptors, queue read/write pointers, ownership and the status-code convention.
#pragma once

#include <cstdint>
#include <string>
#include <utility>
#include <vector>

#include "lower_to_buda/common.hpp"

namespace tt
{

// reference backend_api.cpp:622-625
enum class DEVICE_STATUS_CODE
{
    Success = 0,
    RuntimeError = 1,
    TimeoutError = 2
};

// reference backend_api.cpp:321-329
enum class IO_TYPE
{
    Queue = 0,
    RandomAccess = 1,
    Invalid = 2
};

enum class IO_LAYOUT
{
    Tilized = 0,
    Flat = 1,
    Invalid = 2
};

// reference backend_api.cpp:288-294 (kept so DramIODesc pickles carry the same fields)
enum class DEVICE
{
    Model = 0,
    Versim = 1,
    Silicon = 2,
    Golden = 3,
    Emulation = 4,
    Invalid = 5
};

// reference backend_api.cpp:384-407
struct Stride
{
    std::vector<std::pair<int, int>> xy_offsets;
    int stride = -1;
};

// How a pushed tensor is read when a runtime tensor transform stands between it and the queue (push_input_view).
enum class SOURCE_VIEW : std::uint32_t
{
    Padded = 1,          // zero padding up to the queue's tiles; a size-1 row dimension may be broadcast across its tile
    EmbeddingIndex = 2,  // a vector of row indices laid out for an embedding op
    Prestride = 3        // a convolution activation cut into its stride phases
};

struct tt_SourceView
{
    SOURCE_VIEW mode = SOURCE_VIEW::Padded;
    bool broadcast_rows = false, broadcast_cols = false;  // Padded
    std::uint64_t count = 0, group = 0;                   // EmbeddingIndex: indices per entry; indices per queue tile row
    Stride stride;                                        // Prestride
};

// Queue descriptor: field names of the reference's DramIODesc (backend_api.cpp:409-487).
struct tt_dram_io_desc
{
    std::string netlist_path;
    std::string queue_name;
    std::uint32_t bufq_grid_dim_r = 1, bufq_grid_dim_c = 1;
    std::uint32_t bufq_num_slots = 1;
    std::uint32_t ublock_rt = 1, ublock_ct = 1, mblock_m = 1, mblock_n = 1;
    std::uint32_t tile_height = 32, tile_width = 32;
    std::uint32_t t = 1;
    std::uint32_t input_count = 1;
    std::uint32_t hstack_factor = 1, vstack_factor = 1;
    bool stack_row_major = true;
    DataFormat bufq_target_format = DataFormat::Invalid;
    std::vector<std::pair<std::uint32_t, std::uint16_t>> bufq_start_addr_channel;
    std::uint32_t bufq_entry_size = 0;  // bytes of one entry in one grid buffer
    IO_TYPE io_type = IO_TYPE::Queue;
    Stride s_descriptor;
    DEVICE backend_type = DEVICE::Silicon;
    IO_LAYOUT layout = IO_LAYOUT::Tilized;
    // not in the reference descriptor (its backend reads them from the netlist):
    std::uint32_t ublock_order = 0;  // 0 = r, 1 = c
    bool tile_header = false;        // 32-byte header/pad in front of every tile record

    std::uint64_t tiles_per_entry() const { return (std::uint64_t)t * mblock_m * mblock_n * ublock_rt * ublock_ct; }
    std::uint32_t rows() const { return bufq_grid_dim_r * mblock_m * ublock_rt * tile_height; }
    std::uint32_t cols() const { return bufq_grid_dim_c * mblock_n * ublock_ct * tile_width; }
    std::string key() const { return netlist_path + "::" + queue_name; }
};

namespace backend
{

// Descriptor for a queue that holds a [w, z, R, C] tensor.  The reference only obtains descriptors
// from a compiled netlist (BackendApi.get_queue_descriptor, backend_api.cpp:674); without a
// netlist the caller states the geometry.  Throws std::runtime_error if grid x ublock does not
// divide the tile counts.
tt_dram_io_desc make_queue_desc(const std::string &name, std::array<std::uint32_t, 4> shape, DataFormat df,
                                std::pair<std::uint32_t, std::uint32_t> grid = {1, 1},
                                std::pair<std::uint32_t, std::uint32_t> ublock = {1, 1}, std::uint32_t ublock_order = 0,
                                std::uint32_t num_slots = 0, IO_TYPE io_type = IO_TYPE::Queue, bool tile_header = false,
                                std::uint32_t tile_height = 32);

DEVICE_STATUS_CODE push_input(const tt_dram_io_desc &q, const tt_PytorchTensorDesc &tensor, const bool push_one,
                              const int timeout_in_seconds, const int ram_ptr);
DEVICE_STATUS_CODE push_input(const tt_dram_io_desc &q, const tt_TilizedTensorDesc &tensor, const int timeout_in_seconds,
                              const int ram_ptr);
// ---- not in the reference: a whole set of tensors in one call, and pushes through a runtime transform in one kernel
DEVICE_STATUS_CODE push_input_batch(const std::vector<tt_dram_io_desc> &queues, const std::vector<tt_PytorchTensorDesc> &tensors,
                                    const bool push_one, const int timeout_in_seconds, const std::vector<int> &ram_ptrs);
DEVICE_STATUS_CODE push_input_view(const tt_dram_io_desc &q, const tt_PytorchTensorDesc &tensor, const tt_SourceView &view,
                                   const bool push_one, const int timeout_in_seconds, const int ram_ptr);
DEVICE_STATUS_CODE get_output(const tt_dram_io_desc &q, tt_PytorchTensorDesc &out, const bool pop_one,
                              const int timeout_in_seconds, const int rd_ptr);
DEVICE_STATUS_CODE pop_output(const tt_dram_io_desc &q, const bool pop_one, const int timeout_in_seconds);

tt_TilizedTensorDesc tilize_tensor(const tt_dram_io_desc &q, const tt_PytorchTensorDesc &tensor);

DEVICE_STATUS_CODE free_tensor(tt_PytorchTensorDesc &desc);
DEVICE_STATUS_CODE free_tensor(tt_TilizedTensorDesc &desc);

DEVICE_STATUS_CODE binarize_tensor(const tt_PytorchTensorDesc &desc, const std::string &path);
DEVICE_STATUS_CODE binarize_tensor(const tt_TilizedTensorDesc &desc, const std::string &path);
DEVICE_STATUS_CODE debinarize_tensor(tt_PytorchTensorDesc &desc, const std::string &path);
DEVICE_STATUS_CODE debinarize_tensor(tt_TilizedTensorDesc &desc, const std::string &path);

int get_io_size_in_bytes(DataFormat df, bool is_untilized, int ublock_ct, int ublock_rt, int mblock_m, int mblock_n, int t,
                         int entries, int tile_height = 32, int tile_width = 32);
std::uint32_t get_next_aligned_address(std::uint32_t address);
DEVICE_STATUS_CODE translate_addresses(tt_dram_io_desc &q);

// ---- not in the reference: queue memory lives in this process, so it can be inspected and released
std::uint64_t queue_device_address(const tt_dram_io_desc &q);  // 0 until the first push
std::uint32_t queue_occupancy(const tt_dram_io_desc &q);
DEVICE_STATUS_CODE release_queue(const tt_dram_io_desc &q);
void release_all_queues();
std::string last_error();  // reason for the calling thread's last non-Success status

// C = A @ W with A bfloat16 [M,K] (host or device) and W the newest entry of a Bfp8_b parameter
// queue holding a [1,1,K,N] tensor; C is bfloat16 [M,N] written to `out` (same side as A).
DEVICE_STATUS_CODE matmul_bfp8b(const tt_PytorchTensorDesc &act, const tt_dram_io_desc &weight_q, tt_PytorchTensorDesc &out);

}  // namespace backend
}  // namespace tt
