// Shape-level twins of the descriptor helpers of the reference's torch device plugin
// (pybuda/csrc/tt_torch_device/tt_device.cpp:109-189).  The reference takes a torch::Tensor; this host layer does not
// link against libtorch, so the same rules are stated on (data pointer, element size, sizes, strides).
#pragma once

#include <array>
#include <cstdint>
#include <vector>

#include "lower_to_buda/common.hpp"

namespace tt
{
constexpr std::uint32_t kTileDim = 32;
inline std::uint32_t align_up_tile(std::int64_t v) { return (std::uint32_t)((v + kTileDim - 1) / kTileDim * kTileDim); }

// Descriptor of a tensor of up to 4 dims: sizes right-aligned into [w, z, r, c] with r and c rounded UP to the tile
// (the caller pads the data first: pad_to_buda_shape), byte strides, a 1-D tensor's row stride set to one tile
// row, missing leading strides copied from the outermost given one.  dim is always 4
// (reference to_pytorch_tensor_desc, tt_device.cpp:109-151).  Throws std::invalid_argument on more than 4 dims,
// no dims, or sizes / strides of different lengths.
tt_PytorchTensorDesc to_pytorch_tensor_desc(const void *data, std::uint32_t element_size, DataFormat format,
                                            const std::vector<std::int64_t> &sizes, const std::vector<std::int64_t> &strides);

// The 4-D shape a tensor has after pad_to_buda_shape (tt_device.cpp:153-189): leading 1s up to 4 dims, r and c
// rounded up to the tile; the padded tensor is dense.
std::array<std::uint32_t, 4> buda_padded_shape(const std::vector<std::int64_t> &sizes);
}  // namespace tt
