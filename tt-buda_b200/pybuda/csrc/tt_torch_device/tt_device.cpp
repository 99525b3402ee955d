#include "tt_torch_device/tt_device.hpp"

#include <stdexcept>

namespace tt
{
tt_PytorchTensorDesc to_pytorch_tensor_desc(const void *data, std::uint32_t element_size, DataFormat format,
                                            const std::vector<std::int64_t> &sizes, const std::vector<std::int64_t> &strides)
{
    const int dim = (int)sizes.size();
    if (dim <= 0 || dim > 4)
        throw std::invalid_argument("to_pytorch_tensor_desc: tensors have 1 to 4 dimensions");
    if (strides.size() != sizes.size())
        throw std::invalid_argument("to_pytorch_tensor_desc: sizes and strides differ in length");

    std::array<std::uint32_t, 4> shape = {1, 1, kTileDim, kTileDim};
    std::array<std::uint32_t, 4> byte_strides = {0, 0, 0, 0};
    int i = 4 - dim;
    for (std::int64_t s : sizes)
    {
        shape[i] = i >= 2 ? align_up_tile(s) : (std::uint32_t)s;
        ++i;
    }
    i = 3;
    for (int j = dim - 1; j >= 0; --j, --i) byte_strides[i] = (std::uint32_t)(strides[j] * element_size);
    if (i >= 2)  // a 1-D tensor: its (implied) row is one tile row long
    {
        byte_strides[i] = kTileDim * element_size;
        --i;
    }
    const int last = i + 1;
    while (i >= 0)
    {
        byte_strides[i] = byte_strides[last];
        --i;
    }
    return tt_PytorchTensorDesc(data, element_size, format, shape, byte_strides, 4);
}

std::array<std::uint32_t, 4> buda_padded_shape(const std::vector<std::int64_t> &sizes)
{
    if (sizes.size() > 4)
        throw std::invalid_argument("Tensor has more than 4 dimensions");
    std::array<std::uint32_t, 4> shape = {1, 1, 1, 1};
    const int off = 4 - (int)sizes.size();
    for (std::size_t k = 0; k < sizes.size(); k++) shape[off + k] = (std::uint32_t)sizes[k];
    shape[2] = align_up_tile(shape[2]);
    shape[3] = align_up_tile(shape[3]);
    return shape;
}
}  // namespace tt
