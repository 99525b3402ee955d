// Data-format core of the host layer: the DataFormat / MathFidelity enums with the reference's
// integer values, per-format sizes and the small a/b-exponent helpers the conversion path uses.
// Mirrors the interface of the reference's pybuda/csrc/lower_to_buda/common.hpp:92-258.
#pragma once

#include <array>
#include <cstdint>
#include <iosfwd>
#include <string>

namespace tt
{

// values: reference pybuda/csrc/lower_to_buda/common.hpp:92-111
enum class DataFormat : std::uint8_t
{
    Float32 = 0,
    Float16 = 1,
    Bfp8 = 2,
    Bfp4 = 3,
    Bfp2 = 11,
    Float16_b = 5,
    Bfp8_b = 6,
    Bfp4_b = 7,
    Bfp2_b = 15,
    Lf8 = 10,
    UInt16 = 12,
    Int8 = 14,
    Int32 = 8,
    RawUInt8 = 0xf0,
    RawUInt16 = 0xf1,
    RawUInt32 = 0xf2,
    Invalid = 0xff
};

// values: reference common.hpp:113-120
enum class MathFidelity : std::uint8_t
{
    LoFi = 0,
    HiFi2 = 2,
    HiFi3 = 3,
    HiFi4 = 4,
    Invalid = 0xff
};

// bytes of `elements` values of a format, block-float formats counting their shared exponents
// (reference common.cpp:167-190); throws std::runtime_error for an unknown format
std::uint32_t data_format_byte_size(DataFormat df, int elements = 1);

// bytes of one 32x32 tile in queue memory (reference balancer_utils.hpp:24-51)
std::size_t tile_size_bytes(DataFormat df, bool include_header_padding = true);

// which exponent family a format belongs to (reference common.hpp:175-222)
bool is_b_data_format(DataFormat df);
bool is_a_data_format(DataFormat df);
DataFormat to_a_data_format(DataFormat df);
DataFormat to_b_data_format(DataFormat df);
bool is_integer_data_format(DataFormat df);
bool is_bfp_data_format(DataFormat df);
int get_precision_bits(DataFormat df);
// keep the narrower of two formats, in the exponent family of `to` (reference common.hpp:240-246)
DataFormat preserve_lower_precision_cast(DataFormat from, DataFormat to);

const char *data_format_name(DataFormat df);
const char *math_fidelity_name(MathFidelity mf);
// accepts the enum names, case-insensitively ("Bfp8_b", "float16_b", ...); Invalid if unknown
DataFormat get_format_from_string(const std::string &name);
MathFidelity get_fidelity_from_string(const std::string &name);

std::ostream &operator<<(std::ostream &os, DataFormat const &df);
std::ostream &operator<<(std::ostream &os, MathFidelity const &mf);

// Row-major tensor as the converters see it (reference common.hpp:251-258, extended with the
// owner handle the pybind layer keeps alive, backend_api.cpp:493-503).
struct tt_PytorchTensorDesc
{
    using RefChange = void (*)(const void *handle, bool acquire);

    const void *ptr = nullptr;
    std::uint32_t itemsize = 0;
    DataFormat format = DataFormat::Invalid;
    std::array<std::uint32_t, 4> shape = {1, 1, 1, 1};    // outermost dimension first
    std::array<std::uint32_t, 4> strides = {0, 0, 0, 0};  // outermost first, in BYTES
    std::uint32_t dim = 4;
    const void *owner = nullptr;     // opaque handle of the object that owns ptr (a Python tensor)
    RefChange owner_refchange = nullptr;
    bool backend_owned = false;      // ptr was allocated by get_output and is released by free_tensor

    tt_PytorchTensorDesc() = default;
    // takes over ONE reference to `owner` (the caller has already acquired it)
    tt_PytorchTensorDesc(const void *p, std::uint32_t isz, DataFormat f, std::array<std::uint32_t, 4> sh,
                         std::array<std::uint32_t, 4> st, std::uint32_t d, const void *own = nullptr,
                         RefChange rc = nullptr);
    tt_PytorchTensorDesc(const tt_PytorchTensorDesc &o);
    tt_PytorchTensorDesc(tt_PytorchTensorDesc &&o) noexcept;
    tt_PytorchTensorDesc &operator=(tt_PytorchTensorDesc o) noexcept;
    ~tt_PytorchTensorDesc();

    std::uint64_t numel() const { return (std::uint64_t)shape[0] * shape[1] * shape[2] * shape[3]; }
};

// Queue image produced by tilize_tensor (reference backend_api.cpp:562-591): num_buffers grid
// buffers of buf_size_bytes each, contiguous, in backend-owned host memory.
struct tt_TilizedTensorDesc
{
    const void *ptr = nullptr;
    std::uint32_t num_buffers = 0;
    std::uint32_t buf_size_bytes = 0;
    DataFormat format = DataFormat::Invalid;
    std::uint64_t total_bytes() const { return (std::uint64_t)num_buffers * buf_size_bytes; }
};

}  // namespace tt
