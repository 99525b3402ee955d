#include "lower_to_buda/common.hpp"

#include <algorithm>
#include <cctype>
#include <ostream>
#include <stdexcept>
#include <utility>

#include "buda_cuda.h"

namespace tt
{

std::uint32_t data_format_byte_size(DataFormat df, int elements)
{
    // one table for host and device code: the C ABI owns it
    const std::int64_t n = buda_data_format_byte_size(static_cast<int>(df), elements);
    if (n < 0)
        throw std::runtime_error("Invalid format");
    return static_cast<std::uint32_t>(n);
}

std::size_t tile_size_bytes(DataFormat df, bool include_header_padding)
{
    const std::int64_t n = buda_tile_bytes(static_cast<int>(df), include_header_padding ? 1 : 0);
    return n < 0 ? static_cast<std::size_t>(0xbadface) : static_cast<std::size_t>(n);
}

bool is_bfp_data_format(DataFormat df)
{
    return df == DataFormat::Bfp8 || df == DataFormat::Bfp4 || df == DataFormat::Bfp2 || df == DataFormat::Bfp8_b ||
           df == DataFormat::Bfp4_b || df == DataFormat::Bfp2_b;
}

bool is_b_data_format(DataFormat df)
{
    return df == DataFormat::Float32 || df == DataFormat::Float16_b || df == DataFormat::Bfp8_b ||
           df == DataFormat::Bfp4_b || df == DataFormat::Bfp2_b;
}

bool is_a_data_format(DataFormat df)
{
    return df == DataFormat::Float16 || df == DataFormat::Bfp8 || df == DataFormat::Bfp4 || df == DataFormat::Bfp2;
}

namespace
{
// (a-exponent member, b-exponent member) of each family that has both
constexpr std::pair<DataFormat, DataFormat> kFamilies[] = {
    {DataFormat::Float16, DataFormat::Float16_b},
    {DataFormat::Bfp8, DataFormat::Bfp8_b},
    {DataFormat::Bfp4, DataFormat::Bfp4_b},
    {DataFormat::Bfp2, DataFormat::Bfp2_b},
};
}  // namespace

DataFormat to_a_data_format(DataFormat df)
{
    for (auto const &f : kFamilies)
        if (f.second == df)
            return f.first;
    return df;
}

DataFormat to_b_data_format(DataFormat df)
{
    for (auto const &f : kFamilies)
        if (f.first == df)
            return f.second;
    return df;
}

bool is_integer_data_format(DataFormat df)
{
    switch (df)
    {
        case DataFormat::Lf8:
        case DataFormat::UInt16:
        case DataFormat::Int8:
        case DataFormat::Int32:
        case DataFormat::RawUInt8:
        case DataFormat::RawUInt16:
        case DataFormat::RawUInt32: return true;
        default: return false;
    }
}

int get_precision_bits(DataFormat df)
{
    if (df == DataFormat::Float32)
        return 32;
    switch (to_b_data_format(df))
    {
        case DataFormat::Float16_b: return 16;
        case DataFormat::Bfp8_b: return 8;
        case DataFormat::Bfp4_b: return 4;
        case DataFormat::Bfp2_b: return 2;
        default: return 0;
    }
}

DataFormat preserve_lower_precision_cast(DataFormat from, DataFormat to)
{
    if (get_precision_bits(from) >= get_precision_bits(to))
        return to;
    return is_b_data_format(to) ? to_b_data_format(from) : to_a_data_format(from);
}

namespace
{
struct DfName
{
    DataFormat df;
    const char *name;
};
constexpr DfName kDfNames[] = {
    {DataFormat::Float32, "Float32"},     {DataFormat::Float16, "Float16"},     {DataFormat::Bfp8, "Bfp8"},
    {DataFormat::Bfp4, "Bfp4"},           {DataFormat::Bfp2, "Bfp2"},           {DataFormat::Float16_b, "Float16_b"},
    {DataFormat::Bfp8_b, "Bfp8_b"},       {DataFormat::Bfp4_b, "Bfp4_b"},       {DataFormat::Bfp2_b, "Bfp2_b"},
    {DataFormat::Lf8, "Lf8"},             {DataFormat::UInt16, "UInt16"},       {DataFormat::Int8, "Int8"},
    {DataFormat::Int32, "Int32"},         {DataFormat::RawUInt8, "RawUInt8"},   {DataFormat::RawUInt16, "RawUInt16"},
    {DataFormat::RawUInt32, "RawUInt32"}, {DataFormat::Invalid, "Invalid"},
};
struct MfName
{
    MathFidelity mf;
    const char *name;
};
constexpr MfName kMfNames[] = {{MathFidelity::LoFi, "LoFi"},   {MathFidelity::HiFi2, "HiFi2"},
                               {MathFidelity::HiFi3, "HiFi3"}, {MathFidelity::HiFi4, "HiFi4"},
                               {MathFidelity::Invalid, "Invalid"}};

std::string lower(std::string s)
{
    std::transform(s.begin(), s.end(), s.begin(), [](unsigned char c) { return std::tolower(c); });
    return s;
}
}  // namespace

const char *data_format_name(DataFormat df)
{
    for (auto const &e : kDfNames)
        if (e.df == df)
            return e.name;
    return "Invalid";
}

const char *math_fidelity_name(MathFidelity mf)
{
    for (auto const &e : kMfNames)
        if (e.mf == mf)
            return e.name;
    return "Invalid";
}

DataFormat get_format_from_string(const std::string &name)
{
    const std::string n = lower(name);
    for (auto const &e : kDfNames)
        if (lower(e.name) == n)
            return e.df;
    return DataFormat::Invalid;
}

MathFidelity get_fidelity_from_string(const std::string &name)
{
    const std::string n = lower(name);
    for (auto const &e : kMfNames)
        if (lower(e.name) == n)
            return e.mf;
    return MathFidelity::Invalid;
}

std::ostream &operator<<(std::ostream &os, DataFormat const &df) { return os << data_format_name(df); }
std::ostream &operator<<(std::ostream &os, MathFidelity const &mf) { return os << math_fidelity_name(mf); }

// ---------------------------------------------------------------------------------------------
// tt_PytorchTensorDesc: every copy holds one reference to the owner
// ---------------------------------------------------------------------------------------------
tt_PytorchTensorDesc::tt_PytorchTensorDesc(const void *p, std::uint32_t isz, DataFormat f,
                                           std::array<std::uint32_t, 4> sh, std::array<std::uint32_t, 4> st,
                                           std::uint32_t d, const void *own, RefChange rc) :
    ptr(p), itemsize(isz), format(f), shape(sh), strides(st), dim(d), owner(own), owner_refchange(rc)
{
}

tt_PytorchTensorDesc::tt_PytorchTensorDesc(const tt_PytorchTensorDesc &o) :
    ptr(o.ptr), itemsize(o.itemsize), format(o.format), shape(o.shape), strides(o.strides), dim(o.dim), owner(o.owner),
    owner_refchange(o.owner_refchange), backend_owned(o.backend_owned)
{
    if (owner && owner_refchange)
        owner_refchange(owner, true);
}

tt_PytorchTensorDesc::tt_PytorchTensorDesc(tt_PytorchTensorDesc &&o) noexcept :
    ptr(o.ptr), itemsize(o.itemsize), format(o.format), shape(o.shape), strides(o.strides), dim(o.dim), owner(o.owner),
    owner_refchange(o.owner_refchange), backend_owned(o.backend_owned)
{
    o.owner = nullptr;
    o.owner_refchange = nullptr;
}

tt_PytorchTensorDesc &tt_PytorchTensorDesc::operator=(tt_PytorchTensorDesc o) noexcept
{
    std::swap(ptr, o.ptr);
    std::swap(itemsize, o.itemsize);
    std::swap(format, o.format);
    std::swap(shape, o.shape);
    std::swap(strides, o.strides);
    std::swap(dim, o.dim);
    std::swap(owner, o.owner);
    std::swap(owner_refchange, o.owner_refchange);
    std::swap(backend_owned, o.backend_owned);
    return *this;
}

tt_PytorchTensorDesc::~tt_PytorchTensorDesc()
{
    if (owner && owner_refchange)
        owner_refchange(owner, false);
}

}  // namespace tt
