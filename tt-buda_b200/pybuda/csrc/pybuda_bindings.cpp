// Python module pybuda._C: the DataFormat / MathFidelity enums (same values, json and pickle
// behaviour as the reference's pybuda/csrc/pybuda_bindings.cpp:54-130) and the submodules
// backend_api (converter entry points) and balancer (tile order model).
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <string>

#include "balancer/tile_layout.hpp"
#include "lower_to_buda/common.hpp"

namespace py = pybind11;

namespace tt::backend_api
{
void BackendModule(py::module &m_backend);
}

PYBIND11_MODULE(_C, m)
{
    m.attr("__name__") = "pybuda._C";
    m.doc() = "pybuda host layer for the B200 data-format path";
    m.attr("VERSION") = py::int_(1);
    m.attr("k_dim") = py::int_(32);  // tile dimension

    py::enum_<tt::DataFormat>(m, "DataFormat")
        .value("Float32", tt::DataFormat::Float32)
        .value("Float16", tt::DataFormat::Float16)
        .value("Bfp8", tt::DataFormat::Bfp8)
        .value("Bfp4", tt::DataFormat::Bfp4)
        .value("Bfp2", tt::DataFormat::Bfp2)
        .value("Float16_b", tt::DataFormat::Float16_b)
        .value("Bfp8_b", tt::DataFormat::Bfp8_b)
        .value("Bfp4_b", tt::DataFormat::Bfp4_b)
        .value("Bfp2_b", tt::DataFormat::Bfp2_b)
        .value("Lf8", tt::DataFormat::Lf8)
        .value("UInt16", tt::DataFormat::UInt16)
        .value("Int8", tt::DataFormat::Int8)
        .value("Int32", tt::DataFormat::Int32)
        .value("RawUInt8", tt::DataFormat::RawUInt8)
        .value("RawUInt16", tt::DataFormat::RawUInt16)
        .value("RawUInt32", tt::DataFormat::RawUInt32)
        .value("Invalid", tt::DataFormat::Invalid)
        .export_values()
        .def("to_json", [](tt::DataFormat df) { return std::string(tt::data_format_name(df)); })
        .def_static("from_json",
                    [](std::string const &s)
                    {
                        const tt::DataFormat df = tt::get_format_from_string(s);
                        if (df == tt::DataFormat::Invalid && s != "Invalid")
                            throw py::key_error(s);
                        return df;
                    });

    py::enum_<tt::MathFidelity>(m, "MathFidelity")
        .value("LoFi", tt::MathFidelity::LoFi)
        .value("HiFi2", tt::MathFidelity::HiFi2)
        .value("HiFi3", tt::MathFidelity::HiFi3)
        .value("HiFi4", tt::MathFidelity::HiFi4)
        .value("Invalid", tt::MathFidelity::Invalid)
        .export_values()
        .def("to_json", [](tt::MathFidelity mf) { return std::string(tt::math_fidelity_name(mf)); })
        .def_static("from_json",
                    [](std::string const &s)
                    {
                        const tt::MathFidelity mf = tt::get_fidelity_from_string(s);
                        if (mf == tt::MathFidelity::Invalid && s != "Invalid")
                            throw py::key_error(s);
                        return mf;
                    });

    m.def("data_format_byte_size", &tt::data_format_byte_size, py::arg("df"), py::arg("elements") = 1);
    m.def("tile_size_bytes", &tt::tile_size_bytes, py::arg("df"), py::arg("include_header_padding") = true);
    m.def("is_b_data_format", &tt::is_b_data_format);
    m.def("is_a_data_format", &tt::is_a_data_format);
    m.def("to_a_data_format", &tt::to_a_data_format);
    m.def("to_b_data_format", &tt::to_b_data_format);
    m.def("is_integer_data_format", &tt::is_integer_data_format);
    m.def("get_precision_bits", &tt::get_precision_bits);
    m.def("preserve_lower_precision_cast", &tt::preserve_lower_precision_cast);

    py::module m_backend = m.def_submodule("backend_api", "converter entry points of the backend");
    tt::backend_api::BackendModule(m_backend);

    // tile-order model (reference pybuda/csrc/balancer/types.hpp:642-675)
    py::module m_bal = m.def_submodule("balancer", "tile order of queues and core buffers");
    using namespace tt::balancer;
    py::enum_<UBlockOrder>(m_bal, "UBlockOrder").value("R", UBlockOrder::R).value("C", UBlockOrder::C).export_values();
    py::class_<TileLayout>(m_bal, "TileLayout")
        .def(py::init(
                 [](std::pair<int, int> grid, int t, int mblock_m, int mblock_n, std::pair<int, int> ublock, UBlockOrder order)
                 {
                     BlockShape b;
                     b.t = t;
                     b.mblock_m = mblock_m;
                     b.mblock_n = mblock_n;
                     b.ublock = UBlockShape{ublock.first, ublock.second};
                     return TileLayout(GridShape{grid.first, grid.second}, b, order);
                 }),
             py::arg("grid"), py::arg("t"), py::arg("mblock_m"), py::arg("mblock_n"), py::arg("ublock"),
             py::arg("ublock_order") = UBlockOrder::R)
        .def_property_readonly("t", &TileLayout::t)
        .def_property_readonly("rt", &TileLayout::rt)
        .def_property_readonly("ct", &TileLayout::ct)
        .def("volume", &TileLayout::volume)
        .def("map",
             [](TileLayout const &l, int t, int r, int c)
             {
                 const LinCoord lin = l.map(CanCoord{t, r, c});
                 return py::make_tuple(lin.grid_r, lin.grid_c, lin.address);
             })
        .def("unmap",
             [](TileLayout const &l, int grid_r, int grid_c, std::int64_t address)
             {
                 const CanCoord c = l.map(LinCoord{grid_r, grid_c, address});
                 return py::make_tuple(c.t, c.rt, c.ct);
             });
}
