// Python bindings of the converter entry points: pybuda._C.backend_api.
//
// Names, argument order, pickling and the status-code convention follow the reference's
// pybuda/csrc/backend_api/backend_api.cpp (descriptors 384-591, status enum 622-625, functions
// 688-726).  What is new here: DramIODesc has a public factory (there is no netlist to read it
// from), and a few helpers expose the device-resident queues.
#include "tt_torch_device/tt_device.hpp"
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <iostream>
#include <stdexcept>

#include "backend_api/backend.hpp"

namespace py = pybind11;

namespace tt::backend_api
{

// The descriptor keeps the Python tensor alive: every copy of it owns one reference, taken and
// dropped through this callback (which may run on a thread that does not hold the GIL).
static void python_handle_refchange(const void *handle_ptr, bool acquire)
{
    py::gil_scoped_acquire gil;
    py::handle handle((PyObject *)handle_ptr);
    if (acquire)
        handle.inc_ref();
    else
        handle.dec_ref();
}

void BackendModule(py::module &m_backend)
{
    py::enum_<tt::DEVICE>(m_backend, "BackendType")
        .value("Model", tt::DEVICE::Model)
        .value("Versim", tt::DEVICE::Versim)
        .value("Silicon", tt::DEVICE::Silicon)
        .value("Golden", tt::DEVICE::Golden)
        .value("Emulation", tt::DEVICE::Emulation)
        .value("NoBackend", tt::DEVICE::Invalid);

    py::enum_<tt::IO_TYPE>(m_backend, "IOType")
        .value("Queue", tt::IO_TYPE::Queue)
        .value("RandomAccess", tt::IO_TYPE::RandomAccess)
        .value("Invalid", tt::IO_TYPE::Invalid);

    py::enum_<tt::IO_LAYOUT>(m_backend, "IOLayout")
        .value("Tilized", tt::IO_LAYOUT::Tilized)
        .value("Flat", tt::IO_LAYOUT::Flat)
        .value("Invalid", tt::IO_LAYOUT::Invalid);

    py::enum_<tt::DEVICE_STATUS_CODE>(m_backend, "BackendStatusCode")
        .value("Success", tt::DEVICE_STATUS_CODE::Success)
        .value("RuntimeError", tt::DEVICE_STATUS_CODE::RuntimeError)
        .value("TimeoutError", tt::DEVICE_STATUS_CODE::TimeoutError);

    py::class_<tt::Stride>(m_backend, "StrideDescriptor")
        .def(py::init<>())
        .def_readwrite("xy_offsets", &tt::Stride::xy_offsets)
        .def_readwrite("stride", &tt::Stride::stride)
        .def(py::pickle([](const tt::Stride &s) { return py::make_tuple(s.xy_offsets, s.stride); },
                        [](py::tuple t)
                        {
                            if (t.size() != 2)
                                throw std::runtime_error("Invalid state for tt::Stride");
                            tt::Stride s;
                            s.xy_offsets = t[0].cast<std::vector<std::pair<int, int>>>();
                            s.stride = t[1].cast<int>();
                            return s;
                        }));

    py::class_<tt::tt_dram_io_desc>(m_backend, "DramIODesc")
        .def_static(
            "for_tensor",
            [](const std::string &name, std::array<std::uint32_t, 4> shape, tt::DataFormat df,
               std::pair<std::uint32_t, std::uint32_t> grid, std::pair<std::uint32_t, std::uint32_t> ublock,
               const std::string &ublock_order, std::uint32_t num_slots, tt::IO_TYPE io_type, bool tile_header,
               std::uint32_t tile_height)
            {
                if (ublock_order != "r" && ublock_order != "c")
                    throw std::runtime_error("ublock_order must be 'r' or 'c'");
                return tt::backend::make_queue_desc(name, shape, df, grid, ublock, ublock_order == "c" ? 1 : 0, num_slots,
                                                    io_type, tile_header, tile_height);
            },
            py::arg("name"), py::arg("shape"), py::arg("data_format"), py::arg("grid") = std::make_pair(1u, 1u),
            py::arg("ublock") = std::make_pair(1u, 1u), py::arg("ublock_order") = "r", py::arg("num_slots") = 0,
            py::arg("io_type") = tt::IO_TYPE::Queue, py::arg("tile_header") = false, py::arg("tile_height") = 32,
            "Descriptor of a queue holding [w, z, R, C] tensors of the given format.  num_slots = 0 sizes the "
            "ring for two pushes of w entries.")
        .def_property_readonly("name", [](tt::tt_dram_io_desc &self) { return self.queue_name; })
        .def_property_readonly("data_format", [](tt::tt_dram_io_desc &self) { return self.bufq_target_format; })
        .def_property_readonly("num_slots", [](tt::tt_dram_io_desc &self) { return self.bufq_num_slots; })
        .def_property_readonly("entry_size", [](tt::tt_dram_io_desc &self) { return self.bufq_entry_size; })
        .def_property_readonly("io_type", [](tt::tt_dram_io_desc &self) { return self.io_type; })
        .def_property_readonly("ublock_order", [](tt::tt_dram_io_desc &self) { return self.ublock_order ? "c" : "r"; })
        .def_property_readonly("tile_header", [](tt::tt_dram_io_desc &self) { return self.tile_header; })
        .def_readwrite("bufq_grid_dim_r", &tt::tt_dram_io_desc::bufq_grid_dim_r)
        .def_readwrite("bufq_grid_dim_c", &tt::tt_dram_io_desc::bufq_grid_dim_c)
        .def_readwrite("ublock_rt", &tt::tt_dram_io_desc::ublock_rt)
        .def_readwrite("ublock_ct", &tt::tt_dram_io_desc::ublock_ct)
        .def_readwrite("mblock_m", &tt::tt_dram_io_desc::mblock_m)
        .def_readwrite("mblock_n", &tt::tt_dram_io_desc::mblock_n)
        .def_readwrite("tile_height", &tt::tt_dram_io_desc::tile_height)
        .def_readwrite("tile_width", &tt::tt_dram_io_desc::tile_width)
        .def_readwrite("t", &tt::tt_dram_io_desc::t)
        .def_readwrite("hstack_factor", &tt::tt_dram_io_desc::hstack_factor)
        .def_readwrite("vstack_factor", &tt::tt_dram_io_desc::vstack_factor)
        .def_readwrite("stack_row_major", &tt::tt_dram_io_desc::stack_row_major)
        .def_readwrite("s_descriptor", &tt::tt_dram_io_desc::s_descriptor)
        .def_readwrite("input_count", &tt::tt_dram_io_desc::input_count)
        .def_readwrite("netlist_path", &tt::tt_dram_io_desc::netlist_path)
        .def(py::pickle(
            [](const tt::tt_dram_io_desc &p)
            {
                // the reference's 23 fields in its order, then the two this build adds
                return py::make_tuple(p.netlist_path, p.queue_name, p.bufq_grid_dim_r, p.bufq_grid_dim_c, p.bufq_num_slots,
                                      p.ublock_rt, p.ublock_ct, p.mblock_m, p.mblock_n, p.tile_height, p.tile_width, p.t,
                                      p.input_count, p.hstack_factor, p.vstack_factor, (std::uint32_t)p.stack_row_major,
                                      p.bufq_target_format, p.bufq_start_addr_channel, p.bufq_entry_size, p.io_type,
                                      p.s_descriptor, p.backend_type, p.layout, p.ublock_order, p.tile_header);
            },
            [](py::tuple t)
            {
                if (t.size() != 23 && t.size() != 25)
                    throw std::runtime_error("tt::tt_dram_io_desc: Invalid state!");
                tt::tt_dram_io_desc p;
                p.netlist_path = t[0].cast<std::string>();
                p.queue_name = t[1].cast<std::string>();
                p.bufq_grid_dim_r = t[2].cast<std::uint32_t>();
                p.bufq_grid_dim_c = t[3].cast<std::uint32_t>();
                p.bufq_num_slots = t[4].cast<std::uint32_t>();
                p.ublock_rt = t[5].cast<std::uint32_t>();
                p.ublock_ct = t[6].cast<std::uint32_t>();
                p.mblock_m = t[7].cast<std::uint32_t>();
                p.mblock_n = t[8].cast<std::uint32_t>();
                p.tile_height = t[9].cast<std::uint32_t>();
                p.tile_width = t[10].cast<std::uint32_t>();
                p.t = t[11].cast<std::uint32_t>();
                p.input_count = t[12].cast<std::uint32_t>();
                p.hstack_factor = t[13].cast<std::uint32_t>();
                p.vstack_factor = t[14].cast<std::uint32_t>();
                p.stack_row_major = t[15].cast<std::uint32_t>() != 0;
                p.bufq_target_format = t[16].cast<tt::DataFormat>();
                p.bufq_start_addr_channel = t[17].cast<std::vector<std::pair<std::uint32_t, std::uint16_t>>>();
                p.bufq_entry_size = t[18].cast<std::uint32_t>();
                p.io_type = t[19].cast<tt::IO_TYPE>();
                p.s_descriptor = t[20].cast<tt::Stride>();
                p.backend_type = t[21].cast<tt::DEVICE>();
                p.layout = t[22].cast<tt::IO_LAYOUT>();
                if (t.size() == 25)
                {
                    p.ublock_order = t[23].cast<std::uint32_t>();
                    p.tile_header = t[24].cast<bool>();
                }
                return p;
            }));

    py::class_<tt::tt_PytorchTensorDesc>(m_backend, "PytorchTensorDesc", py::buffer_protocol())
        .def(py::init([]() { return tt::tt_PytorchTensorDesc(); }))
        .def(py::init(
            [](py::object pytorch_tensor, std::uint32_t itemsize, tt::DataFormat format, std::uint32_t dim,
               std::array<std::uint32_t, 4> shape, std::array<std::uint32_t, 4> strides)
            {
                // an integer is taken as a raw address (no owner); anything else must offer data_ptr()
                if (py::isinstance<py::int_>(pytorch_tensor))
                    return tt::tt_PytorchTensorDesc((const void *)pytorch_tensor.cast<std::uintptr_t>(), itemsize, format,
                                                    shape, strides, dim);
                auto ptr = pytorch_tensor.attr("data_ptr")().cast<std::uint64_t>();
                py::handle handle = pytorch_tensor.release();  // the descriptor now owns this reference
                return tt::tt_PytorchTensorDesc((const void *)ptr, itemsize, format, shape, strides, dim,
                                                (const void *)handle.ptr(), python_handle_refchange);
            }))
        .def_readwrite("itemsize", &tt::tt_PytorchTensorDesc::itemsize)
        .def_readwrite("format", &tt::tt_PytorchTensorDesc::format)
        .def_readwrite("shape", &tt::tt_PytorchTensorDesc::shape)
        .def_readwrite("strides", &tt::tt_PytorchTensorDesc::strides)
        .def_readwrite("dim", &tt::tt_PytorchTensorDesc::dim)
        .def_property_readonly("ptr", [](tt::tt_PytorchTensorDesc &self) { return (std::uintptr_t)self.ptr; })
        .def("print",
             [](tt::tt_PytorchTensorDesc &self)
             {
                 std::cout << "Descriptor: ptr=" << (std::uint64_t)self.ptr << ", itemsize=" << self.itemsize
                           << ", format =" << (int)self.format << ", dim =" << self.dim << ", shape =" << self.shape[0] << ","
                           << self.shape[1] << "," << self.shape[2] << "," << self.shape[3] << ", strides =" << self.strides[0]
                           << "," << self.strides[1] << "," << self.strides[2] << "," << self.strides[3] << std::endl;
             })
        .def_buffer(
            [](tt::tt_PytorchTensorDesc &desc) -> py::buffer_info
            {
                // exported as a 4-D float buffer whatever the format, as the reference does; the
                // consumer (torch.frombuffer) re-reads the bytes with its own dtype
                return py::buffer_info(const_cast<void *>(desc.ptr), desc.itemsize, py::format_descriptor<float>::format(), 4,
                                       {desc.shape[0], desc.shape[1], desc.shape[2], desc.shape[3]},
                                       {desc.strides[0], desc.strides[1], desc.strides[2], desc.strides[3]});
            })
        .def(py::pickle(
            [](const tt::tt_PytorchTensorDesc &t)
            { return py::make_tuple(reinterpret_cast<std::uintptr_t>(t.ptr), t.itemsize, t.format, t.shape, t.strides, t.dim); },
            [](py::tuple t)
            {
                if (t.size() != 6)
                    throw std::runtime_error("tt::tt_PytorchTensorDesc: Invalid state!");
                tt::tt_PytorchTensorDesc p;
                p.ptr = reinterpret_cast<const void *>(t[0].cast<std::uintptr_t>());
                p.itemsize = t[1].cast<std::uint32_t>();
                p.format = t[2].cast<tt::DataFormat>();
                p.shape = t[3].cast<std::array<std::uint32_t, 4>>();
                p.strides = t[4].cast<std::array<std::uint32_t, 4>>();
                p.dim = t[5].cast<std::uint32_t>();
                return p;
            }));

    py::class_<tt::tt_TilizedTensorDesc>(m_backend, "TilizedTensorDesc", py::buffer_protocol())
        .def(py::init<>())
        .def_readwrite("num_buffers", &tt::tt_TilizedTensorDesc::num_buffers)
        .def_readwrite("buf_size_bytes", &tt::tt_TilizedTensorDesc::buf_size_bytes)
        .def_readwrite("format", &tt::tt_TilizedTensorDesc::format)
        .def_property_readonly("ptr", [](tt::tt_TilizedTensorDesc &self) { return (std::uintptr_t)self.ptr; })
        .def("print",
             [](tt::tt_TilizedTensorDesc &self)
             {
                 std::cout << "Descriptor: ptr=" << (std::uint64_t)self.ptr << ", num_buffers=" << self.num_buffers
                           << ", buf_size_bytes=" << self.buf_size_bytes << ", format =" << self.format << std::endl;
             })
        .def_buffer(
            [](tt::tt_TilizedTensorDesc &d) -> py::buffer_info
            {
                if (!d.ptr)
                    throw std::runtime_error("TilizedTensorDesc holds no data");
                return py::buffer_info(const_cast<void *>(d.ptr), 1, py::format_descriptor<std::uint8_t>::format(), 1,
                                       {(py::ssize_t)d.total_bytes()}, {(py::ssize_t)1});
            })
        .def(py::pickle([](const tt::tt_TilizedTensorDesc &t) { return py::make_tuple(t.num_buffers, t.buf_size_bytes, t.format); },
                        [](py::tuple t)
                        {
                            if (t.size() != 3)
                                throw std::runtime_error("tt::tt_TilizedTensorDesc: Invalid state!");
                            tt::tt_TilizedTensorDesc d;
                            d.ptr = nullptr;
                            d.num_buffers = t[0].cast<std::uint32_t>();
                            d.buf_size_bytes = t[1].cast<std::uint32_t>();
                            d.format = t[2].cast<tt::DataFormat>();
                            return d;
                        }));

    using namespace tt::backend;
    m_backend.def("push_input",
                  py::overload_cast<const tt::tt_dram_io_desc &, const tt::tt_PytorchTensorDesc &, const bool, const int,
                                    const int>(&push_input),
                  py::call_guard<py::gil_scoped_release>());
    m_backend.def("push_input",
                  py::overload_cast<const tt::tt_dram_io_desc &, const tt::tt_TilizedTensorDesc &, const int, const int>(
                      &push_input),
                  py::call_guard<py::gil_scoped_release>());
    py::enum_<tt::SOURCE_VIEW>(m_backend, "SourceViewMode")
        .value("Padded", tt::SOURCE_VIEW::Padded)
        .value("EmbeddingIndex", tt::SOURCE_VIEW::EmbeddingIndex)
        .value("Prestride", tt::SOURCE_VIEW::Prestride);
    py::class_<tt::tt_SourceView>(m_backend, "SourceView")
        .def(py::init<>())
        .def_readwrite("mode", &tt::tt_SourceView::mode)
        .def_readwrite("broadcast_rows", &tt::tt_SourceView::broadcast_rows)
        .def_readwrite("broadcast_cols", &tt::tt_SourceView::broadcast_cols)
        .def_readwrite("count", &tt::tt_SourceView::count)
        .def_readwrite("group", &tt::tt_SourceView::group)
        .def_readwrite("stride", &tt::tt_SourceView::stride);
    m_backend.def("push_input_view", &push_input_view, py::call_guard<py::gil_scoped_release>(), py::arg("queue"), py::arg("tensor"),
                  py::arg("view"), py::arg("push_one"), py::arg("timeout_in_seconds"), py::arg("ram_ptr"),
                  "push_input of a tensor that a runtime tensor transform stands in front of: the pack kernel reads it through the view");
    m_backend.def("push_input_batch", &push_input_batch, py::call_guard<py::gil_scoped_release>(), py::arg("queues"), py::arg("tensors"),
                  py::arg("push_one"), py::arg("timeout_in_seconds"), py::arg("ram_ptrs") = std::vector<int>{},
                  "push_input for a whole set of (queue, tensor) pairs: one conversion launch per format combination");
    m_backend.def("pop_output", &pop_output, py::call_guard<py::gil_scoped_release>());
    m_backend.def("get_output", &get_output, py::call_guard<py::gil_scoped_release>());
    m_backend.def("free_tensor", py::overload_cast<tt::tt_PytorchTensorDesc &>(&free_tensor));
    m_backend.def("free_tensor", py::overload_cast<tt::tt_TilizedTensorDesc &>(&free_tensor));
    m_backend.def("tilize_tensor", &tilize_tensor, py::call_guard<py::gil_scoped_release>());
    m_backend.def("binarize_tensor", py::overload_cast<const tt::tt_PytorchTensorDesc &, const std::string &>(&binarize_tensor));
    m_backend.def("binarize_tensor", py::overload_cast<const tt::tt_TilizedTensorDesc &, const std::string &>(&binarize_tensor));
    m_backend.def("debinarize_tensor", py::overload_cast<tt::tt_PytorchTensorDesc &, const std::string &>(&debinarize_tensor));
    m_backend.def("debinarize_tensor", py::overload_cast<tt::tt_TilizedTensorDesc &, const std::string &>(&debinarize_tensor));

    // argument names as the reference spells them (backend_api.cpp:710-722)
    m_backend.def("get_io_size_in_bytes", &get_io_size_in_bytes, py::arg("data_formati"), py::arg("is_untilizesd"),
                  py::arg("ublock_ct"), py::arg("ublock_rt"), py::arg("mblock_m"), py::arg("mblock_n"), py::arg("t"),
                  py::arg("entries"), py::arg("tile_height") = 32, py::arg("tile_width") = 32);
    m_backend.def("get_next_aligned_address", &get_next_aligned_address);
    m_backend.def("translate_addresses", &translate_addresses, py::call_guard<py::gil_scoped_release>());
    m_backend.def("get_format_from_string", &tt::get_format_from_string, py::arg("format_str"));

    // device-resident queues are this build's own: inspection and release
    m_backend.def("queue_device_address", &queue_device_address);
    m_backend.def("queue_occupancy", &queue_occupancy);
    m_backend.def("release_queue", &release_queue);
    m_backend.def("release_all_queues", &release_all_queues);
    m_backend.def("last_error", &last_error);
    m_backend.def(
        "to_pytorch_tensor_desc",
        [](std::uintptr_t data, std::uint32_t element_size, tt::DataFormat format, const std::vector<std::int64_t> &sizes,
           const std::vector<std::int64_t> &strides)
        { return tt::to_pytorch_tensor_desc(reinterpret_cast<const void *>(data), element_size, format, sizes, strides); },
        py::arg("data_ptr"), py::arg("element_size"), py::arg("format"), py::arg("sizes"), py::arg("strides"),
        "Descriptor of a tensor of up to 4 dims by the rules of the reference's torch device plugin (borrowed pointer).");
    m_backend.def("buda_padded_shape", &tt::buda_padded_shape, py::arg("sizes"));
    m_backend.def("matmul_bfp8b", &matmul_bfp8b, py::call_guard<py::gil_scoped_release>());
}

}  // namespace tt::backend_api
