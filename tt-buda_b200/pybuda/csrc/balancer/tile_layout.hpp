// Tile-level order of a queue or core buffer: which grid core owns tile (t, r, c) and at which
// tile address inside that core's buffer.  Host-side twin of the index arithmetic the CUDA
// kernels use; same model as the reference's TileLayout (pybuda/csrc/balancer/types.hpp:642-675,
// types.cpp:621-666) and BlockShape (types.hpp:123-150).
#pragma once

#include <cstdint>

#include "buda_cuda.h"

namespace tt::balancer
{

enum class UBlockOrder : std::uint8_t
{
    R = 0,  // ublocks of a macro-block scanned row-major
    C = 1   // column-major
};

struct GridShape
{
    int r = 1, c = 1;
    int volume() const { return r * c; }
};

struct UBlockShape
{
    int rt = 1, ct = 1;
    int volume() const { return rt * ct; }
};

struct BlockShape
{
    int t = 1, mblock_m = 1, mblock_n = 1;
    UBlockShape ublock;
    int rt() const { return mblock_m * ublock.rt; }
    int ct() const { return mblock_n * ublock.ct; }
    int volume_no_t() const { return mblock_m * mblock_n * ublock.volume(); }
    int volume() const { return t * volume_no_t(); }
};

struct CanCoord  // canonical: position of a tile in the whole tensor
{
    int t = 0, rt = 0, ct = 0;
    bool operator==(CanCoord const &o) const { return t == o.t && rt == o.rt && ct == o.ct; }
};

struct LinCoord  // linear: grid core + tile address in that core's buffer
{
    int grid_r = 0, grid_c = 0;
    std::int64_t address = 0;
    bool operator==(LinCoord const &o) const { return grid_r == o.grid_r && grid_c == o.grid_c && address == o.address; }
};

struct TileLayout
{
    GridShape grid_shape;
    BlockShape block_shape;
    UBlockOrder ublock_order = UBlockOrder::R;

    TileLayout() = default;
    TileLayout(GridShape g, BlockShape b, UBlockOrder o) : grid_shape(g), block_shape(b), ublock_order(o) {}

    int t() const { return block_shape.t; }
    int rt() const { return grid_shape.r * block_shape.rt(); }
    int ct() const { return grid_shape.c * block_shape.ct(); }
    int volume() const { return t() * rt() * ct(); }

    buda_queue_geom geom() const;
    LinCoord map(CanCoord c) const;  // throws std::out_of_range outside the layout
    CanCoord map(LinCoord l) const;
    LinCoord operator[](int idx) const;  // idx walks the tensor t-major, then rows, then columns
};

}  // namespace tt::balancer
