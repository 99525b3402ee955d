#include "balancer/tile_layout.hpp"

#include <stdexcept>

namespace tt::balancer
{

buda_queue_geom TileLayout::geom() const
{
    buda_queue_geom g = {};
    g.grid_r = grid_shape.r;
    g.grid_c = grid_shape.c;
    g.mblock_m = block_shape.mblock_m;
    g.mblock_n = block_shape.mblock_n;
    g.ublock_rt = block_shape.ublock.rt;
    g.ublock_ct = block_shape.ublock.ct;
    g.t = block_shape.t;
    g.ublock_order = ublock_order == UBlockOrder::R ? 0u : 1u;
    return g;
}

LinCoord TileLayout::map(CanCoord c) const
{
    // the forward map is the one the kernels use: ask the C ABI so there is a single definition
    const buda_queue_geom g = geom();
    std::uint32_t cr = 0, cc = 0;
    std::uint64_t addr = 0;
    if (c.t < 0 || c.rt < 0 || c.ct < 0 ||
        buda_tile_map(&g, (std::uint32_t)c.t, (std::uint32_t)c.rt, (std::uint32_t)c.ct, &cr, &cc, &addr) != BUDA_SUCCESS)
        throw std::out_of_range("tile coordinate outside the layout");
    return LinCoord{(int)cr, (int)cc, (std::int64_t)addr};
}

CanCoord TileLayout::map(LinCoord l) const
{
    const std::int64_t uvol = block_shape.ublock.volume();
    const std::int64_t mvol = block_shape.volume_no_t();
    if (l.grid_r < 0 || l.grid_r >= grid_shape.r || l.grid_c < 0 || l.grid_c >= grid_shape.c || l.address < 0 ||
        l.address >= (std::int64_t)block_shape.volume())
        throw std::out_of_range("linear coordinate outside the layout");
    const std::int64_t in_t = l.address % mvol;
    const std::int64_t ublock_index = in_t / uvol;  // position of the ublock in the scan of the macro-block
    const std::int64_t in_u = in_t % uvol;
    int m, n;
    if (ublock_order == UBlockOrder::R)
    {
        m = (int)(ublock_index / block_shape.mblock_n);
        n = (int)(ublock_index % block_shape.mblock_n);
    }
    else
    {
        n = (int)(ublock_index / block_shape.mblock_m);
        m = (int)(ublock_index % block_shape.mblock_m);
    }
    CanCoord c;
    c.t = (int)(l.address / mvol);
    c.rt = l.grid_r * block_shape.rt() + m * block_shape.ublock.rt + (int)(in_u / block_shape.ublock.ct);
    c.ct = l.grid_c * block_shape.ct() + n * block_shape.ublock.ct + (int)(in_u % block_shape.ublock.ct);
    return c;
}

LinCoord TileLayout::operator[](int idx) const
{
    const int per_t = rt() * ct();
    return map(CanCoord{idx / per_t, (idx % per_t) / ct(), idx % ct()});
}

}  // namespace tt::balancer
