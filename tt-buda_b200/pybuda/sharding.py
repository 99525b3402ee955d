"""How the data-format path spreads over the GPUs of one box: one process per GPU, independent
units (tensors, layers, tile-row bands) dealt round-robin, no collective on the data path.  The only
exchange step on the whole path is the all-gather of the column-parallel matmul outputs
(parallel_matmul.py)."""
from typing import List, Sequence, Tuple


def units_of_rank(n_units: int, rank: int, world: int) -> List[int]:
    """Unit u belongs to rank u % world (tensor i -> GPU i mod g, layer l -> GPU l mod g)."""
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside a world of {world}")
    return list(range(rank, n_units, world))


def bands_of_rank(tile_rows: int, rank: int, world: int) -> Tuple[int, int, int]:
    """Tile-row bands of ONE tensor dealt over the GPUs: band b (32 tensor rows across the whole width) belongs to
    rank b % world.  Returns (first, step, count), the selection the job-table entry points take
    (buda_tensor_job.band_first / band_step / band_count); count is 0 for a rank that gets nothing."""
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside a world of {world}")
    return rank, world, len(range(rank, tile_rows, world))


def band_record_slice(band: int, tile_rows: int, tile_cols: int, tile_bytes: int, z: int = 0, entry: int = 0,
                      t: int = 1) -> Tuple[int, int]:
    """(offset, length) in bytes of the records of tile row `band` of slice z of entry `entry` inside the queue image,
    for a 1x1 grid with 1x1 ublocks scanned row-major: there a band's records are one contiguous run -- tile (z, r, c)
    sits at address z * rows * cols + r * cols + c (TileLayout::map, pybuda/csrc/balancer/types.cpp:629-648).  With
    any other geometry a band is scattered over the image and the kernels place each record themselves."""
    if not (0 <= band < tile_rows and 0 <= z < t):
        raise ValueError("band or slice outside the tensor")
    first_tile = (entry * t + z) * tile_rows * tile_cols + band * tile_cols
    return first_tile * tile_bytes, tile_cols * tile_bytes


def band_slices(rows: int, bands: int, multiple: int = 32) -> List[Tuple[int, int]]:
    """Split `rows` into at most `bands` contiguous (start, stop) row ranges whose sizes are multiples of
    `multiple` (the last one takes the remainder)."""
    if rows <= 0 or bands <= 0:
        return []
    per = -(-rows // bands)
    per = -(-per // multiple) * multiple
    out, r = [], 0
    while r < rows:
        out.append((r, min(rows, r + per)))
        r += per
    return out


def column_shard(n_cols: int, rank: int, world: int, multiple: int = 256) -> Tuple[int, int]:
    """Columns [start, stop) of a [K, N] weight held by `rank` in a column-parallel matmul."""
    if n_cols % (world * multiple):
        raise ValueError(f"{n_cols} columns do not split into {world} shards of a multiple of {multiple}")
    per = n_cols // world
    return rank * per, (rank + 1) * per


def gather_layout_to_row_major(gathered, out):
    """all_gather leaves [world, rows, cols_per_rank]; the row-major result is [rows, world * cols_per_rank]."""
    world, rows, per = gathered.shape
    out.view(rows, world, per).copy_(gathered.permute(1, 0, 2))
    return out
