"""Token-row sharding of a linear across the GPUs of one box.

Rows of a linear are independent, weights are replicated, so rank g of G owns a
contiguous row range and no collective is needed: the concatenation of the
per-rank outputs is bit-identical to the single-GPU output.  Boundaries are
rounded to multiples of 128 rows (the kernel's row tile) where the row count
allows, so that no rank pays a second partial tile.
"""


def row_range(rows, rank, world, tile=128):
    """[begin, end) of the rows owned by `rank`; ranges partition [0, rows)."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError("rank out of range")

    def boundary(i):
        exact = rows * i // world
        if i in (0, world):
            return exact
        rounded = (exact + tile // 2) // tile * tile
        return min(max(rounded, 0), rows)

    begin, end = boundary(rank), boundary(rank + 1)
    return begin, max(begin, end)


def all_ranges(rows, world, tile=128):
    return [row_range(rows, r, world, tile) for r in range(world)]


def blob_slices(total_bytes, world, align=256):
    """(padded_bytes, piece_bytes): a streamed layer blob cut into `world` equal, `align`-byte aligned slices
    (one per rank over PCIe, assembled by an all-gather); padded_bytes = world * piece_bytes >= total_bytes."""
    if world < 1 or total_bytes < 0:
        raise ValueError("invalid blob split")
    unit = world * align
    padded = (total_bytes + unit - 1) // unit * unit
    return padded, padded // world


def feature_range(features, rank, world, tile=128):
    """[begin, end) of the FFN features owned by `rank` in the tensor-parallel FFN: the rows of the FFN-up
    weight (column-parallel, activation local) and the matching K-slice of the FFN-down weight (row-parallel,
    partial sums all-reduced).  Boundaries are multiples of `tile` so every slice keeps whole k-blocks."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError("rank out of range")
    if features % (tile * world):
        raise ValueError("FFN width must be a multiple of tile * world")
    width = features // world
    return rank * width, (rank + 1) * width


def reduce_chunks(rows, chunks, world, quantum=8):
    """Row chunks [begin, end) of the tensor-parallel FFN's reduction: the partial sums of a chunk are reduce-scattered,
    every rank finishes rows/world of it and the results are all-gathered while the next chunk computes.  Every chunk
    is a multiple of `quantum * world` rows (a rank's share is then whole and keeps 16-byte aligned rows) except the
    last, which takes the remainder and must still divide by `world`."""
    if world < 1 or chunks < 1 or rows < 1:
        raise ValueError("invalid chunking")
    unit = quantum * world
    per_chunk = max(unit, rows // chunks // unit * unit)
    bounds = [min(rows, c * per_chunk) for c in range(chunks)] + [rows]
    out = [(b, e) for b, e in zip(bounds, bounds[1:]) if e > b]
    if any((e - b) % world for b, e in out):
        raise ValueError("rows must be a multiple of the rank count")
    return out
