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
