"""Host-side restatement of the reference's panel arithmetic, for callers that think in its terms.

The reference cuts a matrix into N-row (or N-column) panels dealt round-robin to the members of a group
(CTAs along ``ctaid.x`` / ``ctaid.y``) and returns, per member, a grid-strided iterator over the "bulk" panels
plus ONE ragged "epilogue" panel (crates/maize_tile/src/gmem/row_panel.rs:95-126, col_panel.rs:95-123); its demo
then drops the epilogue panels (src/main.rs:56-57), which is why it only handles sizes that divide evenly.
The kernels of this package need none of this (TMA zero fill makes every tile uniform), but the same split is
kept here so that the two decompositions can be compared, and tested to cover every row exactly once.

``copy_window`` restates what ``GmemTile::collective_cp_async`` copies and what it zero-fills for a tile that
hangs over the edge of the matrix (gmem_tile.rs:155-181): rows past the end are all zeros, a 16-byte copy that
straddles the last column is cut to its valid bytes and padded with zeros.  A TMA box with zero fill delivers
exactly that.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Tuple


@dataclass(frozen=True)
class PanelSplit:
    """What one group member gets: full panels of ``panel`` rows starting at ``bulk`` and one ragged panel."""
    panel: int
    bulk: Tuple[int, ...]        # first row of every full panel of this member
    epilogue_start: int          # first row of its ragged panel
    epilogue_rows: int           # 0 if it has none

    def rows(self) -> List[Tuple[int, int]]:
        out = [(r, r + self.panel) for r in self.bulk]
        if self.epilogue_rows:
            out.append((self.epilogue_start, self.epilogue_start + self.epilogue_rows))
        return out


def aligned_panel_split(extent: int, panel: int, index: int, size: int) -> PanelSplit:
    """Panels of ``panel`` rows (or columns) of an ``extent``-long axis for member ``index`` of ``size``.

    Follows row_panel.rs:95-126 literally: ``rows_per_iter = size * panel``; the last ``extent % rows_per_iter``
    rows are the epilogue region; member ``index`` walks the bulk from ``index * panel`` in steps of
    ``rows_per_iter`` and owns, of the epilogue region, the piece starting at ``index * panel`` of width
    ``min(epilogue - index * panel, panel)`` if that is positive.
    """
    if panel <= 0 or size <= 0 or not 0 <= index < size or extent < 0:
        raise ValueError("bad panel split arguments")
    rows_per_iter = size * panel
    epilogue = extent % rows_per_iter
    bulk_rows = extent - epilogue
    init_row = index * panel
    bulk = tuple(range(init_row, bulk_rows, rows_per_iter))
    width = min(epilogue - init_row, panel) if init_row < epilogue else 0
    return PanelSplit(panel, bulk, bulk_rows + init_row, width)


def copy_window(nrows: int, ncols: int, row0: int, col0: int, tile_rows: int, tile_cols: int, elem_bytes: int = 2,
                copy_bytes: int = 16):
    """For a tile at (row0, col0): (valid_rows, per-copy valid byte counts of one row).

    ``valid_rows`` rows are copied, the other ``tile_rows - valid_rows`` are zero-filled; within a row each
    ``copy_bytes`` copy moves ``min(max(ncols - col, 0) * elem_bytes, copy_bytes)`` bytes and zero-fills the rest
    (gmem_tile.rs:159-170).
    """
    valid_rows = max(0, min(tile_rows, nrows - row0))
    per_copy = copy_bytes // elem_bytes
    counts = []
    for c in range(col0, col0 + tile_cols, per_copy):
        counts.append(min(max(ncols - c, 0) * elem_bytes, copy_bytes))
    return valid_rows, counts


def tile_order(tiles_m: int, tiles_n: int, group_m: int) -> List[Tuple[int, int]]:
    """The order in which the persistent kernels of this package visit their tiles (``tile_coord`` in
    csrc/gemm_common.cuh): groups of ``group_m`` row-blocks sweep all column-blocks."""
    out = []
    per_group = group_m * tiles_n
    for t in range(tiles_m * tiles_n):
        g = t // per_group
        first_m = g * group_m
        rows = min(tiles_m - first_m, group_m)
        r = t - g * per_group
        out.append((first_m + r % rows, r // rows))
    return out
