"""The reference's (bulk, epilogue) panel split restated on the host, and how it relates to this package's tiling."""
import numpy as np
import pytest

from maize_b200.panels import aligned_panel_split, copy_window, tile_order


@pytest.mark.parametrize("extent,panel,size", [(4096, 16, 256), (4111, 16, 7), (3967, 16, 148), (100, 16, 3),
                                               (15, 16, 4), (0, 16, 2), (4104, 64, 5)])
def test_panels_cover_every_row_exactly_once(extent, panel, size):
    seen = np.zeros(extent, dtype=np.int32)
    for index in range(size):
        split = aligned_panel_split(extent, panel, index, size)
        for lo, hi in split.rows():
            assert 0 <= lo < hi <= extent
            seen[lo:hi] += 1
        assert all(r % panel == 0 for r in split.bulk)
    assert np.all(seen == 1)


def test_demo_shape_has_no_epilogue_and_ragged_shape_does():
    # 4096 rows, 16-row panels, 256 CTAs (the demo, src/main.rs:47-57): nothing is dropped
    assert all(aligned_panel_split(4096, 16, i, 256).epilogue_rows == 0 for i in range(256))
    # 4111 rows: the last 15 rows live in epilogue panels, which the demo discards and this package computes
    dropped = sum(aligned_panel_split(4111, 16, i, 256).epilogue_rows for i in range(256))
    assert dropped == 4111 % (16 * 256) == 15


def test_copy_window_matches_zero_fill_rules():
    rows, counts = copy_window(nrows=4111, ncols=4104, row0=4096, col0=4096, tile_rows=16, tile_cols=16)
    assert rows == 15                      # one row of the tile is past the end: zero-filled
    assert counts == [16, 0]               # columns 4096..4103 are valid (8 x 2 B), 4104.. are not
    rows, counts = copy_window(4111, 3967, 0, 3952, 16, 16)
    assert rows == 16 and counts == [16, 14]   # 7 valid elements in the second copy: 14 bytes, 2 zero-filled
    assert copy_window(10, 10, 32, 0, 16, 16) == (0, [16, 4])
    with pytest.raises(ValueError):
        aligned_panel_split(10, 16, 3, 3)


@pytest.mark.parametrize("tiles_m,tiles_n,group_m", [(64, 64, 8), (17, 16, 8), (33, 16, 16), (1, 5, 8), (7, 1, 16)])
def test_kernel_tile_order_visits_every_tile_once(tiles_m, tiles_n, group_m):
    order = tile_order(tiles_m, tiles_n, group_m)
    assert sorted(order) == [(i, j) for i in range(tiles_m) for j in range(tiles_n)]
    # one group = group_m row-blocks x all column-blocks, visited before the next group starts
    first = order[:group_m * tiles_n]
    assert len({i for i, _ in first}) <= group_m
