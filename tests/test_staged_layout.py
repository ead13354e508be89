"""The B200 staged layout on the host: the oracle's repack against the layout's definition, and the library's size
function (no device work)."""
import numpy as np
import pytest

from oracle import api
from tessl_b200 import nn, synth


@pytest.mark.parametrize("rows,cols,group", [(16, 4096, 64), (13, 1024, 32), (5, 2048, 128), (1000, 4096, 128), (8, 1024, 64)])
def test_the_staged_image_holds_every_row_where_the_layout_says(rows, cols, group):
    packed, sb = synth.q4_bank(0x57A6 + rows, rows, cols, group)
    img = api.q4_repack_b200_staged(packed, sb, rows, cols, group)
    row_bytes, sb_row = cols // 2, (cols // group) * 4
    pair_pitch = 2 * row_bytes + 32
    unit = 4 * pair_pitch + 8 * sb_row
    assert img.size == ((rows + 7) // 8) * unit == nn.q4_mlx_staged_bytes(rows, cols, group)
    pb, sbb = packed.view(np.uint8).reshape(rows, row_bytes), sb.view(np.uint8).reshape(rows, sb_row)
    covered = np.zeros(img.size, bool)
    for r in range(rows):
        u, l = divmod(r, 8)
        o = u * unit + (l // 2) * pair_pitch + (l % 2) * row_bytes
        assert np.array_equal(img[o:o + row_bytes], pb[r])
        covered[o:o + row_bytes] = True
        o = u * unit + 4 * pair_pitch + l * sb_row
        assert np.array_equal(img[o:o + sb_row], sbb[r])
        covered[o:o + sb_row] = True
    assert not img[~covered].any(), "pads and rows past the end are zeros"


def test_the_size_function_knows_the_domain():
    assert nn.q4_mlx_staged_bytes(0, 4096, 64) == 0
    assert nn.q4_mlx_staged_bytes(1, 4096, 64) == 4 * (4096 + 32) + 8 * 256
    for cols, group in ((1536, 64), (8192, 64), (4096, 256), (1024, 128), (512, 32)):
        assert nn.q4_mlx_staged_bytes(64, cols, group) == 0
