"""Host model of the GEMM kernels' tile order (``tile_coords`` in ``csrc/gemm_tcgen05.cu`` and ``csrc/gemm_pair_tcgen05.cu``):
tiles are numbered in bands of GROUP row tiles with the column tile varying slowest inside a band, optionally rotated
in m (reduce-scatter: start at the own rows) or n (weight gather: start at the own columns).  Every persistent CTA walks
``tile = blockIdx.x, blockIdx.x + gridDim.x, ...``; the order must be a bijection onto (batch, m tile, n tile), and
concurrently running CTAs (consecutive tile numbers) should share row tiles so that A is re-read from L2."""
import itertools

import pytest


def tile_coords(tile, tiles_m, tiles_n, group, m_rotate=0, n_rotate=0):
    per_batch = tiles_m * tiles_n
    b, t = divmod(tile, per_batch)
    band = t // (group * tiles_n)
    first_m = band * group
    rows = min(group, tiles_m - first_m)
    r = t - band * group * tiles_n
    tm, tn = first_m + (r % rows), r // rows
    if m_rotate:
        tm = (tm + m_rotate) % tiles_m
    if n_rotate:
        tn = (tn + n_rotate) % tiles_n
    return b, tm, tn


@pytest.mark.parametrize("group", [16, 8])
@pytest.mark.parametrize("tiles_m,tiles_n,batch", [(1, 1, 1), (16, 32, 1), (384, 8, 1), (17, 5, 3), (7, 501, 2), (33, 1, 4)])
@pytest.mark.parametrize("rot", [(0, 0), (5, 0), (0, 3)])
def test_every_tile_is_visited_once(group, tiles_m, tiles_n, batch, rot):
    m_rot, n_rot = rot[0] % tiles_m, rot[1] % tiles_n
    seen = {tile_coords(t, tiles_m, tiles_n, group, m_rot, n_rot) for t in range(batch * tiles_m * tiles_n)}
    assert seen == set(itertools.product(range(batch), range(tiles_m), range(tiles_n)))


def test_a_wave_of_ctas_shares_few_row_tiles():
    """148 consecutive tiles of the prefix projection (384 x 32 tiles of 128 x 256) touch at most 2 bands of 16 row tiles
    and 10 + 1 column tiles: each A tile is wanted by about ten CTAs at a time, each B tile by sixteen."""
    tiles_m, tiles_n = 384, 32
    for start in (0, 148, 5 * 148, 40 * 148):
        wave = [tile_coords(t, tiles_m, tiles_n, 16) for t in range(start, start + 148)]
        assert len({tm // 16 for _, tm, _ in wave}) <= 2
        assert len({tn for _, _, tn in wave}) <= 11
