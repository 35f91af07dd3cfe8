"""Host restatement of the index arithmetic of the weight-gather GEMM (``csrc/gemm_tcgen05.cu``, epilogue mode 5): which
16-byte vectors a (block, part) copy unit moves, which rank owns each of them, where the copies and the consumer's k-blocks /
tiles start.  Checked for coverage: every vector of the weight is copied exactly once, from inside its owner's shard."""
import itertools

import pytest

ROWS_PER_BLOCK, BN = 64, 256


def plan(rows, cols, flat_off, shard_elems, world, me, on_k, grid):
    """What ``dttt_gemm_wg_bf16`` decides on the host: (rot, n_rotate, parts)."""
    nblk = -(-rows // ROWS_PER_BLOCK)
    blk_elems = ROWS_PER_BLOCK * cols
    own_lo, own_hi = me * shard_elems, (me + 1) * shard_elems
    w_lo, w_hi = flat_off, flat_off + rows * cols
    if own_lo < w_hi and own_hi > w_lo:
        rot = -(-(own_lo - w_lo) // blk_elems) if own_lo > w_lo else 0
    else:
        rot = me * nblk // world
    if rot >= nblk:
        rot = 0
    n_rotate = 0
    if not on_k:
        n_rotate = rot * ROWS_PER_BLOCK // BN
        rot = n_rotate * (BN // ROWS_PER_BLOCK)
    parts = -(-grid // nblk)
    vec_per_blk = blk_elems // 8
    while parts > 1 and vec_per_blk // parts < 1024:
        parts -= 1
    return rot, n_rotate, max(1, min(16, parts))


def copy_units(rows, cols, flat_off, shard_elems, rot, parts, grid):
    """Yields (cta, block, [(vector index in the weight, owner rank, vector offset inside the owner's shard)])."""
    nblk = -(-rows // ROWS_PER_BLOCK)
    vec_per_blk = ROWS_PER_BLOCK * cols // 8
    vec_total = rows * cols // 8
    shard_vecs, flat0 = shard_elems // 8, flat_off // 8
    vec_per_part = -(-vec_per_blk // parts)
    for cta in range(grid):
        for i in range(cta, nblk * parts, grid):
            blk = i // parts + rot
            part = i % parts
            if blk >= nblk:
                blk -= nblk
            b_lo = blk * vec_per_blk
            v_lo = b_lo + part * vec_per_part
            v_hi = min(v_lo + vec_per_part, b_lo + vec_per_blk, vec_total)
            yield cta, blk, [(v, (flat0 + v) // shard_vecs, (flat0 + v) % shard_vecs) for v in range(v_lo, v_hi)]


@pytest.mark.parametrize("rows,cols", [(256, 512), (1024, 384), (192, 72), (512, 2048), (64, 4096)])
@pytest.mark.parametrize("world", [2, 8])
@pytest.mark.parametrize("on_k", [0, 1])
def test_every_vector_is_copied_once_from_its_owner(rows, cols, world, on_k):
    # the weight sits somewhere in a flat space of three such weights, cut evenly
    for flat_off in (0, 64 * ((rows * cols) // 64), 64 * ((5 * rows * cols // 3) // 64)):
        total = -(-(3 * rows * cols + flat_off) // (64 * world)) * 64 * world
        shard = total // world
        for me, grid in itertools.product(range(world), (7, 148)):
            rot, n_rotate, parts = plan(rows, cols, flat_off, shard, world, me, on_k, grid)
            nblk = -(-rows // ROWS_PER_BLOCK)
            assert 0 <= rot < nblk and 1 <= parts <= 16
            if not on_k:
                assert rot % (BN // ROWS_PER_BLOCK) == 0 and 0 <= n_rotate < max(1, -(-rows // BN))
            seen = [0] * (rows * cols // 8)
            per_block = {}
            for cta, blk, vecs in copy_units(rows, cols, flat_off, shard, rot, parts, grid):
                per_block[blk] = per_block.get(blk, 0) + 1
                for v, owner, off in vecs:
                    seen[v] += 1
                    assert 0 <= owner < world and 0 <= off < shard // 8
                    assert owner * (shard // 8) + off == flat_off // 8 + v          # the vector's flat position
            assert all(c == 1 for c in seen)
            assert per_block == {b: parts for b in range(nblk)}                        # the ready word's count: `parts` arrivals
            # the copies begin where this rank's own part of the weight begins (when it owns one that starts inside it)
            first_block = next(copy_units(rows, cols, flat_off, shard, rot, parts, grid))[1]
            assert first_block == rot
