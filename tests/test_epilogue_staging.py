"""Host model of the GEMM epilogue's staging area (``stage_put_* / stage_flush_*`` in ``csrc/ptx_sm100.cuh``): a warp's
32 rows x 128 bytes go into shared memory lane = row, 16-byte pieces XOR-swizzled by row, and come back eight lanes per row.
Checked here, with the kernel's index arithmetic restated: every piece is written once and read back as the piece of the
row and column it belongs to, no two lanes of an 8-lane phase (one shared-memory wavefront of 16-byte accesses) touch the
same 16-byte bank group, and one flush instruction covers whole 128-byte rows."""
import numpy as np
import pytest


def put_offsets(kind):
    """(lane, piece) -> byte offset in the 4 KB staging area, in the order the kernel writes them.  bf16: two calls of four
    pieces (``half``), f32: one call of eight."""
    out = []
    if kind == "bf16":
        for half in range(2):
            for q in range(4):
                out.append([(lane, half * 4 + q, lane * 128 + (((half * 4 + q) ^ (lane & 7)) * 16)) for lane in range(32)])
    else:
        for q in range(8):
            out.append([(lane, q, lane * 128 + ((q ^ (lane & 7)) * 16)) for lane in range(32)])
    return out


def flush_offsets():
    """Per flush instruction i: (lane, row, piece, byte offset read)."""
    out = []
    for i in range(8):
        ins = []
        for lane in range(32):
            piece, rr = lane & 7, i * 4 + (lane >> 3)
            ins.append((lane, rr, piece, rr * 128 + ((piece ^ (rr & 7)) * 16)))
        out.append(ins)
    return out


def conflict_free(offsets):
    """16-byte accesses are served eight lanes at a time; the eight must fall into eight different 16-byte bank groups."""
    for phase in range(4):
        groups = {(off // 16) % 8 for off in offsets[phase * 8:(phase + 1) * 8]}
        if len(groups) != 8:
            return False
    return True


@pytest.mark.parametrize("kind", ["bf16", "f32"])
def test_every_piece_lands_where_the_flush_reads_it(kind):
    where = {}
    for ins in put_offsets(kind):
        assert conflict_free([off for _, _, off in ins])
        for lane, piece, off in ins:
            assert off not in where and 0 <= off < 4096 and off % 16 == 0
            where[off] = (lane, piece)                       # lane = row of the accumulator
    assert len(where) == 256                                 # 32 rows x 8 pieces of 16 bytes
    seen = set()
    for ins in flush_offsets():
        assert conflict_free([off for *_, off in ins])
        rows = sorted({rr for _, rr, _, _ in ins})
        assert len(rows) == 4                                # one instruction: four complete rows
        for lane, rr, piece, off in ins:
            assert where[off] == (rr, piece)                 # the piece of that row and column
            seen.add((rr, piece))
        for rr in rows:
            assert sorted(p for _, r, p, _ in ins if r == rr) == list(range(8))      # all 128 bytes of the row
    assert len(seen) == 256


def test_values_round_trip_like_the_kernel():
    """Numbers instead of offsets: a 32 x 64 bf16 tile (as uint16) through the bf16 path, a 32 x 32 f32 tile through the f32 path."""
    rng = np.random.default_rng(0)
    tile16 = rng.integers(0, 65535, size=(32, 64), dtype=np.uint16)
    stg = np.zeros(4096, dtype=np.uint8)
    for half in range(2):
        for q in range(4):
            for lane in range(32):
                off = lane * 128 + (((half * 4 + q) ^ (lane & 7)) * 16)
                stg[off:off + 16] = tile16[lane, half * 32 + q * 8: half * 32 + q * 8 + 8].view(np.uint8)
    out = np.zeros_like(tile16)
    for i in range(8):
        for lane in range(32):
            piece, rr = lane & 7, i * 4 + (lane >> 3)
            off = rr * 128 + ((piece ^ (rr & 7)) * 16)
            out[rr, piece * 8: piece * 8 + 8] = stg[off:off + 16].view(np.uint16)
    assert np.array_equal(out, tile16)
    tile32 = rng.standard_normal((32, 32)).astype(np.float32)
    stg[:] = 0
    for q in range(8):
        for lane in range(32):
            off = lane * 128 + ((q ^ (lane & 7)) * 16)
            stg[off:off + 16] = tile32[lane, q * 4: q * 4 + 4].view(np.uint8)
    out32 = np.zeros_like(tile32)
    for i in range(8):
        for lane in range(32):
            piece, rr = lane & 7, i * 4 + (lane >> 3)
            off = rr * 128 + ((piece ^ (rr & 7)) * 16)
            out32[rr, piece * 4: piece * 4 + 4] = stg[off:off + 16].view(np.float32)
    assert np.array_equal(out32, tile32)
