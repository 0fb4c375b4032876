"""Index arithmetic of the persistent grouped-GEMM kernel's tile walk, restated on the CPU.

`build_tile_table` and `decode_tile` in scattermoe_b200/csrc/gemm_tc.cu map a linear tile number to (expert, row
tile, column tile): experts by a prefix sum of their tile counts, inside an expert groups of `group_m` row tiles with
the column tiles between them, and (for launches whose rows leave for other ranks) the row tiles of every expert
rotated by rank / world. The functions below follow that code line by line; the tests check the property the kernel
relies on: whatever the segment sizes, the raster group and the rotation, the walk visits every tile of every expert
exactly once and never a tile outside a segment. (Replaces the reference's `tl.program_id` decomposition,
scattermoe/kernels/ops.py:52-60, whose padded block index list has no counterpart here.)"""
import itertools

import pytest

BM = 128


def build_tile_table(offsets, R, units_per_mtile):
    seg_start = [0]
    for v in offsets:
        seg_start.append(min(max(v, 0), R))
    tile_prefix = [0]
    for e in range(len(offsets)):
        cnt = max(0, seg_start[e + 1] - seg_start[e])
        tile_prefix.append(tile_prefix[-1] + ((cnt + BM - 1) // BM) * units_per_mtile)
    return seg_start, tile_prefix


def decode_tile(t, tile_prefix, seg_start, E, BN, group_m, rot_num=0, rot_den=1):
    lo, hi = 0, E
    while hi - lo > 1:
        mid = (lo + hi) >> 1
        if tile_prefix[mid] <= t:
            lo = mid
        else:
            hi = mid
    local = t - tile_prefix[lo]
    cnt = seg_start[lo + 1] - seg_start[lo]
    m_tiles = (cnt + BM - 1) // BM
    n_tiles_e = (tile_prefix[lo + 1] - tile_prefix[lo]) // m_tiles
    gm = max(1, min(group_m, m_tiles))
    per_group = gm * n_tiles_e
    grp = local // per_group
    in_grp = local - grp * per_group
    gw = min(gm, m_tiles - grp * gm)
    n_tile = in_grp // gw
    m_tile = grp * gm + (in_grp - n_tile * gw)
    if rot_num > 0:
        m_tile += m_tiles * rot_num // rot_den
        if m_tile >= m_tiles:
            m_tile -= m_tiles
    m0 = seg_start[lo] + m_tile * BM
    rows = min(BM, seg_start[lo + 1] - m0)
    return lo, m0, rows, n_tile * BN


SEGMENTS = {
    "even": [512, 512, 512, 512],
    "ragged": [130, 0, 301, 57, 200, 1, 0, 128],
    "one_takes_all": [0, 0, 4097, 0],
    "empty": [0, 0, 0],
    "single_partial_tile": [5],
    "long": [128 * 37 + 3, 128 * 2, 9],
}


@pytest.mark.parametrize("rot", [(0, 1), (1, 2), (3, 8), (7, 8)], ids=lambda r: "rot%d_%d" % r)
@pytest.mark.parametrize("group_m", [1, 3, 16, 1 << 20])
@pytest.mark.parametrize("BN,N", [(256, 256), (256, 1000), (128, 128), (256, 4096)])
@pytest.mark.parametrize("name", sorted(SEGMENTS))
def test_every_tile_once(name, BN, N, group_m, rot):
    counts = SEGMENTS[name]
    offsets = list(itertools.accumulate(counts))
    R, E = sum(counts), len(counts)
    n_tiles = (N + BN - 1) // BN
    seg_start, tile_prefix = build_tile_table(offsets, R, n_tiles)
    total = tile_prefix[E]
    assert total == sum(((c + BM - 1) // BM) * n_tiles for c in counts)
    seen = set()
    for t in range(total):
        e, m0, rows, n0 = decode_tile(t, tile_prefix, seg_start, E, BN, group_m, *rot)
        assert counts[e] > 0 and seg_start[e] <= m0 < seg_start[e + 1]
        assert (m0 - seg_start[e]) % BM == 0 and 1 <= rows <= BM and m0 + rows <= seg_start[e + 1]
        assert 0 <= n0 < N and n0 % BN == 0
        seen.add((e, m0, n0))
    assert len(seen) == total                    # no tile twice, hence (equal counts) none missing


def test_offsets_outside_the_row_count_are_clamped():
    """Malformed offsets (negative, beyond R) must not produce tiles outside [0, R): the kernel clamps them."""
    seg_start, tile_prefix = build_tile_table([-5, 100, 9999, 9999], 300, 2)
    assert seg_start == [0, 0, 100, 300, 300]
    for t in range(tile_prefix[-1]):
        e, m0, rows, _ = decode_tile(t, tile_prefix, seg_start, 4, 256, 16)
        assert 0 <= m0 and m0 + rows <= 300


def test_rotation_starts_each_rank_at_its_own_sender():
    """With rows ordered by the rank they return to and an even load, rank r's first row tile of an expert lies in
    the rows that return to rank r: at any moment the owners address different receivers."""
    world, per_sender = 8, 512                       # 8 senders x 512 rows = 32 row tiles per expert
    seg_start, tile_prefix = build_tile_table([world * per_sender], world * per_sender, 1)
    for r in range(world):
        _, m0, _, _ = decode_tile(0, tile_prefix, seg_start, 1, 256, 1 << 20, r, world)
        assert m0 // per_sender == r
