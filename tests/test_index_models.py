"""Index arithmetic of the kernels restated on the CPU, where every case can be enumerated.

Each function below repeats a formula from a kernel (file and function named beside it) and the
tests enumerate its whole domain: that a tile schedule visits every tile exactly once, that a
shared-memory swizzle is a bijection and free of bank conflicts for the access patterns the kernel
uses, that the planes of the fp8 window never overlap. They guard the formulas, not the compiled
code; the GPU tests compare the kernels' results with PyTorch.
"""

import itertools

import pytest

BAND, PAIR_BAND = 16, 8  # gemm_sm100.cuh


def tile_coords(tiles_m, tiles_n, t):  # gemm_sm100.cuh: tile_coords
    band_tiles = BAND * tiles_n
    band = t // band_tiles
    r = t - band * band_tiles
    rows = min(BAND, tiles_m - band * BAND)
    nt = r // rows
    return band * BAND + (r - nt * rows), nt


def pair_tile_coords(tiles_m2, tiles_n, t):  # gemm_sm100.cuh: pair_tile_coords
    band_tiles = PAIR_BAND * tiles_n
    band = t // band_tiles
    r = t - band * band_tiles
    rows = min(PAIR_BAND, tiles_m2 - band * PAIR_BAND)
    nt = r // rows
    return band * PAIR_BAND + (r - nt * rows), nt


@pytest.mark.parametrize("tiles_m,tiles_n", [(1, 1), (16, 20), (17, 3), (74, 60), (148, 20), (33, 1), (5, 7)])
def test_every_tile_is_visited_exactly_once(tiles_m, tiles_n):
    seen = [tile_coords(tiles_m, tiles_n, t) for t in range(tiles_m * tiles_n)]
    assert sorted(seen) == sorted(itertools.product(range(tiles_m), range(tiles_n)))
    # a wave of consecutive tiles stays inside one band of M-tiles as long as the band lasts: L2 reuse
    first_band = [mt for mt, _ in seen[: min(BAND, tiles_m) * tiles_n]]
    assert max(first_band) < BAND


@pytest.mark.parametrize("tiles_m,tiles_n", [(1, 1), (16, 20), (17, 3), (74, 60), (149, 20), (33, 1)])
def test_every_pair_tile_and_both_halves_are_visited_exactly_once(tiles_m, tiles_n):
    tiles_m2 = (tiles_m + 1) // 2
    seen = []
    for t in range(tiles_m2 * tiles_n):
        mt2, nt = pair_tile_coords(tiles_m2, tiles_n, t)
        for half in (0, 1):  # the two CTAs of the pair: rows (mt2 * 2 + half) * 128 ...
            seen.append((mt2 * 2 + half, nt))
    inside = [x for x in seen if x[0] < tiles_m]
    assert sorted(inside) == sorted(itertools.product(range(tiles_m), range(tiles_n)))
    assert len(seen) - len(inside) == (tiles_m % 2) * tiles_n  # an odd M leaves the odd CTA one empty row block per column


def stage_unit(row, unit):  # gemm_sm100.cu: QkvEpi::tile, the staging buffer's XOR swizzle
    return row * 16 + (unit ^ (row & 15))  # 16-byte units; a row is 256 bytes = 16 units


def test_staging_swizzle_is_a_bijection_and_what_is_written_is_what_is_read():
    cells = {stage_unit(row, u) for row in range(32) for u in range(16)}
    assert cells == set(range(32 * 16))
    # writer: lane = row, four chunks of four units; reader: iteration i, lane l reads row 2 i + l // 16, unit l % 16
    written = {(row, chunk * 4 + q): stage_unit(row, chunk * 4 + q) for row in range(32) for chunk in range(4) for q in range(4)}
    for i in range(16):
        for lane in range(32):
            row, unit = 2 * i + lane // 16, lane % 16
            assert stage_unit(row, unit) == written[(row, unit)]


def banks(cell):  # a 16-byte unit covers four consecutive 4-byte banks
    return {(cell * 4 + k) % 32 for k in range(4)}


def test_staging_swizzle_has_no_bank_conflicts_for_either_access_pattern():
    # 16-byte accesses are served a quarter warp (eight lanes, 128 bytes) at a time
    for chunk, q in itertools.product(range(4), range(4)):  # writes: lane = row, same logical unit
        for quarter in range(4):
            lanes = range(quarter * 8, quarter * 8 + 8)
            used = [b for lane in lanes for b in banks(stage_unit(lane, chunk * 4 + q))]
            assert len(used) == len(set(used)), ("write", chunk, q, quarter)
    for i in range(16):  # reads: half a warp per row
        for quarter in range(4):
            lanes = range(quarter * 8, quarter * 8 + 8)
            used = [b for lane in lanes for b in banks(stage_unit(2 * i + lane // 16, lane % 16))]
            assert len(used) == len(set(used)), ("read", i, quarter)


@pytest.mark.parametrize("win_bytes", [144, 144 * 7, 144 * 1000 + 80, 256 * 1234])
def test_fp8_window_planes_do_not_overlap_and_fit(win_bytes):
    # quant.cu: payload of row i at i * 128, its scale at (win_bytes // 144) * 128 + i * 4
    rows = win_bytes // 144
    scale_off = rows * 128
    assert scale_off % 16 == 0
    assert (rows - 1) * 128 + 128 <= scale_off  # the last payload ends where the scales begin
    assert scale_off + rows * 4 <= win_bytes  # and the last scale lies inside the window
