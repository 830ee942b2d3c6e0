"""Host-side checks of the work decomposition the kernels use (same code, compiled for the host)."""
import ctypes
import itertools

import pytest


def tile_coords(lib, m_blocks, n_blocks, group_m):
    out = []
    m, n = ctypes.c_uint32(), ctypes.c_uint32()
    for t in range(m_blocks * n_blocks):
        lib.b200_sched_tile_coord(t, m_blocks, n_blocks, group_m, ctypes.byref(m), ctypes.byref(n))
        out.append((m.value, n.value))
    return out


@pytest.mark.parametrize("m_blocks,n_blocks,group_m", [
    (1, 1, 1), (2, 1, 16), (1, 7, 1), (64, 32, 16), (64, 32, 8), (13, 5, 4), (5, 13, 16), (33, 3, 16), (128, 64, 16),
])
def test_every_tile_exactly_once(native_lib, m_blocks, n_blocks, group_m):
    group_m = min(group_m, m_blocks)
    coords = tile_coords(native_lib, m_blocks, n_blocks, group_m)
    assert sorted(coords) == sorted(itertools.product(range(m_blocks), range(n_blocks)))


def test_rasterisation_keeps_concurrent_tiles_close(native_lib):
    # 148 consecutive tiles (one wave) of an 8192^3 problem touch few distinct row and column blocks
    coords = tile_coords(native_lib, 64, 32, 16)
    wave = coords[:148]
    rows = {m for m, _ in wave}
    cols = {n for _, n in wave}
    assert len(rows) <= 16 and len(cols) <= 10
    # serpentine: the last column of one band is the first of the next
    band = 16 * 32
    assert coords[band - 1][1] == coords[band][1]


def test_bands_are_even(native_lib):
    # 59 row blocks in bands of about 8: heights 8,8,8,7,7,7,7,7 -- never a thin last band
    n_blocks = 3
    coords = tile_coords(native_lib, 59, n_blocks, 8)
    sizes, idx = [], 0
    while idx < len(coords):
        # a band starts with its rows in order at one column; its height is the length of that run
        h = 1
        while idx + h < len(coords) and coords[idx + h][1] == coords[idx][1]:
            h += 1
        assert [m for m, _ in coords[idx:idx + h]] == list(range(coords[idx][0], coords[idx][0] + h))
        sizes.append(h)
        idx += h * n_blocks
    assert sizes == [8, 8, 8, 7, 7, 7, 7, 7]


def segments(lib, part, parts, tiles, k_blocks):
    buf = (ctypes.c_uint32 * (3 * 64))()
    n = lib.b200_sched_segments(part, parts, tiles, k_blocks, buf, 64)
    assert n <= 64
    return [(buf[3 * i], buf[3 * i + 1], buf[3 * i + 2]) for i in range(n)]


@pytest.mark.parametrize("tiles,k_blocks,parts", [
    (1, 1, 1), (1, 64, 148), (8, 4, 148), (32, 4, 32), (112, 64, 148), (112, 64, 448), (2, 3, 5), (7, 5, 3),
    (224, 224, 148), (56, 64, 147), (3, 1000, 148), (4096, 2, 148),
])
def test_stream_k_ranges_cover_every_unit_once(native_lib, tiles, k_blocks, parts):
    parts = min(parts, tiles * k_blocks)
    covered = {}
    for part in range(parts):
        segs = segments(native_lib, part, parts, tiles, k_blocks)
        partial = [s for s in segs if not (s[1] == 0 and s[2] == k_blocks)]
        # only the first and the last segment of a range can be partial tiles
        for s in partial:
            assert s is segs[0] or s is segs[-1]
        for tile, kb0, kb1 in segs:
            assert 0 <= kb0 < kb1 <= k_blocks and tile < tiles
            for kb in range(kb0, kb1):
                assert (tile, kb) not in covered
                covered[(tile, kb)] = part
    assert len(covered) == tiles * k_blocks
    sizes = [sum(kb1 - kb0 for _, kb0, kb1 in segments(native_lib, p, parts, tiles, k_blocks)) for p in range(parts)]
    assert max(sizes) - min(sizes) <= 1  # equal shares

    # contributors and workspace slots
    first, last = ctypes.c_uint32(), ctypes.c_uint32()
    for tile in range(min(tiles, 300)):
        native_lib.b200_sched_contributors(tile, parts, tiles, k_blocks, ctypes.byref(first), ctypes.byref(last))
        owners = sorted({covered[(tile, kb)] for kb in range(k_blocks)})
        assert owners == list(range(first.value, last.value + 1))
    used = set()
    for part in range(parts):
        for tile, kb0, kb1 in segments(native_lib, part, parts, tiles, k_blocks):
            if kb0 == 0 and kb1 == k_blocks:
                continue
            slot = native_lib.b200_sched_partial_slot(part, parts, tiles, k_blocks, tile)
            assert slot // 2 == part and slot not in used
            used.add(slot)


@pytest.mark.parametrize("tiles,k_blocks,workers", [
    (162, 36, 148),   # 2304^3 with 128 x 256 tiles: one full wave whole, 14 tiles cut
    (324, 4, 148),    # two whole tiles per worker, 28 cut tiles of 4 stages: fewer units than workers
    (450, 4, 148),    # 6 cut tiles, 24 units for 148 workers
    (40, 18, 7), (18, 18, 33), (100, 5, 10), (7, 1, 3), (1, 9, 4),
])
def test_whole_tiles_then_k_ranges_cover_every_unit_once(native_lib, tiles, k_blocks, workers):
    """The HYBRID plan's walk, restated on the host with the library's own range arithmetic: worker w takes
    tiles w, w + W, ... below dp_tiles whole, then (if it is one of the first sk_parts workers) its k-range of
    the remaining tiles. Every (tile, k-block) must come up exactly once, and no k-range may be empty."""
    dp_tiles = (tiles // workers) * workers
    cut_tiles = tiles - dp_tiles
    sk_parts = min(cut_tiles * k_blocks, workers)
    seen = {}
    buf = (ctypes.c_uint32 * (3 * 64))()
    for w in range(workers):
        for t in range(w, dp_tiles, workers):
            for kb in range(k_blocks):
                seen[(t, kb)] = seen.get((t, kb), 0) + 1
        if w < sk_parts:
            n = native_lib.b200_sched_segments(w, sk_parts, cut_tiles, k_blocks, buf, 64)
            assert 1 <= n <= 64, "a worker that owns a k-range must get at least one segment"
            for i in range(n):
                tile, kb0, kb1 = buf[3 * i], buf[3 * i + 1], buf[3 * i + 2]
                assert kb0 < kb1 <= k_blocks and tile < cut_tiles
                for kb in range(kb0, kb1):
                    key = (dp_tiles + tile, kb)
                    seen[key] = seen.get(key, 0) + 1
    assert len(seen) == tiles * k_blocks and set(seen.values()) == {1}


def test_division_by_multiplication_is_exact(native_lib):
    """The kernels divide by launch constants with a multiplication and two shifts: exact for every 32-bit pair."""
    import numpy as np

    rng = np.random.default_rng(5)
    cases = [(0, 1), (1, 1), (2 ** 32 - 1, 1), (2 ** 32 - 1, 2 ** 32 - 1), (2 ** 32 - 1, 2), (2 ** 31, 3), (12345, 2 ** 31)]
    cases += [(int(rng.integers(0, 2 ** 32)), int(rng.integers(1, 2 ** 32))) for _ in range(2000)]
    cases += [(int(rng.integers(0, 2 ** 32)), int(rng.integers(1, 5000))) for _ in range(4000)]
    cases += [(d * q + r, d) for d in (1, 2, 3, 7, 74, 148, 255, 256, 257, 65535, 65536) for q in (0, 1, 999, 16777215 // d)
              for r in (0, d - 1)]
    for n, d in cases:
        n &= 0xFFFFFFFF
        assert native_lib.b200_debug_fast_div(n, d) == n // d, (n, d)


def test_fast_tile_raster_agrees_with_the_plain_one(native_lib):
    import ctypes

    import numpy as np

    rng = np.random.default_rng(6)
    m, n = ctypes.c_uint32(), ctypes.c_uint32()
    m2, n2 = ctypes.c_uint32(), ctypes.c_uint32()
    geometries = [(1, 1, 1), (1, 7, 4), (9, 9, 8), (59, 3, 8), (64, 64, 6), (128, 2, 16), (4, 64, 6), (15, 15, 8), (3, 500, 1)]
    geometries += [(int(rng.integers(1, 200)), int(rng.integers(1, 200)), int(rng.integers(1, 40))) for _ in range(60)]
    for mb, nb, g in geometries:
        tiles = mb * nb
        for t in sorted(set([0, tiles - 1] + [int(x) for x in rng.integers(0, tiles, size=min(tiles, 200))])):
            native_lib.b200_sched_tile_coord(t, mb, nb, min(g, mb), ctypes.byref(m), ctypes.byref(n))
            native_lib.b200_sched_tile_coord_fast(t, mb, nb, min(g, mb), ctypes.byref(m2), ctypes.byref(n2))
            assert (m.value, n.value) == (m2.value, n2.value), (mb, nb, g, t)
