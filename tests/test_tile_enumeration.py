"""Host logic of the two-kernel bf16 path: the encoding launch and its complement must partition the
[query tile x key tile] grid of a head, the encoding launch must meet every query tile and every
key tile, and the 256-row variant must cover the same tiles as the 128-row one.  Runs on CPU (the
enumeration is compiled for the host too)."""
import ctypes as C

import pytest


def tiles(L, big, mode, nqt, nkt):
    qt, kt = C.c_int(-1), C.c_int(-1)
    n = L.b200attn_debug_tile_of(big, mode, -1, nqt, nkt, C.byref(qt), C.byref(kt))
    if n < 0:
        return None
    out = []
    for j in range(n):
        assert L.b200attn_debug_tile_of(big, mode, j, nqt, nkt, C.byref(qt), C.byref(kt)) == n
        out.append((qt.value, kt.value))
    return out


@pytest.fixture(scope="module")
def L(pkg):
    lib = pkg.lib()
    lib.b200attn_debug_tile_of.argtypes = [C.c_int] * 5 + [C.POINTER(C.c_int)] * 2
    lib.b200attn_debug_tile_of.restype = C.c_int
    return lib


@pytest.mark.parametrize("nqt", [1, 2, 3, 4, 5, 6, 8, 16, 32, 64])
@pytest.mark.parametrize("nkt", [1, 2, 3, 4, 7, 8, 16, 32])
def test_encoding_launch_and_complement_partition_the_grid(L, nqt, nkt):
    grid = {(q, k) for q in range(nqt) for k in range(nkt)}
    every = tiles(L, 0, 0, nqt, nkt)
    assert sorted(every) == sorted(grid)
    enc, rest = tiles(L, 0, 1, nqt, nkt), tiles(L, 0, 2, nqt, nkt)
    assert len(enc) == max(nqt, nkt) and len(set(enc)) == len(enc)
    assert {q for q, _ in enc} == set(range(nqt)) and {k for _, k in enc} == set(range(nkt))
    assert len(set(rest)) == len(rest) and set(enc).isdisjoint(rest)
    assert set(enc) | set(rest) == grid
    # positions are shared (kt == qt // 2) for every encoding tile of the square benchmark shapes
    if nqt == 2 * nkt:
        assert all(k == q // 2 for q, k in enc)


@pytest.mark.parametrize("nqt", [2, 4, 6, 8, 16, 32])
@pytest.mark.parametrize("nkt", [1, 2, 3, 4, 8, 16])
def test_256_row_tiles_cover_the_same_tiles(L, nqt, nkt):
    for mode in (0, 2):
        big = tiles(L, 1, mode, nqt, nkt)
        if big is None:
            assert mode == 2 and not (nkt <= nqt and nqt >= 2 * nkt - 1)
            continue
        small = tiles(L, 0, mode, nqt, nkt)
        covered = [(2 * qp + r, k) for qp, k in big for r in (0, 1)]
        assert len(set(covered)) == len(covered)
        assert sorted(covered) == sorted(small)
