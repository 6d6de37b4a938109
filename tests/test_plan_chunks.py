"""Host logic of the work lists: hb200_plan_chunks splits a list of items with costs into contiguous runs for the
persistent CTAs.  No device is needed.  The split must cover every item once, in order, use at most `grid` runs, and
its largest run must be the optimum for a contiguous split (checked against an exhaustive search on small lists and
against the lower bounds max(cost) and ceil(total / grid) on the decode sets of the benchmark)."""
import ctypes as C
import itertools

import numpy as np
import pytest

from hearth_b200 import synth


@pytest.fixture(scope="module")
def lib():
    from hearth_b200 import build, lib as L
    build.build()
    return L.load()


def plan(lib, cost, grid):
    cost = np.ascontiguousarray(cost, dtype=np.int32)
    chunks = np.zeros(grid + 1, dtype=np.int32)
    rc = lib.hb200_plan_chunks(cost.ctypes.data_as(C.POINTER(C.c_int)), cost.size, grid, chunks.ctypes.data_as(C.POINTER(C.c_int)))
    assert rc == 0, lib.hb200_last_error()
    return chunks


def runs_of(cost, chunks):
    return [int(np.sum(cost[a:b])) for a, b in zip(chunks[:-1], chunks[1:])]


def brute_force_optimum(cost, grid):
    n = len(cost)
    best = sum(cost)
    for k in range(0, min(grid, n)):
        for cuts in itertools.combinations(range(1, n), k):
            b = (0,) + cuts + (n,)
            best = min(best, max(sum(cost[x:y]) for x, y in zip(b[:-1], b[1:])))
    return best


@pytest.mark.parametrize("seed", range(12))
def test_small_lists_are_split_optimally(lib, seed):
    rng = np.random.default_rng(seed)
    n = int(rng.integers(1, 10))
    grid = int(rng.integers(1, 6))
    cost = rng.integers(0, 9, n).astype(np.int32)
    chunks = plan(lib, cost, grid)
    assert chunks[0] == 0 and chunks[-1] == n and (np.diff(chunks) >= 0).all()
    assert max(runs_of(cost, chunks)) == brute_force_optimum(list(map(int, cost)), grid)


def test_edge_cases(lib):
    assert plan(lib, [], 4).tolist() == [0, 0, 0, 0, 0]
    assert plan(lib, [5], 3).tolist() == [0, 1, 1, 1]
    c = plan(lib, [1] * 10, 20)
    assert c[0] == 0 and c[-1] == 10 and max(np.diff(c)) == 1
    assert plan(lib, [0, 0, 0], 2)[-1] == 3
    bad = np.array([1, -1], dtype=np.int32)
    out = np.zeros(3, dtype=np.int32)
    assert lib.hb200_plan_chunks(bad.ctypes.data_as(C.POINTER(C.c_int)), 2, 2, out.ctypes.data_as(C.POINTER(C.c_int))) == -4
    assert lib.hb200_plan_chunks(bad.ctypes.data_as(C.POINTER(C.c_int)), 2, 0, out.ctypes.data_as(C.POINTER(C.c_int))) == -4


@pytest.mark.parametrize("name,rows_per_panel", [("c1_q1_1p7b_decode", 256), ("c1_q2_1p7b_decode", 128), ("c2_q1_8b_decode", 256)])
def test_decode_sets_are_balanced_to_the_grain(lib, name, rows_per_panel):
    """296 CTAs (two per SM on 148 SMs); an item is a panel of rows over all of K, its cost the rounds of eight
    128-column blocks.  The largest run may exceed the mean by less than one item."""
    cfg = synth.CONFIGS[name]
    cost = []
    for _ in range(cfg["layers"]):
        for _, n, k in cfg["shapes"]:
            cost += [((k // 128) + 7) // 8] * ((n + rows_per_panel - 1) // rows_per_panel)
    cost = np.array(cost, dtype=np.int32)
    grid = 296
    chunks = plan(lib, cost, grid)
    runs = runs_of(cost, chunks)
    assert sum(runs) == int(cost.sum()) and chunks[-1] == cost.size
    lower = max(int(cost.max()), -(-int(cost.sum()) // grid))
    assert lower <= max(runs) < lower + int(cost.max())
    # the prefix rule this replaced (boundary c where the prefix reaches c/grid of the total) does worse on these sets
    total, run, nxt, b = int(cost.sum()), 0, 1, [0]
    for i, c in enumerate(cost):
        run += int(c)
        while nxt < grid and run * grid >= total * nxt:
            b.append(i + 1)
            nxt += 1
    b += [cost.size] * (grid + 1 - len(b))
    assert max(runs) <= max(runs_of(cost, b))
