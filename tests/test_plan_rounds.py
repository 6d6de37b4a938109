"""Host logic of the decode matvec's list launches: hb200_plan_rounds cuts the rounds of all panels of a launch into
equal shares per CTA and splits a panel between two neighbouring CTAs where a cut falls inside it (the ordered fp32 sum
of the panel is then handed over through a carry slot).  Pure host code: runs without a GPU.

Reference for the semantics being balanced: ThreadPool::par_dot_rows splits rows evenly over its threads
(hearth-llm/src/pool.rs:321-323)."""
import ctypes as C

import numpy as np
import pytest

from hearth_b200 import lib as hl


def plan(op, panel, rounds, grid):
    lib = hl.load()
    op = np.ascontiguousarray(op, dtype=np.int32)
    panel = np.ascontiguousarray(panel, dtype=np.int32)
    rounds = np.ascontiguousarray(rounds, dtype=np.int32)
    cap = len(op) + 2 * grid + 8
    seg_begin = np.zeros(grid + 1, dtype=np.int32)
    segs = np.zeros((cap, 8), dtype=np.int32)
    n = C.c_size_t(0)
    P = C.POINTER(C.c_int)
    rc = lib.hb200_plan_rounds(op.ctypes.data_as(P), panel.ctypes.data_as(P), rounds.ctypes.data_as(P), len(op), grid,
                               seg_begin.ctypes.data_as(P), segs.ctypes.data_as(P), cap, C.byref(n))
    assert rc == 0, hl.last_error()
    return seg_begin, segs[: n.value]


def layer_items(shapes, rows_per_panel, layers):
    """(op, panel, rounds) of every panel of `layers` layers of matrices (n_rows, n_cols)."""
    op, panel, rounds = [], [], []
    o = 0
    for _ in range(layers):
        for n_rows, n_cols in shapes:
            nb = n_cols // 128
            for p in range((n_rows + rows_per_panel - 1) // rows_per_panel):
                op.append(o); panel.append(p); rounds.append(max(1, (nb + 7) // 8))
            o += 1
    return op, panel, rounds


def check(op, panel, rounds, grid, seg_begin, segs):
    rounds_of = {(o, p): r for o, p, r in zip(op, panel, rounds)}
    seen = {}
    per_cta = []
    assert seg_begin[0] == 0 and seg_begin[grid] == len(segs)
    for c in range(grid):
        mine = segs[seg_begin[c]:seg_begin[c + 1]]
        total = 0
        for k, (o, p0, cnt, r0, r1, flags, cin, cout) in enumerate(mine):
            assert cnt >= 1 and 0 <= r0 < r1
            if cnt > 1 or not flags:
                assert r0 == 0 and flags == 0
            for p in range(p0, p0 + cnt):
                assert r1 <= rounds_of[(o, p)]
                if not flags:
                    assert r1 == rounds_of[(o, p)]
                for r in range(r0, r1):
                    assert (o, p, r) not in seen, "a round is planned twice"
                    seen[(o, p, r)] = c
                total += r1 - r0
            if flags & 2:  # hands its sums to the next CTA: first in this CTA's order, slot = index of the next CTA
                assert k == 0 and cout == c + 1 and r1 < rounds_of[(o, p0)]
            if flags & 1:  # continues the previous CTA's sums: slot = this CTA's index
                assert cin == c and r0 > 0
                if not (flags & 2):
                    assert k == len(mine) - 1 and r1 == rounds_of[(o, p0)]
        per_cta.append(total)
    assert len(seen) == sum(rounds), "every round of every panel exactly once"
    # a panel's parts lie in consecutive CTAs, in round order
    for (o, p), r in rounds_of.items():
        owners = [seen[(o, p, k)] for k in range(r)]
        assert owners == sorted(owners) and owners[-1] - owners[0] <= max(1, len(set(owners)) - 1)
    return per_cta


def test_split_plan_balances_a_small_model():
    """The 1.7B decode set (28 layers, 256-row panels of Q1_0): 2240 panels of 2 or 6 rounds over 296 CTAs."""
    shapes = [(2048, 2048), (1024, 2048), (1024, 2048), (2048, 2048), (6144, 2048), (6144, 2048), (2048, 6144)]
    op, panel, rounds = layer_items(shapes, 256, 28)
    grid = 296
    seg_begin, segs = plan(op, panel, rounds, grid)
    per_cta = check(op, panel, rounds, grid, seg_begin, segs)
    total = sum(rounds)
    assert max(per_cta) <= total // grid + 1 and min(per_cta) >= total // grid
    assert any(s[5] for s in segs), "cuts fall inside panels"
    # every hand-over has its two sides
    outs = {(s[0], s[1], s[4], s[7]) for s in segs if s[5] & 2}
    ins = {(s[0], s[1], s[3], s[6]) for s in segs if s[5] & 1}
    assert outs == ins


def test_little_work_is_cut_between_panels():
    op, panel, rounds = layer_items([(2048, 2048)], 256, 3)  # 24 panels of 2 rounds
    seg_begin, segs = plan(op, panel, rounds, 24)
    per_cta = check(op, panel, rounds, 24, seg_begin, segs)
    assert not any(s[5] for s in segs) and per_cta == [2] * 24
    seg_begin, segs = plan(op, panel, rounds, 5)  # 48 rounds over 5 CTAs: 48 >= 2 * 5 * 2, so panels are cut
    per_cta = check(op, panel, rounds, 5, seg_begin, segs)
    assert sorted(per_cta) == [9, 9, 10, 10, 10]


def test_mixed_lengths_and_merging():
    rng = np.random.Generator(np.random.PCG64(7))
    op, panel, rounds = [], [], []
    for o in range(40):
        r = int(rng.integers(1, 18))
        for p in range(int(rng.integers(1, 30))):
            op.append(o); panel.append(p); rounds.append(r)
    for grid in (1, 2, 7, 33):
        seg_begin, segs = plan(op, panel, rounds, grid)
        check(op, panel, rounds, grid, seg_begin, segs)
    seg_begin, segs = plan(op, panel, rounds, 1)
    assert len(segs) == 40, "consecutive whole panels of one op are one segment"


def test_plan_rounds_rejects_bad_input():
    lib = hl.load()
    P = C.POINTER(C.c_int)
    one = np.array([1], dtype=np.int32)
    zero = np.array([0], dtype=np.int32)
    sb = np.zeros(3, dtype=np.int32)
    segs = np.zeros((4, 8), dtype=np.int32)
    n = C.c_size_t(0)
    assert lib.hb200_plan_rounds(zero.ctypes.data_as(P), zero.ctypes.data_as(P), zero.ctypes.data_as(P), 1, 2, sb.ctypes.data_as(P),
                                 segs.ctypes.data_as(P), 4, C.byref(n)) == -4  # zero rounds
    assert lib.hb200_plan_rounds(zero.ctypes.data_as(P), zero.ctypes.data_as(P), one.ctypes.data_as(P), 1, 0, sb.ctypes.data_as(P),
                                 segs.ctypes.data_as(P), 4, C.byref(n)) == -4  # no CTA
    assert lib.hb200_plan_rounds(zero.ctypes.data_as(P), zero.ctypes.data_as(P), one.ctypes.data_as(P), 1, 2, sb.ctypes.data_as(P),
                                 segs.ctypes.data_as(P), 0, C.byref(n)) == -8 and n.value == 1  # no room: the count is still reported
