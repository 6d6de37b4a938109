"""Row sharding of weight matrices across GPUs and the layout of the gathered outputs.

The reference splits the rows of one matrix over worker threads as
chunk = ceil(n / T), worker i -> [i*chunk, min((i+1)*chunk, n))  (hearth-llm/src/pool.rs:321-323).
Here the same split is applied across ranks (one process per GPU).  Every rank writes its output
slices for all matrices of a step into one packed buffer [seq_len, slice_total]; one all-gather
yields [world, seq_len, slice_total], from which `ShardPlan.assemble` rebuilds the token-major
[seq_len, n_rows] result of any matrix.
"""
from __future__ import annotations

from dataclasses import dataclass


def shard_rows(n_rows: int, rank: int, world: int) -> tuple[int, int]:
    """Rows [lo, hi) of an n_rows matrix owned by `rank` of `world`."""
    chunk = -(-n_rows // world)
    lo = min(rank * chunk, n_rows)
    return lo, min(lo + chunk, n_rows)


@dataclass
class ShardPlan:
    """Offsets of every matrix's slice inside the packed per-rank output buffer."""
    world: int
    n_rows: list[int]          # full row count of each matrix
    chunk: list[int]           # ceil(n_rows / world): slot width reserved per matrix (same on every rank)
    offset: list[int]          # start column of each matrix's slot
    slice_total: int           # columns of the packed buffer

    @classmethod
    def build(cls, n_rows: list[int], world: int) -> "ShardPlan":
        chunk = [-(-n // world) for n in n_rows]
        offset, acc = [], 0
        for c in chunk:
            offset.append(acc)
            acc += c
        return cls(world, list(n_rows), chunk, offset, acc)

    def rows_of(self, i: int, rank: int) -> tuple[int, int]:
        return shard_rows(self.n_rows[i], rank, self.world)

    def assemble(self, gathered, i: int):
        """gathered: array-like [world, seq_len, slice_total] (numpy or torch). Returns [seq_len, n_rows[i]]."""
        parts = []
        for r in range(self.world):
            lo, hi = self.rows_of(i, r)
            if hi > lo:
                parts.append(gathered[r][:, self.offset[i]:self.offset[i] + (hi - lo)])
        if hasattr(gathered, "dim"):  # torch
            import torch
            return torch.cat(parts, dim=1)
        import numpy as np
        return np.concatenate(parts, axis=1)
