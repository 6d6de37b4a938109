"""CPU tests of the multi-GPU host logic with two gloo ranks: the row split, the packed output
buffer, the all-gather and the reassembly.  The per-rank compute is the CPU oracle here (the GPU
kernels are exercised by the -m gpu tests); what is under test is everything around it."""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shard_rows_is_the_pool_split():
    from hearth_b200.sharding import ShardPlan, shard_rows
    for n in (0, 1, 7, 1024, 5120, 17408, 1000):
        for world in (1, 2, 3, 4, 8):
            covered = []
            chunk = -(-n // world) if n else 0
            for r in range(world):
                lo, hi = shard_rows(n, r, world)
                assert 0 <= lo <= hi <= n
                assert hi - lo <= chunk
                if lo < n:
                    assert lo == r * chunk  # pool.rs:321-323
                covered.extend(range(lo, hi))
            assert covered == list(range(n))
    plan = ShardPlan.build([5120, 1024, 1000, 3], 8)
    assert plan.chunk == [640, 128, 125, 1]
    assert plan.offset == [0, 640, 768, 893] and plan.slice_total == 894


def _worker(rank: int, world: int, port: int, q):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    from hearth_b200 import synth
    from hearth_b200.sharding import ShardPlan
    from oracle import oracle as O

    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        seq_len, n_cols = 3, 256
        shapes = [(42, 257), (41, 64), (142, 5), (8, 33)]  # ragged on purpose: 5 rows over 2 ranks, odd counts
        plan = ShardPlan.build([n for _, n in shapes], world)
        x = synth.activations(seq_len, n_cols, seed=9)
        a = O.quantize_q8_0(x)  # replicated activation
        local = np.zeros((seq_len, plan.slice_total), dtype=np.float32)
        full = []
        for i, (dt, n) in enumerate(shapes):
            w = synth.weights(dt, n, n_cols, seed=100 + i)
            full.append(O.dot_rows_batched(dt, w, a, n, n_cols))
            lo, hi = plan.rows_of(i, rank)
            if hi > lo:
                local[:, plan.offset[i]:plan.offset[i] + hi - lo] = O.dot_rows_batched(dt, w[lo:hi], a, hi - lo, n_cols)
        flat = torch.zeros((world * seq_len, plan.slice_total), dtype=torch.float32)
        dist.all_gather_into_tensor(flat, torch.from_numpy(local))
        gathered = flat.view(world, seq_len, plan.slice_total)
        ok = True
        for i in range(len(shapes)):
            got = plan.assemble(gathered, i).numpy()
            ok = ok and got.shape == full[i].shape and (got.view(np.uint32) == full[i].view(np.uint32)).all()
        q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


def test_two_rank_gather_reassembles_every_matrix():
    import torch.multiprocessing as mp
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=60) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(results) == [(0, True), (1, True)]
