"""Row-sharded outputs written straight into every rank's buffer (peer stores + flag exchange).

On one GPU the two ranks are emulated inside one process: both output buffers are local, each rank's batch
only publishes (wait=False) and the launches run one after the other, so no kernel ever waits for another.
With two or more GPUs a second test runs two real ranks (one process per GPU, IPC-mapped peer buffers,
wait=True).
"""
import os
import sys

import numpy as np
import pytest

from hearth_b200 import synth
from hearth_b200.sharding import shard_rows

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SPECS = [(42, 1000, 2048), (41, 520, 2048), (142, 7, 1152), (8, 33, 256)]  # (dtype, rows, cols); 7 rows over 2 ranks is ragged


def _expected(oracle, seq):
    outs, xs = [], {}
    for i, (dt, n, k) in enumerate(SPECS):
        x = xs.setdefault(k, synth.activations(seq, k, seed=900 + k))
        w = synth.weights(dt, n, k, seed=800 + i)
        outs.append(oracle.dot_rows_batched(dt, w, oracle.quantize_q8_0(x), n, k))
    return np.concatenate(outs, axis=1), xs


def _build_rank(hb, torch, dev, rank, world, seq, bufs, wait):
    """Uploads this rank's row shards and records a batch that stores into all of bufs."""
    total = sum(n for _, n, _ in SPECS)
    acts, Ws = {}, []
    batch = hb.Batch()
    batch.set_peers(rank, bufs, wait=wait)
    local = bufs[rank].tensor(dev).view(seq, total)
    coff = 0
    for i, (dt, n, k) in enumerate(SPECS):
        if k not in acts:
            acts[k] = hb.Act(seq, k)
            acts[k].quantize(seq, x_dev=torch.from_numpy(synth.activations(seq, k, seed=900 + k)).to(dev))
        lo, hi = shard_rows(n, rank, world)
        w = synth.weights(dt, n, k, seed=800 + i)
        W = hb.Weight.upload(dt, n, k, w, rows=(lo, hi))
        Ws.append(W)
        if hi > lo:
            batch.add(W, acts[k], seq, local[:, coff + lo:], ld_out=total)
        coff += n
    batch.seal()
    return batch, acts, Ws


def test_two_emulated_ranks_fill_both_buffers(hb, oracle):
    import torch
    dev = torch.device("cuda:0")
    seq = 2
    want, _ = _expected(oracle, seq)
    total = want.shape[1]
    bufs = [hb.PeerBuffer.alloc(seq * total) for _ in range(2)]
    built = [_build_rank(hb, torch, dev, r, 2, seq, bufs, wait=False) for r in range(2)]
    try:
        for _ in range(2):  # second pass: epochs advance, results identical
            for b in bufs:
                b.tensor(dev).fill_(float("nan"))
            for batch, _, _ in built:
                batch.launch()
            hb.check_status()
            for b in bufs:
                got = b.tensor(dev).view(seq, total).cpu().numpy()
                assert (got.view(np.uint32) == want.view(np.uint32)).all()
    finally:
        for batch, acts, Ws in built:
            batch.free()
            for a in acts.values():
                a.free()
            for W in Ws:
                W.free()
        for b in bufs:
            b.close()


def _real_rank(rank, world, seq, qs, result_q):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import torch
    from hearth_b200 import api as hb
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    hb.init(rank)
    total = sum(n for _, n, _ in SPECS)
    mine = hb.PeerBuffer.alloc(seq * total)
    for r in range(world):
        if r != rank:
            qs[r].put((rank, mine.handle))
    bufs = [None] * world
    bufs[rank] = mine
    for _ in range(world - 1):
        src, h = qs[rank].get(timeout=60)
        bufs[src] = hb.PeerBuffer.open(h, seq * total)
    batch, acts, Ws = _build_rank(hb, torch, dev, rank, world, seq, bufs, wait=True)
    for _ in range(3):
        batch.launch()
    hb.check_status()
    result_q.put((rank, mine.tensor(dev).view(seq, total).cpu().numpy()))
    # leave only between steps, after every rank has its results
    qs[rank].get(timeout=60)
    batch.free()
    for b in bufs:
        if b is not mine:
            b.close()
    mine.close()


def test_two_real_ranks_over_nvlink(oracle):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    seq, world = 2, 2
    want, _ = _expected(oracle, seq)
    ctx = mp.get_context("spawn")
    qs = [ctx.Queue() for _ in range(world)]
    result_q = ctx.Queue()
    procs = [ctx.Process(target=_real_rank, args=(r, world, seq, qs, result_q)) for r in range(world)]
    for p in procs:
        p.start()
    got = dict(result_q.get(timeout=180) for _ in range(world))
    for r in range(world):
        qs[r].put("done")
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for r in range(world):
        assert (got[r].view(np.uint32) == want.view(np.uint32)).all(), f"rank {r}"


def test_absent_rank_ends_in_a_timeout_status_not_a_hang(hb, oracle):
    """Failure detection without a fault: rank 0 waits (bounded) for the flag of a rank that never launches.  The wait
    runs out, the kernel returns, the next status check reports HB200_ERR_TIMEOUT, and the context stays usable."""
    import time
    import torch
    dev = torch.device("cuda:0")
    seq = 1
    want, _ = _expected(oracle, seq)
    total = want.shape[1]
    bufs = [hb.PeerBuffer.alloc(seq * total) for _ in range(2)]
    batch, acts, Ws = _build_rank(hb, torch, dev, 0, 2, seq, bufs, wait=True)
    try:
        t0 = time.perf_counter()
        batch.launch()
        torch.cuda.synchronize()
        assert time.perf_counter() - t0 < 30.0
        with pytest.raises(hb.Hb200Error) as e:
            hb.check_status()
        assert e.value.code == -9
        hb.check_status()                      # the status word was cleared
        # rank 0's own rows are in place all the same, and the library still works
        got = bufs[0].tensor(dev).view(seq, total).cpu().numpy()
        coff = 0
        for dt, n, k in SPECS:
            lo, hi = shard_rows(n, 0, 2)
            assert (got[:, coff + lo:coff + hi].view(np.uint32) == want[:, coff + lo:coff + hi].view(np.uint32)).all()
            coff += n
        x = synth.activations(1, 256, seed=1)
        assert (hb.quantize_q8_0(x) == oracle.quantize_q8_0(x)).all()
    finally:
        batch.free()
        for a in acts.values():
            a.free()
        for W in Ws:
            W.free()
        for b in bufs:
            b.close()
