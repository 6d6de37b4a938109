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


def _build_rank(hb, torch, dev, rank, world, seq, bufs, wait, specs=None, area_floats=0):
    """Uploads this rank's row shards and records a batch that stores into all of bufs."""
    specs = SPECS if specs is None else specs
    total = sum(n for _, n, _ in specs)
    acts, Ws = {}, []
    batch = hb.Batch()
    batch.set_peers(rank, bufs, wait=wait, area_floats=area_floats)
    local = bufs[rank].tensor(dev)[:seq * total].view(seq, total)
    coff = 0
    for i, (dt, n, k) in enumerate(specs):
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


def _step_inputs(seq, step):
    """Activations of one step, by width: they change from step to step so that a stale or early row shows."""
    return {k: synth.activations(seq, k, seed=900 + k + 7919 * step) for k in sorted({k for _, _, k in SPECS})}


def _step_expected(oracle, seq, step):
    xs = _step_inputs(seq, step)
    outs = []
    for i, (dt, n, k) in enumerate(SPECS):
        w = synth.weights(dt, n, k, seed=800 + i)
        outs.append(oracle.dot_rows_batched(dt, w, oracle.quantize_q8_0(xs[k]), n, k))
    return np.concatenate(outs, axis=1)


N_STEPS = 6


def _real_rank(rank, world, seq, qs, result_q):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import torch
    from hearth_b200 import api as hb
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    hb.init(rank)
    total = sum(n for _, n, _ in SPECS)
    area = seq * total + (-(seq * total)) % 4
    mine = hb.PeerBuffer.alloc(2 * area)          # two output areas, written by alternate launches
    for r in range(world):
        if r != rank:
            qs[r].put((rank, mine.handle))
    bufs = [None] * world
    bufs[rank] = mine
    for _ in range(world - 1):
        src, h = qs[rank].get(timeout=60)
        bufs[src] = hb.PeerBuffer.open(h, 2 * area)
    batch, acts, Ws = _build_rank(hb, torch, dev, rank, world, seq, bufs, wait=True, area_floats=area)
    results = []
    stream = torch.cuda.current_stream()
    for step in range(N_STEPS):
        # no host-side synchronisation between the ranks from here on: a rank may run one launch ahead of the other,
        # and the two output areas keep its stores away from what the slower rank still reads
        for k, x in _step_inputs(seq, step).items():
            acts[k].quantize(seq, x_dev=torch.from_numpy(x).to(dev))
        batch.launch()
        got = mine.tensor(dev)[batch.peer_area * area: batch.peer_area * area + seq * total].view(seq, total)
        results.append(got.to("cpu", non_blocking=False).numpy().copy())  # this rank's read of step `step`, in stream order
        if rank == 0 and step % 2 == 0:
            stream.synchronize()
            import time
            time.sleep(0.05)                      # let one rank fall behind now and then
    hb.check_status()
    result_q.put((rank, np.stack(results)))
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
    want = np.stack([_step_expected(oracle, seq, step) for step in range(N_STEPS)])
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
        for step in range(N_STEPS):
            assert (got[r][step].view(np.uint32) == want[step].view(np.uint32)).all(), f"rank {r}, step {step}"


def test_emulated_ranks_with_empty_shards_keep_one_epoch_per_launch(hb, oracle):
    """One launch is one epoch on every rank, whatever the number of kernels it takes there.  Rank 1's shard of the
    only Q8_0 matrix is empty (1 row over 2 ranks), so rank 0 launches two kernels per step and rank 1 one; in a
    second batch every shard of rank 1 is empty and it only runs the flag exchange.  After three launches every
    control block must read epoch 3 from both ranks."""
    import torch
    dev = torch.device("cuda:0")
    seq = 1
    for specs in ([(42, 100, 1152), (8, 1, 256)], [(42, 1, 1152), (41, 1, 256)]):
        total = sum(n for _, n, _ in specs)
        bufs = [hb.PeerBuffer.alloc(seq * total) for _ in range(2)]
        built = [_build_rank(hb, torch, dev, r, 2, seq, bufs, wait=False, specs=specs) for r in range(2)]
        try:
            for _ in range(3):
                for batch, _, _ in built:
                    batch.launch()
            hb.check_status()
            for b in bufs:
                assert b.flags(dev)[:2].tolist() == [3, 3], (specs, b.flags(dev).tolist())
            want = np.concatenate([oracle.dot_rows_batched(dt, synth.weights(dt, n, k, seed=800 + i),
                                                           oracle.quantize_q8_0(synth.activations(seq, k, seed=900 + k)), n, k)
                                   for i, (dt, n, k) in enumerate(specs)], axis=1)
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


def test_emulated_ranks_alternate_output_areas(hb, oracle):
    """Two output areas per buffer: launch e writes area (e - 1) & 1 and leaves the other one, the previous step's
    results, untouched.  Inputs change every step."""
    import torch
    dev = torch.device("cuda:0")
    seq = 2
    total = sum(n for _, n, _ in SPECS)
    area = seq * total + (-(seq * total)) % 4
    bufs = [hb.PeerBuffer.alloc(2 * area) for _ in range(2)]
    built = [_build_rank(hb, torch, dev, r, 2, seq, bufs, wait=False, area_floats=area) for r in range(2)]
    try:
        prev = None
        for step in range(4):
            want = _step_expected(oracle, seq, step)
            for batch, acts, _ in built:
                for k, x in _step_inputs(seq, step).items():
                    acts[k].quantize(seq, x_dev=torch.from_numpy(x).to(dev))
                batch.launch()
            hb.check_status()
            assert built[0][0].peer_area == built[1][0].peer_area == step & 1
            for b in bufs:
                both = b.tensor(dev).cpu().numpy()
                cur = both[(step & 1) * area:(step & 1) * area + seq * total].reshape(seq, total)
                assert (cur.view(np.uint32) == want.view(np.uint32)).all(), f"step {step}"
                if prev is not None:
                    old = both[((step - 1) & 1) * area:((step - 1) & 1) * area + seq * total].reshape(seq, total)
                    assert (old.view(np.uint32) == prev.view(np.uint32)).all(), f"step {step}: the previous area changed"
            prev = want
    finally:
        for batch, acts, Ws in built:
            batch.free()
            for a in acts.values():
                a.free()
            for W in Ws:
                W.free()
        for b in bufs:
            b.close()


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
