"""One process, several device slots (hb200_init_multi / hb200_init_slots): the shape the reference needs, since it is a
single process with one dispatching thread (hearth-llm/src/pool.rs:398-425).

On one GPU two slots are bound to the same device and emulate two row shards: every object lives in the slot it was
created in, calls switch slots by themselves, each slot's batch stores its rows into both slots' buffers (wait=False:
the launches run one after the other on the one device, so no kernel may wait for another).  With two GPUs the same
is done on two devices from one host thread with wait=True, two output areas and inputs that change every step.
"""
import numpy as np
import pytest

from hearth_b200 import synth
from hearth_b200.sharding import shard_rows

pytestmark = pytest.mark.gpu

SPECS = [(42, 1000, 2048), (41, 520, 2048), (142, 7, 1152), (8, 33, 256)]  # (dtype, rows, cols)


def _inputs(seq, step):
    return {k: synth.activations(seq, k, seed=900 + k + 7919 * step) for k in sorted({k for _, _, k in SPECS})}


def _expected(oracle, seq, step):
    xs = _inputs(seq, step)
    return np.concatenate([oracle.dot_rows_batched(dt, synth.weights(dt, n, k, seed=800 + i), oracle.quantize_q8_0(xs[k]), n, k)
                           for i, (dt, n, k) in enumerate(SPECS)], axis=1)


def _build(hb, torch, slots, devs, seq, wait, area):
    """Per slot: row shards, activations, a peer buffer, and a batch that stores into every slot's buffer."""
    world = len(slots)
    total = sum(n for _, n, _ in SPECS)
    bufs = []
    for r in range(world):
        hb.set_slot(slots[r])
        bufs.append(hb.PeerBuffer.alloc(2 * area if area else seq * total))
    built = []
    for r in range(world):
        hb.set_slot(slots[r])
        with torch.cuda.device(devs[r]):
            batch = hb.Batch()
            batch.set_peers(r, bufs, wait=wait, area_floats=area)
            local = bufs[r].tensor(devs[r])[:seq * total].view(seq, total)
            acts, Ws, coff = {}, [], 0
            for i, (dt, n, k) in enumerate(SPECS):
                if k not in acts:
                    acts[k] = hb.Act(seq, k)
                lo, hi = shard_rows(n, r, world)
                W = hb.Weight.upload(dt, n, k, synth.weights(dt, n, k, seed=800 + i), rows=(lo, hi))
                Ws.append(W)
                if hi > lo:
                    batch.add(W, acts[k], seq, local[:, coff + lo:], ld_out=total)
                coff += n
            batch.seal()
        built.append((batch, acts, Ws))
    return bufs, built


def _free(hb, bufs, built):
    for batch, acts, Ws in built:
        batch.free()
        for a in acts.values():
            a.free()
        for W in Ws:
            W.free()
    for b in bufs:
        b.close()
    hb.set_slot(0)


def test_two_slots_on_one_device_emulate_two_shards(hb, oracle):
    import torch
    dev = torch.device("cuda:0")
    assert hb.init_multi(devices=[0, 0]) >= 2      # slot 0 is the one the other tests use; slot 1 joins it
    seq = 2
    total = sum(n for _, n, _ in SPECS)
    bufs, built = _build(hb, torch, [0, 1], [dev, dev], seq, wait=False, area=0)
    try:
        # an object of another slot is refused, not silently used on the wrong device
        with pytest.raises(hb.Hb200Error) as e:
            built[0][0].add(built[1][2][0], built[1][1][2048], seq, bufs[0].tensor(dev), ld_out=total)
        assert e.value.code == -4
        for step in range(2):
            want = _expected(oracle, seq, step)
            for r, (batch, acts, _) in enumerate(built):
                for k, x in _inputs(seq, step).items():
                    acts[k].quantize(seq, x_dev=torch.from_numpy(x).to(dev))   # switches to the activation's slot by itself
            hb.multi_batch_launch([b for b, _, _ in built], [torch.cuda.current_stream(), torch.cuda.current_stream()])
            torch.cuda.synchronize()
            hb.check_status()
            for b in bufs:
                got = b.tensor(dev)[:seq * total].view(seq, total).cpu().numpy()
                assert (got.view(np.uint32) == want.view(np.uint32)).all(), f"step {step}"
            assert [b.flags(dev)[:2].tolist() for b in bufs] == [[step + 1] * 2] * 2
    finally:
        _free(hb, bufs, built)
    # the single-slot calls of the other tests still work
    x = synth.activations(1, 256, seed=1)
    assert (hb.quantize_q8_0(x) == oracle.quantize_q8_0(x)).all()


def test_two_devices_driven_by_one_host_thread(hb, oracle):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    devs = [torch.device("cuda:0"), torch.device("cuda:1")]
    # slot 1 may already be a second slot on device 0 (the emulation test above): the second GPU becomes slot 2
    hb.init_multi(devices=[0, 0, 1])
    slots = [0, 2]
    seq = 2
    total = sum(n for _, n, _ in SPECS)
    area = seq * total + (-(seq * total)) % 4
    bufs, built = _build(hb, torch, slots, devs, seq, wait=True, area=area)
    try:
        for step in range(5):
            want = _expected(oracle, seq, step)
            for r, (batch, acts, _) in enumerate(built):
                with torch.cuda.device(devs[r]):
                    for k, x in _inputs(seq, step).items():
                        acts[k].quantize(seq, x_dev=torch.from_numpy(x).to(devs[r]))
                    torch.cuda.current_stream().synchronize()
            hb.multi_batch_launch([b for b, _, _ in built])     # default streams: both kernels run at once and exchange flags
            for r in range(2):
                with torch.cuda.device(devs[r]):
                    torch.cuda.synchronize()
            a = built[0][0].peer_area
            assert a == built[1][0].peer_area == step & 1
            for r, b in enumerate(bufs):
                got = b.tensor(devs[r])[a * area:a * area + seq * total].view(seq, total).cpu().numpy()
                assert (got.view(np.uint32) == want.view(np.uint32)).all(), f"device {r}, step {step}"
        for sl in slots:
            hb.set_slot(sl)
            hb.check_status()
    finally:
        _free(hb, bufs, built)
