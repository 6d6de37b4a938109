"""GPU parity tests for the recorded-batch launch paths at the configured sizes.

A recorded batch (hb200_batch_*) puts every tensor-core op of one weight kind into ONE persistent launch: the tiles of
all matrices are numbered consecutively, a CTA walks a contiguous run of them, and its rings and barrier phases carry
on from one matrix into the next (different K-block counts, different tensor maps).  The K-quant ops of a batch share
a launch in the same way.  These tests drive exactly those list launches - not the single-matrix entry points - and
compare with the CPU oracle bit for bit:

  * one full layer of the 8B Q1_0 prefill configuration (512 tokens, seven matrices, prefill tensor-core kernel),
  * one full layer of the 27B PQ2_0 configuration at 32 tokens (few-token tensor-core kernel),
  * small batches that mix matrices with different block counts and ragged last tiles at the token counts where the
    kernels change (12, 33, 64, 65, 130),
  * the K-quant matvec at its configured shapes (14336 x 4096 and 4096 x 14336, Q4_K and Q6_K, 1 / 8 / 32 tokens) with
    two matrices of each kind in one launch.

Reference semantics: token-major output for any seq_len (hearth-llm/src/pool.rs:40-80), scalar dot order
(hearth-quant/src/q1_0g128.rs:1019-1052, q2_0.rs:537-574), K-quant dots (q4_k.rs:51-96, qk_quant.rs:141-176).
The large matrices are checked on sampled rows and tokens (the oracle is scalar C), the small ones in full.
"""
import numpy as np
import pytest

from hearth_b200 import synth

pytestmark = pytest.mark.gpu

RTOL, ATOL = 1e-5, 1e-6
Q4_K, Q6_K, Q1_0, Q2_0, PQ2_0 = 12, 14, 41, 42, 142
GROUP_OF = {"q": 0, "k": 0, "v": 0, "o": 1, "gate": 2, "up": 2, "down": 3}


def assert_bits_equal(got, want, what):
    got = np.ascontiguousarray(got, dtype=np.float32)
    want = np.ascontiguousarray(want, dtype=np.float32)
    assert got.shape == want.shape, (what, got.shape, want.shape)
    np.testing.assert_allclose(got, want, rtol=RTOL, atol=ATOL, err_msg=what)
    diff = got.view(np.uint32) != want.view(np.uint32)
    assert not diff.any(), f"{what}: {int(diff.sum())} of {diff.size} outputs differ in their bits"


def sample(n, count, rng, tile):
    """Indices that always include both ends and both sides of every `tile` boundary near them."""
    must = [0, n - 1, min(tile - 1, n - 1), min(tile, n - 1), max(n - tile - 1, 0), max(n - tile, 0)]
    extra = rng.integers(0, n, max(count - len(must), 0)).tolist()
    return sorted(set(must + extra))


def run_layer(hb, oracle, cfg_name, seq_len, expect_kernel, full_check, n_row_samples, n_tok_samples):
    """All seven projections of one layer of `cfg_name` in one recorded batch, from host f32 inputs."""
    import torch
    dev = torch.device("cuda:0")
    cfg = synth.CONFIGS[cfg_name]
    dtype, shapes = cfg["dtype"], cfg["shapes"]
    assert expect_kernel in hb.selected_kernel(dtype, seq_len)
    rng = np.random.Generator(np.random.PCG64(seq_len))
    widths, xs, acts = {}, {}, {}
    for name, _, n_cols in shapes:
        widths.setdefault(GROUP_OF[name], n_cols)
    for g, k in widths.items():
        xs[g] = synth.activations(seq_len, k, seed=9000 + g)
        acts[g] = hb.Act(seq_len, k)
    ws = [synth.weights(dtype, n, k, seed=9100 + i) for i, (_, n, k) in enumerate(shapes)]
    Ws = [hb.Weight.upload(dtype, n, k, w) for (_, n, k), w in zip(shapes, ws)]
    total = sum(n for _, n, _ in shapes)
    out_dev = torch.full((seq_len, total), float("nan"), dtype=torch.float32, device=dev)
    batch = hb.Batch()
    off = 0
    for (name, n, _), W in zip(shapes, Ws):
        batch.add(W, acts[GROUP_OF[name]], seq_len, out_dev[:, off:], ld_out=total)
        off += n
    batch.seal()
    assert batch.launch_count == 1, "one persistent launch for every matrix of the layer"
    x_host = np.concatenate([xs[g].reshape(-1) for g in sorted(widths)])  # groups are first used in this order
    assert batch.input_floats == x_host.size
    out_host = np.zeros((seq_len, total), dtype=np.float32)
    try:
        batch.run_host(x_host, out_dev, out_host)
        hb.check_status()
        assert not np.isnan(out_host).any(), "an output element was never written"
        q8 = {g: oracle.quantize_q8_0(xs[g]) for g in widths}
        off = 0
        for (name, n, k), w in zip(shapes, ws):
            a = q8[GROUP_OF[name]]
            got = out_host[:, off:off + n]
            if name in full_check:
                assert_bits_equal(got, oracle.dot_rows_batched(dtype, w, a, n, k), f"{cfg_name}:{name} (all rows, all tokens)")
            else:
                rows = sample(n, n_row_samples, rng, 128)
                toks = sample(seq_len, n_tok_samples, rng, 32)
                want = oracle.dot_rows_batched(dtype, np.ascontiguousarray(w[rows]), np.ascontiguousarray(a[toks]), len(rows), k)
                assert len(rows) * len(toks) >= 64
                assert_bits_equal(got[np.ix_(toks, rows)], want, f"{cfg_name}:{name} ({len(rows)} rows x {len(toks)} tokens)")
            off += n
    finally:
        batch.free()
        for a in acts.values():
            a.free()
        for W in Ws:
            W.free()


def test_prefill_layer_in_one_list_launch(hb, oracle):
    """Config 2 (8B Q1_0, 512 tokens): q/k/v/o/gate/up/down of one layer through the prefill tensor-core list launch.
    k and v are compared in full, the others (down with its 96 K-blocks among them) on sampled rows and tokens."""
    run_layer(hb, oracle, "c2_q1_8b_prefill_1layer", 512, "gemm_tcgen05", full_check=("k", "v"), n_row_samples=24, n_tok_samples=12)


def test_27b_layer_at_32_tokens_in_one_list_launch(hb, oracle):
    """Config 4 at M = 32 (27B PQ2_0): one layer through the few-token tensor-core list launch."""
    run_layer(hb, oracle, "c4_pq2_27b_m32_2layers", 32, "_rows_", full_check=("k",), n_row_samples=24, n_tok_samples=32)


@pytest.mark.parametrize("seq_len", [12, 33, 64, 65, 130])
def test_mixed_matrices_cross_tile_rings(hb, oracle, seq_len):
    """Matrices with different K-block counts and ragged last row tiles in one batch: every CTA's rings run on from one
    matrix into the next in mid-stream.  Full comparison."""
    import torch
    dev = torch.device("cuda:0")
    specs = [(Q1_0, 200, 256), (Q1_0, 136, 1152), (Q1_0, 72, 2048), (Q1_0, 1, 128), (Q1_0, 321, 640),
             (Q2_0, 130, 384), (PQ2_0, 260, 1280), (Q2_0, 65, 128), (Q2_0, 515, 2304)]
    acts = {k: hb.Act(seq_len, k) for k in sorted({k for _, _, k in specs})}
    xs = {k: synth.activations(seq_len, k, seed=seq_len * 7 + k) for k in acts}
    ws = [synth.weights(dt, n, k, seed=seq_len + 31 * i, allow_code3=True) for i, (dt, n, k) in enumerate(specs)]
    Ws = [hb.Weight.upload(dt, n, k, w) for (dt, n, k), w in zip(specs, ws)]
    total = sum(n for _, n, _ in specs)
    out_dev = torch.full((seq_len, total), float("nan"), dtype=torch.float32, device=dev)
    batch = hb.Batch()
    off = 0
    for (dt, n, k), W in zip(specs, Ws):
        batch.add(W, acts[k], seq_len, out_dev[:, off:], ld_out=total)
        off += n
    batch.seal()
    assert batch.launch_count == 2  # one per weight kind
    try:
        for k, a in acts.items():
            a.quantize(seq_len, x_dev=torch.from_numpy(xs[k]).to(dev))
        for rep in range(2):
            batch.launch()
            torch.cuda.synchronize()
            hb.check_status()
            got_all = out_dev.cpu().numpy()
            off = 0
            for (dt, n, k), w in zip(specs, ws):
                want = oracle.dot_rows_batched(dt, w, oracle.quantize_q8_0(xs[k]), n, k)
                assert_bits_equal(got_all[:, off:off + n], want, f"{seq_len} tokens, dtype {dt} {n}x{k}, launch {rep}")
                off += n
    finally:
        batch.free()
        for a in acts.values():
            a.free()
        for W in Ws:
            W.free()


@pytest.mark.parametrize("seq_len", [1, 8, 32])
def test_kquant_configured_shapes_in_one_batch(hb, oracle, seq_len):
    """Config 3: 14336 x 4096 and 4096 x 14336, Q4_K and Q6_K, so that each kind's launch carries two matrices.
    Oracle on sampled rows, every token."""
    import torch
    dev = torch.device("cuda:0")
    rng = np.random.Generator(np.random.PCG64(100 + seq_len))
    specs = [(Q4_K, 14336, 4096), (Q4_K, 4096, 14336), (Q6_K, 14336, 4096), (Q6_K, 4096, 14336)]
    acts = {k: hb.Act(seq_len, k) for k in (4096, 14336)}
    xs = {k: synth.activations(seq_len, k, seed=seq_len * 11 + k) for k in acts}
    ws = [synth.weights(dt, n, k, seed=40 + i) for i, (dt, n, k) in enumerate(specs)]
    Ws = [hb.Weight.upload(dt, n, k, w) for (dt, n, k), w in zip(specs, ws)]
    total = sum(n for _, n, _ in specs)
    out_dev = torch.full((seq_len, total), float("nan"), dtype=torch.float32, device=dev)
    batch = hb.Batch()
    off = 0
    for (dt, n, k), W in zip(specs, Ws):
        batch.add(W, acts[k], seq_len, out_dev[:, off:], ld_out=total)
        off += n
    batch.seal()
    assert batch.launch_count == 2
    x_host = np.concatenate([xs[4096].reshape(-1), xs[14336].reshape(-1)])
    out_host = np.zeros((seq_len, total), dtype=np.float32)
    try:
        batch.run_host(x_host, out_dev, out_host)
        assert not np.isnan(out_host).any()
        off = 0
        for (dt, n, k), w in zip(specs, ws):
            rows = sample(n, 40, rng, 32)
            want = oracle.matmul_kquant_f32(dt, np.ascontiguousarray(w[rows]), xs[k], len(rows), k)
            got = out_host[:, off:off + n][:, rows]
            np.testing.assert_allclose(got, want, rtol=RTOL, atol=ATOL, err_msg=f"dtype {dt} {n}x{k} x {seq_len}")
            assert (got.view(np.uint32) == want.view(np.uint32)).all(), "same order as the oracle, same bits expected"
            off += n
    finally:
        batch.free()
        for a in acts.values():
            a.free()
        for W in Ws:
            W.free()


@pytest.mark.parametrize("dtype,seq_len", [(Q1_0, 1), (Q1_0, 2), (Q2_0, 1), (PQ2_0, 4), (Q1_0, 7), (8, 2)])
def test_decode_list_launch_with_cut_panels(hb, oracle, dtype, seq_len):
    """A recorded batch of decode matvecs large enough that the launch's rounds are cut into equal shares per CTA and
    panels are split between neighbouring CTAs (the ordered sum of such a panel continues from a carry in global
    memory).  Matrices with one, two and three rounds per panel (the last one ragged), a ragged last panel, and a
    change of matrix in mid-pipeline in every CTA.  Every row of every matrix is compared with the oracle, twice (the
    second launch reuses the carry slots with a new epoch)."""
    import torch
    dev = torch.device("cuda:0")
    rpp = {Q1_0: 256, Q2_0: 128, PQ2_0: 128, 8: 32}[dtype]  # rows per panel
    scale = 1 if dtype != 8 else 2  # Q8_0 panels are small: more of them
    specs = ([(25 * rpp - 37, 2048)] * (20 * scale) + [(16 * rpp, 2304)] * (16 * scale) + [(8 * rpp, 1024)] * (8 * scale)
             + [(3 * rpp + 1, 128)] * 4)
    ks = sorted({k for _, k in specs})
    acts = {k: hb.Act(seq_len, k) for k in ks}
    xs = {k: synth.activations(seq_len, k, seed=seq_len * 13 + k) for k in ks}
    ws = [synth.weights(dtype, n, k, seed=500 + i, allow_code3=True) for i, (n, k) in enumerate(specs)]
    Ws = [hb.Weight.upload(dtype, n, k, w) for (n, k), w in zip(specs, ws)]
    total = sum(n for n, _ in specs)
    out_dev = torch.full((seq_len, total), float("nan"), dtype=torch.float32, device=dev)
    batch = hb.Batch()
    off = 0
    for (n, k), W in zip(specs, Ws):
        batch.add(W, acts[k], seq_len, out_dev[:, off:], ld_out=total)
        off += n
    batch.seal()
    try:
        for k, a in acts.items():
            a.quantize(seq_len, x_dev=torch.from_numpy(xs[k]).to(dev))
        q8 = {k: oracle.quantize_q8_0(xs[k]) for k in ks}
        want = np.concatenate([oracle.dot_rows_batched(dtype, w, q8[k], n, k) for (n, k), w in zip(specs, ws)], axis=1)
        for rep in range(2):
            out_dev.fill_(float("nan"))
            batch.launch()
            torch.cuda.synchronize()
            hb.check_status()
            assert_bits_equal(out_dev.cpu().numpy(), want, f"dtype {dtype}, {seq_len} tokens, launch {rep}")
    finally:
        batch.free()
        for a in acts.values():
            a.free()
        for W in Ws:
            W.free()


def test_step_from_device_inputs_equals_step_from_host_inputs(hb):
    """hb200_batch_run_dev (inputs already on the device, written on another stream) gives the bits of
    hb200_batch_run_host, through the pipelined runs of a single-token step (64 ops) and through the one-shot path."""
    import torch
    dev = torch.device("cuda:0")
    for n_ops, seq_len in ((64, 1), (6, 3)):
        specs = [((Q1_0, Q2_0, PQ2_0, 8)[i % 4], 256 + 32 * (i % 5), (1024, 2048, 1152)[i % 3]) for i in range(n_ops)]
        ks = sorted({k for _, _, k in specs})
        acts = {k: hb.Act(seq_len, k) for k in ks}
        Ws = [hb.Weight.upload(dt, n, k, synth.weights(dt, n, k, seed=700 + i)) for i, (dt, n, k) in enumerate(specs)]
        total = sum(n for _, n, _ in specs)
        out_dev = torch.zeros((seq_len, total), dtype=torch.float32, device=dev)
        batch = hb.Batch()
        off = 0
        for (dt, n, k), W in zip(specs, Ws):
            batch.add(W, acts[k], seq_len, out_dev[:, off:], ld_out=total)
            off += n
        batch.seal()
        try:
            # the batch lists its activations in order of first use
            order = []
            for _, _, k in specs:
                if k not in order:
                    order.append(k)
            x_host = np.concatenate([synth.activations(seq_len, k, seed=70 + k).reshape(-1) for k in order])
            assert batch.input_floats == x_host.size
            a = np.zeros((seq_len, total), dtype=np.float32)
            b = np.full((seq_len, total), np.nan, dtype=np.float32)
            batch.run_host(x_host, out_dev, a)
            out_dev.fill_(float("nan"))
            side = torch.cuda.Stream(device=dev)
            with torch.cuda.stream(side):
                x_dev = torch.from_numpy(x_host).to(dev, non_blocking=False)
                x_dev = x_dev * 1.0  # produced by a kernel on the side stream
            batch.run_dev(x_dev, out_dev, b, x_stream=side)
            hb.check_status()
            assert_bits_equal(b, a, f"{n_ops} ops, {seq_len} tokens")
        finally:
            batch.free()
            for x in acts.values():
                x.free()
            for W in Ws:
                W.free()
