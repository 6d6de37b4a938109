"""Argmax over the logits: the oracle executes the reference's two-pass reduction literally
(hearth-compute/src/lib.rs:338-450, shaders/argmax.wgsl); the CUDA kernel must return the same index."""
import numpy as np
import pytest

Q1_0 = 41


def _cases():
    rng = np.random.default_rng(3)
    out = [rng.normal(size=151669).astype(np.float32),      # the vocabulary size the reference quotes
           rng.normal(size=2048).astype(np.float32), rng.normal(size=2049).astype(np.float32),
           rng.normal(size=1).astype(np.float32), rng.normal(size=17).astype(np.float32)]
    ties = np.zeros(10000, dtype=np.float32)
    ties[[7000, 300, 9999]] = 5.0                             # equal maxima: the lowest index wins
    out.append(ties)
    nan = rng.normal(size=5000).astype(np.float32)
    nan[[0, 100, 4999]] = np.nan                              # NaN never wins
    nan[2500] = 9.0
    out.append(nan)
    out.append(np.full(4100, -np.inf, dtype=np.float32))      # nothing exceeds -FLT_MAX: index 0
    low = np.full(4100, -np.inf, dtype=np.float32)
    low[3000] = np.float32(-3.4028235e38)                     # equal to the scan's start value: still index 0
    out.append(low)
    inf = rng.normal(size=70000).astype(np.float32)
    inf[[65000, 66000]] = np.inf
    out.append(inf)
    out.append(np.array([np.nan, np.nan, 1.0, np.nan], dtype=np.float32))
    return out


def test_oracle_argmax_semantics(oracle):
    for x in _cases():
        got = oracle.argmax_f32(x)
        with np.errstate(all="ignore"):
            ok = x > np.float32(-3.4028235e38)                # NaN compares false
            want = int(np.flatnonzero(ok & (x == x[ok].max()))[0]) if ok.any() else 0
        assert got == want, (x.size, got, want)


@pytest.mark.gpu
def test_gpu_argmax_matches_oracle(hb, oracle):
    import torch
    for x in _cases():
        xd = torch.from_numpy(x).cuda()
        assert hb.argmax_f32_dev(xd) == oracle.argmax_f32(x), x.size
        idx = torch.full((1,), -1, dtype=torch.int32, device="cuda")
        hb.argmax_f32_dev_async(xd, idx)
        torch.cuda.synchronize()
        assert int(idx.item()) == oracle.argmax_f32(x)
    with pytest.raises(hb.Hb200Error):
        hb.argmax_f32_dev(torch.zeros(0, device="cuda"))


@pytest.mark.gpu
def test_lm_head_then_argmax(hb, oracle):
    """The last step of a decoded token: logits = lm_head (151 669 rows, the reference's vocabulary,
    docs/BENCHMARKS.md:22) x hidden state, then argmax; only the index leaves the GPU."""
    import torch
    from hearth_b200 import synth
    n_rows, n_cols = 151669, 1024
    w = synth.weights(Q1_0, n_rows, n_cols, seed=12)
    x = synth.activations(1, n_cols, seed=13)
    W = hb.Weight.upload(Q1_0, n_rows, n_cols, w)
    A = hb.Act(1, n_cols)
    logits = torch.zeros(1, n_rows, device="cuda")
    A.quantize(1, torch.from_numpy(x).cuda())
    hb.dot_rows_dev(W, A, 1, logits)
    got = hb.argmax_f32_dev(logits)
    want_logits = oracle.dot_rows_batched(Q1_0, w, oracle.quantize_q8_0(x), n_rows, n_cols)
    assert np.array_equal(logits.cpu().numpy().view(np.uint32), want_logits.view(np.uint32))
    assert got == oracle.argmax_f32(want_logits[0])
    A.free(); W.free()
