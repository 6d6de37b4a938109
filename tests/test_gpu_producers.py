"""GPU parity tests of the fused Q8_0 producers (norm, gated activation, rotation) against the CPU oracle.

rms_norm_q8 and the Hadamard rotation use only IEEE operations in the reference's order: every output byte
must equal the oracle's.  silu_mul_q8 goes through exp (CUDA's expf here, libm's in the oracle, `wide`'s
polynomial in the reference), so its bar is the stated tolerance: equal scales within one f16 step and
quantized values within one step, almost all equal.
"""
import numpy as np
import pytest

from hearth_b200 import synth

pytestmark = pytest.mark.gpu

Q8_0, PQ2_0 = 8, 142


def _signs(n, seed):
    return np.random.default_rng(seed).choice(np.array([-1.0, 1.0], dtype=np.float32), size=n)


# ---------------------------------------------------------------------------------- rms_norm_q8

@pytest.mark.parametrize("seq_len,dim", [(1, 2048), (1, 8), (1, 4), (3, 37), (2, 1000), (5, 5120), (1, 4099), (2, 12288),
                                         (1, 32768)])
def test_rms_norm_q8_bytes_match_oracle(hb, oracle, seq_len, dim):
    x = synth.activations(seq_len, dim, seed=300 + dim)
    w = (1.0 + 0.2 * synth.activations(1, dim, seed=301 + dim)[0]).astype(np.float32)
    got = hb.rms_norm_q8(x, w, 1e-6)
    want = oracle.rms_norm_q8(x, w, 1e-6)
    assert got.shape == want.shape
    assert (got == want).all(), f"{int((got != want).sum())} of {got.size} bytes differ"


def test_rms_norm_q8_specials_and_limits(hb, oracle):
    x = np.zeros((1, 64), dtype=np.float32)  # all-zero row: rms = sqrt(eps), every block scale 1
    w = np.ones(64, dtype=np.float32)
    assert (hb.rms_norm_q8(x, w, 1e-5) == oracle.rms_norm_q8(x, w, 1e-5)).all()
    x[0, 3] = np.inf
    with np.errstate(all="ignore"):
        assert (hb.rms_norm_q8(x, w, 1e-5) == oracle.rms_norm_q8(x, w, 1e-5)).all()
    with pytest.raises(RuntimeError):
        hb.rms_norm_q8(np.zeros((1, 32768 + 32), dtype=np.float32), np.ones(32768 + 32, dtype=np.float32), 1e-5)


def test_rms_norm_q8_feeds_the_matvec(hb, oracle):
    """Device form: norm into an activation's planes, then the dot, equals oracle norm -> oracle dot."""
    import torch
    n_rows, n_cols, seq = 96, 2048, 3
    w = synth.weights(Q8_0, n_rows, n_cols, seed=5)
    x = synth.activations(seq, n_cols, seed=6)
    g = (1.0 + 0.1 * synth.activations(1, n_cols, seed=7)[0]).astype(np.float32)
    W = hb.Weight.upload(Q8_0, n_rows, n_cols, w)
    A = hb.Act(seq, n_cols)
    out = torch.zeros(seq, n_rows, device="cuda")
    A.rms_norm_q8(torch.from_numpy(x).cuda(), torch.from_numpy(g).cuda(), 1e-6, seq)
    hb.dot_rows_dev(W, A, seq, out)
    torch.cuda.synchronize()
    want = oracle.dot_rows_batched(Q8_0, w, oracle.rms_norm_q8(x, g, 1e-6), n_rows, n_cols)
    assert np.array_equal(out.cpu().numpy().view(np.uint32), want.view(np.uint32))
    A.free(); W.free()


# ---------------------------------------------------------------------------------- hadamard -> quantize

@pytest.mark.parametrize("seq_len,dim,bs", [(1, 1024, 1024), (2, 5120, 1024), (1, 17408, 1024), (3, 4096, 128), (1, 300, 64),
                                            (2, 2048, 4), (1, 96, 32), (1, 64, 2), (1, 40, 1), (2, 1536, 512), (1, 256, 256),
                                            (1, 1000, 0)])
@pytest.mark.parametrize("with_signs", [False, True])
def test_hadamard_quantize_matches_oracle(hb, oracle, seq_len, dim, bs, with_signs):
    x = synth.activations(seq_len, dim, seed=400 + dim + bs)
    sg = _signs(dim, dim + bs) if with_signs else None
    got, rot = hb.hadamard_quantize_q8_0(x, sg, bs, return_rotated=True)
    want_rot = oracle.hadamard_rotate(x, sg, bs)
    assert np.array_equal(rot.view(np.uint32), want_rot.view(np.uint32)), "rotated f32 rows differ in their bits"
    want = oracle.hadamard_quantize_q8_0(x, sg, bs)
    assert (got == want).all(), f"{int((got != want).sum())} of {got.size} bytes differ"


def test_hadamard_rejects_unsupported_blocks(hb):
    x = np.zeros((1, 4096), dtype=np.float32)
    for bs in (3, 48, 2048):
        with pytest.raises(RuntimeError):
            hb.hadamard_quantize_q8_0(x, None, bs)


def test_folded_matmul_step(hb, oracle):
    """The hybrid models' folded matmul (qwen35.rs:924-975): rotate, quantize, PQ2_0 dot; device form vs oracle."""
    import torch
    n_rows, n_cols, seq = 256, 5120, 2
    w = synth.weights(PQ2_0, n_rows, n_cols, seed=8)
    x = synth.activations(seq, n_cols, seed=9)
    sg = _signs(n_cols, 10)
    W = hb.Weight.upload(PQ2_0, n_rows, n_cols, w)
    A = hb.Act(seq, n_cols)
    out = torch.zeros(seq, n_rows, device="cuda")
    A.hadamard_quantize(seq, 1024, x_dev=torch.from_numpy(x).cuda(), signs_dev=torch.from_numpy(sg).cuda())
    hb.dot_rows_dev(W, A, seq, out)
    torch.cuda.synchronize()
    want = oracle.dot_rows_batched(PQ2_0, w, oracle.hadamard_quantize_q8_0(x, sg, 1024), n_rows, n_cols)
    assert np.array_equal(out.cpu().numpy().view(np.uint32), want.view(np.uint32))
    A.free(); W.free()


# ---------------------------------------------------------------------------------- silu_mul_q8

@pytest.mark.parametrize("seq_len,dim", [(1, 32), (1, 6144), (3, 17408), (2, 167), (1, 31)])
def test_silu_mul_q8_within_one_step_of_oracle(hb, oracle, seq_len, dim):
    g = 3.0 * synth.activations(seq_len, dim, seed=500 + dim)
    u = synth.activations(seq_len, dim, seed=501 + dim)
    got = hb.silu_mul_q8(g, u)
    want = oracle.silu_mul_q8(g, u)
    assert got.shape == want.shape == (seq_len, dim // 32 * 34)
    if got.size == 0:
        return
    gb, wb = got.reshape(-1, 34), want.reshape(-1, 34)
    gs = gb[:, :2].copy().view(np.uint16).astype(np.int32).ravel()
    ws = wb[:, :2].copy().view(np.uint16).astype(np.int32).ravel()
    assert np.abs(gs - ws).max() <= 1, "block scales differ by more than one f16 step"
    gq, wq = gb[:, 2:].view(np.int8).astype(np.int32), wb[:, 2:].view(np.int8).astype(np.int32)
    assert np.abs(gq - wq).max() <= 1, "a quantized value differs by more than one step"
    assert (gq != wq).mean() < 0.01


def test_silu_mul_q8_known_answer(hb):
    g = np.zeros(32, dtype=np.float32)
    g[1], g[2] = 1.0, -1.0
    q8 = hb.silu_mul_q8(g, np.ones(32, dtype=np.float32))
    d = q8[:2].copy().view(np.float16).astype(np.float32)[0]
    out = d * q8[2:].view(np.int8).astype(np.float32)
    assert abs(out[0]) < 0.01 and abs(out[1] - 0.731) < 0.01 and abs(out[2] + 0.269) < 0.01
