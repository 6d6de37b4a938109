"""CPU checks of the oracle's fused-producer restatements (norm, gated activation, rotation).

The reference holds no golden vectors for these three functions; its own tests
assert only unit RMS after the norm and silu(1) = 0.731 (hearth-llm/src/ops.rs
tests test_rms_norm, test_silu).  Those known answers are repeated here, and
the rest pins the restatement against independent numpy arithmetic.
"""
import numpy as np
import pytest

import np_ref


def test_hadamard_matches_the_matrix_definition(oracle):
    # H[i][j] = s * (-1)^popcount(i & j), s = 1/sqrt(n) (qwen35.rs:49-50)
    rng = np.random.default_rng(11)
    for n in (1, 2, 4, 8, 64, 256):
        x = rng.normal(size=n).astype(np.float32)
        idx = np.arange(n)
        H = np.array([[(-1.0) ** bin(i & j).count("1") for j in idx] for i in idx]) / np.sqrt(n)
        got = oracle.hadamard_rotate(x, None, n)
        np.testing.assert_allclose(got, H @ x.astype(np.float64), rtol=0, atol=2e-6 * max(1, np.abs(x).max()) * np.sqrt(n))


@pytest.mark.parametrize("n,bs", [(1024, 1024), (5120, 1024), (4096, 128), (300, 64), (2048, 4), (96, 32)])
def test_hadamard_bit_equal_to_numpy_butterflies(oracle, n, bs):
    rng = np.random.default_rng(n + bs)
    x = (rng.normal(size=n) * 3).astype(np.float32)
    signs = rng.choice(np.array([-1.0, 1.0], dtype=np.float32), size=n)
    for sg in (None, signs):
        got = oracle.hadamard_rotate(x, sg, bs)
        want = np_ref.hadamard_rotate(x, sg, bs)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_hadamard_tail_is_only_sign_multiplied(oracle):
    x = np.arange(1, 301, dtype=np.float32)
    signs = np.where(np.arange(300) % 3 == 0, -1.0, 1.0).astype(np.float32)
    got = oracle.hadamard_rotate(x, signs, 64)
    assert np.array_equal(got[256:], (x * signs)[256:])


def test_hadamard_twice_is_identity_up_to_rounding(oracle):
    x = np.random.default_rng(5).normal(size=4096).astype(np.float32)
    back = oracle.hadamard_rotate(oracle.hadamard_rotate(x, None, 1024), None, 1024)
    np.testing.assert_allclose(back, x, atol=2e-6)


def test_hadamard_quantize_is_rotate_then_quantize(oracle):
    x = np.random.default_rng(6).normal(size=(3, 2048)).astype(np.float32)
    got = oracle.hadamard_quantize_q8_0(x, None, 1024)
    want = np.stack([np_ref.quantize_q8_0(np_ref.hadamard_rotate(r, None, 1024)) for r in x])
    assert np.array_equal(got, want)


def test_rms_norm_q8_known_answer_unit_rms(oracle):
    # the reference's test_rms_norm: x = 1..4, w = 1 -> output of unit RMS
    x = np.array([1.0, 2.0, 3.0, 4.0], dtype=np.float32)
    q8 = oracle.rms_norm_q8(x, np.ones(4, dtype=np.float32), 1e-5)
    assert q8.size == 34
    out = np_ref.dequantize_q8_0(q8, 4)
    assert abs(np.sqrt((out * out).mean()) - 1.0) < 0.01
    assert np.all(q8[2 + 4:] == 0)  # lanes past dim are zero (ops.rs:481-483)
    assert q8.view(np.int8)[2 + 3] == 127


@pytest.mark.parametrize("dim", [8, 40, 2048, 5120, 4099])
def test_rms_norm_q8_close_to_f64(oracle, dim):
    rng = np.random.default_rng(dim)
    x = rng.normal(size=(2, dim)).astype(np.float32)
    w = rng.normal(1.0, 0.2, size=dim).astype(np.float32)
    q8 = oracle.rms_norm_q8(x, w, 1e-6)
    for s in range(2):
        want = np_ref.rms_norm_values(x[s], w, 1e-6)
        got = np_ref.dequantize_q8_0(q8[s], dim)
        blocks = (dim + 31) // 32
        pad = np.zeros(blocks * 32)
        pad[:dim] = np.abs(want)
        step = np.repeat(pad.reshape(blocks, 32).max(axis=1) / 127.0, 32)[:dim]
        assert np.all(np.abs(got - want) <= 0.6 * step + 1e-7)  # half a step + the f16 rounding of the scale


def test_rms_norm_q8_equals_quantizer_on_exact_inputs(oracle):
    # Powers of two keep every product exact, so the fused path must reproduce quantize_q8_0(w*x*inv) bit for bit.
    x = np.tile(np.array([2.0, -2.0, 2.0, 2.0, -2.0, 2.0, 2.0, -2.0], dtype=np.float32), 8)
    w = np.tile(np.array([0.5, 1.0, 2.0, 4.0], dtype=np.float32), 16)
    q8 = oracle.rms_norm_q8(x, w, 0.0)
    normed = (w * x * np.float32(0.5)).astype(np.float32)  # rms = 2 exactly
    assert np.array_equal(q8, oracle.quantize_q8_0(normed))


def test_silu_mul_q8_known_answer(oracle):
    # the reference's test_silu: silu(0) = 0, silu(1) = 0.731
    g = np.zeros(32, dtype=np.float32)
    g[1] = 1.0
    g[2] = -1.0
    out = np_ref.dequantize_q8_0(oracle.silu_mul_q8(g, np.ones(32, dtype=np.float32)), 32)
    assert abs(out[0]) < 0.01 and abs(out[1] - 0.731) < 0.01 and abs(out[2] + 0.269) < 0.01


def test_silu_mul_q8_drops_partial_block_and_tracks_f64(oracle):
    rng = np.random.default_rng(9)
    dim = 32 * 5 + 7
    g = rng.normal(size=(2, dim)).astype(np.float32) * 3
    u = rng.normal(size=(2, dim)).astype(np.float32)
    q8 = oracle.silu_mul_q8(g, u)
    assert q8.shape == (2, 5 * 34)
    want = (g.astype(np.float64) / (1 + np.exp(-g.astype(np.float64))) * u)[:, :160]
    for s in range(2):
        got = np_ref.dequantize_q8_0(q8[s], 160)
        step = np.repeat(np.abs(want[s]).reshape(5, 32).max(axis=1) / 127.0, 32)
        assert np.all(np.abs(got - want[s]) <= 0.6 * step + 1e-6)
