"""GPU parity tests for PTQ1_0 (dense base-3 ternary, GGML id 143) x Q8_0 against the CPU oracle.

The weights are re-coded to 2-bit codes when they are uploaded, so every integer sub-block dot and
every fp32 output must equal the scalar reference order bit for bit, as for Q2_0.
"""
import numpy as np
import pytest

from hearth_b200 import synth
from test_gpu_parity import assert_bits_equal
from test_ptq1_0_oracle import _lcg

pytestmark = pytest.mark.gpu

PTQ1_0 = 143


@pytest.mark.parametrize("n_rows,n_cols", [(6144, 2048), (300, 2048), (7, 128), (1, 128), (257, 6144), (129, 256), (33, 5120)])
def test_ptq1_0_single_token(hb, oracle, n_rows, n_cols):
    w = synth.weights(PTQ1_0, n_rows, n_cols, seed=n_rows + n_cols)
    a = oracle.quantize_q8_0(synth.activations(1, n_cols, seed=n_cols))[0]
    W = hb.Weight.upload(PTQ1_0, n_rows, n_cols, w)
    try:
        assert W.packed_bytes == n_rows * (n_cols // 128) * 28
        got = hb.par_dot_rows(W, a)
        want = oracle.dot_rows_batched(PTQ1_0, w, a, n_rows, n_cols)[0]
        assert_bits_equal(got, want, f"PTQ1_0 {n_rows}x{n_cols}")
        assert np.abs(want).max() > 1e-6
    finally:
        W.free()


@pytest.mark.parametrize("seq_len", [2, 5, 9, 50, 130])
def test_ptq1_0_batched_including_the_tensor_core_path(hb, oracle, seq_len):
    n_rows, n_cols = 200, 1152
    w = synth.weights(PTQ1_0, n_rows, n_cols, seed=seq_len)
    a = oracle.quantize_q8_0(synth.activations(seq_len, n_cols, seed=100 + seq_len))
    W = hb.Weight.upload(PTQ1_0, n_rows, n_cols, w)
    try:
        got = hb.par_dot_rows_batched(W, a)
        assert_bits_equal(got, oracle.dot_rows_batched(PTQ1_0, w, a, n_rows, n_cols), f"PTQ1_0 seq {seq_len}")
    finally:
        W.free()


def test_ptq1_0_every_byte_value_and_raw_activation_bytes(hb, oracle):
    n_rows, n_cols = 64, 1024
    rng = np.random.Generator(np.random.PCG64(9))
    w = rng.integers(0, 256, (n_rows, n_cols // 128, 28), dtype=np.uint8)  # any byte is a legal digit group
    w[:, :, 26:28] = np.frombuffer(np.float16(0.03125).tobytes(), dtype=np.uint8)
    w[0, 0, :26] = np.arange(26) * 9  # includes bytes 0 and 225..
    w = w.reshape(n_rows, -1)
    a = rng.integers(0, 256, (2, n_cols // 32, 34), dtype=np.uint8)
    a[:, :, 0:2] = np.frombuffer(np.float16(0.01).tobytes(), dtype=np.uint8)
    a[0, 0, 2:34] = 0x80
    a = a.reshape(2, -1)
    W = hb.Weight.upload(PTQ1_0, n_rows, n_cols, w)
    try:
        got = hb.block_dots_i32(W, a)
        for s in range(2):
            for r in range(n_rows):
                assert (got[s, r] == oracle.block_dots_i32(PTQ1_0, w[r], a[s], n_cols)).all(), (s, r)
        assert_bits_equal(hb.par_dot_rows_batched(W, a), oracle.dot_rows_batched(PTQ1_0, w, a, n_rows, n_cols), "raw bytes")
    finally:
        W.free()


def test_ptq1_0_reference_lcg_fixture(hb, oracle):
    """The fixture of paired_matches_two_single_calls (hearth-quant/src/ptq1_0.rs:747-819): real packer, LCG inputs."""
    for n_blocks in (1, 3, 11):
        n = n_blocks * 128
        wf, _ = _lcg(0x12345678, n)
        w = oracle.quantize_ptq1_0(wf).reshape(1, -1)
        a0f, _ = _lcg(0x0BADF00D, n)
        a1f, _ = _lcg(0x5EED1234, n)
        a = np.stack([oracle.quantize_q8_0(a0f * np.float32(3.0)), oracle.quantize_q8_0(a1f * np.float32(3.0))])
        W = hb.Weight.upload(PTQ1_0, 1, n, w)
        try:
            got = hb.par_dot_rows_batched(W, a)  # paired call == two single calls, by construction of the kernel
            want = oracle.dot_rows_batched(PTQ1_0, w, a, 1, n)
            assert_bits_equal(got, want, f"LCG fixture n={n}")
            assert_bits_equal(hb.par_dot_rows(W, a[1]), want[1], "single call, token 1")
            assert abs(want[0, 0]) > 1.0 and abs(want[1, 0]) > 1.0
        finally:
            W.free()


def test_ptq1_0_folded_matmul_and_row_split(hb, oracle):
    """rotate -> quantize -> PTQ1_0 dot (qwen35.rs:924-975), with the weight uploaded as two row ranges."""
    n_rows, n_cols = 300, 2048
    w = synth.weights(PTQ1_0, n_rows, n_cols, seed=21)
    x = synth.activations(1, n_cols, seed=22)
    a = hb.hadamard_quantize_q8_0(x, None, 1024)
    assert (a == oracle.hadamard_quantize_q8_0(x, None, 1024)).all()
    want = oracle.dot_rows_batched(PTQ1_0, w, a, n_rows, n_cols)[0]
    parts = []
    for lo, hi in ((0, 150), (150, 300)):
        W = hb.Weight.upload(PTQ1_0, n_rows, n_cols, w, rows=(lo, hi))
        parts.append(hb.par_dot_rows(W, a[0]))
        W.free()
    assert_bits_equal(np.concatenate(parts), want, "row split")
