"""GPU parity tests for the two tcgen05 (tensor-core) matmuls of Q1_0 / Q2_0 weights: the few-token kernel with the
weight rows on the MMA's M side (11 .. 64 tokens of Q1_0, 12 .. 64 of Q2_0) and the prefill kernel with the tokens on
the M side (more than 64).  Fewer tokens run as passes of the streaming decode kernel; a few such cases are kept
here on purpose.

Same bar as the decode kernel: the int32 sub-block dots are exact and the fp32 scaling replays the scalar
order, so the outputs must equal the oracle's bits (1e-5 rel / 1e-6 abs asserted as the outer bound).
"""
import numpy as np
import pytest

from hearth_b200 import synth

pytestmark = pytest.mark.gpu

RTOL, ATOL = 1e-5, 1e-6
Q1_0, Q2_0, PQ2_0 = 41, 42, 142


def check(got, want, what):
    np.testing.assert_allclose(got, want, rtol=RTOL, atol=ATOL, err_msg=what)
    diff = got.view(np.uint32) != want.view(np.uint32)
    assert not diff.any(), f"{what}: {int(diff.sum())} of {diff.size} outputs differ in their bits"


@pytest.mark.parametrize("dtype", [Q1_0, Q2_0])
@pytest.mark.parametrize("n_rows,n_cols,seq_len", [
    (64, 128, 48), (200, 2048, 65), (264, 1152, 128), (1000, 2048, 130), (96, 6144, 49), (8, 256, 300), (520, 2048, 33),
    (130, 1152, 17), (130, 1152, 25), (72, 256, 24), (72, 256, 16),
    (300, 1152, 5), (300, 1152, 7), (129, 128, 8), (300, 1152, 10), (300, 1152, 11), (300, 1152, 12), (300, 1152, 13), (128, 2304, 31), (1, 256, 32), (257, 640, 64), (384, 1152, 96), (100, 512, 97),
    (64, 128, 4), (700, 4096, 40), (260, 384, 200)])
def test_tensor_core_matches_oracle(hb, oracle, dtype, n_rows, n_cols, seq_len):
    min_tokens = 11 if dtype == Q1_0 else 12
    name = hb.selected_kernel(dtype, seq_len)
    assert name.startswith("gemm_tcgen05_i8" if seq_len >= min_tokens else "gemv_dp4a")
    assert ("_rows_" in name) == (min_tokens <= seq_len <= 64)
    w = synth.weights(dtype, n_rows, n_cols, seed=dtype * 3 + n_rows, allow_code3=True)
    a = oracle.quantize_q8_0(synth.activations(seq_len, n_cols, seed=seq_len))
    W = hb.Weight.upload(dtype, n_rows, n_cols, w)
    try:
        got = hb.par_dot_rows_batched(W, a)
        want = oracle.dot_rows_batched(dtype, w, a, n_rows, n_cols)
        assert got.shape == (seq_len, n_rows)
        check(got, want, f"dtype {dtype} {n_rows}x{n_cols} x {seq_len} tokens")
        assert np.abs(want).max() > 1e-6
    finally:
        W.free()


def test_tensor_core_raw_bytes_with_minus_128(hb, oracle):
    """Activation bytes the quantizer never emits (0x80) and negative / zero scales must still be exact."""
    n_rows, n_cols, seq_len = 130, 512, 50
    rng = np.random.Generator(np.random.PCG64(8))
    a = rng.integers(0, 256, (seq_len, n_cols // 32, 34), dtype=np.uint8)
    scales = rng.normal(0, 0.02, (seq_len, n_cols // 32)).astype(np.float16)
    scales[0, 0] = 0.0
    a[:, :, 0:2] = scales.view(np.uint8).reshape(seq_len, n_cols // 32, 2)
    a[1, 3, 2:] = 0x80
    a = a.reshape(seq_len, -1)
    for dtype in (Q1_0, PQ2_0):
        w = synth.weights(dtype, n_rows, n_cols, seed=70 + dtype, allow_code3=True)
        W = hb.Weight.upload(dtype, n_rows, n_cols, w)
        try:
            check(hb.par_dot_rows_batched(W, a), oracle.dot_rows_batched(dtype, w, a, n_rows, n_cols), f"raw bytes dtype {dtype}")
        finally:
            W.free()


def test_tensor_core_equals_decode_kernel_token_by_token(hb, oracle):
    """The paired-token contract of the reference (x2 == two single calls, q1_0g128.rs:1504-1552) extended to
    many tokens: a batched call over 72 tokens equals single-token calls bit for bit."""
    n_rows, n_cols, seq_len = 520, 2048, 72
    for dtype in (Q1_0, Q2_0):
        w = synth.weights(dtype, n_rows, n_cols, seed=5 + dtype)
        a = oracle.quantize_q8_0(synth.activations(seq_len, n_cols, seed=6))
        W = hb.Weight.upload(dtype, n_rows, n_cols, w)
        try:
            batched = hb.par_dot_rows_batched(W, a)
            for s in (0, 1, 17, 71):
                single = hb.par_dot_rows(W, a[s])
                assert (single.view(np.uint32) == batched[s].view(np.uint32)).all()
        finally:
            W.free()


def test_prefill_shape_sampled_rows(hb, oracle):
    """Config 2 shape (8B, M=512): the k projection in full and the gate projection on sampled tokens."""
    seq_len = 512
    for n_rows, n_cols, toks in ((1024, 4096, None), (12288, 4096, [0, 5, 127, 128, 300, 511])):
        w = synth.weights(Q1_0, n_rows, n_cols, seed=n_rows)
        x = synth.activations(seq_len, n_cols, seed=n_cols)
        W = hb.Weight.upload(Q1_0, n_rows, n_cols, w)
        try:
            got = hb.matmul(W, x)
        finally:
            W.free()
        a = oracle.quantize_q8_0(x)
        if toks is None:
            check(got, oracle.dot_rows_batched(Q1_0, w, a, n_rows, n_cols), "k projection, 512 tokens")
        else:
            check(got[toks], oracle.dot_rows_batched(Q1_0, w, a[toks], n_rows, n_cols), "gate projection, sampled tokens")


def test_int8_peak_measurement_is_plausible(hb):
    """A bare run of kind::i8 MMAs: between the promotion-bound kernel's rate and the 4.5 POP/s nominal figure."""
    tops = hb.measure_i8_peak()
    assert 1000.0 < tops < 5000.0, tops
    hb.check_status()
