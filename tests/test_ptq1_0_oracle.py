"""CPU checks of the oracle's PTQ1_0 restatement, following the reference's own tests
(hearth-quant/src/ptq1_0.rs:652-819): ternary round trip, every byte pattern decodes to a trit,
f32 dot equals the dot of the dequantized row, all-ones block sums to 128, and the LCG fixture
built with the real packer has real signal.
"""
import numpy as np

PTQ1_0, Q2_0 = 143, 42


def _lcg(seed, n):
    out = np.zeros(n, dtype=np.float32)
    for i in range(n):
        seed = (seed * 1664525 + 1013904223) & 0xFFFFFFFF
        out[i] = np.float32(((seed >> 8) & 0xFFFF)) / np.float32(32768.0) - np.float32(1.0)
    return out, seed


def test_dequantize_ternary_values(oracle):
    src = np.zeros(128, dtype=np.float32)
    src[0], src[1], src[2], src[3], src[127] = -1.0, 1.0, 0.4, -0.4, 1.0
    data = oracle.quantize_ptq1_0(src)
    assert data.size == 28
    out = oracle.dequantize(PTQ1_0, data, 128)
    assert out[0] == -1.0 and out[1] == 1.0 and out[2] == 0.0 and out[3] == 0.0 and out[4] == 0.0 and out[127] == 1.0


def test_every_byte_pattern_is_ternary(oracle):
    data = np.zeros(28, dtype=np.uint8)
    data[:24] = (np.arange(24) * 37 + 11) & 0xFF
    data[24], data[25] = 0xAB, 0xC3
    data[26:28] = np.frombuffer(np.float16(0.25).tobytes(), dtype=np.uint8)
    out = oracle.dequantize(PTQ1_0, data, 128)
    assert set(np.unique(out / 0.25).tolist()) <= {-1.0, 0.0, 1.0}
    # and for all 256 byte values in every position of the block
    for b in range(256):
        data[:26] = b
        out = oracle.dequantize(PTQ1_0, data, 128)
        assert set(np.unique(out / 0.25).tolist()) <= {-1.0, 0.0, 1.0}


def test_dot_f32_matches_dequantized_dot(oracle):
    data = np.zeros(28 * 4, dtype=np.uint8)
    for i in range(data.size):
        data[i] = (i * 91 + 7) & 0xFF
    for b in range(4):
        data[b * 28 + 26:b * 28 + 28] = np.frombuffer(np.float16(0.5 + b * 0.25).tobytes(), dtype=np.uint8)
    vec = np.sin(np.arange(512, dtype=np.float32) * np.float32(0.173)).astype(np.float32)
    deq = oracle.dequantize(PTQ1_0, data, 512)
    expected = float((deq.astype(np.float64) * vec).sum())
    got = oracle.dot_ptq1_0_f32(data, vec, 512)
    assert abs(got - expected) < 1e-3 * max(abs(expected), 1.0)


def test_all_ones_block_sums_to_128(oracle):
    ones = np.ones(128, dtype=np.float32)
    q = oracle.quantize_ptq1_0(ones)
    assert np.all(oracle.dequantize(PTQ1_0, q, 128) == 1.0)
    assert abs(oracle.dot_ptq1_0_f32(q, ones, 128) - 128.0) < 0.1


def test_lcg_fixture_has_signal_and_block_dots_agree(oracle):
    # the fixture of paired_matches_two_single_calls (ptq1_0.rs:747-819)
    for n_blocks in (1, 3, 11):
        n = n_blocks * 128
        wf, _ = _lcg(0x12345678, n)
        w = oracle.quantize_ptq1_0(wf)
        assert w.size == n_blocks * 28
        a0f, _ = _lcg(0x0BADF00D, n)
        a1f, _ = _lcg(0x5EED1234, n)
        a0, a1 = oracle.quantize_q8_0(a0f * np.float32(3.0)), oracle.quantize_q8_0(a1f * np.float32(3.0))
        d0 = oracle.dot_rows_batched(PTQ1_0, w.reshape(1, -1), a0, 1, n)[0, 0]
        d1 = oracle.dot_rows_batched(PTQ1_0, w.reshape(1, -1), a1, 1, n)[0, 0]
        assert abs(d0) > 1.0 and abs(d1) > 1.0 and d0 != d1
        # integer sub-block dots against an independent numpy decode
        deq = oracle.dequantize(PTQ1_0, w, n)
        d = np.frombuffer(w.reshape(-1, 28)[:, 26:28].tobytes(), dtype=np.float16).astype(np.float32)
        trits = np.round(deq.reshape(-1, 128) / d[:, None]).astype(np.int32).reshape(-1, 32)
        aq = a0.reshape(-1, 34)[:, 2:].view(np.int8).astype(np.int32)
        assert np.array_equal(oracle.block_dots_i32(PTQ1_0, w, a0, n), (trits * aq).sum(axis=1))


def test_recoding_to_q2_0_gives_the_same_dot(oracle):
    """A PTQ1_0 row and the Q2_0 row with code = trit + 1 and the same scale have bit-identical scalar dots."""
    from hearth_b200 import synth
    n = 128 * 9
    w = synth.weights(PTQ1_0, 3, n, seed=77)
    a = oracle.quantize_q8_0(synth.activations(2, n, seed=78))
    q2 = np.zeros((3, 9, 34), dtype=np.uint8)
    for r in range(3):
        blocks = w[r].reshape(9, 28)
        q2[r, :, 0:2] = blocks[:, 26:28]
        deq = oracle.dequantize(PTQ1_0, w[r], n).reshape(9, 128)
        d = np.frombuffer(blocks[:, 26:28].tobytes(), dtype=np.float16).astype(np.float32)
        codes = (np.round(deq / d[:, None]).astype(np.int32) + 1).astype(np.uint8).reshape(9, 32, 4)
        q2[r, :, 2:] = codes[..., 0] | (codes[..., 1] << 2) | (codes[..., 2] << 4) | (codes[..., 3] << 6)
    got = oracle.dot_rows_batched(PTQ1_0, w, a, 3, n)
    want = oracle.dot_rows_batched(Q2_0, q2.reshape(3, -1), a, 3, n)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
