"""CPU tests: the oracle against the reference's known answers and golden fixtures,
and against the independent numpy restatement."""
import numpy as np
import pytest

import np_ref


def f16b(v):
    return np.frombuffer(np.float16(v).tobytes(), dtype=np.uint8)


def test_h2f_matches_ieee_for_every_half(oracle):
    hs = np.arange(65536, dtype=np.uint16)
    want = hs.view(np.float16).astype(np.float32)
    got = np.array([oracle.h2f(int(h)) for h in hs], dtype=np.float32)
    nan = np.isnan(want)
    assert (np.isnan(got) == nan).all()
    assert (got[~nan].view(np.uint32) == want[~nan].view(np.uint32)).all()


def test_f2h_is_round_to_nearest_even(oracle):
    rng = np.random.Generator(np.random.PCG64(1))
    vals = np.concatenate([
        rng.normal(0, 1, 4000), rng.normal(0, 1e-5, 2000), rng.normal(0, 3e4, 1000),
        np.array([0.0, -0.0, 65504.0, 65520.0, 65519.99, 1e-8, 5.96e-8, 2.98e-8, 2.9802322e-8, 6.1e-5, 1.0, 1.00048828125,
                  1.0009765625, 1.00146484375, np.inf, -np.inf])]).astype(np.float32)
    with np.errstate(over="ignore"):
        want = vals.astype(np.float16).view(np.uint16)
    got = np.array([oracle.f2h(float(v)) for v in vals], dtype=np.uint16)
    assert (got == want).all()


def test_block_geometry(oracle):
    # hearth-gguf/src/ggml.rs:105-176
    geo = {8: (32, 34), 12: (256, 144), 14: (256, 210), 39: (128, 18), 41: (128, 18), 43: (128, 18), 42: (128, 34),
           142: (128, 34), 143: (128, 28)}
    L = oracle.lib()
    for dt, (bs, bb) in geo.items():
        assert L.ho_block_size(dt) == bs and L.ho_block_bytes(dt) == bb
        assert oracle.byte_size(dt, 2048) == 2048 // bs * bb
        assert oracle.byte_size(dt, bs + 1) == 2 * bb  # div_ceil
    assert oracle.byte_size(13, 128) == 0  # Q5_K is outside this path


def test_q2_0_code_mapping_known_answer(oracle):
    # q2_0.rs:738-766: byte 0b00100100 with scale 2.0 dequantizes to -2, 0, +2, -2
    data = np.zeros(68, dtype=np.uint8)
    data[0:2] = f16b(2.0)
    data[2] = 0b00100100
    out = oracle.dequantize(oracle.Q2_0, data, 256)
    assert out[:4].tolist() == [-2.0, 0.0, 2.0, -2.0]
    # code 3 -> +2 (Q2V table, q2_0.rs:9-23)
    data[3] = 0b11
    assert oracle.dequantize(oracle.PQ2_0, data, 256)[4] == 4.0


def test_q1_0_sign_mapping_known_answer(oracle):
    # q1_0g128.rs:1206-1220: bits 0b00001011 -> +1, +1, -1, +1, then -1...
    data = np.zeros(18, dtype=np.uint8)
    data[0:2] = f16b(1.0)
    data[2] = 0b00001011
    out = oracle.dequantize(oracle.Q1_0_G128, data, 128)
    assert out[:8].tolist() == [1.0, 1.0, -1.0, 1.0, -1.0, -1.0, -1.0, -1.0]


def test_q4_k_zero_block_known_answer(oracle):
    # q4_k.rs:102-110
    out = oracle.dequantize(oracle.Q4_K, np.zeros(288, dtype=np.uint8), 512)
    assert (np.abs(out) < 1e-6).all()


def test_q8_0_roundtrip_bound_and_bytes(oracle, golden):
    # q8_0.rs:177-194: |src - dequant| < 1.0
    src = golden["q8_roundtrip_src"]
    q = oracle.quantize_q8_0(src)
    assert (q == golden["q8_roundtrip_q"]).all()
    deq = oracle.dequantize(oracle.Q8_0, q, 64)
    assert (np.abs(src - deq) < 1.0).all()
    # hand-derived: block 0 is -16..-0.5, max 16 -> scale 16/127; -16 -> -127, -0.5 -> round(-3.96875) = -4
    assert q[0:2].tolist() == f16b(np.float32(16.0) / np.float32(127.0)).tolist()
    assert np.int8(q[2]) == -127 and np.int8(q[33]) == -4
    # block 1 is 0..15.5, max 15.5: 0 -> 0, 15.5 -> 127
    assert np.int8(q[36]) == 0 and np.int8(q[67]) == 127


def test_quantizer_matches_numpy_restatement(oracle, golden):
    for key in ("benchk", "quant_seeded"):
        x = golden[f"{key}_x"]
        with np.errstate(over="ignore"):
            want = np_ref.quantize_q8_0(x)
        got = oracle.quantize_q8_0(x)
        assert (got == want).all()
        assert (got == golden[f"{key}_q8"]).all()


def test_quantizer_never_emits_minus_128(oracle):
    rng = np.random.Generator(np.random.PCG64(5))
    x = rng.normal(0, 1, (64, 4096)).astype(np.float32)
    q = oracle.quantize_q8_0(x).reshape(64, -1, 34)[:, :, 2:].view(np.int8)
    assert q.min() >= -127 and q.max() <= 127


def test_quantizer_ragged_tail_and_specials(oracle):
    x = np.array([1.0, -2.0, np.nan, 0.5] + [0.0] * 33, dtype=np.float32)  # 37 values: second block has 5
    q = oracle.quantize_q8_0(x)
    assert q.size == 68
    v = q.reshape(2, 34)[:, 2:].view(np.int8)
    assert v[0, 2] == 0                       # NaN -> 0
    assert v[0, 1] == -127 and v[0, 0] == 64  # round(63.5) away from zero
    assert (v[1] == 0).all()
    assert q[34:36].tolist() == f16b(1.0).tolist()  # all-zero block stores scale 1.0


@pytest.mark.parametrize("kind,dtype", [("q1", 43), ("q2", 42)])
@pytest.mark.parametrize("n", [128, 256, 2048, 6144])
def test_reference_x2_fixtures(oracle, golden, kind, dtype, n):
    """The paired-token fixtures of q1_0g128.rs:1504-1552 / q2_0.rs:939-986: the oracle's dot equals
    the golden value bit for bit, is not degenerate, and the numpy restatement agrees."""
    w = golden[f"x2_{kind}_{n}_w"]
    for t in (0, 1):
        a = golden[f"x2_{kind}_{n}_a{t}"]
        got = oracle.dot_rows_batched(dtype, w, a, 1, n)[0, 0]
        assert np.float32(got).tobytes() == golden[f"x2_{kind}_{n}_out{t}"].tobytes()
        assert abs(got) > 1e-6
        want, ints = np_ref.dot_q8x(kind, w, a, n)
        assert np.float32(want).tobytes() == np.float32(got).tobytes()
        assert (oracle.block_dots_i32(dtype, w, a, n) == ints).all()
    # two tokens through the batched entry point == two single calls (token-major output)
    a2 = np.stack([golden[f"x2_{kind}_{n}_a0"], golden[f"x2_{kind}_{n}_a1"]])
    both = oracle.dot_rows_batched(dtype, w, a2, 1, n)
    assert both.shape == (2, 1)
    assert both[0, 0].tobytes() == golden[f"x2_{kind}_{n}_out0"].tobytes()
    assert both[1, 0].tobytes() == golden[f"x2_{kind}_{n}_out1"].tobytes()


def test_q2_0_q8_path_close_to_f32_path(oracle, golden):
    # q2_0.rs:787-818
    import ctypes as C
    w, x = golden["q2_vs_f32_w"], golden["q2_vs_f32_x"]
    a = oracle.quantize_q8_0(x)
    dq8 = oracle.dot_rows_batched(oracle.Q2_0, w, a, 1, 256)[0, 0]
    df32 = oracle.lib().ho_dot_q2_0_f32(w.ctypes.data_as(C.POINTER(C.c_uint8)), x.ctypes.data_as(C.POINTER(C.c_float)), 256)
    assert abs(dq8 - df32) < max(abs(df32), 1.0) * 0.01 + 0.5


def test_q8_0_dot_against_numpy(oracle):
    from hearth_b200 import synth
    w = synth.weights(8, 3, 256, seed=11)
    a = oracle.quantize_q8_0(synth.activations(2, 256, seed=12))
    got = oracle.dot_rows_batched(8, w, a, 3, 256)
    for s in range(2):
        for r in range(3):
            want, _ = np_ref.dot_q8x("q8", w[r], a[s], 256)
            assert np.float32(want).tobytes() == got[s, r].tobytes()


def test_tail_columns_are_dropped(oracle):
    # n/128 blocks: a 200-column Q1_0 row uses only its first block (q1_0g128.rs:997-1002)
    from hearth_b200 import synth
    w = synth.weights(43, 2, 256, seed=3)
    a = oracle.quantize_q8_0(synth.activations(1, 256, seed=4))
    full = oracle.dot_rows_batched(43, w, a, 2, 128)
    import ctypes as C
    f = oracle.lib().ho_dot_q1_0g128_q8_0
    p = lambda arr: arr.ctypes.data_as(C.POINTER(C.c_uint8))
    assert np.float32(f(p(w[0]), p(a[0]), 200)).tobytes() == full[0, 0].tobytes()


def test_kquant_dot_matches_dequantized_dot(oracle):
    """Unpinned by the reference (no Q6_K tests, Q4_K zero block only): check the fused dots against
    dequantize-then-dot in float64 to a tolerance."""
    from hearth_b200 import synth
    for dt in (12, 14):
        w = synth.weights(dt, 4, 512, seed=21 + dt)
        x = synth.activations(2, 512, seed=22)
        got = oracle.matmul_kquant_f32(dt, w, x, 4, 512)
        for r in range(4):
            deq = oracle.dequantize(dt, w[r], 512).astype(np.float64)
            for s in range(2):
                want = float((deq * x[s].astype(np.float64)).sum())
                assert abs(got[s, r] - want) <= 1e-4 * max(1.0, abs(want))


def test_simd_baseline_agrees_with_scalar_oracle(oracle):
    """The restated SIMD arms: integer-identical by construction; fp32 association differs, so compare
    loosely (the reference bounds arm-vs-arm agreement at 1e-2, q1_0g128.rs:1402-1412)."""
    from hearth_b200 import synth
    S = oracle.simd()
    S.hs_pool_start(2)
    try:
        for dt in (43, 42, 8, 143):
            n_rows, n_cols = 70, 2048
            w = synth.weights(dt, n_rows, n_cols, seed=31 + dt, allow_code3=True)
            a = oracle.quantize_q8_0(synth.activations(3, n_cols, seed=32))
            want = oracle.dot_rows_batched(dt, w, a, n_rows, n_cols)
            got = oracle.simd_dot_rows_batched(dt, w, a, n_rows, n_cols)
            assert got.shape == want.shape == (3, n_rows)
            err = np.abs(got - want)
            assert (err <= 1e-4 * np.maximum(1.0, np.abs(want))).all(), (dt, err.max())
            assert S.hs_selected_kernel(dt).decode() in ("vnni256", "avx2_shuffle", "vnni512x2", "avx2_lut", "scalar",
                                                          "avx512", "avx2")
        # K-quants: the same eight-lane order as the scalar oracle, so the bits agree
        for dt in (12, 14):
            n_rows, n_cols = 37, 1024
            w = synth.weights(dt, n_rows, n_cols, seed=41 + dt)
            x = synth.activations(2, n_cols, seed=42)
            want = oracle.matmul_kquant_f32(dt, w, x, n_rows, n_cols)
            got = oracle.simd_matmul_kquant_f32(dt, w, x, n_rows, n_cols)
            assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), dt
    finally:
        S.hs_pool_stop()


def test_ptq1_0_simd_arms_share_the_integer_dots(oracle):
    """hs_dot for id 143 on rows with one non-zero activation block isolates the integer sub-block sums."""
    from hearth_b200 import synth
    n = 1152
    w = synth.weights(143, 5, n, seed=3)
    a = oracle.quantize_q8_0(synth.activations(1, n, seed=4))[0]
    S = oracle.simd()
    for r in range(5):
        got = S.hs_dot(143, w[r].ctypes.data_as(oracle._u8p), a.ctypes.data_as(oracle._u8p), n)
        want = oracle.dot_rows_batched(143, w[r:r + 1], a, 1, n)[0, 0]
        assert abs(got - want) <= 1e-4 * max(1.0, abs(want))
