"""GPU parity tests: the CUDA path, called through the C ABI, against the CPU oracle.

Bit-exact for the quantizer bytes, the integer sub-block dots and (because the kernels replay the
scalar float order) the fp32 outputs of the Q8_0-activation dots; the stated tolerance
1e-5 relative / 1e-6 absolute is asserted as well, as the contract's outer bound.
"""
import numpy as np
import pytest

from hearth_b200 import synth

pytestmark = pytest.mark.gpu

RTOL, ATOL = 1e-5, 1e-6

Q8_0, Q4_K, Q6_K, Q1_0, Q2_0, Q1_0_G128, PQ2_0 = 8, 12, 14, 41, 42, 43, 142


def assert_bits_equal(got: np.ndarray, want: np.ndarray, what: str):
    got = np.ascontiguousarray(got, dtype=np.float32)
    want = np.ascontiguousarray(want, dtype=np.float32)
    assert got.shape == want.shape, (what, got.shape, want.shape)
    np.testing.assert_allclose(got, want, rtol=RTOL, atol=ATOL, err_msg=what)
    diff = got.view(np.uint32) != want.view(np.uint32)
    assert not diff.any(), f"{what}: {int(diff.sum())} of {diff.size} outputs differ in their bits"


# ---------------------------------------------------------------------------------- quantizer

@pytest.mark.parametrize("seq_len,dim", [(1, 2048), (1, 32), (3, 37), (7, 4096), (2, 1000), (1, 12288), (5, 5120)])
def test_quantizer_bytes_match_oracle(hb, oracle, seq_len, dim):
    x = synth.activations(seq_len, dim, seed=100 + dim)
    got = hb.quantize_q8_0(x)
    want = oracle.quantize_q8_0(x)
    assert got.shape == want.shape
    assert (got == want).all(), f"{int((got != want).sum())} bytes differ"


def test_quantizer_golden_and_specials(hb, oracle, golden):
    for key in ("q8_roundtrip_src", "benchk_x", "quant_seeded_x"):
        x = golden[key]
        want = golden[key.replace("_src", "_q").replace("_x", "_q8")]
        assert (hb.quantize_q8_0(x) == want).all(), key
    x = np.zeros(128, dtype=np.float32)
    x[0], x[1], x[2] = np.nan, np.inf, -1.0
    x[40] = np.float32(1e-45)  # subnormal: scale underflows f16 to zero
    x[70] = -0.0
    x[96:128] = np.float32(127.5)
    with np.errstate(all="ignore"):
        assert (hb.quantize_q8_0(x) == oracle.quantize_q8_0(x)).all()


def test_quantizer_half_way_cases_round_away_from_zero(hb, oracle):
    # max 127 -> scale exactly 1: x.5 values must round away from zero, not to even
    x = np.array([127.0, 0.5, 1.5, 2.5, -0.5, -1.5, -2.5, 63.5] + [0.0] * 24, dtype=np.float32)
    got = hb.quantize_q8_0(x)
    assert (got == oracle.quantize_q8_0(x)).all()
    assert got[2:10].view(np.int8).tolist() == [127, 1, 2, 3, -1, -2, -3, 64]


def test_quantizer_empty(hb):
    assert hb.quantize_q8_0(np.zeros((0, 64), dtype=np.float32)).shape == (0, 68)


# ---------------------------------------------------------------------------------- Q8_0-activation dots

SHAPES = [(6144, 2048), (300, 2048), (7, 128), (1, 128), (257, 6144), (1000, 1152), (129, 256), (33, 5120)]


@pytest.mark.parametrize("dtype", [Q1_0, Q1_0_G128, Q2_0, PQ2_0, Q8_0])
@pytest.mark.parametrize("n_rows,n_cols", SHAPES)
def test_dot_rows_single_token(hb, oracle, dtype, n_rows, n_cols):
    w = synth.weights(dtype, n_rows, n_cols, seed=7 * dtype + n_rows, allow_code3=True)
    a = oracle.quantize_q8_0(synth.activations(1, n_cols, seed=n_cols))[0]
    W = hb.Weight.upload(dtype, n_rows, n_cols, w)
    try:
        got = hb.par_dot_rows(W, a)
        want = oracle.dot_rows_batched(dtype, w, a, n_rows, n_cols)[0]
        assert_bits_equal(got, want, f"dtype {dtype} {n_rows}x{n_cols}")
        assert np.abs(want).max() > 1e-6, "degenerate fixture"
    finally:
        W.free()


@pytest.mark.parametrize("dtype", [Q1_0, Q2_0, Q8_0])
@pytest.mark.parametrize("seq_len", [2, 3, 4, 5, 9])
def test_dot_rows_batched_token_major(hb, oracle, dtype, seq_len):
    n_rows, n_cols = 520, 2048
    w = synth.weights(dtype, n_rows, n_cols, seed=dtype, allow_code3=True)
    a = oracle.quantize_q8_0(synth.activations(seq_len, n_cols, seed=seq_len))
    W = hb.Weight.upload(dtype, n_rows, n_cols, w)
    try:
        got = hb.par_dot_rows_batched(W, a)
        want = oracle.dot_rows_batched(dtype, w, a, n_rows, n_cols)
        assert got.shape == (seq_len, n_rows)
        assert_bits_equal(got, want, f"dtype {dtype} seq {seq_len}")
        # a q8_stride wider than a row (padding between tokens)
        wide = np.zeros((seq_len, a.shape[1] + 6), dtype=np.uint8)
        wide[:, :a.shape[1]] = a
        got2 = hb.par_dot_rows_batched(W, wide, seq_len, wide.shape[1])
        assert_bits_equal(got2, want, "padded stride")
    finally:
        W.free()


@pytest.mark.parametrize("dtype", [Q1_0, Q2_0, Q8_0])
def test_integer_block_dots_exact(hb, oracle, dtype):
    n_rows, n_cols = 77, 1152
    w = synth.weights(dtype, n_rows, n_cols, seed=900 + dtype, allow_code3=True)
    rng = np.random.Generator(np.random.PCG64(4))
    # raw Q8_0 rows with every byte value, -128 included, which the quantizer itself never produces
    a = rng.integers(0, 256, (2, n_cols // 32, 34), dtype=np.uint8)
    a[:, :, 0:2] = np.frombuffer(np.float16(0.01).tobytes(), dtype=np.uint8)
    a[0, 0, 2:34] = 0x80
    a = a.reshape(2, -1)
    W = hb.Weight.upload(dtype, n_rows, n_cols, w)
    try:
        got = hb.block_dots_i32(W, a)
        for s in range(2):
            for r in range(n_rows):
                want = oracle.block_dots_i32(dtype, w[r], a[s], n_cols)
                assert (got[s, r] == want).all(), (dtype, s, r)
        out = hb.par_dot_rows_batched(W, a)
        assert_bits_equal(out, oracle.dot_rows_batched(dtype, w, a, n_rows, n_cols), "fp32 with 0x80 bytes")
    finally:
        W.free()


@pytest.mark.parametrize("kind,dtype", [("q1", Q1_0_G128), ("q2", Q2_0)])
@pytest.mark.parametrize("n", [128, 256, 2048, 6144])
def test_reference_x2_fixtures_on_gpu(hb, golden, kind, dtype, n):
    """The fixtures of q1_0g128.rs:1504-1552 / q2_0.rs:939-986: both tokens in one batched call
    (the paired-token contract) and one at a time give the golden bits."""
    w = golden[f"x2_{kind}_{n}_w"]
    a = np.stack([golden[f"x2_{kind}_{n}_a0"], golden[f"x2_{kind}_{n}_a1"]])
    W = hb.Weight.upload(dtype, 1, n, w)
    try:
        both = hb.par_dot_rows_batched(W, a)
        for t in (0, 1):
            want = golden[f"x2_{kind}_{n}_out{t}"]
            assert both[t, 0].tobytes() == want.tobytes()
            assert hb.par_dot_rows(W, a[t])[0].tobytes() == want.tobytes()
            assert (hb.block_dots_i32(W, a[t])[0, 0] == golden[f"x2_{kind}_{n}_int{t}"]).all()
    finally:
        W.free()


def test_matmul_quantizes_then_dots(hb, oracle):
    """LlamaModel::matmul with x_q8 = None: quantize_act then par_dot_rows (matmul.rs:569-573)."""
    for dtype in (Q1_0, PQ2_0, Q8_0):
        n_rows, n_cols = 264, 2048
        w = synth.weights(dtype, n_rows, n_cols, seed=55 + dtype)
        x = synth.activations(3, n_cols, seed=56)
        W = hb.Weight.upload(dtype, n_rows, n_cols, w)
        try:
            got = hb.matmul(W, x)
            want = oracle.dot_rows_batched(dtype, w, oracle.quantize_q8_0(x), n_rows, n_cols)
            assert_bits_equal(got, want, f"matmul dtype {dtype}")
            assert_bits_equal(hb.matmul(W, x[0]), want[0], "matmul single vector")
        finally:
            W.free()


def test_tail_columns_dropped_like_reference(hb, oracle):
    # 200 columns of Q1_0: two blocks are stored, only the first full one is used (n/128)
    n_rows, n_cols = 40, 200
    w = synth.weights(Q1_0, n_rows, n_cols, seed=77)
    a = oracle.quantize_q8_0(synth.activations(1, n_cols, seed=78))[0]
    W = hb.Weight.upload(Q1_0, n_rows, n_cols, w)
    try:
        got = hb.par_dot_rows(W, a)
        want = oracle.dot_rows_batched(Q1_0, w, a, n_rows, n_cols)[0]
        assert_bits_equal(got, want, "tail")
    finally:
        W.free()


def test_row_range_upload_is_the_pool_row_split(hb, oracle):
    n_rows, n_cols = 1000, 2048
    w = synth.weights(Q2_0, n_rows, n_cols, seed=5)
    a = oracle.quantize_q8_0(synth.activations(1, n_cols, seed=6))[0]
    want = oracle.dot_rows_batched(Q2_0, w, a, n_rows, n_cols)[0]
    parts = []
    T = 3
    chunk = -(-n_rows // T)  # ceil(n / T), pool.rs:321-323
    for i in range(T):
        lo, hi = i * chunk, min((i + 1) * chunk, n_rows)
        W = hb.Weight.upload(Q2_0, n_rows, n_cols, w, rows=(lo, hi))
        parts.append(hb.par_dot_rows(W, a))
        W.free()
    assert_bits_equal(np.concatenate(parts), want, "row split")


# ---------------------------------------------------------------------------------- K-quants

@pytest.mark.parametrize("dtype", [Q4_K, Q6_K])
@pytest.mark.parametrize("n_rows,n_cols,seq_len", [(64, 4096, 1), (37, 512, 3), (5, 14336, 2), (1, 256, 1),
                                                    (33, 1280, 9), (40, 768, 5), (70, 2304, 1), (3, 1792, 2),
                                                    # eight and more tokens: the two-rows-per-lane kernel, Q4_K with 8, 16 or
                                                    # 32 tokens per pass; ragged last rounds (5, 9, 3, 1 blocks), ragged token tiles
                                                    (1, 256, 8), (33, 1280, 12), (70, 2304, 16), (37, 512, 17), (64, 4096, 32),
                                                    (40, 768, 33), (5, 14336, 40), (96, 2048, 64)])
def test_kquant_f32_matvec(hb, oracle, dtype, n_rows, n_cols, seq_len):
    """Tolerance-level parity (the 8-lane reduce order is an assumption shared with the oracle)."""
    w = synth.weights(dtype, n_rows, n_cols, seed=dtype + n_rows)
    x = synth.activations(seq_len, n_cols, seed=n_cols + 1)
    W = hb.Weight.upload(dtype, n_rows, n_cols, w)
    try:
        got = hb.matmul(W, x)
        want = oracle.matmul_kquant_f32(dtype, w, x, n_rows, n_cols)
        np.testing.assert_allclose(got, want, rtol=RTOL, atol=ATOL)
        assert (got.view(np.uint32) == want.view(np.uint32)).all(), "same order, same bits expected"
    finally:
        W.free()


@pytest.mark.parametrize("dtype", [Q4_K, Q6_K])
@pytest.mark.parametrize("seq_len", [1, 3, 8, 16, 32])
def test_kquant_non_finite_block_scales(hb, oracle, dtype, seq_len):
    """Blocks whose f16 d (or dmin) is inf or NaN leave the fast nibble-to-float path: inf and NaN must come out in the
    rows the reference puts them in, and every other row keeps its bits."""
    n_rows, n_cols = 40, 1024
    w = synth.weights(dtype, n_rows, n_cols, seed=77).copy()
    bb, d_off = (144, 0) if dtype == Q4_K else (210, 208)
    inf16, nan16, ninf16 = 0x7C00, 0x7E00, 0xFC00
    for row, blk, bits, off in [(3, 0, inf16, d_off), (7, 2, nan16, d_off), (11, 3, ninf16, d_off), (12, 1, inf16, 2 if dtype == Q4_K else d_off)]:
        o = blk * bb + off
        w[row, o], w[row, o + 1] = bits & 0xFF, bits >> 8
    x = synth.activations(seq_len, n_cols, seed=5)
    W = hb.Weight.upload(dtype, n_rows, n_cols, w)
    try:
        got = hb.matmul(W, x)
        want = oracle.matmul_kquant_f32(dtype, w, x, n_rows, n_cols)
        assert (np.isnan(got) == np.isnan(want)).all()
        fin = ~np.isnan(want)
        assert (got[fin].view(np.uint32) == want[fin].view(np.uint32)).all()
        assert not np.isfinite(want[:, [3, 7, 11, 12]]).all(), "the case must exercise non-finite outputs"
    finally:
        W.free()


# ---------------------------------------------------------------------------------- device calls and batches

def test_device_calls_and_batch_match_host_calls(hb, oracle):
    import torch
    dev = torch.device("cuda:0")
    n_cols = 2048
    x = synth.activations(2, n_cols, seed=1)
    q8 = oracle.quantize_q8_0(x)
    shapes = [(Q2_0, 2048), (Q2_0, 1024), (Q2_0, 1000), (Q1_0, 6144), (Q8_0, 96)]
    ws = [synth.weights(dt, n, n_cols, seed=10 + i) for i, (dt, n) in enumerate(shapes)]
    Ws = [hb.Weight.upload(dt, n, n_cols, w) for (dt, n), w in zip(shapes, ws)]
    act = hb.Act(2, n_cols)
    try:
        xd = torch.from_numpy(x).to(dev)
        act.quantize(2, x_dev=xd)
        # planes -> reference bytes round trip
        raw = torch.zeros((2, q8.shape[1]), dtype=torch.uint8, device=dev)
        act.store_q8_0(raw, 2, q8.shape[1])
        torch.cuda.synchronize()
        assert (raw.cpu().numpy() == q8).all()
        act.load_q8_0(raw, 2, q8.shape[1])

        # fused q|k|v style: three weights write one [seq, 4072] buffer at column offsets
        total = sum(n for _, n in shapes[:3])
        fused = torch.zeros((2, total), dtype=torch.float32, device=dev)
        batch = hb.Batch()
        off = 0
        for W in Ws[:3]:
            batch.add(W, act, 2, fused[:, off:], ld_out=total)
            off += W.n_rows
        outs = [torch.zeros((2, W.n_rows), dtype=torch.float32, device=dev) for W in Ws[3:]]
        for W, o in zip(Ws[3:], outs):
            batch.add(W, act, 2, o)
        batch.seal()
        assert batch.launch_count == 3  # one launch per (format, tokens-per-op) group
        batch.launch()
        single = torch.zeros((2, Ws[0].n_rows), dtype=torch.float32, device=dev)
        hb.dot_rows_dev(Ws[0], act, 2, single)
        torch.cuda.synchronize()
        off = 0
        for (dt, n), w in zip(shapes[:3], ws[:3]):
            want = oracle.dot_rows_batched(dt, w, q8, n, n_cols)
            assert_bits_equal(fused[:, off:off + n].cpu().numpy(), want, f"fused slice {off}")
            off += n
        for (dt, n), w, o in zip(shapes[3:], ws[3:], outs):
            assert_bits_equal(o.cpu().numpy(), oracle.dot_rows_batched(dt, w, q8, n, n_cols), f"batch dtype {dt}")
        assert_bits_equal(single.cpu().numpy(), oracle.dot_rows_batched(Q2_0, ws[0], q8, 2048, n_cols), "dot_rows_dev")
        # running the sealed batch again gives the same bits (no state carried between launches)
        before = fused.clone()
        batch.launch()
        torch.cuda.synchronize()
        assert torch.equal(before, fused)
        batch.free()
    finally:
        act.free()
        for W in Ws:
            W.free()


def test_fused_matmul_is_one_upload_for_several_weights(hb, oracle):
    """hb200_matmul_f32_fused (matmul_fused_qkv / matmul_fused2, hearth-llm/src/model/matmul.rs:383-567): q|k|v and a
    K-quant weight against one input, each result equal to the single-weight call and to the oracle."""
    n_cols = 2048
    for seq in (1, 3, 70):
        x = synth.activations(seq, n_cols, seed=50 + seq)
        specs = [(Q1_0, 2048), (Q1_0, 1024), (Q2_0, 1022), (Q6_K, 40), (Q8_0, 5)]
        ws = [synth.weights(dt, n, n_cols, seed=60 + i) for i, (dt, n) in enumerate(specs)]
        Ws = [hb.Weight.upload(dt, n, n_cols, w) for (dt, n), w in zip(specs, ws)]
        try:
            outs = hb.matmul_fused(Ws, x)
            for (dt, n), w, W, got in zip(specs, ws, Ws, outs):
                if dt == Q6_K:
                    want = oracle.matmul_kquant_f32(dt, w, x, n, n_cols)
                else:
                    want = oracle.dot_rows_batched(dt, w, oracle.quantize_q8_0(x), n, n_cols)
                assert_bits_equal(got, want, f"fused, dtype {dt}, {seq} tokens")
                assert_bits_equal(got, hb.matmul(W, x), "fused equals the single call")
            with pytest.raises(hb.Hb200Error) as e:
                other = hb.Weight.upload(Q1_0, 8, 256, synth.weights(Q1_0, 8, 256, seed=1))
                try:
                    hb.matmul_fused([Ws[0], other], x)
                finally:
                    other.free()
            assert e.value.code == -4
        finally:
            for W in Ws:
                W.free()


# ---------------------------------------------------------------------------------- errors and empties

def test_error_behaviour(hb):
    E = hb.Hb200Error
    w = synth.weights(Q1_0, 4, 256, seed=1)
    with pytest.raises(E) as e:
        hb.Weight.upload(13, 4, 256, w)  # Q5_K: outside this path
    assert e.value.code == -3
    with pytest.raises(E) as e:
        hb.Weight.upload(Q1_0, 5, 256, w)  # byte count mismatch
    assert e.value.code == -4
    with pytest.raises(E) as e:
        hb.Weight.upload(Q1_0, 4, 0, np.zeros(0, dtype=np.uint8))  # n_cols == 0 (matmul.rs:66)
    assert e.value.code == -4
    W = hb.Weight.upload(Q1_0, 4, 256, w)
    try:
        with pytest.raises(E) as e:
            hb.matmul(W, np.zeros(128, dtype=np.float32))  # x.len != n_cols
        assert e.value.code == -4
        with pytest.raises(E) as e:
            hb.par_dot_rows_batched(W, np.zeros((1, 10), dtype=np.uint8), 1, 10)  # stride shorter than a row
        assert e.value.code == -4
        act = hb.Act(1, 128)
        import torch
        out = torch.zeros(4, device="cuda:0")
        with pytest.raises(E) as e:
            hb.dot_rows_dev(W, act, 1, out)  # activation width != weight width
        assert e.value.code == -4
        act.free()
    finally:
        W.free()
    Wk = hb.Weight.upload(Q4_K, 2, 256, synth.weights(Q4_K, 2, 256, seed=2))
    with pytest.raises(E) as e:
        hb.par_dot_rows(Wk, np.zeros(8 * 34, dtype=np.uint8))  # no Q8_0 dot for K-quants in the reference
    assert e.value.code == -7
    Wk.free()


def test_empty_inputs_are_no_ops(hb):
    # par_dot_rows returns at once for n == 0 (pool.rs:520), par_dot_rows_batched for seq_len == 0 (:581)
    W0 = hb.Weight.upload(Q2_0, 0, 256, np.zeros(0, dtype=np.uint8))
    assert hb.par_dot_rows(W0, np.zeros(8 * 34, dtype=np.uint8)).shape == (0,)
    W0.free()
    W = hb.Weight.upload(Q2_0, 3, 256, synth.weights(Q2_0, 3, 256, seed=1))
    assert hb.par_dot_rows_batched(W, np.zeros((0, 8 * 34), dtype=np.uint8), 0, 8 * 34).shape == (0, 3)
    W.free()


# ---------------------------------------------------------------------------------- full-size cases

@pytest.mark.parametrize("name", ["c0_q1_single", "c1_q2_1p7b_decode", "c4_pq2_27b_decode"])
def test_full_size_layer_against_oracle(hb, oracle, name):
    """One whole layer of the named configuration (all seven projections at their real shapes), M = 1."""
    cfg = synth.CONFIGS[name]
    for i, (pname, n_rows, n_cols) in enumerate(cfg["shapes"]):
        w = synth.weights(cfg["dtype"], n_rows, n_cols, seed=1000 + i)
        a = oracle.quantize_q8_0(synth.activations(1, n_cols, seed=2000 + i))[0]
        W = hb.Weight.upload(cfg["dtype"], n_rows, n_cols, w)
        try:
            got = hb.par_dot_rows(W, a)
        finally:
            W.free()
        want = oracle.dot_rows_batched(cfg["dtype"], w, a, n_rows, n_cols)[0]
        assert_bits_equal(got, want, f"{name}:{pname}")


def test_full_size_linearity_of_integer_dots(hb, oracle):
    """Size-independent property at the 27B gate shape: the integer dots are linear in the activation
    bytes, so dots(a + b) == dots(a) + dots(b) exactly when a + b stays inside int8."""
    n_rows, n_cols = 17408, 5120
    w = synth.weights(PQ2_0, n_rows, n_cols, seed=3)
    rng = np.random.Generator(np.random.PCG64(9))
    def raw(vals):
        r = np.zeros((n_cols // 32, 34), dtype=np.uint8)
        r[:, 0:2] = np.frombuffer(np.float16(1.0).tobytes(), dtype=np.uint8)
        r[:, 2:] = vals.astype(np.int8).view(np.uint8).reshape(-1, 32)
        return r.reshape(-1)
    a = rng.integers(-60, 61, n_cols)
    b = rng.integers(-60, 61, n_cols)
    W = hb.Weight.upload(PQ2_0, n_rows, n_cols, w)
    try:
        da, db, dab = (hb.block_dots_i32(W, raw(v))[0] for v in (a, b, a + b))
        assert (da + db == dab).all()
        rows = rng.integers(0, n_rows, 16)
        for r in rows:
            assert (da[r] == oracle.block_dots_i32(PQ2_0, w[r], raw(a), n_cols)).all()
    finally:
        W.free()


def test_batch_run_from_host_buffers(hb, oracle):
    """hb200_batch_run_host: all inputs in one host buffer, one readback; K-quant and Q8_0-activation ops together."""
    import torch
    dev = torch.device("cuda:0")
    seq = 2
    specs = [(Q2_0, 300, 2048, 0), (Q1_0, 64, 2048, 0), (Q2_0, 100, 1152, 1), (Q6_K, 24, 512, 2), (Q1_0, 40, 256, 3)]
    widths = {0: 2048, 1: 1152, 2: 512, 3: 256}
    xs = {g: synth.activations(seq, k, seed=300 + g) for g, k in widths.items()}
    acts = {g: hb.Act(seq, k) for g, k in widths.items()}
    ws = [synth.weights(dt, n, k, seed=400 + i) for i, (dt, n, k, _) in enumerate(specs)]
    Ws = [hb.Weight.upload(dt, n, k, w) for (dt, n, k, _), w in zip(specs, ws)]
    total = sum(n for _, n, _, _ in specs)
    out_dev = torch.zeros((seq, total), dtype=torch.float32, device=dev)
    batch = hb.Batch()
    off = 0
    for (dt, n, k, g), W in zip(specs, Ws):
        batch.add(W, acts[g], seq, out_dev[:, off:], ld_out=total)
        off += n
    batch.seal()
    assert batch.input_floats == sum(seq * k for k in widths.values())
    x_host = np.concatenate([xs[g].reshape(-1) for g in sorted(widths)])  # order of first use: groups 0, 1, 2, 3
    out_host = np.zeros((seq, total), dtype=np.float32)
    try:
        for _ in range(2):
            batch.run_host(x_host, out_dev, out_host)
            off = 0
            for (dt, n, k, g), w in zip(specs, ws):
                if dt == Q6_K:
                    want = oracle.matmul_kquant_f32(dt, w, xs[g], n, k)
                else:
                    want = oracle.dot_rows_batched(dt, w, oracle.quantize_q8_0(xs[g]), n, k)
                assert_bits_equal(out_host[:, off:off + n], want, f"run_host op dtype {dt}")
                off += n
    finally:
        batch.free()
        for a in acts.values():
            a.free()
        for W in Ws:
            W.free()


def test_batch_run_host_pipelined(hb, oracle):
    """Forty single-token ops: hb200_batch_run_host splits them into runs and overlaps upload, compute and readback.
    Same results as the oracle, and the same on every repetition (buffers are reused)."""
    import torch
    dev = torch.device("cuda:0")
    kinds = [Q2_0, Q1_0, Q8_0, Q6_K, Q4_K]
    specs = []
    for i in range(40):
        dt = kinds[i % len(kinds)]
        k = 512 if dt in (Q4_K, Q6_K) else (1152 if i % 3 else 2048)
        specs.append((dt, 40 + 8 * (i % 7), k, i // 2))            # two ops share each activation
    n_acts = 20
    widths = {}
    for dt, n, k, g in specs:
        widths.setdefault(g, k)
    # ops of one activation must agree on its width: give every op the width of its group
    specs = [(dt, n, widths[g], g) for dt, n, k, g in specs]
    specs = [(dt, n, k, g) for dt, n, k, g in specs if not (dt in (Q4_K, Q6_K) and k % 256)]
    xs = {g: synth.activations(1, k, seed=700 + g) for g, k in widths.items()}
    acts = {g: hb.Act(1, k) for g, k in widths.items()}
    ws = [synth.weights(dt, n, k, seed=800 + i, allow_code3=True) for i, (dt, n, k, _) in enumerate(specs)]
    Ws = [hb.Weight.upload(dt, n, k, w) for (dt, n, k, _), w in zip(specs, ws)]
    total = sum(n for _, n, _, _ in specs)
    out_dev = torch.zeros((1, total), dtype=torch.float32, device=dev)
    batch = hb.Batch()
    off = 0
    for (dt, n, k, g), W in zip(specs, Ws):
        batch.add(W, acts[g], 1, out_dev[:, off:], ld_out=total)
        off += n
    batch.seal()
    order = []
    for _, _, _, g in specs:
        if g not in order:
            order.append(g)
    pieces = []
    for g in order:                                              # first-use order, each start 16-byte aligned
        pieces.append(xs[g].reshape(-1))
        pad = (-xs[g].size) % 4
        if pad:
            pieces.append(np.zeros(pad, dtype=np.float32))
    x_host = np.concatenate(pieces)
    assert batch.input_floats == x_host.size
    out_host = np.zeros((1, total), dtype=np.float32)
    try:
        for rep in range(3):
            out_host[:] = np.nan
            batch.run_host(x_host, out_dev, out_host)
            off = 0
            for (dt, n, k, g), w in zip(specs, ws):
                if dt in (Q4_K, Q6_K):
                    want = oracle.matmul_kquant_f32(dt, w, xs[g], n, k)
                else:
                    want = oracle.dot_rows_batched(dt, w, oracle.quantize_q8_0(xs[g]), n, k)
                assert_bits_equal(out_host[:, off:off + n], want, f"pipelined run_host op dtype {dt} rep {rep}")
                off += n
    finally:
        batch.free()
        for a in acts.values():
            a.free()
        for W in Ws:
            W.free()
