"""The f32-activation matmul (the arithmetic of the reference's GPU shaders): oracle known answers from the
reference's own tests (hearth-compute/src/lib.rs:1819-2080) and GPU parity, bit for bit, against the oracle."""
import numpy as np
import pytest

from hearth_b200 import synth

Q1_0, Q1_0_G128, Q2_0, PQ2_0, Q8_0, PTQ1_0 = 41, 43, 42, 142, 8, 143


def q1_row(vals: np.ndarray) -> np.ndarray:
    """quantize_q1_0_row of the reference's tests (lib.rs:1707-1739): scale = max |x| (1 if zero), bit = x >= 0."""
    out = bytearray()
    for b in range(vals.size // 128):
        blk = vals[b * 128:(b + 1) * 128]
        m = float(np.abs(blk).max())
        out += np.float16(1.0 if m == 0 else m).tobytes()
        bits = (blk >= 0).astype(np.uint8).reshape(16, 8)
        out += bytes(int((row << np.arange(8)).sum()) for row in bits)
    return np.frombuffer(bytes(out), dtype=np.uint8)


def _known_answer_cases():
    ones256, ones128 = np.ones(256, np.float32), np.ones(128, np.float32)
    alt = np.where(np.arange(128) % 2 == 0, 1.0, -1.0).astype(np.float32)
    return [
        (np.stack([q1_row(ones256)] * 4), ones256, None, [256.0] * 4),                                  # test_q1_0_matmul_correctness
        (np.stack([q1_row(ones128), q1_row(-ones128)]), np.arange(128, dtype=np.float32), None, [8128.0, -8128.0]),  # _mixed_weights
        (np.stack([q1_row(ones128)] * 2), ones128, np.full((1, 2), 3.0, np.float32), [131.0, 131.0]),   # _add_inplace
        (np.stack([q1_row(ones128)] * 4), ones128, None, [128.0] * 4),                                  # fused_gate_up: gate
        (np.stack([q1_row(alt)] * 4), ones128, None, [0.0] * 4),                                        # fused_gate_up: up
    ]


def test_oracle_known_answers(oracle):
    for w, x, accum, want in _known_answer_cases():
        got = oracle.matmul_f32act(Q1_0_G128, w, x, w.shape[0], x.size, accum=accum)
        assert np.abs(got[0] - np.array(want)).max() < 0.1


def test_oracle_matches_dequantized_dot_and_shader_scale_quirk(oracle):
    rng = np.random.default_rng(1)
    for dt in (Q1_0, Q2_0):
        n_rows, n_cols = 5, 512
        w = synth.weights(dt, n_rows, n_cols, seed=dt, allow_code3=True)
        x = rng.normal(size=n_cols).astype(np.float32)
        got = oracle.matmul_f32act(dt, w, x, n_rows, n_cols)[0]
        for r in range(n_rows):
            ref = float((oracle.dequantize(dt, w[r], n_cols).astype(np.float64) * x).sum())
            assert abs(got[r] - ref) < 1e-3 * max(1.0, abs(ref))      # the bound the reference's cross-check uses
    # a zero f16 scale is widened to 2^-15 by the shader's bit formula, not to 0
    w = q1_row(np.ones(128, np.float32)).copy()
    w[0:2] = 0
    assert oracle.matmul_f32act(Q1_0, w.reshape(1, -1), np.ones(128, np.float32), 1, 128)[0, 0] == np.float32(128.0 * 2.0 ** -15)


@pytest.mark.gpu
def test_gpu_known_answers(hb):
    for w, x, accum, want in _known_answer_cases():
        W = hb.Weight.upload(Q1_0_G128, w.shape[0], x.size, w)
        got = hb.dequant_matmul_f32act(W, x, accum=accum)
        assert np.abs(got[0] - np.array(want)).max() < 0.1
        W.free()


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [Q1_0, Q1_0_G128, Q2_0, PQ2_0])
@pytest.mark.parametrize("n_rows,n_cols,batch", [(300, 2048, 1), (7, 128, 3), (257, 1152, 2), (1024, 4096, 1), (33, 5120, 4)])
def test_gpu_bits_match_oracle(hb, oracle, dtype, n_rows, n_cols, batch):
    w = synth.weights(dtype, n_rows, n_cols, seed=dtype + n_rows, allow_code3=True)
    x = synth.activations(batch, n_cols, seed=n_cols + batch)
    W = hb.Weight.upload(dtype, n_rows, n_cols, w)
    try:
        got = hb.dequant_matmul_f32act(W, x)
        want = oracle.matmul_f32act(dtype, w, x, n_rows, n_cols)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), f"{int((got != want).sum())} of {got.size} differ"
        acc = synth.activations(batch, n_rows, seed=5)
        got = hb.dequant_matmul_f32act(W, x, accum=acc)
        want = oracle.matmul_f32act(dtype, w, x, n_rows, n_cols, accum=acc)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), "add-in-place form"
    finally:
        W.free()


@pytest.mark.gpu
def test_gpu_fused_gate_up_shares_an_output_buffer_and_specials(hb, oracle):
    import torch
    n_cols, m = 1024, 200
    wg, wu = synth.weights(Q1_0, m, n_cols, seed=1), synth.weights(Q1_0, m, n_cols, seed=2)
    wg[3, 0:2] = 0                                    # zero scale: the shader's formula gives 2^-15
    wu[5, 18:20] = np.frombuffer(np.float16(np.inf).tobytes(), dtype=np.uint8)  # exp = 31: a finite number there
    x = synth.activations(2, n_cols, seed=3)
    x[0, 7] = 0.0
    x[1, 9] = -0.0
    G, U = hb.Weight.upload(Q1_0, m, n_cols, wg), hb.Weight.upload(Q1_0, m, n_cols, wu)
    out = torch.zeros(2, 2 * m, device="cuda")
    xd = torch.from_numpy(x).cuda()
    hb.dequant_matmul_f32act_dev(G, xd, 2, out, ld_out=2 * m)
    hb.dequant_matmul_f32act_dev(U, xd, 2, out[:, m:], ld_out=2 * m)
    torch.cuda.synchronize()
    got = out.cpu().numpy()
    assert np.array_equal(got[:, :m].view(np.uint32), oracle.matmul_f32act(Q1_0, wg, x, m, n_cols).view(np.uint32))
    assert np.array_equal(got[:, m:].view(np.uint32), oracle.matmul_f32act(Q1_0, wu, x, m, n_cols).view(np.uint32))
    for bad in (Q8_0, PTQ1_0):                        # no shader for these: the reference returns None
        W = hb.Weight.upload(bad, 4, 128, synth.weights(bad, 4, 128, seed=4))
        with pytest.raises(hb.Hb200Error) as e:
            hb.dequant_matmul_f32act(W, x[0, :128])
        assert e.value.code == -7
        W.free()
    G.free(); U.free()
