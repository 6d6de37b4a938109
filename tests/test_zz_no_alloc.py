"""hb200_matmul_f32_noalloc, the entry point for callers that must not allocate device memory
(hosts whose device memory is already fully owned by something else, or that cannot afford the
device-wide synchronisation an allocation brings in the middle of a decode loop).

Collected last on purpose: a run that stops at the first failure has then already run every other test.
The entry point is called through the C ABI and its output is compared with hb200_matmul_f32_dev, the
allocating entry point, and with the CPU oracle, under the same bar the other GPU tests use (same bits;
1e-5 rel / 1e-6 abs).
Two calls in a row with different widths check that nothing left in the shared scratch array by the
first call leaks into the second.
"""
import ctypes as C

import numpy as np
import pytest

from hearth_b200 import synth

pytestmark = pytest.mark.gpu

RTOL, ATOL = 1e-5, 1e-6


def _oracle(oracle, dtype, w, x, n_rows, n_cols):
    if dtype in (12, 14):
        return oracle.matmul_kquant_f32(dtype, w, x, n_rows, n_cols)
    return oracle.dot_rows_batched(dtype, w, oracle.quantize_q8_0(x), n_rows, n_cols)


def _run_pair(hb, oracle, torch, dtype, n_rows, n_cols, seq_len, seed, through_binding=False):
    from hearth_b200 import lib as L
    lib = L.load()
    dev = torch.device("cuda:0")
    w = synth.weights(dtype, n_rows, n_cols, seed=seed)
    x_host = synth.activations(seq_len, n_cols, seed=seed + 1)
    x = torch.from_numpy(x_host).to(dev)
    W = hb.Weight.upload(dtype, n_rows, n_cols, w)
    act = hb.Act(seq_len, n_cols)
    try:
        want = torch.zeros((seq_len, n_rows), dtype=torch.float32, device=dev)
        act.set_f32(x)
        hb.matmul_f32_dev(W, act, seq_len, want)
        got = torch.full((seq_len, n_rows), float("nan"), dtype=torch.float32, device=dev)
        if through_binding:
            hb.matmul_f32_noalloc(W, x, got)
        else:
            stream = C.c_void_p(int(torch.cuda.current_stream().cuda_stream))
            rc = lib.hb200_matmul_f32_noalloc(W._h, C.c_void_p(x.data_ptr()), seq_len, C.c_void_p(got.data_ptr()), n_rows, stream)
            assert rc == 0, lib.hb200_last_error()
        torch.cuda.synchronize()
        g, t = got.cpu().numpy(), want.cpu().numpy()
        np.testing.assert_allclose(g, t, rtol=RTOL, atol=ATOL)
        assert (g.view(np.uint32) == t.view(np.uint32)).all()
        assert np.abs(t).max() > 1e-6
        o = _oracle(oracle, dtype, w, x_host, n_rows, n_cols)
        np.testing.assert_allclose(g, o, rtol=RTOL, atol=ATOL)
        assert (g.view(np.uint32) == o.view(np.uint32)).all(), "the oracle's bits"
    finally:
        act.free()
        W.free()


def test_noalloc_matches_allocating_entry_point_twice_in_a_row(hb, oracle):
    import torch
    # first call: wide rows, four tokens, 1-bit weights; second call right after: narrower rows (the
    # scratch still holds the first call's planes beyond this call's width), one token, 2-bit weights
    _run_pair(hb, oracle, torch, 41, 300, 6144, 4, seed=11)
    _run_pair(hb, oracle, torch, 142, 257, 1152, 1, seed=21)
    _run_pair(hb, oracle, torch, 8, 64, 2048, 2, seed=31)
    _run_pair(hb, oracle, torch, 14, 16, 512, 1, seed=41)  # K-quant: f32 activations, no scratch involved
    _run_pair(hb, oracle, torch, 42, 96, 2048, 3, seed=51, through_binding=True)  # the Python binding of the same call


def test_noalloc_rejects_sizes_beyond_its_fixed_scratch(hb):
    import torch
    from hearth_b200 import lib as L
    lib = L.load()
    dev = torch.device("cuda:0")
    W = hb.Weight.upload(41, 8, 128, synth.weights(41, 8, 128, seed=1))
    x = torch.zeros((5, 128), dtype=torch.float32, device=dev)
    out = torch.zeros((5, 8), dtype=torch.float32, device=dev)
    rc = lib.hb200_matmul_f32_noalloc(W._h, C.c_void_p(x.data_ptr()), 5, C.c_void_p(out.data_ptr()), 8, None)
    assert rc == -8 and b"at most 4 tokens" in lib.hb200_last_error()
    W.free()
    wide = 32768 + 128
    Ww = hb.Weight.upload(41, 8, wide, synth.weights(41, 8, wide, seed=2))
    x = torch.zeros((1, wide), dtype=torch.float32, device=dev)
    rc = lib.hb200_matmul_f32_noalloc(Ww._h, C.c_void_p(x.data_ptr()), 1, C.c_void_p(out.data_ptr()), 8, None)
    assert rc == -8
    Ww.free()
