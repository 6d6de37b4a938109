"""CPU tests of the C-ABI library: it loads, exports every symbol the header declares,
answers geometry queries, and refuses to compute without a device (no fallback)."""
import ctypes as C
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "hb200.h")).read()
    return sorted(set(re.findall(r"HB200_API\s+[\w\s\*]+?\b(hb200_\w+)\s*\(", text)))


@pytest.fixture(scope="module")
def lib():
    from hearth_b200 import build, lib as L
    build.build()
    return L.load()


def test_header_and_bindings_agree(lib):
    from hearth_b200 import lib as L
    syms = declared_symbols()
    assert len(syms) >= 30
    assert sorted(L.SIGNATURES) == syms
    for s in syms:
        assert hasattr(lib, s), f"{s} not exported"


def test_geometry_matches_reference_table(lib):
    # hearth-gguf/src/ggml.rs:105-176
    geo = {8: (32, 34), 12: (256, 144), 14: (256, 210), 39: (128, 18), 41: (128, 18), 43: (128, 18), 42: (128, 34),
           142: (128, 34), 143: (128, 28)}
    for dt, (bs, bb) in geo.items():
        assert lib.hb200_block_size(dt) == bs
        assert lib.hb200_block_bytes(dt) == bb
        assert lib.hb200_byte_size(dt, 6144) == 6144 // bs * bb
        assert lib.hb200_byte_size(dt, bs + 1) == 2 * bb
    for dt in (0, 1, 2, 13, 144, 9999):
        assert lib.hb200_block_size(dt) == 0 and lib.hb200_byte_size(dt, 128) == 0


def test_selected_kernel_names(lib):
    assert lib.hb200_selected_kernel(41, 1).decode().startswith("gemv_dp4a_q1_0")
    assert lib.hb200_selected_kernel(142, 1).decode().startswith("gemv_dp4a_q2_0")
    assert lib.hb200_selected_kernel(12, 1).decode() == "kquant_gemv_q4_k_f32"
    assert lib.hb200_selected_kernel(143, 1).decode().startswith("gemv_dp4a_q2_0")  # trits re-coded at upload
    assert lib.hb200_selected_kernel(13, 1).decode() == "none"


def test_no_device_means_error_not_fallback(lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present; this test is about the device-less case")
    rc = lib.hb200_init(0)
    assert rc == -2, "hb200_init must fail with HB200_ERR_NO_DEVICE without a GPU"
    assert b"CUDA" in lib.hb200_last_error() or b"device" in lib.hb200_last_error()
    x = np.zeros(64, dtype=np.float32)
    out = np.zeros(68, dtype=np.uint8)
    rc = lib.hb200_quantize_q8_0(C.c_void_p(x.ctypes.data), 1, 64, C.c_void_p(out.ctypes.data))
    assert rc == -1, "compute calls must report HB200_ERR_NOT_INITIALIZED"
    h = C.c_void_p()
    w = np.zeros(18, dtype=np.uint8)
    assert lib.hb200_weight_upload(41, 1, 128, C.c_void_p(w.ctypes.data), 18, C.byref(h)) == -1
    assert lib.hb200_act_create(1, 128, C.byref(h)) == -1


def test_python_api_raises_without_device():
    import torch
    if torch.cuda.is_available():
        pytest.skip("device present")
    from hearth_b200 import api
    with pytest.raises(api.Hb200Error):
        api.init(0)
    with pytest.raises(api.Hb200Error):
        api.quantize_q8_0(np.zeros(32, dtype=np.float32))


def test_synthetic_layouts_decode(oracle):
    from hearth_b200 import synth
    w = synth.weights(42, 5, 256, seed=1)
    assert w.shape == (5, 68)
    vals = oracle.dequantize(42, w[0], 256)
    scale0 = np.frombuffer(bytes(w[0, 0:2]), dtype=np.float16)[0].astype(np.float32)
    assert set(np.unique(np.round(vals[:128] / scale0)).tolist()) <= {-1.0, 0.0, 1.0}
    w1 = synth.weights(41, 3, 384, seed=2)
    assert w1.shape == (3, 54)
    assert synth.row_bytes(12, 4096) == 16 * 144 and synth.row_bytes(14, 4096) == 16 * 210
    assert synth.config_weight_bytes("c0_q1_single") == 1769472
    assert synth.config_weight_bytes("c1_q2_1p7b_decode") == 374341632
    assert synth.config_weight_bytes("c2_q1_8b_prefill") == 976748544
    assert synth.config_weight_bytes("c4_pq2_27b_decode") == 5615124480
