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


def test_dispatch_report_and_banner(lib):
    """hb200_dispatch_report / _banner: the analogue of hearth_quant::dispatch_report (hearth-quant/src/lib.rs:449-473).
    Keys are lowercase format names, repeats collapse, formats outside the path are skipped; needs no device."""
    import json
    from hearth_b200 import api
    rep = api.dispatch_report([41, 142, 142, 13, 12, 8, 0])
    assert list(rep["kernels"]) == ["q1_0", "pq2_0", "q4_k", "q8_0"]
    q1 = rep["kernels"]["q1_0"]
    assert [r["tokens"] for r in q1] == ["1-10", "11-64", "65+"]
    for r in q1:
        lo = int(r["tokens"].rstrip("+").split("-")[0])
        assert r["kernel"] == lib.hb200_selected_kernel(41, lo).decode()
    assert rep["kernels"]["q4_k"] == [{"tokens": "1+", "kernel": "kquant_gemv_q4_k_f32"}]
    banner = api.dispatch_banner([143, 41])
    assert banner.startswith("[kernel] PTQ1_0=gemv_dp4a_q2_0(1-11),") and " Q1_0=gemv_dp4a_q1_0(1-10)," in banner
    # a buffer that is too small: the needed length comes back with HB200_ERR_TOO_LARGE
    need = C.c_size_t()
    arr = (C.c_int * 1)(41)
    buf = C.create_string_buffer(8)
    assert lib.hb200_dispatch_report(arr, 1, buf, 8, C.byref(need)) == -8
    assert need.value > 8
    buf = C.create_string_buffer(need.value + 1)
    assert lib.hb200_dispatch_report(arr, 1, buf, need.value + 1, C.byref(need)) == 0
    json.loads(buf.value.decode())


def test_token_count_limit_is_a_clear_error(lib):
    """More than HB200_MAX_SEQ_LEN tokens: HB200_ERR_TOO_LARGE with a message, checked before any device work."""
    h = C.c_void_p()
    assert lib.hb200_act_create(65536, 128, C.byref(h)) == -8
    assert b"65535" in lib.hb200_last_error()
    assert lib.hb200_act_create(0, 128, C.byref(h)) == -4


def test_device_slots_without_a_device(lib):
    """hb200_init_multi / hb200_init_slots / hb200_set_slot: clear errors when no GPU is present, nothing bound."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present; this test is about the device-less case")
    assert lib.hb200_slot_count() == 0
    assert lib.hb200_init_multi(2) == -2
    assert lib.hb200_init_multi(0) == -4 and lib.hb200_init_multi(9) == -4
    arr = (C.c_int * 2)(0, 0)
    assert lib.hb200_init_slots(arr, 2) == -2
    assert lib.hb200_init_slots(None, 2) == -5
    assert lib.hb200_set_slot(1) == -1 and b"slot 1" in lib.hb200_last_error()
    assert lib.hb200_slot_count() == 0
    assert lib.hb200_multi_batch_launch(None, 0, None) == -5
