"""The GGUF reader behind the C ABI against files written by tests/gguf_writer.py: header, metadata, tensor infos
and data offsets as hearth_gguf::GgufFile reports them (hearth-gguf/src/gguf.rs:137-259); parsing needs no GPU."""
import os
import struct

import numpy as np
import pytest

import gguf_writer as gw
from hearth_b200 import synth

Q1_0, PQ2_0, PTQ1_0, Q8_0 = 41, 142, 143, 8


@pytest.fixture(scope="module")
def api():
    from hearth_b200 import api as hb
    return hb


def _model(tmp_path, version=3, alignment=None):
    w1 = synth.weights(Q1_0, 96, 256, seed=1)
    w2 = synth.weights(PQ2_0, 40, 1152, seed=2)
    w3 = synth.weights(PTQ1_0, 8, 128, seed=3)
    norm = np.arange(256, dtype=np.float32)
    signs = [1.0, -1.0, -1.0, 1.0]
    meta = [("general.architecture", gw.T_STR, "qwen35"), ("general.name", gw.T_STR, "synthetic é"),
            ("qwen35.block_count", gw.T_U32, 2), ("prism.hadamard.block_size", gw.T_U32, 1024),
            ("qwen35.rope.freq_base", gw.T_F32, 10000.0), ("some.i8", gw.T_I8, -5), ("some.u64", gw.T_U64, 1 << 40),
            ("some.i64", gw.T_I64, -7), ("some.f64", gw.T_F64, 0.25), ("some.flag", gw.T_BOOL, 1), ("some.u16", gw.T_U16, 65535),
            ("prism.hadamard.signs.4", gw.T_ARR, (gw.T_F32, signs)), ("tokenizer.tokens", gw.T_ARR, (gw.T_STR, ["a", "bc", ""])),
            ("some.i32s", gw.T_ARR, (gw.T_I32, [-1, 2, -3]))]
    tensors = [("blk.0.attn_q.weight", [256, 96], Q1_0, w1.reshape(-1)), ("blk.0.ffn_down.weight", [1152, 40], PQ2_0, w2.reshape(-1)),
               ("blk.1.ssm_out.weight", [128, 8], PTQ1_0, w3.reshape(-1)), ("output_norm.weight", [256], 0, norm.view(np.uint8))]
    path = str(tmp_path / f"m{version}.gguf")
    layout = gw.write_gguf(path, meta, tensors, version=version, alignment=alignment)
    return path, layout, dict(w1=w1, w2=w2, w3=w3, norm=norm, signs=signs)


@pytest.mark.parametrize("version,alignment", [(3, None), (3, 64), (2, None)])
def test_header_metadata_and_tensor_infos(api, tmp_path, version, alignment):
    path, layout, ref = _model(tmp_path, version, alignment)
    g = api.Gguf(path)
    try:
        assert g.version == version and g.data_offset == layout["data_offset"]
        assert [t["name"] for t in g.tensors] == ["blk.0.attn_q.weight", "blk.0.ffn_down.weight", "blk.1.ssm_out.weight",
                                                  "output_norm.weight"]
        t = g.tensors[g.find_tensor("blk.0.ffn_down.weight")]
        assert t["dtype"] == PQ2_0 and t["shape"] == [1152, 40] and t["bytes"] == 40 * 9 * 34
        assert t["offset"] == layout["offsets"]["blk.0.ffn_down.weight"]
        assert g.tensors[2]["bytes"] == 8 * 28 and g.tensors[3]["bytes"] == 1024
        assert np.array_equal(g.tensor_data(0), ref["w1"].reshape(-1))
        assert np.array_equal(g.tensor_data(2), ref["w3"].reshape(-1))
        assert np.array_equal(g.tensor_data(3).view(np.float32), ref["norm"])
        assert g.meta_str("general.architecture") == "qwen35" and g.meta_str("general.name") == "synthetic é"
        assert g.meta_u64("qwen35.block_count") == 2 and g.meta_u64("prism.hadamard.block_size") == 1024
        assert g.meta_u64("some.u64") == 1 << 40 and g.meta_u64("some.flag") == 1 and g.meta_u64("some.u16") == 65535
        assert g.meta_u64("some.i8") == (1 << 64) - 5 and g.meta_u64("some.i64") == (1 << 64) - 7  # sign-extended
        assert g.meta_f64("qwen35.rope.freq_base") == 10000.0 and g.meta_f64("some.f64") == 0.25
        assert g.meta_array_f32("prism.hadamard.signs.4").tolist() == ref["signs"]
        assert g.meta_array_f32("some.i32s").tolist() == [-1.0, 2.0, -3.0]
        with pytest.raises(api.Hb200Error) as e:
            g.meta_u64("missing.key")
        assert e.value.code == -12
        with pytest.raises(api.Hb200Error) as e:
            g.meta_u64("general.name")
        assert e.value.code == -3
        with pytest.raises(api.Hb200Error):
            g.meta_array_f32("tokenizer.tokens")  # strings are not numeric
        with pytest.raises(api.Hb200Error) as e:
            g.find_tensor("nope")
        assert e.value.code == -12
    finally:
        g.close()


def test_malformed_files_are_rejected(api, tmp_path):
    p = tmp_path / "bad.gguf"
    for blob, code in [(b"GG", -11), (b"GGML" + b"\0" * 40, -11), (b"GGUF" + struct.pack("<IQQ", 1, 0, 0), -11),
                       (b"GGUF" + struct.pack("<IQQ", 3, 5, 0), -11)]:  # too small, magic, version 1, truncated infos
        p.write_bytes(blob)
        with pytest.raises(api.Hb200Error) as e:
            api.Gguf(str(p))
        assert e.value.code == code, blob[:8]
    with pytest.raises(api.Hb200Error) as e:
        api.Gguf(str(tmp_path / "does-not-exist.gguf"))
    assert e.value.code == -10
    # an array whose element count exceeds the bytes that remain, flat and nested, and a huge string length: rejected
    # before anything of that size is allocated, and (repeated many times) without leaking the mapping or descriptor
    head = b"GGUF" + struct.pack("<IQQ", 3, 0, 1) + struct.pack("<Q", 1) + b"k" + struct.pack("<I", 9)
    huge_flat = head + struct.pack("<IQ", 0, 1 << 40) + b"\0" * 64
    huge_nested = head + struct.pack("<IQ", 9, 2) + struct.pack("<IQ", 0, 1 << 33) + b"\0" * 32
    huge_str = b"GGUF" + struct.pack("<IQQ", 3, 0, 1) + struct.pack("<Q", 1 << 50) + b"k"
    n_fds = len(os.listdir("/proc/self/fd"))
    for _ in range(20):
        for blob in (huge_flat, huge_nested, huge_str):
            p.write_bytes(blob)
            with pytest.raises(api.Hb200Error) as e:
                api.Gguf(str(p))
            assert e.value.code == -11
    assert len(os.listdir("/proc/self/fd")) <= n_fds + 1
    # a tensor type id GgmlDType::from_id does not know (hearth-gguf/src/ggml.rs:58-103)
    gw.write_gguf(str(p), [], [("t", [32], 40, np.zeros(4, np.uint8))])
    with pytest.raises(api.Hb200Error) as e:
        api.Gguf(str(p))
    assert e.value.code == -3
    # truncated data section: infos parse, the data call fails
    path, layout, _ = _model(tmp_path)
    blob = open(path, "rb").read()
    p.write_bytes(blob[:layout["data_offset"] + 100])
    g = api.Gguf(str(p))
    with pytest.raises(api.Hb200Error) as e:
        g.tensor_data(1)
    assert e.value.code == -11
    g.close()


@pytest.mark.gpu
def test_upload_from_gguf_and_dot(hb, oracle, tmp_path):
    path, _, ref = _model(tmp_path)
    g = hb.Gguf(path)
    try:
        for name, w, dt, n_rows, n_cols in [("blk.0.attn_q.weight", ref["w1"], Q1_0, 96, 256),
                                            ("blk.0.ffn_down.weight", ref["w2"], PQ2_0, 40, 1152),
                                            ("blk.1.ssm_out.weight", ref["w3"], PTQ1_0, 8, 128)]:
            W = g.upload(name)
            assert (W.dtype, W.n_rows, W.n_cols) == (dt, n_rows, n_cols)
            a = oracle.quantize_q8_0(synth.activations(1, n_cols, seed=n_cols))[0]
            got = hb.par_dot_rows(W, a)
            want = oracle.dot_rows_batched(dt, w, a, n_rows, n_cols)[0]
            assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), name
            W.free()
        with pytest.raises(hb.Hb200Error):
            g.upload("output_norm.weight")  # F32: not a format of this path
    finally:
        g.close()
