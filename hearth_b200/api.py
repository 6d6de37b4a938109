"""Python face of the C ABI, named after the reference interfaces it stands in for.

Host-buffer calls take and return numpy arrays and follow the reference's call
shapes (hearth-llm/src/pool.rs, hearth-llm/src/model/matmul.rs,
hearth-quant/src/lib.rs).  Device-buffer calls take torch CUDA tensors; torch is
used for device memory and streams only.  Everything computes in the CUDA
library; a missing library or device raises.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import lib as _l
from .lib import PQ2_0, PTQ1_0, Q1_0, Q1_0_G128, Q2_0, Q4_K, Q6_K, Q8_0, Hb200Error, check  # noqa: F401

_initialized_device = None


def init(device: int = 0) -> None:
    """GpuCompute::new (hearth-compute/src/lib.rs:127): bind this process to one B200."""
    global _initialized_device
    check(_l.load().hb200_init(device))
    _initialized_device = device


def init_multi(n_devices: int | None = None, devices: list[int] | None = None) -> int:
    """One process, several GPUs: binds device slots 0 .. n-1 (to `devices`, default 0 .. n-1) and enables peer access
    between them.  Returns the number of slots.  Objects are created in the current slot (set_slot)."""
    global _initialized_device
    L = _l.load()
    if devices is None:
        check(L.hb200_init_multi(int(n_devices)))
    else:
        arr = (C.c_int * len(devices))(*devices)
        check(L.hb200_init_slots(arr, len(devices)))
    _initialized_device = 0
    return int(L.hb200_slot_count())


def set_slot(slot: int) -> None:
    check(_l.load().hb200_set_slot(slot))


def multi_batch_launch(batches: list, streams: list | None = None) -> None:
    """hb200_multi_batch_launch: one recorded batch per device slot, launched one after the other by this thread."""
    arr = (C.c_void_p * len(batches))(*[b._h for b in batches])
    st = None
    if streams is not None:
        st = (C.c_void_p * len(streams))(*[C.c_void_p(int(x.cuda_stream)) if x is not None else C.c_void_p(0) for x in streams])
    check(_l.load().hb200_multi_batch_launch(arr, len(batches), st))


def shutdown() -> None:
    global _initialized_device
    check(_l.load().hb200_shutdown())
    _initialized_device = None


def sm_count() -> int:
    return int(_l.load().hb200_sm_count())


def block_size(dtype: int) -> int:
    return int(_l.load().hb200_block_size(dtype))


def block_bytes(dtype: int) -> int:
    return int(_l.load().hb200_block_bytes(dtype))


def byte_size(dtype: int, n_cols: int) -> int:
    """GgmlDType::byte_size (hearth-gguf/src/ggml.rs:173-176)."""
    return int(_l.load().hb200_byte_size(dtype, n_cols))


def selected_kernel(dtype: int, seq_len: int = 1) -> str:
    """hearth_quant::selected_kernel (hearth-quant/src/lib.rs:411-418)."""
    return _l.load().hb200_selected_kernel(dtype, seq_len).decode()


def _text_call(fn, dtypes) -> str:
    arr = (C.c_int * len(dtypes))(*dtypes)
    need = C.c_size_t()
    rc = fn(arr, len(dtypes), None, 0, C.byref(need))
    if rc not in (0, -8):
        check(rc)
    buf = C.create_string_buffer(need.value + 1)
    check(fn(arr, len(dtypes), buf, need.value + 1, C.byref(need)))
    return buf.value.decode()


def dispatch_report(dtypes) -> dict:
    """hearth_quant::dispatch_report (hearth-quant/src/lib.rs:449-473): kernels per weight format and token range."""
    import json
    return json.loads(_text_call(_l.load().hb200_dispatch_report, list(dtypes)))


def dispatch_banner(dtypes) -> str:
    """DispatchReport::banner (hearth-quant/src/lib.rs:438-447)."""
    return _text_call(_l.load().hb200_dispatch_banner, list(dtypes))


def _np_ptr(a: np.ndarray) -> C.c_void_p:
    assert a.flags["C_CONTIGUOUS"]
    return C.c_void_p(a.ctypes.data)


def _stream_ptr(stream) -> C.c_void_p:
    if stream is None:
        import torch
        stream = torch.cuda.current_stream()
    return C.c_void_p(int(stream.cuda_stream))


def measure_i8_peak() -> float:
    """Dense int8 tensor-core rate of the device in use, measured, in TOP/s."""
    v = C.c_double()
    check(_l.load().hb200_measure_i8_peak(C.byref(v)))
    return float(v.value)


class Weight:
    """A weight tensor resident on the device (GpuCompute::upload_bytes residency)."""

    def __init__(self, handle, dtype, n_rows, n_cols):
        self._h = handle
        self.dtype, self.n_rows, self.n_cols = dtype, n_rows, n_cols

    @classmethod
    def upload(cls, dtype: int, n_rows: int, n_cols: int, packed: np.ndarray, rows: tuple[int, int] | None = None):
        packed = np.ascontiguousarray(packed, dtype=np.uint8).reshape(-1)
        h = C.c_void_p()
        L = _l.load()
        if rows is None:
            check(L.hb200_weight_upload(dtype, n_rows, n_cols, _np_ptr(packed), packed.size, C.byref(h)))
            return cls(h, dtype, n_rows, n_cols)
        check(L.hb200_weight_upload_rows(dtype, n_rows, n_cols, _np_ptr(packed), packed.size, rows[0], rows[1], C.byref(h)))
        return cls(h, dtype, rows[1] - rows[0], n_cols)

    @classmethod
    def upload_dev(cls, dtype: int, n_rows: int, n_cols: int, packed_dev, stream=None):
        """packed_dev: torch.uint8 CUDA tensor holding the reference's packed bytes."""
        assert packed_dev.is_cuda and packed_dev.is_contiguous()
        h = C.c_void_p()
        check(_l.load().hb200_weight_upload_dev(dtype, n_rows, n_cols, C.c_void_p(packed_dev.data_ptr()),
                                                packed_dev.numel(), _stream_ptr(stream), C.byref(h)))
        return cls(h, dtype, n_rows, n_cols)

    @property
    def resident_bytes(self) -> int:
        d, r, c, b = C.c_int(), C.c_size_t(), C.c_size_t(), C.c_size_t()
        check(_l.load().hb200_weight_info(self._h, C.byref(d), C.byref(r), C.byref(c), C.byref(b)))
        return int(b.value)

    @property
    def packed_bytes(self) -> int:
        return self.n_rows * byte_size(self.dtype, self.n_cols)

    def free(self) -> None:
        if self._h:
            check(_l.load().hb200_weight_free(self._h))
            self._h = None


class Act:
    """A resident activation: an f32 staging area plus its Q8_0 planes."""

    def __init__(self, max_seq_len: int, n_cols: int):
        self._h = C.c_void_p()
        check(_l.load().hb200_act_create(max_seq_len, n_cols, C.byref(self._h)))
        self.max_seq_len, self.n_cols = max_seq_len, n_cols

    def f32_ptr(self) -> int:
        p = C.c_void_p()
        check(_l.load().hb200_act_f32_ptr(self._h, C.byref(p)))
        return int(p.value)

    def set_f32(self, x, stream=None) -> None:
        """Copy a torch CUDA f32 tensor [seq, n_cols] into the staging area (device to device)."""
        import torch
        assert x.is_cuda and x.dtype == torch.float32 and x.is_contiguous()
        n = x.numel()
        dst = _as_torch_f32(self.f32_ptr(), n, x.device)
        dst.copy_(x.reshape(-1))

    def quantize(self, seq_len: int, x_dev=None, stream=None) -> None:
        """par_quantize (hearth-llm/src/pool.rs:467) on the device."""
        xp = C.c_void_p(x_dev.data_ptr()) if x_dev is not None else C.c_void_p(0)
        check(_l.load().hb200_act_quantize_dev(self._h, xp, seq_len, _stream_ptr(stream)))

    def rms_norm_q8(self, x_dev, weight_dev, eps: float, seq_len: int, stream=None) -> None:
        """ops::rms_norm_q8_batch (hearth-llm/src/ops.rs:489) on the device, into this activation's planes."""
        check(_l.load().hb200_act_rms_norm_q8_dev(self._h, C.c_void_p(x_dev.data_ptr()), C.c_void_p(weight_dev.data_ptr()),
                                                  eps, seq_len, _stream_ptr(stream)))

    def silu_mul_q8(self, gate_dev, up_dev, seq_len: int, stream=None) -> None:
        """ops::silu_mul_q8 (hearth-llm/src/ops.rs:273) per token on the device."""
        check(_l.load().hb200_act_silu_mul_q8_dev(self._h, C.c_void_p(gate_dev.data_ptr()), C.c_void_p(up_dev.data_ptr()),
                                                  seq_len, _stream_ptr(stream)))

    def hadamard_quantize(self, seq_len: int, block_size: int, x_dev=None, signs_dev=None, rotated_dev=None, stream=None) -> None:
        """hadamard_rotate + quantize_q8_0 (hearth-llm/src/model/qwen35.rs:924-943) on the device."""
        p = lambda t: C.c_void_p(t.data_ptr()) if t is not None else C.c_void_p(0)
        check(_l.load().hb200_act_hadamard_quantize_dev(self._h, p(x_dev), p(signs_dev), block_size, seq_len, p(rotated_dev),
                                                        _stream_ptr(stream)))

    def load_q8_0(self, q8_dev, seq_len: int, q8_stride: int, stream=None) -> None:
        check(_l.load().hb200_act_load_q8_0_dev(self._h, C.c_void_p(q8_dev.data_ptr()), seq_len, q8_stride, _stream_ptr(stream)))

    def store_q8_0(self, q8_dev, seq_len: int, q8_stride: int, stream=None) -> None:
        check(_l.load().hb200_act_store_q8_0_dev(self._h, C.c_void_p(q8_dev.data_ptr()), seq_len, q8_stride, _stream_ptr(stream)))

    def free(self) -> None:
        if self._h:
            check(_l.load().hb200_act_free(self._h))
            self._h = None


def _as_torch_f32(ptr: int, n: int, device):
    """View n floats of library-owned device memory as a torch tensor (no copy)."""
    import torch

    class _Holder:
        pass

    h = _Holder()
    h.__cuda_array_interface__ = {"shape": (n,), "typestr": "<f4", "data": (ptr, False), "version": 3}
    return torch.as_tensor(h, device=device)


def dequant_matmul_f32act(w: "Weight", x: np.ndarray, accum: np.ndarray | None = None) -> np.ndarray:
    """GpuCompute::dequant_matmul_fused / _batch (hearth-compute/src/lib.rs:483, :1153): f32 activations, the shaders'
    arithmetic; with `accum` the add-in-place form (lib.rs:1123).  f32 [batch, n_rows]."""
    x2 = _rows(x)
    out = np.zeros((x2.shape[0], w.n_rows), dtype=np.float32) if accum is None else np.array(accum, dtype=np.float32).reshape(x2.shape[0], w.n_rows)
    check(_l.load().hb200_matmul_f32act(w._h, _np_ptr(x2), x2.shape[0], _np_ptr(out), 0 if accum is None else 1))
    return out


def dequant_matmul_f32act_dev(w: "Weight", x_dev, seq_len: int, out_dev, ld_out: int | None = None, accumulate: bool = False,
                              stream=None) -> None:
    """Device-buffer form; ld_out > n_rows lets gate|up or q|k|v share one output buffer (fused_gate_up, fused_qkv)."""
    check(_l.load().hb200_matmul_f32act_dev(w._h, C.c_void_p(x_dev.data_ptr()), seq_len, C.c_void_p(out_dev.data_ptr()),
                                            w.n_rows if ld_out is None else ld_out, 1 if accumulate else 0, _stream_ptr(stream)))


class Gguf:
    """A mapped GGUF model file (hearth_gguf::GgufFile, hearth-gguf/src/gguf.rs:137-259).  Parsing needs no device."""

    def __init__(self, path: str):
        self._h = C.c_void_p()
        check(_l.load().hb200_gguf_open(os.fsencode(path), C.byref(self._h)))
        L = _l.load()
        self.version = int(L.hb200_gguf_version(self._h))
        self.data_offset = int(L.hb200_gguf_data_offset(self._h))
        self.tensors = []
        for i in range(L.hb200_gguf_tensor_count(self._h)):
            name, dt, nd, off, nb = C.c_char_p(), C.c_int(), C.c_size_t(), C.c_uint64(), C.c_size_t()
            shape = (C.c_uint64 * 8)()
            check(L.hb200_gguf_tensor_info(self._h, i, C.byref(name), C.byref(dt), C.byref(nd), shape, C.byref(off), C.byref(nb)))
            self.tensors.append(dict(name=name.value.decode(), dtype=dt.value, shape=[int(shape[k]) for k in range(nd.value)],
                                     offset=int(off.value), bytes=int(nb.value)))

    def find_tensor(self, name: str) -> int:
        idx = C.c_size_t()
        check(_l.load().hb200_gguf_find_tensor(self._h, name.encode(), C.byref(idx)))
        return int(idx.value)

    def tensor_data(self, index: int) -> np.ndarray:
        p, n = C.c_void_p(), C.c_size_t()
        check(_l.load().hb200_gguf_tensor_data(self._h, index, C.byref(p), C.byref(n)))
        return np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_uint8)), shape=(n.value,)).copy()

    def upload(self, name_or_index) -> "Weight":
        i = self.find_tensor(name_or_index) if isinstance(name_or_index, str) else int(name_or_index)
        h = C.c_void_p()
        check(_l.load().hb200_gguf_upload_tensor(self._h, i, C.byref(h)))
        t = self.tensors[i]
        return Weight(h, t["dtype"], t["shape"][1] if len(t["shape"]) > 1 else 1, t["shape"][0])

    def meta_u64(self, key: str) -> int:
        v = C.c_uint64()
        check(_l.load().hb200_gguf_meta_u64(self._h, key.encode(), C.byref(v)))
        return int(v.value)

    def meta_f64(self, key: str) -> float:
        v = C.c_double()
        check(_l.load().hb200_gguf_meta_f64(self._h, key.encode(), C.byref(v)))
        return float(v.value)

    def meta_str(self, key: str) -> str:
        p, n = C.c_char_p(), C.c_size_t()
        check(_l.load().hb200_gguf_meta_str(self._h, key.encode(), C.byref(p), C.byref(n)))
        return C.string_at(p, n.value).decode("utf-8", "replace")

    def meta_array_f32(self, key: str) -> np.ndarray:
        n = C.c_size_t()
        check(_l.load().hb200_gguf_meta_array_f32(self._h, key.encode(), None, 0, C.byref(n)))
        out = np.zeros(n.value, dtype=np.float32)
        check(_l.load().hb200_gguf_meta_array_f32(self._h, key.encode(), _np_ptr(out), out.size, C.byref(n)))
        return out

    def close(self) -> None:
        if self._h:
            _l.load().hb200_gguf_close(self._h)
            self._h = None


def argmax_f32_dev(x_dev, n: int | None = None, stream=None) -> int:
    """GpuCompute::argmax_f32 (hearth-compute/src/lib.rs:338): index of the largest value of a CUDA f32 tensor."""
    import torch
    assert x_dev.is_cuda and x_dev.dtype == torch.float32 and x_dev.is_contiguous()
    idx = C.c_uint32()
    check(_l.load().hb200_argmax_f32_dev(C.c_void_p(x_dev.data_ptr()), x_dev.numel() if n is None else n, C.byref(idx),
                                         _stream_ptr(stream)))
    return int(idx.value)


def argmax_f32_dev_async(x_dev, index_dev, n: int | None = None, stream=None) -> None:
    """The same without a synchronisation; index_dev is a CUDA int32 / uint32 tensor of one element."""
    check(_l.load().hb200_argmax_f32_dev_async(C.c_void_p(x_dev.data_ptr()), x_dev.numel() if n is None else n,
                                               C.c_void_p(index_dev.data_ptr()), _stream_ptr(stream)))


# ---- host-buffer calls --------------------------------------------------------------------------

def quantize_q8_0(x: np.ndarray) -> np.ndarray:
    """quantize_q8_0_into / par_quantize: f32 [seq, dim] (or [dim]) -> uint8 [seq, ceil(dim/32)*34]."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    x2 = x.reshape(1, -1) if x.ndim == 1 else x
    seq_len, dim = x2.shape
    out = np.zeros((seq_len, byte_size(Q8_0, dim)), dtype=np.uint8)
    check(_l.load().hb200_quantize_q8_0(_np_ptr(x2), seq_len, dim, _np_ptr(out)))
    return out[0] if x.ndim == 1 else out


def _rows(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    return x.reshape(1, -1) if x.ndim == 1 else x


def rms_norm_q8(x: np.ndarray, weight: np.ndarray, eps: float) -> np.ndarray:
    """ops::rms_norm_q8 / rms_norm_q8_batch: f32 [seq, dim] (or [dim]) -> uint8 [seq, ceil(dim/32)*34]."""
    x2 = _rows(x)
    w = np.ascontiguousarray(weight, dtype=np.float32)
    seq_len, dim = x2.shape
    assert w.size == dim
    out = np.zeros((seq_len, byte_size(Q8_0, dim)), dtype=np.uint8)
    check(_l.load().hb200_rms_norm_q8(_np_ptr(x2), _np_ptr(w), eps, _np_ptr(out), seq_len, dim))
    return out[0] if np.ndim(x) == 1 else out


def silu_mul_q8(gate: np.ndarray, up: np.ndarray) -> np.ndarray:
    """ops::silu_mul_q8 per token: f32 [seq, dim] x2 -> uint8 [seq, (dim/32)*34]."""
    g2, u2 = _rows(gate), _rows(up)
    assert g2.shape == u2.shape
    seq_len, dim = g2.shape
    out = np.zeros((seq_len, dim // 32 * 34), dtype=np.uint8)
    check(_l.load().hb200_silu_mul_q8(_np_ptr(g2), _np_ptr(u2), _np_ptr(out), seq_len, dim))
    return out[0] if np.ndim(gate) == 1 else out


def hadamard_quantize_q8_0(x: np.ndarray, signs: np.ndarray | None, block_size: int, return_rotated: bool = False):
    """hadamard_rotate then quantize_q8_0 (hearth-llm/src/model/qwen35.rs:924-943) per token."""
    x2 = _rows(x)
    seq_len, dim = x2.shape
    sg = np.ascontiguousarray(signs, dtype=np.float32) if signs is not None else None
    assert sg is None or sg.size == dim
    out = np.zeros((seq_len, byte_size(Q8_0, dim)), dtype=np.uint8)
    rot = np.zeros_like(x2) if return_rotated else None
    check(_l.load().hb200_hadamard_quantize_q8_0(_np_ptr(x2), _np_ptr(sg) if sg is not None else None, block_size, _np_ptr(out),
                                                 _np_ptr(rot) if rot is not None else None, seq_len, dim))
    if np.ndim(x) == 1:
        out = out[0]
        rot = rot[0] if rot is not None else None
    return (out, rot) if return_rotated else out


def par_dot_rows(w: Weight, a_q8: np.ndarray) -> np.ndarray:
    """ThreadPool::par_dot_rows: one Q8_0 activation -> f32 [n_rows]."""
    a_q8 = np.ascontiguousarray(a_q8, dtype=np.uint8)
    out = np.zeros(w.n_rows, dtype=np.float32)
    check(_l.load().hb200_dot_rows(w._h, _np_ptr(a_q8), _np_ptr(out)))
    return out


def par_dot_rows_batched(w: Weight, a_q8: np.ndarray, seq_len: int | None = None, q8_stride: int | None = None) -> np.ndarray:
    """ThreadPool::par_dot_rows_batched: uint8 [seq, stride] -> token-major f32 [seq, n_rows]."""
    a_q8 = np.ascontiguousarray(a_q8, dtype=np.uint8)
    if seq_len is None:
        seq_len = a_q8.shape[0]
    if q8_stride is None:
        q8_stride = a_q8.shape[-1] if a_q8.ndim == 2 else byte_size(Q8_0, w.n_cols)
    out = np.zeros((seq_len, w.n_rows), dtype=np.float32)
    check(_l.load().hb200_dot_rows_batched(w._h, _np_ptr(a_q8), seq_len, q8_stride, _np_ptr(out)))
    return out


def matmul(w: Weight, x: np.ndarray) -> np.ndarray:
    """LlamaModel::matmul / matmul_batch with x_q8=None: f32 [seq, n_cols] (or [n_cols]) -> f32 [seq, n_rows]."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    x2 = x.reshape(1, -1) if x.ndim == 1 else x
    if x2.shape[1] != w.n_cols:
        raise Hb200Error(-4, f"Matmul dim mismatch: cols={w.n_cols} x.len={x2.shape[1]}")
    out = np.zeros((x2.shape[0], w.n_rows), dtype=np.float32)
    check(_l.load().hb200_matmul_f32(w._h, _np_ptr(x2), x2.shape[0], _np_ptr(out)))
    return out[0] if x.ndim == 1 else out


def matmul_fused(ws: list, x: np.ndarray) -> list:
    """LlamaModel::matmul_fused2 / matmul_fused_qkv: several weights against one input; one upload and one
    quantization of x.  Returns one f32 [seq, n_rows_i] (or [n_rows_i]) array per weight."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    x2 = x.reshape(1, -1) if x.ndim == 1 else x
    outs = [np.zeros((x2.shape[0], w.n_rows), dtype=np.float32) for w in ws]
    harr = (C.c_void_p * len(ws))(*[w._h for w in ws])
    oarr = (C.c_void_p * len(ws))(*[C.c_void_p(o.ctypes.data) for o in outs])
    check(_l.load().hb200_matmul_f32_fused(harr, len(ws), _np_ptr(x2), x2.shape[0], oarr))
    return [o[0] if x.ndim == 1 else o for o in outs]


def block_dots_i32(w: Weight, a_q8: np.ndarray) -> np.ndarray:
    """Exact int32 dots per (token, row, 32-column block): int32 [seq, n_rows, n_cols // 32]."""
    a_q8 = np.ascontiguousarray(a_q8, dtype=np.uint8)
    a2 = a_q8.reshape(1, -1) if a_q8.ndim == 1 else a_q8
    seq_len, stride = a2.shape
    n_sub = (w.n_cols // 32) if w.dtype == Q8_0 else (w.n_cols // 128) * 4
    out = np.zeros((seq_len, w.n_rows, n_sub), dtype=np.int32)
    check(_l.load().hb200_block_dots_i32(w._h, _np_ptr(a2), seq_len, stride, _np_ptr(out)))
    return out


# ---- device-buffer calls ------------------------------------------------------------------------

def dot_rows_dev(w: Weight, a: Act, seq_len: int, out_dev, ld_out: int | None = None, stream=None) -> None:
    check(_l.load().hb200_dot_rows_dev(w._h, a._h, seq_len, C.c_void_p(out_dev.data_ptr()),
                                       ld_out if ld_out is not None else w.n_rows, _stream_ptr(stream)))


def matmul_f32_dev(w: Weight, a: Act, seq_len: int, out_dev, ld_out: int | None = None, stream=None) -> None:
    check(_l.load().hb200_matmul_f32_dev(w._h, a._h, seq_len, C.c_void_p(out_dev.data_ptr()),
                                         ld_out if ld_out is not None else w.n_rows, _stream_ptr(stream)))


def matmul_f32_noalloc(w: Weight, x_dev, out_dev, ld_out: int | None = None, stream=None) -> None:
    """hb200_matmul_f32_noalloc: x_dev is a torch CUDA f32 tensor [seq_len, n_cols] owned by the caller; the
    call allocates nothing on the device (at most 4 tokens of 32768 columns)."""
    seq_len = 1 if x_dev.dim() == 1 else x_dev.shape[0]
    check(_l.load().hb200_matmul_f32_noalloc(w._h, C.c_void_p(x_dev.data_ptr()), seq_len, C.c_void_p(out_dev.data_ptr()),
                                             ld_out if ld_out is not None else w.n_rows, _stream_ptr(stream)))


class Batch:
    """begin_batch / end_batch (hearth-compute/src/lib.rs:206-224): record ops, launch them together."""

    def __init__(self):
        self._h = C.c_void_p()
        check(_l.load().hb200_batch_create(C.byref(self._h)))
        self._keep = []

    def add(self, w: Weight, a: Act, seq_len: int, out_dev, ld_out: int | None = None) -> None:
        self._keep.append((w, a, out_dev))
        check(_l.load().hb200_batch_add(self._h, w._h, a._h, seq_len, C.c_void_p(out_dev.data_ptr()),
                                        ld_out if ld_out is not None else w.n_rows))

    def set_peers(self, my_rank: int, buffers: list, wait: bool = True, area_floats: int = 0) -> None:
        """Row-sharded run: buffers[r] is rank r's PeerBuffer (local or opened); outputs are stored into all of them.
        area_floats > 0: every buffer holds two output areas that far apart, written by alternate launches."""
        arr = (C.c_void_p * len(buffers))(*[C.c_void_p(b.ptr) for b in buffers])
        check(_l.load().hb200_batch_set_peers(self._h, len(buffers), my_rank, arr, area_floats * 4, 1 if wait else 0))
        self._keep.append(buffers)

    @property
    def peer_area(self) -> int:
        """Index (0 or 1) of the output area the latest launch wrote."""
        return int(_l.load().hb200_batch_peer_area(self._h))

    def seal(self) -> None:
        check(_l.load().hb200_batch_seal(self._h))

    def launch(self, stream=None) -> None:
        check(_l.load().hb200_batch_launch(self._h, _stream_ptr(stream)))

    @property
    def input_floats(self) -> int:
        return int(_l.load().hb200_batch_input_floats(self._h))

    def run_host(self, x_host: np.ndarray, out_dev, out_host: np.ndarray) -> None:
        """One recorded step from host memory: x_host (float32, input_floats long) holds every distinct activation's
        rows in order of first use; out_dev is the device tensor the ops write into, copied whole into out_host."""
        assert x_host.dtype == np.float32 and x_host.size >= self.input_floats and out_host.dtype == np.float32
        check(_l.load().hb200_batch_run_host(self._h, _np_ptr(x_host), C.c_void_p(out_dev.data_ptr()), out_host.size, _np_ptr(out_host)))

    def run_dev(self, x_dev, out_dev, out_host: np.ndarray, x_stream=None) -> None:
        """The same step with its inputs already on the device (float32 tensor of input_floats values in run_host's
        layout, written on x_stream): a device copy, the list quantizer, the recorded batch, the outputs back."""
        assert out_host.dtype == np.float32 and x_dev.numel() >= self.input_floats
        check(_l.load().hb200_batch_run_dev(self._h, C.c_void_p(x_dev.data_ptr()), _stream_ptr(x_stream),
                                            C.c_void_p(out_dev.data_ptr()), out_host.size, _np_ptr(out_host)))

    @property
    def launch_count(self) -> int:
        return int(_l.load().hb200_batch_launch_count(self._h))

    def free(self) -> None:
        if self._h:
            check(_l.load().hb200_batch_free(self._h))
            self._h = None
            self._keep = []


class PeerBuffer:
    """An output buffer other ranks can store into (hb200_peer_alloc / hb200_peer_open)."""

    def __init__(self, ptr: int, n_floats: int, handle: bytes | None, owned: bool):
        self.ptr, self.n_floats, self.handle, self.owned = ptr, n_floats, handle, owned

    @classmethod
    def alloc(cls, n_floats: int) -> "PeerBuffer":
        p = C.c_void_p()
        h = (C.c_uint8 * 64)()
        check(_l.load().hb200_peer_alloc(n_floats * 4, C.byref(p), h))
        return cls(int(p.value), n_floats, bytes(h), True)

    @classmethod
    def open(cls, handle: bytes, n_floats: int) -> "PeerBuffer":
        p = C.c_void_p()
        h = (C.c_uint8 * 64).from_buffer_copy(handle)
        check(_l.load().hb200_peer_open(h, C.byref(p)))
        return cls(int(p.value), n_floats, None, False)

    def tensor(self, device):
        """The output area(s) as a torch float32 tensor (no copy)."""
        return _as_torch_f32(self.ptr, self.n_floats, device)

    def flags(self, device):
        """The eight epoch flags of the control block in front of the output area (int32, no copy)."""
        import torch
        return _as_torch_f32(self.ptr - 512, 8, device).view(torch.int32)

    def close(self) -> None:
        if self.ptr:
            L = _l.load()
            check(L.hb200_peer_free(C.c_void_p(self.ptr)) if self.owned else L.hb200_peer_close(C.c_void_p(self.ptr)))
            self.ptr = 0


def check_status() -> None:
    check(_l.load().hb200_check_status())
