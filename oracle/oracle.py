"""ctypes bindings for the CPU checker (libhearth_oracle.so / libhearth_simd.so).

Test infrastructure only: imported by tests/, by the smoke check and by the
benchmark's CPU-baseline leg.  The product package never imports this module.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))

Q8_0, Q4_K, Q6_K, Q1_0, Q2_0, Q1_0_G128, PQ2_0, PTQ1_0 = 8, 12, 14, 41, 42, 43, 142, 143

_u8p = C.POINTER(C.c_uint8)
_f32p = C.POINTER(C.c_float)
_i32p = C.POINTER(C.c_int32)


def build(force: bool = False) -> None:
    """Compile both shared objects with the Makefile beside this file."""
    so = [os.path.join(_HERE, n) for n in ("libhearth_oracle.so", "libhearth_simd.so")]
    if force or not all(os.path.exists(p) for p in so):
        subprocess.check_call(["make", "-s", "-C", _HERE, "all"])


def _load(name: str) -> C.CDLL:
    path = os.path.join(_HERE, name)
    if not os.path.exists(path):
        build()
    return C.CDLL(path)


_lib = None
_simd = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        L = _load("libhearth_oracle.so")
        L.ho_h2f.restype = C.c_float
        L.ho_h2f.argtypes = [C.c_uint16]
        L.ho_f2h.restype = C.c_uint16
        L.ho_f2h.argtypes = [C.c_float]
        for fn in ("ho_block_size", "ho_block_bytes"):
            getattr(L, fn).restype = C.c_size_t
            getattr(L, fn).argtypes = [C.c_int]
        L.ho_byte_size.restype = C.c_size_t
        L.ho_byte_size.argtypes = [C.c_int, C.c_size_t]
        L.ho_quantize_q8_0_into.restype = None
        L.ho_quantize_q8_0_into.argtypes = [_f32p, C.c_size_t, _u8p]
        L.ho_par_quantize.restype = None
        L.ho_par_quantize.argtypes = [C.c_size_t, C.c_size_t, _f32p, _u8p]
        for fn in ("ho_dequantize_q8_0", "ho_dequantize_q1_0g128", "ho_dequantize_q2_0", "ho_dequantize_q4_k",
                   "ho_dequantize_q6_k", "ho_dequantize_ptq1_0"):
            getattr(L, fn).restype = None
            getattr(L, fn).argtypes = [_u8p, C.c_size_t, _f32p, C.c_size_t]
        L.ho_block_dots_i32.restype = C.c_int
        L.ho_block_dots_i32.argtypes = [C.c_int, _u8p, _u8p, C.c_size_t, _i32p]
        for fn in ("ho_dot_q1_0g128_q8_0", "ho_dot_q2_0_q8_0", "ho_dot_q8_0_q8_0", "ho_dot_ptq1_0_q8_0"):
            getattr(L, fn).restype = C.c_float
            getattr(L, fn).argtypes = [_u8p, _u8p, C.c_size_t]
        for fn in ("ho_dot_q2_0_f32", "ho_dot_q4_k_f32", "ho_dot_q6_k_f32", "ho_dot_ptq1_0_f32"):
            getattr(L, fn).restype = C.c_float
            getattr(L, fn).argtypes = [_u8p, _f32p, C.c_size_t]
        L.ho_par_dot_rows_batched.restype = C.c_int
        L.ho_par_dot_rows_batched.argtypes = [C.c_int, C.c_size_t, C.c_size_t, C.c_size_t, _u8p, _u8p, _f32p,
                                              C.c_size_t, C.c_size_t]
        L.ho_matmul_kquant_f32.restype = C.c_int
        L.ho_matmul_kquant_f32.argtypes = [C.c_int, C.c_size_t, C.c_size_t, _u8p, _f32p, _f32p, C.c_size_t]
        L.ho_matmul_f32act.restype = C.c_int
        L.ho_matmul_f32act.argtypes = [C.c_int, C.c_size_t, C.c_size_t, _u8p, _f32p, _f32p, C.c_size_t, C.c_int]
        L.ho_argmax_f32.restype = C.c_uint32
        L.ho_argmax_f32.argtypes = [_f32p, C.c_size_t]
        L.ho_quantize_ptq1_0.restype = None
        L.ho_quantize_ptq1_0.argtypes = [_f32p, C.c_size_t, _u8p]
        L.ho_hadamard_rotate.restype = None
        L.ho_hadamard_rotate.argtypes = [_f32p, C.c_size_t, _f32p, C.c_size_t]
        L.ho_hadamard_quantize_q8_0.restype = None
        L.ho_hadamard_quantize_q8_0.argtypes = [_f32p, C.c_size_t, _f32p, C.c_size_t, _f32p, _u8p]
        L.ho_rms_norm_q8.restype = None
        L.ho_rms_norm_q8.argtypes = [_f32p, _f32p, C.c_float, _u8p, C.c_size_t]
        L.ho_silu_mul_q8.restype = None
        L.ho_silu_mul_q8.argtypes = [_f32p, _f32p, _u8p, C.c_size_t]
        _lib = L
    return _lib


def simd() -> C.CDLL:
    global _simd
    if _simd is None:
        L = _load("libhearth_simd.so")
        L.hs_selected_kernel.restype = C.c_char_p
        L.hs_selected_kernel.argtypes = [C.c_int]
        L.hs_dot.restype = C.c_float
        L.hs_dot.argtypes = [C.c_int, _u8p, _u8p, C.c_size_t]
        L.hs_logical_cores.restype = C.c_int
        L.hs_physical_cores.restype = C.c_int
        L.hs_pool_start.restype = C.c_int
        L.hs_pool_start.argtypes = [C.c_int]
        L.hs_pool_stop.restype = None
        L.hs_par_dot_rows_batched.restype = C.c_int
        L.hs_par_dot_rows_batched.argtypes = [C.c_int, C.c_size_t, C.c_size_t, C.c_size_t, _u8p, _u8p, _f32p,
                                              C.c_size_t, C.c_size_t]
        _simd = L
    return _simd


def _u8(a: np.ndarray):
    assert a.dtype == np.uint8 and a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(_u8p)


def _f32(a: np.ndarray):
    assert a.dtype == np.float32 and a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(_f32p)


def byte_size(dtype: int, n: int) -> int:
    return int(lib().ho_byte_size(dtype, n))


def h2f(h: int) -> float:
    return float(lib().ho_h2f(h))


def f2h(f: float) -> int:
    return int(lib().ho_f2h(f))


def quantize_q8_0(x: np.ndarray) -> np.ndarray:
    """f32[seq_len, dim] (or f32[dim]) -> uint8[seq_len, ceil(dim/32)*34] (par_quantize layout)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    x2 = x.reshape(1, -1) if x.ndim == 1 else x
    seq_len, dim = x2.shape
    out = np.zeros((seq_len, (dim + 31) // 32 * 34), dtype=np.uint8)
    lib().ho_par_quantize(seq_len, dim, _f32(x2), _u8(out))
    return out[0] if x.ndim == 1 else out


def dequantize(dtype: int, data: np.ndarray, n_out: int) -> np.ndarray:
    fn = {Q8_0: "ho_dequantize_q8_0", Q1_0: "ho_dequantize_q1_0g128", Q1_0_G128: "ho_dequantize_q1_0g128",
          Q2_0: "ho_dequantize_q2_0", PQ2_0: "ho_dequantize_q2_0", Q4_K: "ho_dequantize_q4_k",
          Q6_K: "ho_dequantize_q6_k", PTQ1_0: "ho_dequantize_ptq1_0"}[dtype]
    data = np.ascontiguousarray(data, dtype=np.uint8)
    out = np.zeros(n_out, dtype=np.float32)
    getattr(lib(), fn)(_u8(data), data.size, _f32(out), n_out)
    return out


def block_dots_i32(dtype: int, w_row: np.ndarray, a_q8: np.ndarray, n_cols: int) -> np.ndarray:
    out = np.zeros(n_cols // 32, dtype=np.int32)
    rc = lib().ho_block_dots_i32(dtype, _u8(w_row), _u8(a_q8), n_cols, out.ctypes.data_as(_i32p))
    assert rc == 0
    return out


def dot_rows_batched(dtype: int, w: np.ndarray, a_q8: np.ndarray, n_rows: int, n_cols: int) -> np.ndarray:
    """Scalar-order results, token-major f32[seq_len, n_rows]."""
    a2 = a_q8.reshape(1, -1) if a_q8.ndim == 1 else a_q8
    a2 = np.ascontiguousarray(a2)
    seq_len, stride = a2.shape
    out = np.zeros((seq_len, n_rows), dtype=np.float32)
    rb = byte_size(dtype, n_cols)
    rc = lib().ho_par_dot_rows_batched(dtype, n_rows, seq_len, stride, _u8(w), _u8(a2), _f32(out), rb, n_cols)
    assert rc == 0
    return out


def matmul_kquant_f32(dtype: int, w: np.ndarray, x: np.ndarray, n_rows: int, n_cols: int) -> np.ndarray:
    x2 = np.ascontiguousarray(x.reshape(1, -1) if x.ndim == 1 else x, dtype=np.float32)
    out = np.zeros((x2.shape[0], n_rows), dtype=np.float32)
    rc = lib().ho_matmul_kquant_f32(dtype, n_rows, x2.shape[0], _u8(w), _f32(x2), _f32(out), n_cols)
    assert rc == 0
    return out


def simd_dot_rows_batched(dtype: int, w: np.ndarray, a_q8: np.ndarray, n_rows: int, n_cols: int,
                          out: np.ndarray | None = None) -> np.ndarray:
    """Same call through the restated SIMD arms and pool (hs_pool_start first)."""
    a2 = a_q8.reshape(1, -1) if a_q8.ndim == 1 else a_q8
    seq_len, stride = a2.shape
    if out is None:
        out = np.zeros((seq_len, n_rows), dtype=np.float32)
    rb = byte_size(dtype, n_cols)
    rc = simd().hs_par_dot_rows_batched(dtype, n_rows, seq_len, stride, _u8(w), _u8(a2), _f32(out), rb, n_cols)
    assert rc == 0, rc
    return out


def hadamard_rotate(x: np.ndarray, signs: np.ndarray | None, block_size: int) -> np.ndarray:
    """qwen35.rs:49-87 on every row of x (f32 [seq, n] or [n]); returns the rotated copy."""
    x2 = np.array(x, dtype=np.float32, copy=True)
    rows = x2.reshape(1, -1) if x2.ndim == 1 else x2
    sp = _f32(np.ascontiguousarray(signs, dtype=np.float32)) if signs is not None else None
    for r in rows:
        lib().ho_hadamard_rotate(_f32(r), r.size, sp, block_size)
    return x2


def hadamard_quantize_q8_0(x: np.ndarray, signs: np.ndarray | None, block_size: int) -> np.ndarray:
    return quantize_q8_0(hadamard_rotate(x, signs, block_size))


def rms_norm_q8(x: np.ndarray, weight: np.ndarray, eps: float) -> np.ndarray:
    """ops::rms_norm_q8_batch: f32 [seq, dim] -> uint8 [seq, ceil(dim/32)*34]."""
    x2 = np.ascontiguousarray(x.reshape(1, -1) if x.ndim == 1 else x, dtype=np.float32)
    w = np.ascontiguousarray(weight, dtype=np.float32)
    out = np.zeros((x2.shape[0], (x2.shape[1] + 31) // 32 * 34), dtype=np.uint8)
    for s in range(x2.shape[0]):
        lib().ho_rms_norm_q8(_f32(x2[s]), _f32(w), eps, _u8(out[s]), x2.shape[1])
    return out[0] if x.ndim == 1 else out


def silu_mul_q8(gate: np.ndarray, up: np.ndarray) -> np.ndarray:
    g2 = np.ascontiguousarray(gate.reshape(1, -1) if gate.ndim == 1 else gate, dtype=np.float32)
    u2 = np.ascontiguousarray(up.reshape(1, -1) if up.ndim == 1 else up, dtype=np.float32)
    out = np.zeros((g2.shape[0], g2.shape[1] // 32 * 34), dtype=np.uint8)
    for s in range(g2.shape[0]):
        lib().ho_silu_mul_q8(_f32(g2[s]), _f32(u2[s]), _u8(out[s]), g2.shape[1])
    return out[0] if gate.ndim == 1 else out


def quantize_ptq1_0(x: np.ndarray) -> np.ndarray:
    """ptq1_0::quantize: f32 [n] -> uint8 [(n/128)*28]."""
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1)
    out = np.zeros(x.size // 128 * 28, dtype=np.uint8)
    lib().ho_quantize_ptq1_0(_f32(x), x.size, _u8(out))
    return out


def dot_ptq1_0_f32(w_row: np.ndarray, x: np.ndarray, n: int) -> float:
    return float(lib().ho_dot_ptq1_0_f32(_u8(np.ascontiguousarray(w_row)), _f32(np.ascontiguousarray(x, dtype=np.float32)), n))


def simd_matmul_kquant_f32(dtype: int, w: np.ndarray, x: np.ndarray, n_rows: int, n_cols: int,
                           out: np.ndarray | None = None) -> np.ndarray:
    """Q4_K / Q6_K rows against f32 activations through the restated eight-lane FMA loops and the pool."""
    x2 = np.ascontiguousarray(x.reshape(1, -1) if x.ndim == 1 else x, dtype=np.float32)
    if out is None:
        out = np.zeros((x2.shape[0], n_rows), dtype=np.float32)
    rb = byte_size(dtype, n_cols)
    rc = simd().hs_par_dot_rows_batched(dtype, n_rows, x2.shape[0], x2.shape[1] * 4, _u8(w),
                                        x2.ctypes.data_as(_u8p), _f32(out), rb, n_cols)
    assert rc == 0, rc
    return out


def argmax_f32(x: np.ndarray) -> int:
    """GpuCompute::argmax_f32 executed literally on the CPU."""
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1)
    return int(lib().ho_argmax_f32(_f32(x), x.size))


def matmul_f32act(dtype: int, w: np.ndarray, x: np.ndarray, n_rows: int, n_cols: int, accum: np.ndarray | None = None) -> np.ndarray:
    """The GPU shaders' f32-activation matmul (dequant_matmul_fused / _batch / _add_inplace): f32 [batch, n_rows]."""
    x2 = np.ascontiguousarray(x.reshape(1, -1) if x.ndim == 1 else x, dtype=np.float32)
    out = np.zeros((x2.shape[0], n_rows), dtype=np.float32) if accum is None else np.array(accum, dtype=np.float32).reshape(x2.shape[0], n_rows)
    rc = lib().ho_matmul_f32act(dtype, n_rows, x2.shape[0], _u8(np.ascontiguousarray(w)), _f32(x2), _f32(out), n_cols, 0 if accum is None else 1)
    assert rc == 0
    return out
