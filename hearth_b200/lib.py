"""ctypes loader for libhearth_b200.so (the C ABI declared in include/hb200.h).

There is no fallback of any kind: if the shared object is missing or a symbol
cannot be bound, import fails with an explicit message.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
# HB200_LIB in the environment selects another build of the same library (the bounds-checked debug build,
# libhearth_b200_bounds.so); there is no fallback either way.
LIB_PATH = os.environ.get("HB200_LIB") or os.path.join(HERE, "libhearth_b200.so")

# GGML type ids on this path (hearth-gguf/src/ggml.rs:49-101 of the reference).
Q8_0, Q4_K, Q6_K, Q1_0_G128_LEGACY, Q1_0, Q2_0, Q1_0_G128, PQ2_0, PTQ1_0 = 8, 12, 14, 39, 41, 42, 43, 142, 143

STATUS = {
    0: "HB200_OK", -1: "HB200_ERR_NOT_INITIALIZED", -2: "HB200_ERR_NO_DEVICE", -3: "HB200_ERR_BAD_DTYPE",
    -4: "HB200_ERR_BAD_SHAPE", -5: "HB200_ERR_NULL", -6: "HB200_ERR_CUDA", -7: "HB200_ERR_UNSUPPORTED",
    -8: "HB200_ERR_TOO_LARGE", -9: "HB200_ERR_TIMEOUT", -10: "HB200_ERR_IO", -11: "HB200_ERR_BAD_FORMAT",
    -12: "HB200_ERR_NOT_FOUND",
}

_vp = C.c_void_p
_sz = C.c_size_t
_int = C.c_int

# name -> (restype, argtypes); must list every symbol include/hb200.h declares.
SIGNATURES = {
    "hb200_init": (_int, [_int]),
    "hb200_init_multi": (_int, [_int]),
    "hb200_init_slots": (_int, [C.POINTER(_int), _int]),
    "hb200_set_slot": (_int, [_int]),
    "hb200_slot_count": (_int, []),
    "hb200_shutdown": (_int, []),
    "hb200_last_error": (C.c_char_p, []),
    "hb200_sm_count": (_int, []),
    "hb200_block_size": (_sz, [_int]),
    "hb200_block_bytes": (_sz, [_int]),
    "hb200_measure_i8_peak": (_int, [C.POINTER(C.c_double)]),
    "hb200_bounds_checked": (_int, []),
    "hb200_bounds_selftest": (_int, []),
    "hb200_plan_chunks": (_int, [C.POINTER(C.c_int), C.c_size_t, _int, C.POINTER(C.c_int)]),
    "hb200_plan_rounds": (_int, [C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(C.c_int), C.c_size_t, _int, C.POINTER(C.c_int),
                                 C.POINTER(C.c_int), C.c_size_t, C.POINTER(C.c_size_t)]),
    "hb200_byte_size": (_sz, [_int, _sz]),
    "hb200_selected_kernel": (C.c_char_p, [_int, _sz]),
    "hb200_dispatch_report": (_int, [C.POINTER(_int), _sz, C.c_char_p, _sz, C.POINTER(_sz)]),
    "hb200_dispatch_banner": (_int, [C.POINTER(_int), _sz, C.c_char_p, _sz, C.POINTER(_sz)]),
    "hb200_weight_upload": (_int, [_int, _sz, _sz, _vp, _sz, C.POINTER(_vp)]),
    "hb200_weight_upload_dev": (_int, [_int, _sz, _sz, _vp, _sz, _vp, C.POINTER(_vp)]),
    "hb200_weight_upload_rows": (_int, [_int, _sz, _sz, _vp, _sz, _sz, _sz, C.POINTER(_vp)]),
    "hb200_weight_free": (_int, [_vp]),
    "hb200_weight_info": (_int, [_vp, C.POINTER(_int), C.POINTER(_sz), C.POINTER(_sz), C.POINTER(_sz)]),
    "hb200_act_create": (_int, [_sz, _sz, C.POINTER(_vp)]),
    "hb200_act_free": (_int, [_vp]),
    "hb200_act_f32_ptr": (_int, [_vp, C.POINTER(_vp)]),
    "hb200_act_q8_planes": (_int, [_vp, C.POINTER(_vp), C.POINTER(_vp), C.POINTER(_vp), C.POINTER(_sz), C.POINTER(_sz)]),
    "hb200_act_quantize_dev": (_int, [_vp, _vp, _sz, _vp]),
    "hb200_act_load_q8_0_dev": (_int, [_vp, _vp, _sz, _sz, _vp]),
    "hb200_act_store_q8_0_dev": (_int, [_vp, _vp, _sz, _sz, _vp]),
    "hb200_act_rms_norm_q8_dev": (_int, [_vp, _vp, _vp, C.c_float, _sz, _vp]),
    "hb200_act_silu_mul_q8_dev": (_int, [_vp, _vp, _vp, _sz, _vp]),
    "hb200_act_hadamard_quantize_dev": (_int, [_vp, _vp, _vp, _sz, _sz, _vp, _vp]),
    "hb200_matmul_f32act_dev": (_int, [_vp, _vp, _sz, _vp, _sz, _int, _vp]),
    "hb200_matmul_f32act": (_int, [_vp, _vp, _sz, _vp, _int]),
    "hb200_argmax_f32_dev": (_int, [_vp, _sz, C.POINTER(C.c_uint32), _vp]),
    "hb200_argmax_f32_dev_async": (_int, [_vp, _sz, _vp, _vp]),
    "hb200_gguf_open": (_int, [C.c_char_p, C.POINTER(_vp)]),
    "hb200_gguf_close": (_int, [_vp]),
    "hb200_gguf_version": (C.c_uint32, [_vp]),
    "hb200_gguf_data_offset": (C.c_uint64, [_vp]),
    "hb200_gguf_tensor_count": (_sz, [_vp]),
    "hb200_gguf_tensor_info": (_int, [_vp, _sz, C.POINTER(C.c_char_p), C.POINTER(_int), C.POINTER(_sz), C.POINTER(C.c_uint64),
                                      C.POINTER(C.c_uint64), C.POINTER(_sz)]),
    "hb200_gguf_find_tensor": (_int, [_vp, C.c_char_p, C.POINTER(_sz)]),
    "hb200_gguf_tensor_data": (_int, [_vp, _sz, C.POINTER(_vp), C.POINTER(_sz)]),
    "hb200_gguf_upload_tensor": (_int, [_vp, _sz, C.POINTER(_vp)]),
    "hb200_gguf_meta_u64": (_int, [_vp, C.c_char_p, C.POINTER(C.c_uint64)]),
    "hb200_gguf_meta_f64": (_int, [_vp, C.c_char_p, C.POINTER(C.c_double)]),
    "hb200_gguf_meta_str": (_int, [_vp, C.c_char_p, C.POINTER(C.c_char_p), C.POINTER(_sz)]),
    "hb200_gguf_meta_array_f32": (_int, [_vp, C.c_char_p, _vp, _sz, C.POINTER(_sz)]),
    "hb200_quantize_q8_0": (_int, [_vp, _sz, _sz, _vp]),
    "hb200_rms_norm_q8": (_int, [_vp, _vp, C.c_float, _vp, _sz, _sz]),
    "hb200_silu_mul_q8": (_int, [_vp, _vp, _vp, _sz, _sz]),
    "hb200_hadamard_quantize_q8_0": (_int, [_vp, _vp, _sz, _vp, _vp, _sz, _sz]),
    "hb200_dot_rows": (_int, [_vp, _vp, _vp]),
    "hb200_dot_rows_batched": (_int, [_vp, _vp, _sz, _sz, _vp]),
    "hb200_matmul_f32": (_int, [_vp, _vp, _sz, _vp]),
    "hb200_matmul_f32_fused": (_int, [C.POINTER(_vp), _sz, _vp, _sz, C.POINTER(_vp)]),
    "hb200_block_dots_i32": (_int, [_vp, _vp, _sz, _sz, _vp]),
    "hb200_dot_rows_dev": (_int, [_vp, _vp, _sz, _vp, _sz, _vp]),
    "hb200_matmul_f32_dev": (_int, [_vp, _vp, _sz, _vp, _sz, _vp]),
    "hb200_matmul_f32_noalloc": (_int, [_vp, _vp, _sz, _vp, _sz, _vp]),
    "hb200_batch_create": (_int, [C.POINTER(_vp)]),
    "hb200_batch_add": (_int, [_vp, _vp, _vp, _sz, _vp, _sz]),
    "hb200_batch_seal": (_int, [_vp]),
    "hb200_batch_launch": (_int, [_vp, _vp]),
    "hb200_batch_free": (_int, [_vp]),
    "hb200_multi_batch_launch": (_int, [C.POINTER(_vp), _int, C.POINTER(_vp)]),
    "hb200_batch_launch_count": (_int, [_vp]),
    "hb200_batch_run_host": (_int, [_vp, _vp, _vp, _sz, _vp]),
    "hb200_batch_run_dev": (_int, [_vp, _vp, _vp, _vp, _sz, _vp]),
    "hb200_batch_input_floats": (_sz, [_vp]),
    "hb200_peer_alloc": (_int, [_sz, C.POINTER(_vp), _vp]),
    "hb200_peer_free": (_int, [_vp]),
    "hb200_peer_open": (_int, [_vp, C.POINTER(_vp)]),
    "hb200_peer_close": (_int, [_vp]),
    "hb200_batch_set_peers": (_int, [_vp, _int, _int, C.POINTER(_vp), _sz, _int]),
    "hb200_batch_peer_area": (_int, [_vp]),
    "hb200_check_status": (_int, []),
    "hb200_stream_synchronize": (_int, [_vp]),
}


class Hb200Error(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"{STATUS.get(code, code)}: {message}")
        self.code = code
        self.message = message


_lib = None


def load() -> C.CDLL:
    """Load the library and bind every declared symbol; raises if anything is missing."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m hearth_b200.build` (nvcc, sm_100a). "
            "There is no CPU or PyTorch fallback for this path.")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        try:
            fn = getattr(lib, name)
        except AttributeError as e:
            raise ImportError(f"{LIB_PATH} does not export {name}") from e
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(code: int) -> None:
    if code != 0:
        raise Hb200Error(code, load().hb200_last_error().decode("utf-8", "replace"))
