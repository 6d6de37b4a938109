"""A minimal GGUF writer for the tests (the format hearth-gguf/src/gguf.rs:137-224 reads): header, metadata
key/values of every GGUF value type, tensor infos, aligned data section."""
from __future__ import annotations

import struct

import numpy as np

T_U8, T_I8, T_U16, T_I16, T_U32, T_I32, T_F32, T_BOOL, T_STR, T_ARR, T_U64, T_I64, T_F64 = range(13)
_FMT = {T_U8: "<B", T_I8: "<b", T_U16: "<H", T_I16: "<h", T_U32: "<I", T_I32: "<i", T_F32: "<f", T_BOOL: "<B", T_U64: "<Q",
        T_I64: "<q", T_F64: "<d"}


def _s(text: str) -> bytes:
    b = text.encode()
    return struct.pack("<Q", len(b)) + b


def _value(t: int, v) -> bytes:
    if t == T_STR:
        return _s(v)
    if t == T_ARR:
        et, items = v
        return struct.pack("<IQ", et, len(items)) + b"".join(_value(et, x) for x in items)
    return struct.pack(_FMT[t], v)


def write_gguf(path: str, meta: list[tuple[str, int, object]], tensors: list[tuple[str, list[int], int, np.ndarray]],
               version: int = 3, alignment: int | None = None) -> dict:
    """tensors: (name, shape innermost-first, dtype id, uint8 payload).  Returns each tensor's offset in the data section."""
    align = alignment or 32
    if alignment is not None:
        meta = list(meta) + [("general.alignment", T_U32, alignment)]
    out = bytearray(b"GGUF" + struct.pack("<IQQ", version, len(tensors), len(meta)))
    for key, t, v in meta:
        out += _s(key) + struct.pack("<I", t) + _value(t, v)
    offsets, off = {}, 0
    for name, shape, dt, payload in tensors:
        off = (off + align - 1) // align * align
        offsets[name] = off
        out += _s(name) + struct.pack("<I", len(shape)) + b"".join(struct.pack("<Q", d) for d in shape)
        out += struct.pack("<IQ", dt, off)
        off += payload.size
    if version == 3:
        out += b"\0" * ((align - len(out) % align) % align)
    base = len(out)
    for name, _, _, payload in tensors:
        out += b"\0" * (base + offsets[name] - len(out))
        out += payload.tobytes()
    with open(path, "wb") as f:
        f.write(out)
    return dict(offsets=offsets, data_offset=base)
