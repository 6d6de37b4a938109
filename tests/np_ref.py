"""A second, independent restatement of the scalar arithmetic in numpy.

Its only job is to cross-check the C oracle (two implementations written
separately, from the same reference lines, must agree bit for bit).  Loops are
per block, so keep inputs small.
"""
from __future__ import annotations

import numpy as np

f32 = np.float32


def h2f(lo_hi: np.ndarray) -> np.float32:
    return np.frombuffer(bytes(lo_hi[:2]), dtype="<f2")[0].astype(f32)


def quantize_q8_0(x: np.ndarray) -> np.ndarray:
    """hearth-quant/src/q8_0.rs:20-51."""
    x = np.asarray(x, dtype=f32)
    n = x.size
    nb = (n + 31) // 32
    out = np.zeros(nb * 34, dtype=np.uint8)
    for b in range(nb):
        blk = x[b * 32:min(n, b * 32 + 32)]
        a = np.abs(blk)
        a = a[~np.isnan(a)]
        max_abs = f32(a.max()) if a.size else f32(0)
        scale = f32(1.0) if max_abs == 0 else f32(max_abs / f32(127.0))
        out[b * 34:b * 34 + 2] = np.frombuffer(np.float16(scale).tobytes(), dtype=np.uint8)
        with np.errstate(all="ignore"):
            r = (blk / scale).astype(f32).astype(np.float64)  # the f32 quotient, held exactly
            r = np.where(np.isnan(r), 0.0, np.copysign(np.floor(np.abs(r) + 0.5), r))  # half away from zero
            q = np.clip(r, -128, 127).astype(np.int8)
        out[b * 34 + 2:b * 34 + 2 + blk.size] = q.view(np.uint8)
    return out


def _q1_signs(bits16: np.ndarray) -> np.ndarray:
    b = np.unpackbits(bits16.astype(np.uint8), bitorder="little")
    return np.where(b == 1, 1, -1).astype(np.int32)


def _q2_vals(qs32: np.ndarray) -> np.ndarray:
    q = qs32.astype(np.uint8)
    codes = np.stack([(q >> (2 * j)) & 3 for j in range(4)], axis=1).reshape(-1)
    return codes.astype(np.int32) - 1


def dot_q8x(kind: str, w: np.ndarray, a: np.ndarray, n: int):
    """Scalar-order dot; returns (f32 result, int32 sub-block dots).
    kind: 'q1' (q1_0g128.rs:1019-1052), 'q2' (q2_0.rs:537-574), 'q8' (q8_0.rs:154-171)."""
    ints = []
    if kind == "q8":
        sumf = f32(0)
        for b in range(n // 32):
            d0, d1 = h2f(w[b * 34:]), h2f(a[b * 34:])
            wi = w[b * 34 + 2:b * 34 + 34].view(np.int8).astype(np.int32)
            ai = a[b * 34 + 2:b * 34 + 34].view(np.int8).astype(np.int32)
            s = int((wi * ai).sum())
            ints.append(s)
            sumf = f32(sumf + f32(f32(f32(s) * d0) * d1))
        return sumf, np.array(ints, dtype=np.int32)
    bb = 18 if kind == "q1" else 34
    total = f32(0)
    for b in range(n // 128):
        ws = h2f(w[b * bb:])
        vals = _q1_signs(w[b * bb + 2:b * bb + 18]) if kind == "q1" else _q2_vals(w[b * bb + 2:b * bb + 34])
        acc = f32(0)
        for s in range(4):
            ab = a[(b * 4 + s) * 34:(b * 4 + s + 1) * 34]
            ai = ab[2:].view(np.int8).astype(np.int32)
            d = int((vals[s * 32:s * 32 + 32] * ai).sum())
            ints.append(d)
            acc = f32(acc + f32(f32(d) * h2f(ab)))
        total = f32(total + f32(acc * ws))
    return total, np.array(ints, dtype=np.int32)


def hadamard_rotate(x: np.ndarray, signs, block_size: int) -> np.ndarray:
    """Independent float32 restatement of qwen35.rs:49-87 for one row (vectorised butterflies)."""
    v = np.array(x, dtype=np.float32, copy=True)
    if signs is not None:
        v = (v * np.asarray(signs, dtype=np.float32)).astype(np.float32)
    n_whole = (v.size // block_size) * block_size if block_size else 0
    if n_whole:
        blk = v[:n_whole].reshape(-1, block_size)
        h = 1
        while h < block_size:
            t = blk.reshape(blk.shape[0], block_size // (2 * h), 2, h)
            a, b = t[:, :, 0, :].copy(), t[:, :, 1, :].copy()
            t[:, :, 0, :] = a + b
            t[:, :, 1, :] = a - b
            h *= 2
        s = np.float32(1.0) / np.sqrt(np.float32(block_size))
        v[:n_whole] = (blk * np.float32(s)).reshape(-1)
    return v


def rms_norm_values(x: np.ndarray, weight: np.ndarray, eps: float) -> np.ndarray:
    """f64 normed values of ops::rms_norm_q8 (for tolerance checks, not bit parity)."""
    x64 = x.astype(np.float64)
    inv = 1.0 / np.sqrt((x64 * x64).mean() + eps)
    return weight.astype(np.float64) * x64 * inv


def dequantize_q8_0(q8: np.ndarray, n: int) -> np.ndarray:
    blocks = q8.reshape(-1, 34)
    d = blocks[:, :2].copy().view(np.float16).astype(np.float32)
    return (d * blocks[:, 2:].view(np.int8).astype(np.float32)).reshape(-1)[:n]
