"""Seeded synthetic weights and activations in the reference's byte layouts.

Stand-ins for the Bonsai GGUF tensors the reference benchmarks (no model file
is available offline): same shapes, block formats and value distributions.
numpy versions feed the parity tests; the torch versions build the multi-GB
benchmark layer sets directly in device memory.

Layouts (all little-endian):
  Q1_0 / Q1_0_G128  18 B per 128 columns: [f16 d][16 B sign bits, LSB first]   hearth-quant/src/q1_0g128.rs:76-98
  Q2_0 / PQ2_0      34 B per 128: [f16 d][32 B, four 2-bit codes per byte]      hearth-quant/src/q2_0.rs:9-23
  Q8_0              34 B per 32:  [f16 d][32 x i8]                              hearth-quant/src/q8_0.rs:4-18
  Q4_K (Hearth)     144 B per 256: [f16 d][f16 dmin][12 B scales][128 B nibbles] hearth-quant/src/q4_k.rs:9-49
  Q6_K (Hearth)     210 B per 256: [128 B ql][64 B qh][16 x i8 scales][f16 d]    hearth-quant/src/qk_quant.rs:102-137
"""
from __future__ import annotations

import numpy as np

from .lib import PQ2_0, PTQ1_0, Q1_0, Q1_0_G128, Q2_0, Q4_K, Q6_K, Q8_0

_BLOCK = {Q1_0: (128, 18), Q1_0_G128: (128, 18), 39: (128, 18), Q2_0: (128, 34), PQ2_0: (128, 34), Q8_0: (32, 34), PTQ1_0: (128, 28),
          Q4_K: (256, 144), Q6_K: (256, 210)}


def row_bytes(dtype: int, n_cols: int) -> int:
    bs, bb = _BLOCK[dtype]
    return (n_cols + bs - 1) // bs * bb


def _rng(seed: int) -> np.random.Generator:
    return np.random.Generator(np.random.PCG64(seed))


def _f16_bytes(vals: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(vals.astype(np.float16)).view(np.uint8).reshape(vals.shape + (2,))


def weights(dtype: int, n_rows: int, n_cols: int, seed: int, *, allow_code3: bool = False) -> np.ndarray:
    """uint8 [n_rows, row_bytes] of one weight tensor."""
    g = _rng(seed)
    bs, bb = _BLOCK[dtype]
    nb = (n_cols + bs - 1) // bs
    out = np.zeros((n_rows, nb, bb), dtype=np.uint8)
    if dtype in (Q1_0, Q1_0_G128, 39):
        out[:, :, 0:2] = _f16_bytes(np.abs(g.normal(0.0, 0.02, (n_rows, nb))))
        out[:, :, 2:] = g.integers(0, 256, (n_rows, nb, 16), dtype=np.uint8)
    elif dtype in (Q2_0, PQ2_0):
        out[:, :, 0:2] = _f16_bytes(np.abs(g.normal(0.0, 0.02, (n_rows, nb))))
        # codes 0/1/2 with P = 77/256, 102/256, 77/256 (0.30 / 0.40 / 0.30 to within 0.1 %), from one byte each;
        # allow_code3 also emits the code 3 (+2) that real files do not use but the kernels must handle.
        u = g.integers(0, 256, (n_rows, nb, 32, 4), dtype=np.uint8)
        t0, t1, t2 = (72, 174, 246) if allow_code3 else (77, 179, 256)
        codes = (u >= t0).astype(np.uint8) + (u >= t1).astype(np.uint8) + (u.astype(np.uint16) >= t2).astype(np.uint8)
        out[:, :, 2:] = codes[..., 0] | (codes[..., 1] << 2) | (codes[..., 2] << 4) | (codes[..., 3] << 6)
    elif dtype == PTQ1_0:
        # digits 0/1/2 (weights -1/0/+1) with P = 0.30/0.40/0.30, packed as the reference's own packer does
        # (hearth-quant/src/ptq1_0.rs:604-646): Q = sum of digit * 3^k, most significant first, byte = ceil(256 Q / 243).
        out[:, :, 26:28] = _f16_bytes(np.abs(g.normal(0.0, 0.02, (n_rows, nb))))
        u = g.integers(0, 256, (n_rows, nb, 26, 5), dtype=np.uint8)
        dig = (u >= 77).astype(np.uint16) + (u >= 179).astype(np.uint16)
        qv = np.zeros((n_rows, nb, 26), dtype=np.uint16)
        for k in range(5):
            use = dig[..., k] if k < 4 else np.concatenate([dig[..., :24, 4], np.zeros((n_rows, nb, 2), np.uint16)], axis=2)
            qv = qv * 3 + use  # the two qh bytes carry four digits and a trailing zero
        out[:, :, 0:26] = ((qv * 256 + 242) // 243).astype(np.uint8)
    elif dtype == Q8_0:
        out[:, :, 0:2] = _f16_bytes(np.abs(g.normal(0.0, 0.02, (n_rows, nb))) / 127.0 + 1e-6)
        out[:, :, 2:] = g.integers(-127, 128, (n_rows, nb, 32)).astype(np.int8).view(np.uint8)
    elif dtype == Q4_K:
        out[:, :, 0:2] = _f16_bytes(np.abs(g.normal(0.0, 0.01, (n_rows, nb))))
        out[:, :, 2:4] = _f16_bytes(np.abs(g.normal(0.0, 0.01, (n_rows, nb))))
        out[:, :, 4:] = g.integers(0, 256, (n_rows, nb, 140), dtype=np.uint8)
    elif dtype == Q6_K:
        out[:, :, 0:208] = g.integers(0, 256, (n_rows, nb, 208), dtype=np.uint8)
        out[:, :, 208:210] = _f16_bytes(np.abs(g.normal(0.0, 0.01, (n_rows, nb))))
    else:
        raise ValueError(f"dtype {dtype}")
    return out.reshape(n_rows, nb * bb)


def activations(seq_len: int, n_cols: int, seed: int) -> np.ndarray:
    """f32 [seq_len, n_cols] ~ N(0, 1)."""
    return _rng(seed).normal(0.0, 1.0, (seq_len, n_cols)).astype(np.float32)


# ---- torch (device) generators for the benchmark -------------------------------------------------

def weights_torch(dtype: int, n_rows: int, n_cols: int, seed: int, device):
    """uint8 CUDA tensor [n_rows * row_bytes] in the reference layout, generated on the device."""
    import torch

    g = torch.Generator(device=device)
    g.manual_seed(seed)
    bs, bb = _BLOCK[dtype]
    nb = (n_cols + bs - 1) // bs
    out = torch.empty((n_rows, nb, bb), dtype=torch.uint8, device=device)

    def f16_bytes(std):
        v = torch.empty((n_rows, nb), dtype=torch.float32, device=device).normal_(0.0, std, generator=g).abs_()
        return v.to(torch.float16).view(torch.uint8).reshape(n_rows, nb, 2)

    if dtype in (Q1_0, Q1_0_G128, 39):
        out[:, :, 0:2] = f16_bytes(0.02)
        out[:, :, 2:] = torch.randint(0, 256, (n_rows, nb, 16), dtype=torch.uint8, device=device, generator=g)
    elif dtype in (Q2_0, PQ2_0):
        out[:, :, 0:2] = f16_bytes(0.02)
        packed = torch.zeros((n_rows, nb, 32), dtype=torch.uint8, device=device)
        for j in range(4):
            u = torch.rand((n_rows, nb, 32), device=device, generator=g)
            code = (u >= 0.3).to(torch.uint8) + (u >= 0.7).to(torch.uint8)  # P = 0.3 / 0.4 / 0.3
            packed |= code << (2 * j)
            del u, code
        out[:, :, 2:] = packed
    elif dtype == PTQ1_0:
        # every byte value decodes to valid base-3 digits (ptq1_0.rs:22-57), so uniform bytes are legal blocks
        out[:, :, 0:26] = torch.randint(0, 256, (n_rows, nb, 26), dtype=torch.uint8, device=device, generator=g)
        out[:, :, 26:28] = f16_bytes(0.02)
    elif dtype == Q8_0:
        v = torch.empty((n_rows, nb), dtype=torch.float32, device=device).normal_(0.0, 0.02, generator=g).abs_() / 127.0 + 1e-6
        out[:, :, 0:2] = v.to(torch.float16).view(torch.uint8).reshape(n_rows, nb, 2)
        out[:, :, 2:] = torch.randint(0, 256, (n_rows, nb, 32), dtype=torch.uint8, device=device, generator=g)
    elif dtype == Q4_K:
        out[:, :, 0:2] = f16_bytes(0.01)
        out[:, :, 2:4] = f16_bytes(0.01)
        out[:, :, 4:] = torch.randint(0, 256, (n_rows, nb, 140), dtype=torch.uint8, device=device, generator=g)
    elif dtype == Q6_K:
        out[:, :, 0:208] = torch.randint(0, 256, (n_rows, nb, 208), dtype=torch.uint8, device=device, generator=g)
        out[:, :, 208:210] = f16_bytes(0.01)
    else:
        raise ValueError(f"dtype {dtype}")
    return out.reshape(-1)


# ---- benchmark configurations ---------------------------------------------------------------------

def layer_shapes(d_model: int, ffn: int, kv: int) -> list[tuple[str, int, int]]:
    """(name, n_rows, n_cols) of the seven projections of one transformer layer."""
    return [("q", d_model, d_model), ("k", kv, d_model), ("v", kv, d_model), ("o", d_model, d_model),
            ("gate", ffn, d_model), ("up", ffn, d_model), ("down", d_model, ffn)]


CONFIGS = {
    # name: dtype, layer shapes, layers, tokens
    "c0_q1_single": dict(dtype=Q1_0, shapes=[("up", 6144, 2048)], layers=1, seq_len=1),
    # the same matvec over 160 distinct copies of the weight (283 MB, more than twice the L2) in one launch: the way to
    # time an operation that is shorter than a kernel launch and L2-resident when repeated
    "c0_q1_single_x160": dict(dtype=Q1_0, shapes=[("up", 6144, 2048)], layers=160, seq_len=1),
    # Q8_0 weights at the 1.7B shapes (the reference's scalar dot_q8_0_q8_0, hearth-quant/src/q8_0.rs:154-171)
    "c1_q8_1p7b_decode": dict(dtype=Q8_0, shapes=layer_shapes(2048, 6144, 1024), layers=28, seq_len=1),
    "c1_q2_1p7b_decode": dict(dtype=Q2_0, shapes=layer_shapes(2048, 6144, 1024), layers=28, seq_len=1),
    "c1_q1_1p7b_decode": dict(dtype=Q1_0, shapes=layer_shapes(2048, 6144, 1024), layers=28, seq_len=1),
    "c2_q1_8b_prefill": dict(dtype=Q1_0, shapes=layer_shapes(4096, 12288, 1024), layers=36, seq_len=512),
    "c2_q1_8b_prefill_1layer": dict(dtype=Q1_0, shapes=layer_shapes(4096, 12288, 1024), layers=1, seq_len=512),
    "c2_q1_8b_decode": dict(dtype=Q1_0, shapes=layer_shapes(4096, 12288, 1024), layers=36, seq_len=1),
    "c2_q2_8b_decode": dict(dtype=Q2_0, shapes=layer_shapes(4096, 12288, 1024), layers=36, seq_len=1),
    # config 3: K-quant decode matvec, f32 activations; eight copies of the pair so a step streams 5x the L2
    "c3_q4k_m1": dict(dtype=Q4_K, shapes=[("a", 14336, 4096), ("b", 4096, 14336)], layers=8, seq_len=1),
    "c3_q4k_m8": dict(dtype=Q4_K, shapes=[("a", 14336, 4096), ("b", 4096, 14336)], layers=8, seq_len=8),
    "c3_q4k_m32": dict(dtype=Q4_K, shapes=[("a", 14336, 4096), ("b", 4096, 14336)], layers=8, seq_len=32),
    "c3_q6k_m1": dict(dtype=Q6_K, shapes=[("a", 14336, 4096), ("b", 4096, 14336)], layers=8, seq_len=1),
    "c3_q6k_m8": dict(dtype=Q6_K, shapes=[("a", 14336, 4096), ("b", 4096, 14336)], layers=8, seq_len=8),
    "c3_q6k_m32": dict(dtype=Q6_K, shapes=[("a", 14336, 4096), ("b", 4096, 14336)], layers=8, seq_len=32),
    "c4_pq2_27b_decode": dict(dtype=PQ2_0, shapes=layer_shapes(5120, 17408, 1024), layers=64, seq_len=1),
    "c4_ptq1_27b_decode": dict(dtype=PTQ1_0, shapes=layer_shapes(5120, 17408, 1024), layers=64, seq_len=1),
    "c4_pq2_27b_m4": dict(dtype=PQ2_0, shapes=layer_shapes(5120, 17408, 1024), layers=64, seq_len=4),
    "c4_pq2_27b_m8": dict(dtype=PQ2_0, shapes=layer_shapes(5120, 17408, 1024), layers=64, seq_len=8),
    "c4_pq2_27b_m16": dict(dtype=PQ2_0, shapes=layer_shapes(5120, 17408, 1024), layers=64, seq_len=16),
    "c4_pq2_27b_m32": dict(dtype=PQ2_0, shapes=layer_shapes(5120, 17408, 1024), layers=64, seq_len=32),
    "c4_pq2_27b_m32_2layers": dict(dtype=PQ2_0, shapes=layer_shapes(5120, 17408, 1024), layers=2, seq_len=32),
    "c2_q1_8b_m8": dict(dtype=Q1_0, shapes=layer_shapes(4096, 12288, 1024), layers=36, seq_len=8),
    "c2_q1_8b_m32": dict(dtype=Q1_0, shapes=layer_shapes(4096, 12288, 1024), layers=36, seq_len=32),
}


def config_weight_bytes(name: str) -> int:
    c = CONFIGS[name]
    return c["layers"] * sum(r * row_bytes(c["dtype"], k) for _, r, k in c["shapes"])
