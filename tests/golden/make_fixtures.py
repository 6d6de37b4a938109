"""Generates tests/golden/fixtures.npz.

Inputs are the deterministic fixtures of the reference's own unit tests,
re-created from their formulas (no reference code is executed: the reference is
Rust and no Rust toolchain exists here):

  x2 / single fixtures   hearth-quant/src/q1_0g128.rs:1504-1552, q2_0.rs:939-986
      weight byte  ((b*16 + j) * 37 ^ 0xAB) as u8   (Q1_0: 16 per block)
                   ((b*32 + j) * 37 ^ 0xAB) as u8   (Q2_0: 32 per block)
      weight scale f16(((b % 7) + 0.5) * 0.25)
      act scale    f16(((b % 5) + 0.5) * 0.125)
      act bytes    (b * salt * 2654435761) as u8, salt 53 / 97, constant inside a block
      n in {128, 256, 2048, 6144}
  Q8_0 round-trip input  (i - 32) * 0.5, i < 64                q8_0.rs:178-194
  Q2_0-vs-f32 fixture    scale 1.5 / 2.0, bytes (j*37)^0xAB, x = sin(0.13 i)   q2_0.rs:787-818
  benchk activation      ((i * 2654435761 mod 1000) / 500) - 1                 hearth-llm/examples/benchk.rs:165-169

Expected outputs are produced by the C oracle and accepted only if the numpy
restatement in tests/np_ref.py yields the same bits.  Run from the repo root:
    python tests/golden/make_fixtures.py
"""
from __future__ import annotations

import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from oracle import oracle as O  # noqa: E402
import np_ref  # noqa: E402


def f16b(v: float) -> np.ndarray:
    return np.frombuffer(np.float16(v).tobytes(), dtype=np.uint8)


def x2_fixture(kind: str, n: int):
    nb = n // 128
    bb, per = (18, 16) if kind == "q1" else (34, 32)
    w = np.zeros(nb * bb, dtype=np.uint8)
    for b in range(nb):
        w[b * bb:b * bb + 2] = f16b(((b % 7) + 0.5) * 0.25)
        for j in range(per):
            w[b * bb + 2 + j] = (((b * per + j) * 37) ^ 0xAB) & 0xFF
    acts = []
    for salt in (53, 97):
        a = np.zeros(nb * 4 * 34, dtype=np.uint8)
        for b in range(nb * 4):
            a[b * 34:b * 34 + 2] = f16b(((b % 5) + 0.5) * 0.125)
            a[b * 34 + 2:b * 34 + 34] = ((b * salt) & 0xFFFFFFFF) * 2654435761 & 0xFF
        acts.append(a)
    return w, acts


def main() -> None:
    out = {}
    for kind, dtype in (("q1", O.Q1_0_G128), ("q2", O.Q2_0)):
        for n in (128, 256, 2048, 6144):
            w, acts = x2_fixture(kind, n)
            out[f"x2_{kind}_{n}_w"] = w
            for t, a in enumerate(acts):
                got = O.dot_rows_batched(dtype, w, a, 1, n)[0, 0]
                ints = O.block_dots_i32(dtype, w, a, n)
                want, want_i = np_ref.dot_q8x(kind, w, a, n)
                assert np.float32(got).tobytes() == np.float32(want).tobytes(), (kind, n, t, got, want)
                assert (ints == want_i).all()
                assert abs(got) > 1e-6, "degenerate fixture"
                out[f"x2_{kind}_{n}_a{t}"] = a
                out[f"x2_{kind}_{n}_out{t}"] = np.float32(got)
                out[f"x2_{kind}_{n}_int{t}"] = ints

    src = ((np.arange(64, dtype=np.float32) - np.float32(32.0)) * np.float32(0.5)).astype(np.float32)
    q = O.quantize_q8_0(src)
    assert (q == np_ref.quantize_q8_0(src)).all()
    out["q8_roundtrip_src"] = src
    out["q8_roundtrip_q"] = q

    # benchk computes ((i*K % 1000) as f32 / 500.0) - 1.0 in f32
    benchk = (np.array([(i * 2654435761) % 1000 for i in range(2048)], dtype=np.float32) / np.float32(500.0)) - np.float32(1.0)
    qb = O.quantize_q8_0(benchk)
    assert (qb == np_ref.quantize_q8_0(benchk)).all()
    out["benchk_x"] = benchk
    out["benchk_q8"] = qb

    rng = np.random.Generator(np.random.PCG64(20240607))
    x = rng.normal(0, 1, 4096).astype(np.float32)
    x[17] = 0.0
    x[64:96] = 0.0                      # an all-zero block (scale 1.0)
    x[200] = np.float32(3.4e38)         # huge value: scale overflows f16 to inf
    x[300] = np.float32(1e-30)
    qx = O.quantize_q8_0(x)
    assert (qx == np_ref.quantize_q8_0(x)).all()
    out["quant_seeded_x"] = x
    out["quant_seeded_q8"] = qx

    w = np.zeros(68, dtype=np.uint8)
    for b in range(2):
        w[b * 34:b * 34 + 2] = f16b(1.5 if b == 0 else 2.0)
        for j in range(32):
            w[b * 34 + 2 + j] = ((j * 37) & 0xFF) ^ 0xAB
    xs = np.sin(np.arange(256, dtype=np.float32) * np.float32(0.13)).astype(np.float32)
    out["q2_vs_f32_w"] = w
    out["q2_vs_f32_x"] = xs

    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "fixtures.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes,", len(out), "arrays")


if __name__ == "__main__":
    main()
