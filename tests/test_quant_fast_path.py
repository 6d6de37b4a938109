"""The Q8_0 quantizer's division-free path (hearth_b200/csrc/quantize_core.cuh, quant_fast) restated in numpy float32 and
compared with the reference arithmetic (q8_0::quantize_into, hearth-quant/src/q8_0.rs:20-51: q = clamp(round-half-away(
x / scale))) on inputs aimed at the rounding boundaries.  The device takes the fast result only when t = x * inv is at least
2^-13 away from every k + 0.5; this test checks that whenever that condition holds the fast result equals the reference's,
for a reciprocal that is off by up to one ulp in either direction (the stated error of rcp.approx).  Runs without a GPU."""
import numpy as np

F = np.float32


def reference_q(x, scale):
    r = (x / scale).astype(F)  # IEEE division, rounded to fp32
    q = np.where(r >= 0, np.floor(r.astype(np.float64) + 0.5), np.ceil(r.astype(np.float64) - 0.5))  # half away from zero
    return np.clip(q, -128, 127).astype(np.int32)


def fast_q(x, inv):
    t = (x * inv).astype(F)
    y = (np.abs(t) - F(0.5)).astype(F)
    dist = np.abs((y - np.rint(y).astype(F)).astype(F))
    ok = dist >= F(0.0001220703125)
    return ok, np.rint(t).astype(np.int32)


def check(scale, x):
    scale = scale.astype(F)
    x = x.astype(F)
    inv0 = (F(1.0) / scale).astype(F)
    want = reference_q(x, scale)
    for inv in (inv0, np.nextafter(inv0, F(np.inf)), np.nextafter(inv0, F(0))):
        ok, got = fast_q(x, inv.astype(F))
        bad = ok & (got != want)
        assert not bad.any(), (scale[bad][:3], x[bad][:3], got[bad][:3], want[bad][:3])
    return float(np.mean(~fast_q(x, inv0)[0]))


def test_fast_path_agrees_wherever_it_is_taken():
    rng = np.random.Generator(np.random.PCG64(2024))
    n = 2_000_000
    # scales over the whole range the device admits (1e-30 .. 1e30), the block maximum is 127 * scale up to rounding
    scale = np.exp(rng.uniform(np.log(1e-30), np.log(1e30), n)).astype(F)
    amax = (scale * F(127)).astype(F)
    scale = (amax / F(127)).astype(F)
    # (a) uniformly inside the block's range
    x = (rng.uniform(-1, 1, n) * amax).astype(F)
    slow = check(scale, x)
    assert 0.0 < slow < 0.001, "the exact path should be rare on ordinary data, the fast one the rule"
    # (b) right at and a few ulps around every tie k + 0.5
    k = rng.integers(0, 127, n).astype(F) + F(0.5)
    base = (k * scale).astype(F) * np.where(rng.random(n) < 0.5, F(-1), F(1))
    for step in range(-6, 7):
        xx = base.copy()
        for _ in range(abs(step)):
            xx = np.nextafter(xx, F(np.inf) if step > 0 else F(-np.inf)).astype(F)
        check(scale, xx)
    # (c) the extremes of the block: +-amax and its neighbours
    for step in (-2, -1, 0):
        xx = amax.copy()
        for _ in range(-step):
            xx = np.nextafter(xx, F(0)).astype(F)
        check(scale, xx)
        check(scale, -xx)
    # (d) zeros and values far below the scale
    check(scale, np.zeros(n, dtype=F))
    check(scale, (scale * F(1e-6)).astype(F))
