"""The integer identity behind the Q2_0 one-token decode kernel's fourth accumulator (hearth_b200/csrc/gemv_dp4a.cu,
round_terms): a lane's word holds, per column byte, the 2-bit codes of its four rows (row g at bits 2g..2g+1), so

    dp4a(word, a) = S_0 + 4 S_1 + 16 S_2 + 64 S_3,      S_g = sum_i a_i * code_g,i

and the kernel takes the fourth row's 64 S_3 as dp4a(word, a) minus the three masked dots, every accumulator biased by
MAGIC_I and the total started at 4 * MAGIC_I modulo 2^32.  Checked here with numpy on random and extreme sub-blocks
(32 columns = 8 words), in the same modular 32-bit arithmetic."""
import numpy as np

MAGIC_I = 0x4B400000
MAGIC_F = np.float32(12582912.0)


def dp4a_u8s8(word, a4):
    b = np.array([(int(word) >> (8 * k)) & 0xFF for k in range(4)], dtype=np.int64)
    return int((b * a4.astype(np.int64)).sum())


def sub_block(words, a):
    """Returns what the kernel's four accumulators hold after one 32-column sub-block (as unsigned 32-bit)."""
    acc = [MAGIC_I, MAGIC_I, MAGIC_I, (4 * MAGIC_I) & 0xFFFFFFFF]
    for j, w in enumerate(words):
        a4 = a[4 * j:4 * j + 4]
        for g in range(3):
            acc[g] = (acc[g] + dp4a_u8s8(int(w) & (0x03030303 << (2 * g)), a4)) & 0xFFFFFFFF
        acc[3] = (acc[3] + dp4a_u8s8(int(w), a4)) & 0xFFFFFFFF
    acc[3] = (acc[3] - acc[0] - acc[1] - acc[2]) & 0xFFFFFFFF
    return acc


def check(codes, a):
    # codes[g][i]: code of row g, column i
    words = []
    for j in range(8):
        w = 0
        for k in range(4):
            byte = sum(int(codes[g][4 * j + k]) << (2 * g) for g in range(4))
            w |= byte << (8 * k)
        words.append(w)
    acc = sub_block(words, a)
    for g in range(4):
        s = int((codes[g].astype(np.int64) * a.astype(np.int64)).sum())
        assert acc[g] == (MAGIC_I + (4 ** g) * s) & 0xFFFFFFFF
        # the widening: as_float(acc) - MAGIC_F is the exact float of 4^g * S_g
        f = np.array([acc[g]], dtype=np.uint32).view(np.float32)[0]
        assert np.float32(f - MAGIC_F) == np.float32((4 ** g) * s)


def test_random_sub_blocks():
    rng = np.random.default_rng(7)
    for _ in range(200):
        check(rng.integers(0, 4, size=(4, 32)), rng.integers(-127, 128, size=32).astype(np.int8))


def test_extreme_sub_blocks():
    for code in (0, 3):
        for av in (-127, 127):
            check(np.full((4, 32), code), np.full(32, av, dtype=np.int8))
    codes = np.zeros((4, 32), dtype=np.int64)
    codes[3] = 3  # only the unmasked row is non-zero
    check(codes, np.full(32, -127, dtype=np.int8))
    codes = np.full((4, 32), 3)
    codes[3] = 0  # the total is made of the other three rows alone
    check(codes, np.full(32, 127, dtype=np.int8))
