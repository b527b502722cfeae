"""Arithmetic shortcuts of the Q4_0 kernels restated in numpy and checked on the CPU.  The tensor-core mat-mat
(csrc/pi_gemv_mma_q4.cu) relies on:

* operand order: the low nibbles of a block's 16 bytes pair with Q8_0 values 0..15, the high nibbles with 16..31, so one
  integer dot per block over (nibbles, int8) minus 8 x (sum of the int8) is the block term of vec_dot_q4_0_q8_0
  (ggml-quants.c:2586-2610); summed over the blocks in FP32 it must agree with the CPU checker's mat-vec;
* the integer-to-float trick: the word {FP16 scale | 0x8000 - 8 s} yields the mma's C operand 0x4B400000 | low half, and
  as_float(C + dot) - (12582912 + 32768) equals float(dot - 8 s) exactly for every reachable s and dot."""
import numpy as np

from oracle import pio
from powerinfer_b200 import synth

MAGIC = 0x4B400000
BIAS = np.float32(12582912.0 + 32768.0)


def test_magic_number_conversion_is_exact_over_the_whole_range():
    rng = np.random.default_rng(0)
    s = np.arange(-127 * 32, 127 * 32 + 1, dtype=np.int64)                       # every possible block sum of 32 int8
    low = (0x8000 - 8 * s) & 0xFFFF
    assert low.min() >= 0 and low.max() <= 0xFFFF and np.array_equal(low, 0x8000 - 8 * s)   # fits 16 bits, no wrap
    c_operand = MAGIC | low
    assert np.array_equal(c_operand, MAGIC + low)                                 # the OR is an add: the low mantissa bits are free
    for dot in (np.full_like(s, -15 * 127 * 32), np.full_like(s, 15 * 127 * 32), rng.integers(-15 * 127 * 32, 15 * 127 * 32 + 1, s.size)):
        acc = (c_operand + dot).astype(np.uint32)                                 # what the integer mma leaves in the accumulator
        got = acc.view(np.float32) - BIAS
        assert np.array_equal(got, (dot - 8 * s).astype(np.float32))
        assert np.all(np.abs(dot - 8 * s) < 2 ** 22)


def test_block_dot_operand_order_matches_the_cpu_dot():
    rng = np.random.default_rng(1)
    o = pio.Oracle()
    rows, cols, T = 24, 512, 3
    W = synth.quantize_q4_0(rng.standard_normal((rows, cols), dtype=np.float32) * np.float32(0.02))
    x = rng.standard_normal((T, cols), dtype=np.float32)
    ref = o.mul_mat(synth.Q4_0, W, rows, cols, x)                                 # CPU checker, the reference's lane order
    nb = cols // 32
    wb = W.reshape(rows, nb, 18)
    d4 = wb[:, :, :2].copy().view(np.float16).astype(np.float32)[:, :, 0]         # [rows, nb]
    qs = wb[:, :, 2:]
    lo_n, hi_n = (qs & 0x0F).astype(np.int32), (qs >> 4).astype(np.int32)         # values 0..15 | 16..31 of the block
    out = np.zeros((T, rows), np.float32)
    for t in range(T):
        q8 = o.quantize_q8_0(x[t]).reshape(nb, 34)
        d8 = q8[:, :2].copy().view(np.float16).astype(np.float32)[:, 0]           # [nb]
        v = q8[:, 2:].view(np.int8).astype(np.int32)                              # [nb, 32]
        s8 = v.sum(axis=1)
        dot = (lo_n * v[None, :, :16]).sum(axis=2) + (hi_n * v[None, :, 16:]).sum(axis=2)   # [rows, nb]: u8 x s8 -> s32
        term = (dot - 8 * s8[None, :]).astype(np.float32) * (d4 * d8[None, :])    # float(sumi) * (d4 * d8), as the CPU path
        acc = np.zeros(rows, np.float32)
        for b in range(nb):                                                       # FP32 accumulation over the blocks
            acc = acc + term[:, b]
        out[t] = acc
    assert np.abs(out - ref).max() <= 2e-5, np.abs(out - ref).max()


def test_batch_1_axpy_nibble_to_float_trick_costs_about_four_bits():
    """csrc/pi_sparse.cu (k_axpy_pipe, Q4_0 rows): nibble q becomes the float 0.5 + q/256 by one byte permute, the weight
    term is accumulated as (0.5 + q/256) * (256 c d) and 0.53125 * sum(256 c d) is subtracted once per column at the end.
    Restated in float32 (fma emulated through float64): the result stays within 5e-6 of sum |8 c d| of the exact sum."""
    rng = np.random.default_rng(0)

    def fmaf(a, b, c):
        return np.float32(np.float64(a) * np.float64(b) + np.float64(c))

    worst = 0.0
    for _ in range(200):
        n = int(rng.integers(1, 64))                                              # rows one CTA accumulates
        q = rng.integers(0, 16, n)
        c = (rng.standard_normal(n) * 0.5).astype(np.float32)                     # coefficient of the row
        d = np.float16(np.abs(rng.standard_normal(n)) * 0.01 + 1e-3).astype(np.float32)
        acc, corr = np.float32(0), np.float32(0)
        for i in range(n):
            sc = np.float32(np.float32(np.float32(256.0) * c[i]) * d[i])
            corr = np.float32(corr + sc)
            val = np.array([0x3F000000 | (int(q[i]) << 16)], np.uint32).view(np.float32)[0]
            assert val == np.float32(0.5 + q[i] / 256.0)
            acc = fmaf(val, sc, acc)
        acc = fmaf(np.float32(-0.53125), corr, acc)
        exact = np.sum((q - 8).astype(np.float64) * c.astype(np.float64) * d.astype(np.float64))
        scale = np.sum(np.abs(c.astype(np.float64) * d.astype(np.float64))) * 8
        worst = max(worst, abs(float(acc) - exact) / scale)
    assert worst <= 5e-6, worst
