"""Arithmetic facts the tensor-core GEMM kernel (kronos-2t_b200/csrc/k2t_gemm_tc.cu) relies on, checked on the CPU.

Its epilogue turns the int32 chunk dot d into a float without a conversion instruction: the integer add
`0x4B400000 + d` is reinterpreted as a float (1.5 * 2^23 + d exactly, while |d| < 2^22) and 12582912.0f is subtracted,
which must give (float)d exactly - the value `sdot_one_stripe_neon` (src/kernels/simd_lut.rs:3763-3868) feeds its fma chain.
For bit-plane matrices the same add also folds the correction: d = 2a - (2^B - 1) * xsum."""
import numpy as np

MAGIC_I = 0x4B400000
MAGIC_F = np.float32(12582912.0)


def via_magic(d):
    bits = (np.int64(MAGIC_I) + d.astype(np.int64)).astype(np.uint32)
    return bits.view(np.float32) - MAGIC_F


def test_magic_constant_is_one_and_a_half_times_two_to_the_23():
    assert np.array([MAGIC_I], np.uint32).view(np.float32)[0] == MAGIC_F == np.float32(1.5 * 2 ** 23)


def test_magic_conversion_is_exact_over_the_whole_range_of_chunk_dots():
    # every value near the ends and a dense sample in between; |d| < 2^22 is the range the trick covers
    lim = 2 ** 22
    d = np.concatenate([np.arange(-lim + 1, -lim + 70000), np.arange(-70000, 70000), np.arange(lim - 70000, lim),
                        np.random.Generator(np.random.PCG64(1)).integers(-lim + 1, lim, 2_000_000)]).astype(np.int64)
    assert np.array_equal(via_magic(d), d.astype(np.float32))
    assert np.all(d.astype(np.float32).astype(np.int64) == d)          # and (float)d is itself exact there


def test_chunk_dots_of_every_format_stay_inside_the_exact_range():
    # 64 columns, int8 activations in [-127, 127] (the quantizer never emits -128), xsum = sum of the chunk's activations
    worst = {}
    for planes in (4, 5, 6):                      # codes 0 .. 2^B - 1, dot = 2a - (2^B - 1) * xsum = sum((2u - (2^B - 1)) q)
        worst[f"b{planes}"] = 64 * (2 ** planes - 1) * 127
    for name, cmax in (("nf", 127), ("e8q2", 0x60)):      # signed centroids up to 127; E8Q2 magnitudes up to 96
        worst[name] = 64 * cmax * 127
    assert max(worst.values()) < 2 ** 22, worst
    # the two terms of the bit-plane form separately (the kernel adds them in one integer multiply-add)
    assert 2 * 64 * 63 * 127 + 63 * 64 * 127 < 2 ** 31


def test_correction_folded_into_the_constant_equals_the_reference_form():
    rng = np.random.Generator(np.random.PCG64(7))
    for planes in (4, 5, 6):
        max_odd = 2 ** planes - 1
        u = rng.integers(0, max_odd + 1, (4096, 64))
        q = rng.integers(-127, 128, (4096, 64))
        a = (u * q).sum(1)
        xsum = q.sum(1)
        dot = 2 * a - max_odd * xsum                                   # reference: exact int32
        bias = np.int64(MAGIC_I) - max_odd * xsum                      # the kernel's per-(chunk, token) constant
        got = ((2 * a + bias).astype(np.uint32)).view(np.float32) - MAGIC_F
        assert np.array_equal(got, dot.astype(np.float32))
