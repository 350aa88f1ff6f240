"""
Known answers for the CPU restatement of the rounding-on-store rules
(oracle/sround.py).  Everything here is hand-derivable from the kernel text it
restates (neon/backends/cuda_templates.py:189-358, float_ew.py:833-844,
944-1037), including the one case neon's own test holds for stochastic rounding
(tests/test_backend_sr.py:52-71: 1.0 + 0.1 stored at one mantissa bit is 1.0 or
1.5 and nothing else).
"""
import numpy as np

from oracle import sround

U32 = np.uint32


def test_mantissa_bit_selection():
    """float_ew.py:833-844: True means 10 bits, fp32 is capped at 15, fp16 at 10, never below 1."""
    assert sround.mantissa_bits(0, np.float16) == 0
    assert sround.mantissa_bits(False, np.float32) == 0
    assert sround.mantissa_bits(True, np.float16) == 10
    assert sround.mantissa_bits(True, np.float32) == 10
    assert sround.mantissa_bits(23, np.float32) == 15
    assert sround.mantissa_bits(12, np.float16) == 10
    assert sround.mantissa_bits(3, np.float16) == 3
    assert sround.mantissa_bits(1, np.float32) == 1


def test_one_mantissa_bit_case_of_the_reference_test():
    """1.1 with one kept mantissa bit lies between 1.0 and 1.5: the discarded fraction is
    0.2, so random words below 0.8 * 2^32 keep 1.0 and the rest give 1.5."""
    val = np.float32(np.float16(1.0)) + np.float32(np.float16(0.1))
    edge = int((1.5 - float(val)) / 0.5 * 2.0 ** 32)
    ur = np.array([0, 1 << 31, edge - 4096, edge + 4096, 0xFFFFFFFF], U32)
    got = sround.sr_f16(np.full(5, val, np.float32), ur, 1)
    assert got.dtype == np.float16
    assert got.tolist() == [1.0, 1.0, 1.0, 1.5, 1.5]
    # over uniformly spread random words the up-probability is the discarded fraction
    ur = (np.arange(1 << 16, dtype=np.uint64) << np.uint64(16)).astype(U32)
    got = sround.sr_f16(np.full(ur.size, val, np.float32), ur, 1)
    assert set(got.tolist()) == {1.0, 1.5}
    assert abs((got == 1.5).mean() - (float(val) - 1.0) / 0.5) < 1e-3
    # negative values round the magnitude the same way
    got = sround.sr_f16(np.full(2, -val, np.float32), np.array([0, 0xFFFFFFFF], U32), 1)
    assert got.tolist() == [-1.0, -1.5]


def test_representable_values_are_never_moved():
    vals = np.array([1.0, -2.5, 0.375, 1024.0, 0.0], np.float32)
    for ur in (0, 0x7FFFFFFF, 0xFFFFFFFF):
        u = np.full(vals.size, ur, U32)
        assert np.array_equal(sround.sr_f32(vals, u, 10), vals)
        assert np.array_equal(sround.sr_f16(vals, u, 10), vals.astype(np.float16))


def test_fp32_rounding_keeps_the_requested_bits():
    """1 + 2^-12 at 10 bits: the tail is 1/4 of a 10-bit ulp, so the top quarter of the
    random range rounds up to 1 + 2^-10; the low 13 mantissa bits are always clear."""
    val = np.float32(1.0 + 2.0 ** -12)
    ur = np.array([0, 0xBFFFFFFF - 8192, 0xC0000000 + 8192, 0xFFFFFFFF], U32)
    got = sround.sr_f32(np.full(4, val, np.float32), ur, 10)
    assert got.tolist() == [1.0, 1.0, 1.0 + 2.0 ** -10, 1.0 + 2.0 ** -10]
    rng = np.random.RandomState(0)
    v = rng.uniform(-100, 100, 4096).astype(np.float32)
    got = sround.sr_f32(v, rng.randint(0, 2 ** 32, 4096, dtype=np.uint64).astype(U32), 12)
    assert not (got.view(U32) & U32((1 << 11) - 1)).any()
    ulp = 2.0 ** (np.floor(np.log2(np.abs(v))) - 12)
    assert (np.abs(got.astype(np.float64) - v) <= ulp).all()
    assert (np.abs(got) >= np.abs(v) - ulp).all()


def test_integer_stores():
    """Nearest: round half to even, saturating (cvt.rni.sat).  Stochastic: a uniform fraction
    is added to the magnitude before truncation; unsigned types always round to nearest."""
    v = np.array([0.5, 1.5, 2.5, -0.5, -1.5, 300.0, -300.0, 126.7], np.float32)
    assert sround.nearest_int(v, np.int8).tolist() == [0, 2, 2, 0, -2, 127, -128, 127]
    assert sround.nearest_int(v, np.uint8).tolist() == [0, 2, 2, 0, 0, 255, 0, 127]
    assert sround.nearest_int(v, np.int16).tolist() == [0, 2, 2, 0, -2, 300, -300, 127]
    w = np.array([2.25, 2.25, -2.25, -2.25], np.float32)
    ur = np.array([0, 0xFFFFFFFF, 0, 0xFFFFFFFF], U32)
    assert sround.sr_int(w, ur, np.int32).tolist() == [2, 3, -2, -3]
    assert sround.sr_int(w, ur, np.uint8).tolist() == [2, 2, 0, 0]
    assert sround.store(w, np.int16, True, ur).tolist() == [2, 3, -2, -3]
    assert sround.store(w, np.int16).tolist() == [2, 2, -2, -2]


def test_nearest_float_stores():
    v = np.array([1.0 + 2.0 ** -11, 1.0 + 3 * 2.0 ** -11, 70000.0], np.float32)
    with np.errstate(over="ignore"):
        got = sround.store(v, np.float16)
    assert got[0] == 1.0 and got[1] == np.float16(1.0 + 2.0 ** -9) and np.isinf(got[2])
    assert np.array_equal(sround.store(v, np.float32), v)


def test_generator_is_a_pure_function_of_seed_launch_and_index():
    k = sround.launch_key(1234, 0)
    assert k == sround.launch_key(1234, 0)
    assert k != sround.launch_key(1234, 1) and k != sround.launch_key(1235, 0)
    idx = np.arange(1 << 16, dtype=np.uint64)
    a = sround.rng_bits(k[0], k[1], idx)
    assert np.array_equal(a, sround.rng_bits(k[0], k[1], idx))
    assert np.array_equal(a[100:200], sround.rng_bits(k[0], k[1], idx[100:200]))
    # indices past 2^32 give different words from their low halves
    assert not np.array_equal(a[:64], sround.rng_bits(k[0], k[1], idx[:64] + np.uint64(1 << 32)))
    # roughly uniform: mean of the top bit and of the word
    assert abs((a >> U32(31)).mean() - 0.5) < 0.01
    assert abs(a.astype(np.float64).mean() / 2.0 ** 32 - 0.5) < 0.01
    f = sround.frand(a)
    assert f.dtype == np.float32 and 0.0 <= f.min() and f.max() <= 1.0


def test_pair_words_of_sixteen_bit_stores():
    """Eight neighbours share one hash: element 0 of a group reads it unchanged, an odd element
    reads its pair's word rotated left by 19 bits, later pairs step a congruential chain."""
    k = sround.launch_key(7, 3)
    idx = np.arange(64, dtype=np.uint64)
    w = sround.rng_bits_pair(k[0], k[1], idx)
    h = sround.rng_bits(k[0], k[1], idx >> np.uint64(3))
    assert np.array_equal(w[0::8], h[0::8])
    assert np.array_equal(w[1::2], ((w[0::2] << U32(19)) | (w[0::2] >> U32(13))).astype(U32))
    h1 = (h[2::8].astype(np.uint64) * np.uint64(0x2C9277B5) + np.uint64(0xAC564B05)) & np.uint64(0xFFFFFFFF)
    assert np.array_equal(w[2::8], (h1 ^ (h1 >> np.uint64(16))).astype(U32))
    # the top 13 bits, which decide an fp16 store at 10 bits, are uniform per element
    big = sround.rng_bits_pair(k[0], k[1], np.arange(1 << 18, dtype=np.uint64))
    top = big >> U32(19)
    for lane in range(8):
        assert abs(top[lane::8].mean() / 8192.0 - 0.5) < 0.01, lane


def test_compensated_sum_known_answers():
    """Kahan step of float_ew.py:958-993 at fp16: 2048 + 1 is a tie that rounds to 2048 and
    the lost 1 lands (negated) in cmp; the next step adds it back."""
    s = np.array([2048.0], np.float16)
    c = np.array([0.0], np.float16)
    a = np.array([1.0], np.float16)
    s, c = sround.compensated_sum(s, c, a)
    assert s[0] == 2048.0 and c[0] == -1.0 and s.dtype == np.float16
    s, c = sround.compensated_sum(s, c, a)
    assert s[0] == 2050.0 and c[0] == 0.0
    # scales (cmp_scale = 0 drops the compensation, as the periodic reset does)
    s, c = sround.compensated_sum(np.array([1.0], np.float32), np.array([0.25], np.float32),
                                  np.array([2.0], np.float32), cmp_scale=0.0, add_scale=0.5)
    assert s[0] == 2.0 and c[0] == 0.0
    # stochastic rounding of the sum at one mantissa bit: 1.0 + 0.1 becomes 1.0 or 1.5
    ur = np.array([0, 0xFFFFFFFF], U32)
    s, c = sround.compensated_sum(np.ones(2, np.float32), np.zeros(2, np.float32),
                                  np.full(2, 0.1, np.float32), rounding=1, urand=ur)
    assert s.tolist() == [1.0, 1.5]
    assert np.allclose(c, [-0.1, 0.4], atol=1e-7)
