"""
copy_transpose (any rank, views) against numpy.transpose, and the Kahan
accumulation kernel against its restatement in oracle/sround.py.
"""
import itertools

import numpy as np
import pytest

from oracle import sround

pytestmark = pytest.mark.gpu


def _fill(rng, shape, dtype):
    if np.dtype(dtype).kind == "f":
        return rng.uniform(-4, 4, shape).astype(dtype)
    info = np.iinfo(dtype)
    return rng.randint(max(info.min, -1000), min(info.max, 1000), shape).astype(dtype)


@pytest.mark.parametrize("dtype", [np.float32, np.float16, np.uint8, np.int32, np.int16])
def test_copy_transpose_two_dimensions(b200, dtype):
    be = b200
    rng = np.random.RandomState(0)
    for shape in [(1, 1), (1, 7), (7, 1), (3, 5), (32, 32), (33, 65), (100, 257), (128, 64), (1000, 513), (2048, 1024)]:
        h = _fill(rng, shape, dtype)
        a = be.array(h, dtype=dtype)
        out = be.empty(shape[::-1], dtype=dtype)
        be.copy_transpose(a, out)
        assert np.array_equal(out.get(), h.T), (shape, dtype)


@pytest.mark.parametrize("dtype", [np.float32, np.float16, np.uint8])
def test_copy_transpose_every_permutation_of_three_and_four_dimensions(b200, dtype):
    be = b200
    rng = np.random.RandomState(1)
    for shape in [(5, 6, 7), (16, 33, 40), (3, 64, 130), (2, 3, 4, 5), (6, 17, 9, 32)]:
        h = _fill(rng, shape, dtype)
        a = be.array(h, dtype=dtype)
        for axes in itertools.permutations(range(len(shape))):
            oshape = tuple(shape[x] for x in axes)
            out = be.empty(oshape, dtype=dtype)
            be.copy_transpose(a, out, axes=axes)
            assert np.array_equal(out.get(), np.transpose(h, axes)), (shape, axes, dtype)


def test_copy_transpose_five_dimensions_and_default_axes(b200):
    be = b200
    rng = np.random.RandomState(2)
    shape = (3, 4, 5, 6, 8)
    h = _fill(rng, shape, np.float32)
    a = be.array(h)
    out = be.empty(shape[::-1])
    be.copy_transpose(a, out)                       # axes=None reverses the dimensions
    assert np.array_equal(out.get(), np.transpose(h))
    axes = [4, 0, 3, 1, 2]                          # a list is accepted as well
    out = be.empty(tuple(shape[x] for x in axes))
    be.copy_transpose(a, out, axes=axes)
    assert np.array_equal(out.get(), np.transpose(h, axes))


@pytest.mark.parametrize("dtype", [np.float32, np.float16, np.uint8])
def test_copy_transpose_between_views_as_the_data_iterator_does(b200, dtype):
    """ArrayIterator (neon/data/dataiterator.py:144-202) keeps (examples, features) rows on
    the device and per minibatch transposes a row slice into a column slice of the
    (features, batch) buffer; at the end of an epoch the batch wraps around."""
    be = b200
    rng = np.random.RandomState(3)
    ndata, nfeat, bsz = 1000, 77, 128
    h = _fill(rng, (ndata, nfeat), dtype)
    dev = be.array(h, dtype=dtype)
    buf = be.zeros((nfeat, bsz), dtype=dtype)
    want = np.zeros((nfeat, bsz), dtype)
    for i1 in range(0, ndata, bsz):
        n = min(bsz, ndata - i1)
        be.copy_transpose(dev[i1:i1 + n], buf[:, 0:n])
        want[:, 0:n] = h[i1:i1 + n].T
        if n < bsz:
            be.copy_transpose(dev[0:bsz - n], buf[:, n:])
            want[:, n:] = h[0:bsz - n].T
        assert np.array_equal(buf.get(), want), (i1, dtype)


def test_copy_transpose_leaves_the_rest_of_a_view_alone_and_checks_arguments(b200):
    be = b200
    rng = np.random.RandomState(4)
    h = _fill(rng, (40, 50), np.float16)
    a = be.array(h, dtype=np.float16)
    base = be.zeros((60, 70), dtype=np.float16)
    be.copy_transpose(a[3:33, 5:45], base[10:50, 20:50])
    want = np.zeros((60, 70), np.float16)
    want[10:50, 20:50] = h[3:33, 5:45].T
    assert np.array_equal(base.get(), want)
    with pytest.raises(AssertionError):
        be.copy_transpose(a, be.empty((50, 41), dtype=np.float16))
    with pytest.raises(AssertionError):
        be.copy_transpose(a, be.empty((50, 40), dtype=np.float32))
    with pytest.raises(AssertionError):
        be.copy_transpose(a, a)


def test_copy_transpose_large_matrix(b200):
    """64 MiB each way: past the L2, tile path with 32-bit accesses on 2-byte elements."""
    be = b200
    rng = np.random.RandomState(5)
    h = rng.randint(0, 65535, (4096, 8192)).astype(np.uint16).view(np.float16)
    a = be.array(h, dtype=np.float16)
    out = be.empty((8192, 4096), dtype=np.float16)
    be.copy_transpose(a, out)
    assert np.array_equal(out.get().view(np.uint16), h.T.view(np.uint16))


@pytest.mark.parametrize("dtype", [np.float16, np.uint8, np.int16, np.int8])
def test_copy_transpose_of_aligned_one_and_two_byte_matrices(b200, dtype):
    """Shapes whose pitches are multiples of 16 bytes (whole 16-byte vectors on both sides of the
    tile kernel: edges in both directions, batches, views that keep the alignment) next to
    neighbours that break the alignment by one element."""
    be = b200
    rng = np.random.RandomState(6)
    es = np.dtype(dtype).itemsize
    n = 16 // es
    for shape in [(256, 128), (1008, 528), (2048 + n, 1024 + 16), (16 * n, 4096), (4096, 16 * n), (1008 + 1, 528), (1008, 528 + 1)]:
        h = _fill(rng, shape, dtype)
        a = be.array(h, dtype=dtype)
        out = be.empty(shape[::-1], dtype=dtype)
        be.copy_transpose(a, out)
        assert np.array_equal(out.get(), h.T), (shape, dtype)
    for shape, axes in [((4, 512, 272), (0, 2, 1)), ((3, 2, 256, 192), (0, 1, 3, 2)), ((3, 2, 256, 192), (1, 0, 3, 2)),
                        ((8, 256, 128), (2, 0, 1)), ((8, 256, 128), (1, 2, 0)), ((2, 3, 4, 128, 256), (2, 0, 1, 4, 3))]:
        h = _fill(rng, shape, dtype)
        a = be.array(h, dtype=dtype)
        out = be.empty(tuple(shape[x] for x in axes), dtype=dtype)
        be.copy_transpose(a, out, axes=axes)
        assert np.array_equal(out.get(), np.transpose(h, axes)), (shape, axes, dtype)
    # views: row and column offsets that keep 16-byte alignment, inside larger tensors
    h = _fill(rng, (700, 1200), dtype)
    a = be.array(h, dtype=dtype)
    base = be.zeros((1100, 800), dtype=dtype)
    want = np.zeros((1100, 800), dtype)
    be.copy_transpose(a[32:32 + 640, 64:64 + 1008], base[16:16 + 1008, 48:48 + 640])
    want[16:16 + 1008, 48:48 + 640] = h[32:32 + 640, 64:64 + 1008].T
    assert np.array_equal(base.get(), want), dtype
    # ... and one that does not (odd column offset)
    be.copy_transpose(a[32:32 + 640, 65:65 + 1008], base[16:16 + 1008, 48:48 + 640])
    want[16:16 + 1008, 48:48 + 640] = h[32:32 + 640, 65:65 + 1008].T
    assert np.array_equal(base.get(), want), dtype


# ---------------------------------------------------------------- Kahan accumulation
@pytest.mark.parametrize("dtype", ["float32", "float16", "bfloat16"])
def test_compensated_sum_nearest_matches_the_restated_kernel(b200, dtype):
    if dtype == "bfloat16":
        dtype = pytest.importorskip("ml_dtypes").bfloat16
    be = b200
    rng = np.random.RandomState(6)
    for n in (1, 7, 8, 1000, 4099, 1 << 16):
        sh = rng.uniform(-8, 8, (n, 1)).astype(dtype)
        ch = (rng.uniform(-1, 1, (n, 1)) * 2.0 ** -9).astype(dtype)
        ah = rng.uniform(-1, 1, (n, 1)).astype(dtype)
        s, c, a = be.array(sh, dtype=dtype), be.array(ch, dtype=dtype), be.array(ah, dtype=dtype)
        be.compensated_sum(s, c, a, cmp_scale=0.5, add_scale=0.25)
        ws, wc = sround.compensated_sum(sh, ch, ah, 0.5, 0.25)
        assert np.array_equal(s.get().astype(np.float32), ws.astype(np.float32)), (n, dtype)
        assert np.array_equal(c.get().astype(np.float32), wc.astype(np.float32)), (n, dtype)
        assert np.array_equal(a.get().astype(np.float32), ah.astype(np.float32))


def test_compensated_sum_stochastic_rounding_bit_exact(b200):
    be = b200
    rng = np.random.RandomState(7)
    n = 40000 + 3                                   # vector part and a scalar tail
    for dtype, bits, pair in ((np.float16, True, True), (np.float16, 6, True), (np.float32, 12, False)):
        sh = rng.uniform(-8, 8, (n, 1)).astype(dtype)
        ch = (rng.uniform(-1, 1, (n, 1)) * 2.0 ** -9).astype(dtype)
        ah = (rng.uniform(-1, 1, (n, 1)) * 2.0 ** -6).astype(dtype)
        s, c, a = be.array(sh, dtype=dtype), be.array(ch, dtype=dtype), be.array(ah, dtype=dtype)
        s.rounding = bits
        seed, launch = be.rng_get_state()[1]
        be.compensated_sum(s, c, a)
        assert be.rng_get_state()[1][1] == launch + 1          # one launch number per call
        key = sround.launch_key(int(seed), int(launch))
        idx = np.arange(n, dtype=np.uint64)
        ur = (sround.rng_bits_pair if pair else sround.rng_bits)(key[0], key[1], idx).reshape(n, 1)
        ws, wc = sround.compensated_sum(sh, ch, ah, 1.0, 1.0, rounding=bits, urand=ur)
        assert np.array_equal(s.get().view(np.uint8), ws.view(np.uint8)), (dtype, bits)
        assert np.array_equal(c.get().view(np.uint8), wc.view(np.uint8)), (dtype, bits)


def test_compensated_sum_keeps_what_plain_fp16_accumulation_loses(b200):
    """Adding 1e-3-sized increments to values near 8 in fp16 (ulp 2^-7) loses most of each
    increment; with the compensation tensor the running sum follows the exact one."""
    be = b200
    rng = np.random.RandomState(8)
    n, steps = 4096, 200
    s0 = rng.uniform(8, 12, (n, 1)).astype(np.float16)
    s, c = be.array(s0, dtype=np.float16), be.zeros((n, 1), dtype=np.float16)
    plain = be.array(s0, dtype=np.float16)
    exact = s0.astype(np.float64)
    for k in range(steps):
        ah = (rng.uniform(0.5, 1.5, (n, 1)) * 1e-3).astype(np.float16)
        a = be.array(ah, dtype=np.float16)
        be.compensated_sum(s, c, a)
        plain[:] = plain + a
        exact += ah.astype(np.float64)
    err_kahan = np.abs(s.get().astype(np.float64) - exact).max()
    err_plain = np.abs(plain.get().astype(np.float64) - exact).max()
    assert err_kahan <= 2.0 ** -7                   # within one ulp of the stored sum
    assert err_plain > 10 * err_kahan
    assert c.kahan_count == steps


def test_compensated_sum_reset_period_and_argument_checks(b200):
    be = b200
    sh = np.full((64, 1), 3.0, np.float32)
    s, c, a = be.array(sh), be.array(np.full((64, 1), 0.5, np.float32)), be.array(np.full((64, 1), 1.0, np.float32))
    c.kahan_reset = 2
    c.kahan_count = 3                               # past the period: this call ignores cmp
    be.compensated_sum(s, c, a)
    assert np.array_equal(s.get(), np.full((64, 1), 4.0, np.float32)) and c.kahan_count == 1
    assert np.array_equal(c.get(), np.zeros((64, 1), np.float32))
    with pytest.raises(AssertionError):
        be.compensated_sum(s, c, be.zeros((64, 1), dtype=np.float16))
    big = be.zeros((64, 4))
    with pytest.raises(ValueError):
        be.compensated_sum(big[:, 0:1], c, a)


# ---------------------------------------------------------------- log2 histogram
def _values_away_from_bin_edges(rng, n, lo=-30, hi=12):
    """Magnitudes 2^(k + f) with f at least 0.02 away from the rounding edge at 0.5."""
    k = rng.randint(lo, hi, n)
    f = rng.uniform(-0.48, 0.48, n)
    return (np.exp2(k + f) * rng.choice([-1.0, 1.0], n)).astype(np.float32)


@pytest.mark.parametrize("dtype", [np.float32, np.float16])
def test_log2_histogram_matches_the_restated_kernel(b200, dtype):
    from oracle.numpy_backend import OracleBackend
    be = b200
    rng = np.random.RandomState(9)
    lo, hi = (-30, 12) if dtype == np.float32 else (-12, 12)
    for n in (1, 7, 1000, 100003, 1 << 20):
        h = _values_away_from_bin_edges(rng, n, lo, hi).astype(dtype).reshape(n, 1)
        if n >= 1000:
            h[5] = 0.0
            h[6] = np.inf
            h[7] = np.nan
            h[8] = -np.inf
        t = be.array(h, dtype=dtype)
        got = t.hist("n%d" % n)
        assert tuple(got.shape) == (1, be.hist_bins) and got.dtype == np.int32
        want = OracleBackend.log2_hist(h, be.hist_bins, be.hist_offset)
        assert np.array_equal(got.get().ravel(), want), (n, dtype)
        assert int(got.get().sum()) == n
    data, tags = be.dump_hist_data()
    assert tuple(data.shape) == (5, be.hist_bins) and sorted(tags) == sorted("n%d" % n for n in (1, 7, 1000, 100003, 1 << 20))
    assert int(data.get()[tags["n1000"]].sum()) == 1000
    assert be.hist_idx == 0 and be.hist_map == {}


def test_log2_histogram_bins_and_offset_can_be_changed(b200):
    from oracle.numpy_backend import OracleBackend
    be = b200
    old = (be.hist_bins, be.hist_offset)
    try:
        be.set_hist_buffers(16, -8)
        rng = np.random.RandomState(10)
        h = _values_away_from_bin_edges(rng, 5000, -20, 20).reshape(50, 100)
        got = be.array(h).hist("w")
        assert tuple(got.shape) == (1, 16)
        assert np.array_equal(got.get().ravel(), OracleBackend.log2_hist(h, 16, -8))
        with pytest.raises(ValueError):
            be.array(h)[:, 0:10].hist("view")
    finally:
        be.set_hist_buffers(*old)


def test_log2_histogram_on_the_reference_tests_inputs(b200):
    """tests/test_backend_hist.py: the edge cases, dump_hist_data, and normal(64, 4) data stored as
    float32 and as uint8 with (64, -48) and (32, 0) bins."""
    from oracle.numpy_backend import OracleBackend
    from tests.test_oracle import HIST_EDGE_INPUTS
    be = b200
    old = (be.hist_bins, be.hist_offset)
    try:
        for tag, inp in HIST_EDGE_INPUTS:
            got = be.array(inp.reshape(-1, 1), dtype=inp.dtype).hist(tag)
            assert np.array_equal(got.get().ravel(), OracleBackend.log2_hist(inp)), tag
        data, tags = be.dump_hist_data()
        for tag, inp in HIST_EDGE_INPUTS:
            assert np.array_equal(data.get()[tags[tag]], OracleBackend.log2_hist(inp)), tag
        rng = np.random.RandomState(0)
        for nbins, offset in ((64, -48), (32, 0)):
            be.set_hist_buffers(nbins, offset)
            for dim in ((64, 32768), (64, 1)):
                for dtype in (np.float32, np.uint8, np.float16, np.int8):
                    inp = rng.normal(64, 4, dim[0] * dim[1]).reshape(dim).astype(dtype)
                    got = be.array(inp, dtype=dtype).hist("x")
                    assert np.array_equal(got.get().ravel(), OracleBackend.log2_hist(inp, nbins, offset)), (nbins, dim, dtype)
            be.dump_hist_data()
    finally:
        be.set_hist_buffers(*old)
