"""GPU parity tests: the CUDA backend against the numpy checker and against the
committed NervanaCPU fingerprints, on the same seeded inputs.  Every call goes
python -> ctypes -> libb200ew.so."""
import numpy as np
import pytest

from oracle import sround
from oracle.numpy_backend import OracleBackend
from tests import cases
from tests.parity import check_fingerprint, check_output

pytestmark = pytest.mark.gpu

STANDARD = cases.standard_cases()


def _oracle64(case):
    with np.errstate(all="ignore"):
        return cases.run_case(OracleBackend(default_dtype=np.float64), case, compute_dtype=np.float64)


def _compare(case, got, want):
    for k, (shape, dt) in case.outputs.items():
        if k in case.derived:
            expect, scale = case.derived[k](got)
            check_output("%s/%s(derived)" % (case.name, k), got[k], expect, dt, scale=scale)
        else:
            check_output("%s/%s" % (case.name, k), got[k], want[k], dt)
    for k in got:
        if k in case.outputs or k.startswith("grad"):
            continue
        check_output("%s/%s(in place)" % (case.name, k), got[k], want[k], got[k].dtype)


@pytest.mark.parametrize("case", STANDARD, ids=lambda c: c.name)
def test_case_matches_checker(case, b200):
    got = cases.run_case(b200, case)
    _compare(case, got, _oracle64(case))


@pytest.mark.parametrize("case", STANDARD[:5], ids=lambda c: c.name)
def test_benchmark_configs_match_nervanacpu_golden(case, b200, golden):
    """The five configurations against fingerprints made by neon's own NervanaCPU."""
    got = cases.run_case(b200, case)
    for k, (shape, dt) in case.outputs.items():
        if k in case.derived:
            continue
        g, w = check_fingerprint(k, got[k], golden, "%s/float64/%s" % (case.name, k))
        check_output("%s/%s vs golden" % (case.name, k), np.asarray(g), np.asarray(w), dt)


@pytest.mark.parametrize("case", [cases.cfg2(), cases.cfg4(256, 56 * 56 * 16),
                                  cases.cfg5(2048, 2048), cases.cfg3(n=1000000, steps=3)],
                         ids=lambda c: c.name)
def test_large_configs_match_checker(case, b200):
    """Benchmark shapes at (or scaled towards) their quoted sizes: split reductions,
    several blocks per row/column, more than one wave of blocks."""
    got = cases.run_case(b200, case)
    _compare(case, got, _oracle64(case))


def _rowres_cases():
    def in1(shape, dtype=np.float32, scale=1.0):
        return lambda rng: {"x": (scale * rng.uniform(-1, 1, shape)).astype(dtype)}

    out = [cases.cfg4(256, 56 * 56 * 128), cases.cfg4(64, 100352), cases.cfg4(300, 8192)]

    def softmax1(be, t):
        x = t["x"]
        t["out"][:] = be.exp(x - be.max(x, axis=1)) / be.sum(be.exp(x - be.max(x, axis=1)), axis=1)
    out.append(cases.Case("softmax_axis1_200x16384", in1((200, 16384), scale=3.0),
                          {"out": ((200, 16384), np.float32)}, softmax1))

    def logsumexp_rows(be, t):
        x = t["x"]
        mx = be.max(x, axis=1)
        t["out"][:] = be.log(be.sum(be.exp(x - mx), axis=1)) + mx
    out.append(cases.Case("logsumexp_axis1_red_out_150x40000", in1((150, 40000), scale=3.0),
                          {"out": ((150, 1), np.float32)}, logsumexp_rows))

    def argmax_center(be, t):
        x = t["x"]
        t["out"][:] = (x - be.mean(x, axis=1)) * be.argmax(x, axis=1)
    out.append(cases.Case("center_times_argmax_128x65536_f16", in1((128, 65536), np.float16),
                          {"out": ((128, 65536), np.float32)}, argmax_center))
    return out


@pytest.mark.parametrize("case", _rowres_cases(), ids=lambda c: c.name)
def test_row_resident_cluster_kernel_matches_checker(case, b200):
    """Statements whose rows fit in cluster shared memory run as one kernel (TMA-staged
    rows, reductions exchanged through distributed shared memory)."""
    b200.launch_log = []
    got = cases.run_case(b200, case)
    kinds = [k for k, _ in b200.launch_log]
    b200.launch_log = None
    assert kinds == ["rowres"], kinds
    b200.check_status()
    _compare(case, got, _oracle64(case))


def _moment_cases():
    """Statements whose second sum is centred on a value that needs the first (variance and its
    relatives): computed from one pass (moments pair).  Sub-warp rows, whole blocks, rows split
    over blocks, scalar tails, 16-bit storage, a compound operand, a centre that is not the
    mean, an arg reduction sharing the pass, data far from zero."""
    def in1(shape, dtype=np.float32, scale=1.0, offset=0.0):
        return lambda rng: {"x": (offset + scale * rng.standard_normal(shape)).astype(dtype)}

    def var_rows(be, t):
        t["out"][:] = be.var(t["x"], axis=1)

    def std_rows(be, t):
        x = t["x"]
        t["out"][:] = (x - be.mean(x, axis=1)) / (be.std(x, axis=1) + 1e-3)

    def about_max(be, t):
        x = t["x"]
        t["out"][:] = be.sum(be.square(be.max(x, axis=1) - x), axis=1)

    def compound(be, t):
        x = t["x"]
        t["out"][:] = be.var(x * x + 0.5 * x, axis=1)

    def with_argmax(be, t):
        x = t["x"]
        t["out"][:] = be.var(x, axis=1) + be.argmax(x, axis=1)

    out = []
    for shape in ((300, 40), (37, 1000), (64, 2051), (5, 100003), (3, 1 << 21)):
        out.append(cases.Case("var_rows_%dx%d" % shape, in1(shape), {"out": ((shape[0], 1), np.float32)}, var_rows))
    out.append(cases.Case("var_rows_far_from_zero_40x30000", in1((40, 30000), offset=100.0),
                          {"out": ((40, 1), np.float32)}, var_rows))
    out.append(cases.Case("var_rows_f16_33x4099", in1((33, 4099), np.float16, 2.0, 1.0),
                          {"out": ((33, 1), np.float32)}, var_rows))
    out.append(cases.Case("standardise_rows_f16_20x12345", in1((20, 12345), np.float16, 2.0, 1.0),
                          {"out": ((20, 12345), np.float16)}, std_rows))
    out.append(cases.Case("squares_about_max_64x5000", in1((64, 5000)), {"out": ((64, 1), np.float32)}, about_max))
    out.append(cases.Case("var_of_compound_50x3000", in1((50, 3000)), {"out": ((50, 1), np.float32)}, compound))
    out.append(cases.Case("var_plus_argmax_48x2500", in1((48, 2500)), {"out": ((48, 1), np.float32)}, with_argmax))
    return out


@pytest.mark.parametrize("case", _moment_cases(), ids=lambda c: c.name)
def test_single_pass_moments_match_checker(case, b200):
    got = cases.run_case(b200, case)
    _compare(case, got, _oracle64(case))
    # the same statement evaluated as written (one pass per sum) agrees too
    b200._planner.fuse_moments = False
    b200._plans.clear()
    try:
        plain = cases.run_case(b200, case)
    finally:
        b200._planner.fuse_moments = True
        b200._plans.clear()
    _compare(case, plain, _oracle64(case))


def test_checked_mode_refuses_out_of_range_operands_without_launching():
    """Checked mode: a view that reaches past its allocation, or an index vector that points
    outside the indexed axis, raises B200_ERR_INVALID before anything is launched."""
    from neon_b200 import runtime as rt
    from neon_b200.backend import B200Backend
    from neon_b200.tensor import B200Tensor
    be = B200Backend(rng_seed=0, check_bounds=True)
    t = be.array(np.arange(400, dtype=np.float32).reshape(4, 100))
    out = be.empty((4, 100))
    out[:] = t * 2.0                                              # in range: runs
    assert np.array_equal(out.get(), 2.0 * np.arange(400, dtype=np.float32).reshape(4, 100))
    bad = B200Tensor(be, (4, 100), np.float32, gpudata=t.gpudata, strides=(200, 1), base=t, _block=t._block)
    before = be.launches
    with pytest.raises(rt.B200Error) as e:
        out[:] = bad + 1.0
    assert e.value.status == -1 and be.launches == before
    idx = be.array(np.array([[0, 3, 7]], dtype=np.int32), dtype=np.int32)     # rows 0..3 exist
    got = be.empty((3, 100))
    with pytest.raises(rt.B200Error) as e:
        got[:] = t.take(idx, axis=0) * 1.0
    assert e.value.status == -1 and be.launches == before
    idx.set(np.array([[0, 3, 2]], dtype=np.int32))
    got[:] = t.take(idx, axis=0) * 1.0
    assert np.array_equal(got.get(), np.arange(400, dtype=np.float32).reshape(4, 100)[[0, 3, 2]])


def test_view_and_fuzz_statements_pass_checked_mode(b200):
    """The random views and random statements of the other tests once more with every operand
    checked against its allocation before each launch."""
    from tests import fuzz
    b200.check_bounds = True
    try:
        for seed in range(0, 160, 4):
            spec = fuzz.Spec(seed)
            fuzz.build(b200, spec, fuzz.host_arrays(spec))
        base = b200.array(np.arange(6 * 7 * 8, dtype=np.float32).reshape(6, 56))
        host = np.arange(6 * 7 * 8, dtype=np.float32).reshape(6, 56)
        for sub in ((slice(1, 5), slice(3, 50, 3)), (slice(None), slice(55, None, -2)), (2, slice(None)), (slice(None), 7)):
            out = b200.empty(base[sub].shape)
            out[:] = base[sub] + 1.0
            assert np.array_equal(out.get().reshape(-1), (host[sub] + 1.0).reshape(-1)), sub
    finally:
        b200.check_bounds = False


def test_bounded_wait_reports_instead_of_hanging():
    """The one software wait in the kernels (a block waiting for its TMA-staged row slice)
    has a time limit.  Announce 16 bytes that never arrive, give it 20 ms: the kernel must
    end by itself, the host must see the status, and the backend must keep working."""
    from neon_b200 import runtime as rt
    from neon_b200.backend import B200Backend
    be = B200Backend(rng_seed=0)
    x = be.array(np.random.RandomState(0).randn(64, 16384).astype(np.float32))
    y = be.empty((64, 16384))

    def stmt():
        y[:] = (x - be.mean(x, axis=1)) / (be.std(x, axis=1) + 1e-3)

    be._planner.wait_limit_ns = 20 * 1000 * 1000
    be._planner.debug_starve_bytes = 16
    be.launch_log = []
    stmt()
    assert [k for k, _ in be.launch_log] == ["rowres"]
    with pytest.raises(rt.B200Error) as e:
        be.synchronize()
    assert e.value.status == -6
    # same context, same backend: a clean statement afterwards gives the right answer
    be._planner.debug_starve_bytes = 0
    be._planner.wait_limit_ns = 2000000000
    be._plans.clear()
    stmt()
    be.synchronize()
    xh = x.get().astype(np.float64)
    want = (xh - xh.mean(1, keepdims=True)) / (xh.std(1, keepdims=True) + 1e-3)
    np.testing.assert_allclose(y.get(), want, rtol=1e-4, atol=1e-5)


def test_full_size_adam_against_checker_on_a_sample(b200):
    """Config 3 at its quoted size and length: 1e8 elements (param/m/v fp32, grad fp16), 100
    steps, a different gradient every step.  The update is element-wise, so the checker run on
    one column (every 1000th element, 1e5 of them) must agree with the same elements of the
    full-size device result.  Gradients are made on the device (a pool of four seeded arrays,
    rescaled per step and stored as fp16) and the checker is fed the very values the device
    stored, read back from that column."""
    be = b200
    n_rows, n_cols, col = 100000, 1000, 123
    rng = np.random.RandomState(3)
    ph = (0.02 * rng.standard_normal((n_rows, n_cols))).astype(np.float32)
    param = be.array(ph)
    m, v = be.zeros((n_rows, n_cols)), be.zeros((n_rows, n_cols))
    grad = be.empty((n_rows, n_cols), dtype=np.float16)
    pool = [be.array((1e-3 * np.random.RandomState(1000 + i).standard_normal((n_rows, n_cols))).astype(np.float16),
                     dtype=np.float16) for i in range(4)]
    ob = OracleBackend(default_dtype=np.float64)
    op = ob.array(ph[:, col:col + 1], dtype=np.float64)
    om, ov = ob.zeros(op.shape, dtype=np.float64), ob.zeros(op.shape, dtype=np.float64)
    be.bsz = ob.bsz = 1
    for step in range(1, 101):
        grad[:] = pool[step % 4] * (1.0 + 0.01 * step)
        cases.adam_step(be, param, grad, m, v, step)
        og = ob.array(grad[:, col:col + 1].get(), dtype=np.float64)
        cases.adam_step(ob, op, og, om, ov, step)
        if step in (1, 3, 10, 30, 100):
            for name, dev, ref in (("param", param, op), ("m", m, om), ("v", v, ov)):
                check_output("adam 1e8 step %d/%s" % (step, name), dev[:, col:col + 1].get(), ref.get(), np.float32)
    # the other columns moved too: the whole tensor, not just the sampled column, was updated
    moved = np.abs(param.get() - ph)
    assert (moved == 0).mean() < 1e-5 and abs(np.median(moved[:, col]) / np.median(moved[:, 7]) - 1) < 0.05


def test_full_size_properties_cfg5(b200):
    """Config 5 at its quoted size, 2^30 elements (32768 x 32768 fp16, stochastic rounding):
    size-independent checks, the host side working through the arrays in row blocks.
    total must equal the float64 sum of the device-produced z (relative to sum|z|), peak must
    equal max|z| exactly, every stored value must be one of the two fp16 neighbours of the exact
    value, and the mean signed rounding error over all 2^30 outputs must be far below one ulp."""
    from tests.parity import ulp16
    be = b200
    rows = cols = 32768
    block = 1024                                          # rows per host block (2^25 elements)
    x, y = be.empty((rows, cols), dtype=np.float16), be.empty((rows, cols), dtype=np.float16)
    rng = np.random.default_rng(5)

    def host_block():
        return (rng.random((block, cols), dtype=np.float32) * np.float32(8) - np.float32(4)).astype(np.float16)
    xs, ys = [], []
    for r0 in range(0, rows, block):                      # 2 GiB each, kept for the checks below
        xs.append(host_block())
        ys.append(host_block())
        x[r0:r0 + block].set(xs[-1])
        y[r0:r0 + block].set(ys[-1])
    z = be.empty((rows, cols), dtype=np.float16)
    z.rounding = True
    total, peak = be.empty((1, 1)), be.empty((1, 1))
    z[:] = be.tanh(x) * be.sqrt(be.absolute(y)) + 0.5 * x * y
    total[:] = be.sum(z)
    peak[:] = be.max(be.absolute(z))
    zsum = zabs = bias = 0.0
    zmax, worst = 0.0, 0.0
    for i, r0 in enumerate(range(0, rows, block)):
        zh = z[r0:r0 + block].get()
        z64 = zh.astype(np.float64)
        zsum += z64.sum()
        zabs += np.abs(z64).sum()
        zmax = max(zmax, float(np.abs(zh).max()))
        a, b = xs[i].astype(np.float64), ys[i].astype(np.float64)
        exact = np.tanh(a) * np.sqrt(np.abs(b)) + 0.5 * a * b
        ulp = ulp16(exact)
        bias += ((z64 - exact) / ulp).sum()
        if i % 8 == 0:                                    # neighbour check on an eighth of the blocks
            worst = max(worst, float(((np.abs(z64 - exact) - 1e-6 * 10.0) / ulp).max()))
    assert abs(float(total.get()[0, 0]) - zsum) <= 1e-5 * zabs
    assert float(peak.get()[0, 0]) == zmax
    assert worst <= 1.0 + 1e-2
    bias /= float(rows) * cols
    assert abs(bias) < 1e-4, "mean rounding bias %.3g ulp" % bias


def test_stochastic_rounding_bit_exact_against_restated_rule(b200):
    """z = 0.5*x + y is exact in fp32 for these inputs, so the stored fp16 must equal
    the restated rounding rule applied to the same random words, bit for bit."""
    be = b200
    rng = np.random.RandomState(11)
    shape = (300, 1000)
    xh = rng.uniform(-4, 4, shape).astype(np.float16)
    yh = (rng.uniform(-1, 1, shape) * 2.0 ** -6).astype(np.float16)
    x, y = be.array(xh, dtype=np.float16), be.array(yh, dtype=np.float16)
    for bits in (True, 5, 1):
        z = be.empty(shape, dtype=np.float16)
        z.rounding = bits
        seed, launch = be.rng_get_state()[1]
        z[:] = 0.5 * x + y
        val = (np.float32(0.5) * xh.astype(np.float32) + yh.astype(np.float32)).astype(np.float32)
        key = sround.launch_key(int(seed), int(launch))
        ur = sround.rng_bits_pair(key[0], key[1], np.arange(val.size, dtype=np.uint64)).reshape(shape)
        want = sround.store(val, np.float16, bits, ur)
        got = z.get()
        assert np.array_equal(got.view(np.uint16), want.view(np.uint16)), bits
    # fp32 output, 12 bits
    zf = be.empty(shape, dtype=np.float32)
    zf.rounding = 12
    seed, launch = be.rng_get_state()[1]
    zf[:] = 0.5 * x + y
    key = sround.launch_key(int(seed), int(launch))
    ur = sround.rng_bits(key[0], key[1], np.arange(val.size, dtype=np.uint64)).reshape(shape)
    assert np.array_equal(zf.get().view(np.uint32), sround.store(val, np.float32, 12, ur).view(np.uint32))


def test_stochastic_rounding_odd_width_uses_same_random_words(b200):
    """A tensor whose row length is odd takes the per-lane path of the kernels; the
    stored values must still be the restated rule on the words of the element indices."""
    be = b200
    rng = np.random.RandomState(12)
    shape = (37, 333)
    xh = rng.uniform(-4, 4, shape).astype(np.float16)
    x = be.array(xh, dtype=np.float16)
    c = be.array(rng.uniform(-1, 1, (shape[0], 1)).astype(np.float16).astype(np.float32))
    z = be.empty(shape, dtype=np.float16)
    z.rounding = True
    seed, launch = be.rng_get_state()[1]
    z[:] = 0.25 * x + c                       # broadcast operand: the 2-d kernel, exact in fp32
    val = (np.float32(0.25) * xh.astype(np.float32) + c.get()).astype(np.float32)
    key = sround.launch_key(int(seed), int(launch))
    ur = sround.rng_bits_pair(key[0], key[1], np.arange(val.size, dtype=np.uint64)).reshape(shape)
    assert np.array_equal(z.get().view(np.uint16), sround.store(val, np.float16, True, ur).view(np.uint16))


def test_precise_math_mode_matches_checker():
    """IEEE division / libm tanh, sqrt instead of the few-ulp fast versions."""
    from neon_b200.backend import B200Backend
    be = B200Backend(rng_seed=0, precise_math=True)
    for case in (cases.cfg5(128, 192), cases.cfg4(32, 4096), cases.cfg2(2000, 96), cases.adam_small(),
                 cases.unary_case("tanh"), cases.unary_case("sig"), cases.binary_case("div")):
        got = cases.run_case(be, case)
        _compare(case, got, _oracle64(case))


def test_fast_math_stays_within_a_few_ulp(b200):
    be = b200
    xs = np.concatenate([np.linspace(-9, 9, 200001), np.linspace(-0.7, 0.7, 100001),
                         np.array([0.0, 1e-6, -1e-6, 1e-20, 30.0, -30.0, 88.0])]).astype(np.float32)
    xs = xs[: (xs.size // 8) * 8].reshape(8, -1)
    x = be.array(xs)
    out = be.empty(xs.shape)
    out[:] = be.tanh(x)
    ref = np.tanh(xs.astype(np.float64))
    err = np.abs(out.get().astype(np.float64) - ref) / np.maximum(np.spacing(np.abs(ref).astype(np.float32)), 1e-45)
    assert err.max() <= 4.0, err.max()
    pos = np.abs(xs) + np.float32(1e-3)
    out[:] = be.sqrt(be.array(pos))
    ref = np.sqrt(pos.astype(np.float64))
    assert (np.abs(out.get() - ref) / np.spacing(ref.astype(np.float32))).max() <= 2.0
    out[:] = x / be.array(pos)
    ref = xs.astype(np.float64) / pos.astype(np.float64)
    assert (np.abs(out.get() - ref) / np.maximum(np.spacing(np.abs(ref).astype(np.float32)), 1e-45)).max() <= 3.0
    # exp over the whole range of normal results, sig, exp2
    es = np.concatenate([np.linspace(-87.0, 88.5, 300001), np.linspace(-1, 1, 100001)]).astype(np.float32)
    es = es[: (es.size // 8) * 8].reshape(8, -1)
    e, eo = be.array(es), be.empty(es.shape)
    eo[:] = be.exp(e)
    ref = np.exp(es.astype(np.float64))
    assert (np.abs(eo.get() - ref) / np.spacing(ref.astype(np.float32))).max() <= 4.0
    eo[:] = be.exp2(e)
    ref = np.exp2(es.astype(np.float64))
    assert (np.abs(eo.get() - ref) / np.spacing(ref.astype(np.float32))).max() <= 3.0
    eo[:] = be.sig(e)
    ref = 1.0 / (1.0 + np.exp(-es.astype(np.float64)))
    ok = ref > 1e-37
    assert (np.abs(eo.get() - ref)[ok] / np.spacing(ref.astype(np.float32))[ok]).max() <= 6.0
    big = be.array(np.array([[100.0, -104.0, 89.0, -200.0]], np.float32))
    bo = be.empty((1, 4))
    bo[:] = be.exp(big)
    assert np.isinf(bo.get()[0, 0]) and bo.get()[0, 1] == 0.0 and np.isinf(bo.get()[0, 2]) and bo.get()[0, 3] == 0.0


def test_stochastic_rounding_one_bit_distribution(b200):
    """neon tests/test_backend_sr.py:52-71: ones + 0.1 at one mantissa bit gives only
    1.0 and 1.5, more than 10% of them 1.5 and more than 70% 1.0."""
    be = b200
    n = 10
    a = be.ones((n * n * 100, 1), dtype=np.float16) if False else be.ones((1000, 100))
    c = be.empty((1000, 100), dtype=np.float16)
    c.rounding = 1
    c[:] = a + 0.1
    got = c.get()
    assert set(np.unique(got).tolist()) <= {1.0, 1.5}
    frac = float((got == 1.5).mean())
    assert 0.1 < frac < 0.3


def test_integer_stores_round_to_nearest_even_and_saturate(b200):
    be = b200
    vals = np.array([[0.5, 1.5, 2.5, -0.5, -1.5, 126.6, 127.5, 300.0, -129.0, -1000.0, 3.49, -3.51]], np.float32)
    x = be.array(vals)
    for dt in (np.int8, np.uint8, np.int16, np.uint16, np.int32, np.uint32):
        out = be.empty(vals.shape, dtype=dt)
        out[:] = x * 1.0
        assert np.array_equal(out.get(), sround.nearest_int(vals, dt)), dt


def test_rng_reproducible_after_reset_and_state_restore(b200):
    """neon tests/test_backend_randomstate.py:23-74,145-178 for the device generator."""
    be = b200
    be.rng_reset()
    a = be.empty((200, 300))
    a[:] = be.rand()
    first = a.get()
    assert 0.0 <= first.min() and first.max() <= 1.0 and abs(first.mean() - 0.5) < 0.01
    state = be.rng_get_state()
    a[:] = be.rand()
    second = a.get()
    assert not np.array_equal(first, second)
    be.rng_set_state(state)
    a[:] = be.rand()
    assert np.array_equal(a.get(), second)
    be.rng_reset()
    a[:] = be.rand()
    assert np.array_equal(a.get(), first)
    mask = be.empty((200, 300))
    be.make_binary_mask(mask, keepthresh=0.3)
    m = mask.get()
    assert set(np.unique(m).tolist()) <= {0.0, 1.0} and abs(m.mean() - 0.3) < 0.02


def test_take_addressing(b200):
    """Fancy-indexed operands and outputs (neon in1/in2/out1/out2 modes,
    cuda_templates.py:448-478); LookupTable.fprop is ``out[:] = W.take(idx, axis=0)``."""
    be = b200
    rng = np.random.RandomState(4)
    Wh = rng.randn(1000, 64).astype(np.float32)
    ih = rng.randint(0, 1000, (1, 200)).astype(np.int32)
    W, idx = be.array(Wh), be.array(ih, dtype=np.int32)
    out = be.empty((200, 64))
    out[:] = W.take(idx, axis=0)
    assert np.array_equal(out.get(), Wh[ih[0]])
    Wt = be.array(np.ascontiguousarray(Wh.T))
    o2 = be.empty((64, 200))
    o2[:] = Wt.take(idx, axis=1) * 2.0 + 1.0
    assert np.allclose(o2.get(), Wh.T[:, ih[0]] * 2.0 + 1.0, rtol=1e-6)
    s = be.empty((1, 64))
    s[:] = be.sum(W.take(idx, axis=0), axis=0)
    np.testing.assert_allclose(s.get(), Wh[ih[0]].sum(0, keepdims=True), rtol=1e-5, atol=1e-5)
    m = be.empty((200, 1))
    m[:] = be.max(W.take(idx, axis=0), axis=1)
    assert np.array_equal(m.get(), Wh[ih[0]].max(1, keepdims=True))
    perm = rng.permutation(1000)[:200].astype(np.int32).reshape(1, -1)
    dW = be.zeros((1000, 64))
    dW[be.array(perm, dtype=np.int32), :] = out * 0.5
    want = np.zeros((1000, 64), np.float32)
    want[perm[0]] = Wh[ih[0]] * 0.5
    assert np.array_equal(dW.get(), want)
    # the plan cache re-aims at a new index vector
    ih2 = rng.randint(0, 1000, (1, 200)).astype(np.int32)
    out[:] = W.take(be.array(ih2, dtype=np.int32), axis=0)
    assert np.array_equal(out.get(), Wh[ih2[0]])


def _bn_case(rows, cols, dtype, relu, accumbeta):
    def inputs(rng):
        return {"x": (1.0 + 2.0 * rng.randn(rows, cols)).astype(dtype),
                "delta": rng.randn(rows, cols).astype(dtype),
                "gamma": rng.uniform(0.5, 1.5, (rows, 1)).astype(np.float32),
                "beta": rng.uniform(-0.5, 0.5, (rows, 1)).astype(np.float32),
                "gmean": rng.randn(rows, 1).astype(np.float32),
                "gvar": rng.uniform(0.5, 1.5, (rows, 1)).astype(np.float32),
                "y": rng.randn(rows, cols).astype(np.float32)}

    def run(be, t):
        be.compound_fprop_bn(t["x"], t["xsum"], t["xvar"], t["gmean"], t["gvar"], t["gamma"], t["beta"],
                             t["y"], 1e-3, 0.9, True, accumbeta=accumbeta, relu=relu)
        be.compound_bprop_bn(t["dx"], t["ggamma"], t["gbeta"], t["delta"], t["x"], t["xsum"], t["xvar"],
                             t["gamma"], 1e-3)
        t["yinf"][:] = 0
        be.compound_fprop_bn(t["x"], t["xsum"], t["xvar"], t["gmean"], t["gvar"], t["gamma"], t["beta"],
                             t["yinf"], 1e-3, 0.9, True, inference=True)

    col = ((rows, 1), np.float32)
    return cases.Case("compound_bn_%dx%d_%s_relu%d_acc%g" % (rows, cols, np.dtype(dtype).name, relu, accumbeta),
                      inputs, {"xsum": col, "xvar": col, "ggamma": col, "gbeta": col,
                               "dx": ((rows, cols), np.float32), "yinf": ((rows, cols), np.float32)}, run)


@pytest.mark.parametrize("case", [_bn_case(32, 1024, np.float32, False, 0.0),
                                  _bn_case(64, 50176, np.float16, True, 0.0),
                                  _bn_case(16, 333, np.float32, False, 0.5)], ids=lambda c: c.name)
def test_compound_batchnorm_entry_points(case, b200):
    """The calls the BatchNorm layer makes (layers/layer.py:2483-2520) against the same
    calls on the checker."""
    got = cases.run_case(b200, case)
    _compare(case, got, _oracle64(case))


def test_dot_inside_op_trees(b200):
    """Trees that contain a matrix product (tests/test_backend_compound_optree.py:39-58):
    the product runs as its own launch between the fused element-wise statements."""
    be = b200
    rng = np.random.RandomState(9)
    ah, bh, ch = rng.randn(37, 53).astype(np.float32), rng.randn(53, 29).astype(np.float32), rng.randn(37, 29).astype(np.float32)
    a, b, c = be.array(ah), be.array(bh), be.array(ch)
    out = be.empty((37, 29))
    out[:] = be.dot(a, b)
    np.testing.assert_allclose(out.get(), ah.dot(bh), rtol=1e-5, atol=1e-5)
    out[:] = be.dot(a * 2.0, b) + c
    np.testing.assert_allclose(out.get(), (ah * 2).dot(bh) + ch, rtol=1e-5, atol=1e-5)
    col = be.empty((37, 1))
    col[:] = be.sum(be.dot(a, b), axis=1) * 0.5
    np.testing.assert_allclose(col.get(), ah.dot(bh).sum(1, keepdims=True) * 0.5, rtol=1e-5, atol=1e-4)
    sq = be.empty((53, 53))
    sq[:] = be.dot(a.T, a)
    np.testing.assert_allclose(sq.get(), ah.T.dot(ah), rtol=1e-5, atol=1e-4)
    h = be.array(ah.astype(np.float16), dtype=np.float16)
    out[:] = be.dot(h, b)
    np.testing.assert_allclose(out.get(), ah.astype(np.float16).astype(np.float32).dot(bh), rtol=1e-5, atol=1e-4)


def _bf16_cases():
    import ml_dtypes
    bf = ml_dtypes.bfloat16
    out = [cases.unary_case("tanh", (64, 328), bf), cases.unary_case("exp", (33, 77), bf),
           cases.binary_case("mul", (64, 328), (64, 1), bf), cases.binary_case("add", (4, 3), (4, 3), bf),
           cases.reduce_case("sum", (64, 4096), 1, bf), cases.reduce_case("max", (4096, 64), 0, bf),
           cases.reduce_case("argmax", (300, 40), 0, bf, ties=True)]

    def chain(be, t):
        x, y = t["x"], t["y"]
        t["z"][:] = be.tanh(x) * be.sqrt(be.absolute(y)) + 0.5 * x * y
    out.append(cases.Case("bf16_chain_256x512",
                          lambda rng: {"x": rng.uniform(-4, 4, (256, 512)).astype(bf),
                                       "y": rng.uniform(-4, 4, (256, 512)).astype(bf)},
                          {"z": ((256, 512), bf)}, chain))
    return out


@pytest.mark.parametrize("case", _bf16_cases(), ids=lambda c: c.name)
def test_bfloat16_storage(case, b200):
    """bf16 storage with fp32 arithmetic (no counterpart in neon, which predates the format)."""
    got = cases.run_case(b200, case)
    _compare(case, got, _oracle64(case))


def test_bfloat16_stochastic_rounding_bit_exact(b200):
    import ml_dtypes
    bf = ml_dtypes.bfloat16
    be = b200
    rng = np.random.RandomState(21)
    shape = (200, 512)
    xh = rng.uniform(-4, 4, shape).astype(np.float16)
    x = be.array(xh, dtype=np.float16)
    z = be.empty(shape, dtype=bf)
    z.rounding = True                       # capped at the 7 mantissa bits bf16 has
    seed, launch = be.rng_get_state()[1]
    z[:] = x * 1.0
    key = sround.launch_key(int(seed), int(launch))
    ur = sround.rng_bits_pair(key[0], key[1], np.arange(xh.size, dtype=np.uint64)).reshape(shape)
    want32 = sround.sr_f32(xh.astype(np.float32), ur, 7)          # exactly representable in bf16
    assert np.array_equal(z.get().astype(np.float32).view(np.uint32), want32.view(np.uint32))


def test_graph_replay_of_a_statement_sequence(b200):
    """A captured sequence replays with one call and computes the same values; inputs
    changed in place between replays are seen (addresses are frozen, contents are not)."""
    be = b200
    rng = np.random.RandomState(1)
    ah, bh = rng.randn(512, 128).astype(np.float32), rng.randn(512, 128).astype(np.float32)
    ch = rng.uniform(-.5, .5, (512, 1)).astype(np.float32)
    a, b, c = be.array(ah), be.array(bh), be.array(ch)
    out, s, m = be.empty((512, 128)), be.empty((1, 128)), be.empty((1, 128), dtype=np.int32)

    def step():
        out[:] = be.maximum(a * b + c, 0)
        s[:] = be.sum(out, axis=0)
        m[:] = be.argmax(out, axis=0)

    graph = be.capture(step)
    assert graph.launches == 3
    for trial in range(3):
        ah = rng.randn(512, 128).astype(np.float32)
        a.set(ah)
        graph.replay()
        want = np.maximum(ah.astype(np.float64) * bh + ch, 0)
        np.testing.assert_allclose(out.get(), want, rtol=1e-5, atol=1e-6)
        np.testing.assert_allclose(s.get(), want.sum(0, keepdims=True), rtol=1e-5, atol=1e-4)
        assert np.array_equal(m.get(), out.get().argmax(0).reshape(1, -1))
    # eager execution still works afterwards
    step()
    be.synchronize()


def test_graph_replay_draws_the_random_words_eager_execution_would(b200):
    """Stochastic rounding, a dropout mask and rand inside a recorded sequence: every replay is
    bit for bit what the next eager execution of the sequence would have produced."""
    be = b200
    rng = np.random.RandomState(2)
    xh = rng.uniform(-4, 4, (300, 257)).astype(np.float32)
    x = be.array(xh)
    z = be.empty((300, 257), dtype=np.float16)
    z.rounding = True
    mask, noisy = be.empty((300, 257)), be.empty((300, 257))

    def step():
        z[:] = x * 1.0009765625 + 0.3
        be.make_binary_mask(mask, keepthresh=0.6)
        noisy[:] = x + be.rand() * 0.5
        x[:] = x * 0.5 + 1.0                       # the sequence feeds itself

    def snapshot():
        return [t.get().copy() for t in (z, mask, noisy, x)]

    state = be.rng_get_state()
    eager = []
    for _ in range(4):
        step()
        eager.append(snapshot())
    # the same four steps again: one eager (inside capture), three replayed
    x.set(xh)
    be.rng_set_state(state)
    graph = be.capture(step)
    assert graph.rng_count == 3
    got = [snapshot()]
    for _ in range(3):
        graph.replay()
        got.append(snapshot())
    for i, (want, have) in enumerate(zip(eager, got)):
        for name, w, h in zip(("z", "mask", "noisy", "x"), want, have):
            assert np.array_equal(w.view(np.uint8), h.view(np.uint8)), (i, name)
    assert not np.array_equal(got[1][1], got[2][1])            # and the masks do change between replays
    # eager execution carries on from the same point of the random stream
    step()
    after_replays = snapshot()
    x.set(xh)
    be.rng_set_state(state)
    for _ in range(5):
        step()
    for w, h in zip(snapshot(), after_replays):
        assert np.array_equal(w.view(np.uint8), h.view(np.uint8))


def test_bench_flag_records_every_launch(tmp_path):
    """be.bench turns on per-launch timing (the reference prints msecs per compound kernel,
    float_ew.py:917-938); here the records are kept and can be dumped as JSON."""
    import json
    from neon_b200.backend import B200Backend
    be = B200Backend(rng_seed=0, bench=True)
    x = be.array(np.random.RandomState(0).randn(1000, 64).astype(np.float32))
    y = be.empty((1000, 64))
    y[:] = be.exp(x - be.max(x, axis=0)) / be.sum(be.exp(x - be.max(x, axis=0)), axis=0)
    assert [r["kind"] for r in be.trace] == ["red_cols", "red_cols", "ew_2d"]
    assert all(r["ms"] > 0 and r["kernel"].startswith("ot_") for r in be.trace)
    be.dump_trace(str(tmp_path / "trace.json"))
    assert len(json.load(open(str(tmp_path / "trace.json")))) == 3


def test_onehot_and_views(b200):
    be = b200
    idx = np.random.RandomState(3).randint(0, 10, (1, 64)).astype(np.int32)
    out = be.zeros((10, 64))
    out[:] = be.onehot(be.array(idx, dtype=np.int32), axis=0)
    want = np.zeros((10, 64), np.float32)
    want[idx[0], np.arange(64)] = 1
    assert np.array_equal(out.get(), want)
    x = be.array(np.arange(48, dtype=np.float32).reshape(6, 8))
    assert np.array_equal(x[1:5, 2:7].get(), np.arange(48).reshape(6, 8)[1:5, 2:7])
    assert np.array_equal(x.T.get(), np.arange(48).reshape(6, 8).T)
    assert np.array_equal(x.reshape(8, 6).get(), np.arange(48).reshape(8, 6))
    assert np.array_equal(x[3].get(), np.arange(48).reshape(6, 8)[3:4])


def test_more_than_two_to_the_32_elements(b200):
    """Element indices past 2^32 (the 64-bit paths of the flat element-wise kernel, the
    whole-tensor reduction, a row reduction and the random words of a stochastic store): a
    (65536, 65540) fp16 tensor, 4.3e9 elements, checked through values planted near its end."""
    be = b200
    rows, cols = 65536, 65540
    x = be.empty((rows, cols), dtype=np.float16)
    x[:] = 0.5
    tail = np.arange(1, 11, dtype=np.float16).reshape(1, 10)
    x[rows - 1:rows, cols - 10:cols] = be.array(tail, dtype=np.float16)        # the very last ten elements
    x[rows - 2:rows - 1, 0:10] = be.array(-tail, dtype=np.float16)
    z = be.empty((rows, cols), dtype=np.float16)
    z[:] = x * 2.0 + 1.0                                    # flat kernel, indices up to 2^32 + 2^18
    assert np.array_equal(z[rows - 1:rows, cols - 12:cols].get().ravel(),
                          np.concatenate([[2.0, 2.0], 2.0 * np.arange(1, 11) + 1.0]).astype(np.float16))
    assert np.array_equal(z[rows - 2:rows - 1, 0:12].get().ravel(),
                          np.concatenate([-2.0 * np.arange(1, 11) + 1.0, [2.0, 2.0]]).astype(np.float16))
    assert float(z[0:1, 0:1].get()[0, 0]) == 2.0
    peak, low, total = be.empty((1, 1)), be.empty((1, 1)), be.empty((1, 1))
    peak[:] = be.max(z)
    low[:] = be.min(z)
    total[:] = be.sum(x)
    assert float(peak.get()[0, 0]) == 21.0 and float(low.get()[0, 0]) == -19.0
    want = 0.5 * (rows * cols - 20)                         # the planted values cancel
    assert abs(float(total.get()[0, 0]) - want) <= 1e-5 * want
    rowsum = be.empty((rows, 1))
    rowsum[:] = be.sum(x, axis=1)
    got = rowsum.get().ravel()
    assert got[0] == 0.5 * cols and abs(got[-1] - (0.5 * (cols - 10) + 55.0)) < 1e-3 * cols
    assert abs(got[-2] - (0.5 * (cols - 10) - 55.0)) < 1e-3 * cols
    # stochastic store: the words used at the far end are those of the far element indices
    from oracle import sround
    z.rounding = True
    seed, launch = be.rng_get_state()[1]
    z[:] = x * 1.0009765625                                 # 0.5 * (1 + 2^-10): needs rounding at 10 bits
    key = sround.launch_key(int(seed), int(launch))
    last = np.arange(rows * cols - 16, rows * cols, dtype=np.uint64)
    vals = (x[rows - 1:rows, cols - 16:cols].get().astype(np.float32) * np.float32(1.0009765625)).ravel()
    ur = sround.rng_bits_pair(key[0], key[1], last)
    want = sround.store(vals, np.float16, True, ur)
    assert np.array_equal(z[rows - 1:rows, cols - 16:cols].get().ravel().view(np.uint16), want.view(np.uint16))


def test_stochastic_rounding_bit_exact_over_random_shapes(b200):
    """The stored bits are the restated rule applied to the random word of each element's
    row-major index, whatever the shape (vector width, scalar tails), the kernel (flat, 2-d with a
    broadcast operand, store into a view), the storage type and the number of kept bits."""
    be = b200
    rng = np.random.RandomState(0)
    dims = (1, 2, 3, 7, 8, 9, 15, 16, 17, 31, 33, 64, 100, 127, 129, 255, 257, 1000, 1024, 4099)
    try:
        import ml_dtypes
        bf = ml_dtypes.bfloat16
    except ImportError:
        bf = None
    for trial in range(90):
        R, C = int(rng.choice(dims)), int(rng.choice(dims))
        odt = (bf or np.float16) if trial % 5 == 0 else (np.float16, np.float32)[trial % 2]
        bits = (True, 3, 7, 10, 12)[trial % 5]
        mode = trial % 3                      # 0 flat, 1 broadcast column operand, 2 output view
        xh = rng.uniform(-4, 4, (R, C)).astype(np.float16)
        x = be.array(xh, dtype=np.float16)
        z = be.zeros((R + 3, C + 5), dtype=odt)[1:1 + R, 2:2 + C] if mode == 2 else be.empty((R, C), dtype=odt)
        z.rounding = bits
        seed, launch = be.rng_get_state()[1]
        if mode == 1:
            ch = rng.uniform(-1, 1, (R, 1)).astype(np.float16).astype(np.float32)
            z[:] = 0.3330078125 * x + be.array(ch)
            val = (np.float32(0.3330078125) * xh.astype(np.float32) + ch).astype(np.float32)
        else:
            z[:] = x * 1.0009765625
            val = (xh.astype(np.float32) * np.float32(1.0009765625)).astype(np.float32)
        key = sround.launch_key(int(seed), int(launch))
        idx = np.arange(R * C, dtype=np.uint64)
        two_byte = np.dtype(odt).itemsize == 2
        ur = (sround.rng_bits_pair if two_byte else sround.rng_bits)(key[0], key[1], idx).reshape(R, C)
        want = sround.store(val, odt, bits, ur)
        got = z.get()
        assert np.array_equal(got.view(np.uint8), want.view(np.uint8)), (trial, (R, C), np.dtype(odt).name, bits, mode)


def test_random_views_read_and_write_like_numpy(b200):
    """Slices with steps, integer subscripts (kept as extent-1 axes, nervanagpu.py:262-275),
    negative indices, transposes of views and reshapes: ``get`` returns what numpy indexing
    returns, and assigning through the view changes exactly the viewed elements."""
    be = b200
    rng = np.random.RandomState(42)
    for trial in range(60):
        R, C = int(rng.randint(2, 70)), int(rng.randint(2, 90))
        dtype = (np.float32, np.float16, np.int32)[trial % 3]
        h = (rng.randn(R, C) * 8).astype(dtype)
        t = be.array(h, dtype=dtype)

        def rand_slice(n):
            a, b = sorted(rng.randint(0, n + 1, 2))
            if a == b:
                b = min(n, a + 1)
                a = b - 1
            step = int(rng.choice([1, 1, 2, 3]))
            start = int(a) - n if (a > 0 and rng.rand() < 0.2) else int(a)      # sometimes counted from the end
            return slice(start, int(b), step)
        kind = trial % 5
        if kind == 0:
            key = (rand_slice(R), rand_slice(C))
        elif kind == 1:
            key = (int(rng.randint(-R, R)), rand_slice(C))
        elif kind == 2:
            key = (rand_slice(R), int(rng.randint(-C, C)))
        elif kind == 3:
            key = (rand_slice(R),)
        else:
            key = (Ellipsis, rand_slice(C))
        view = t[key]
        want = h[key]
        if want.ndim == 1:                    # an integer subscript keeps its axis with extent 1
            want = want.reshape((1, -1)) if isinstance(key[0], (int, np.integer)) else want.reshape((-1, 1))
        assert tuple(view.shape) == want.shape, (trial, key, view.shape, want.shape)
        assert np.array_equal(view.get(), want), (trial, key)
        assert np.array_equal(view.T.get(), want.T), (trial, key)
        # write through the view
        new = (rng.randn(*want.shape) * 8).astype(dtype)
        view[:] = be.array(new, dtype=dtype)
        ref = h.copy()
        ref[key] = new.reshape(ref[key].shape)
        assert np.array_equal(t.get(), ref), (trial, key)
        view[:] = 3
        ref[key] = 3
        assert np.array_equal(t.get(), ref), (trial, key)
    # reshape of a contiguous tensor and of a row slice; refusal for a column slice
    h = rng.randn(12, 10).astype(np.float32)
    t = be.array(h)
    assert np.array_equal(t.reshape((20, 6)).get(), h.reshape(20, 6))
    assert np.array_equal(t[2:8].reshape((6, 10)).get(), h[2:8])
    assert np.array_equal(t[2:8].reshape((30, 2)).get(), h[2:8].reshape(30, 2))
    with pytest.raises(ValueError):
        t[:, 2:8].reshape((36, 2))
