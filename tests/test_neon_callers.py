"""
neon's own classes computing on this package's backend.

``tests/neon_cases.py`` holds the cases: neon's optimizers (with gradient /
parameter clipping and schedules), Bias / Activation / Dropout / BatchNorm layers,
GeneralizedCost with its cost functions, the ArrayIterator, and the backend entry
points ``compound_fprop_bn`` / ``compound_bprop_bn``.  The reference side is the
same neon code on neon's NervanaCPU with float64 tensors, run live and, in
addition, taken from the committed fingerprints ``tests/golden/neon_callers_golden.npz``
(made by ``tests/golden/make_golden.py``).

* GPU tests: the b200 backend against both, tolerances of ``tests/parity.py``
  (fp32 within 1e-5 relative of the float64 result).
* CPU tests: the numpy checker -- which shares this package's op-tree front end --
  stands in for the device, so that the cases themselves, the front end as neon's
  classes use it, and the committed fingerprints are checked on every machine.

All of them need a neon source tree (``oracle/neon_ref.py`` says where it is
looked for); without one they are skipped, because the callers are neon's code.
"""
import os

import numpy as np
import pytest

from oracle import neon_ref
from tests.parity import check_output

HAVE_NEON = neon_ref.find_reference() is not None
pytestmark = pytest.mark.skipif(not HAVE_NEON, reason="no neon source tree on this machine "
                                                      "(set NEON_REFERENCE or run oracle/make_ref.py)")

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "neon_callers_golden.npz")


def _case_names():
    if not HAVE_NEON:
        return []
    neon_ref.import_neon()
    from tests.neon_cases import neon_caller_cases
    return sorted(neon_caller_cases())


@pytest.fixture(scope="module")
def neon_env():
    neon_ref.import_neon()
    import neon_b200.neon_plugin as plugin
    from neon import NervanaObject
    with neon_ref.numpy_compat():
        old = NervanaObject.be
        yield plugin
        NervanaObject.be = old


@pytest.fixture(scope="module")
def callers_golden():
    return np.load(GOLDEN)


def _reference(name):
    from neon.backends.nervanacpu import NervanaCPU
    from tests.neon_cases import neon_caller_cases
    with np.errstate(all="ignore"):
        return neon_caller_cases()[name](NervanaCPU(default_dtype=np.float64, rng_seed=0))


def _compare(name, got, want, golden, exact_reference):
    from tests.cases import summarize
    assert sorted(got) == sorted(want), name
    for k in want:
        label = "%s/%s" % (name, k)
        if exact_reference:
            np.testing.assert_allclose(got[k], want[k], rtol=1e-9, atol=1e-12, err_msg=label)
        else:
            check_output(label, np.asarray(got[k]), want[k], np.float32)
        # the committed fingerprint of the same array
        fp = summarize(np.asarray(want[k]))
        for field, val in fp.items():
            stored = golden["%s/%s/%s" % (name, k, field)]
            np.testing.assert_allclose(val, stored, rtol=1e-7, atol=1e-10, err_msg=label + " vs golden")


# --------------------------------------------------------------------------- CPU: checker as executor
@pytest.mark.parametrize("name", _case_names())
def test_case_on_checker_matches_nervanacpu_and_golden(name, neon_env, callers_golden):
    from oracle.numpy_backend import OracleBackend
    from tests.neon_cases import GPU_ONLY, neon_caller_cases
    if name in GPU_ONLY:
        pytest.skip("needs the eager shift of the GPU backends")
    neon_env.register(backend_cls=OracleBackend)
    want = _reference(name)
    with np.errstate(all="ignore"):
        got = neon_caller_cases()[name](OracleBackend(default_dtype=np.float64, rng_seed=0))
    _compare(name, got, want, callers_golden, exact_reference=True)


def test_array_iterator_on_checker(neon_env):
    from oracle.numpy_backend import OracleBackend
    from tests.neon_cases import NUMPY_CHECKED
    neon_env.register(backend_cls=OracleBackend)
    run = NUMPY_CHECKED["array_iterator"]
    got, want = run(OracleBackend(rng_seed=0)), run.expected()
    assert sorted(got) == sorted(want)
    for k in want:
        assert np.array_equal(got[k], want[k]), k


# --------------------------------------------------------------------------- GPU
@pytest.fixture(scope="module")
def b200_neon(neon_env):
    neon_env.register()
    from neon_b200 import gen_backend
    return gen_backend(backend="b200", rng_seed=0)


@pytest.mark.gpu
@pytest.mark.parametrize("name", _case_names())
def test_neon_callers_on_b200_match_nervanacpu(name, b200_neon, callers_golden):
    from tests.neon_cases import GPU_ONLY, neon_caller_cases
    before = b200_neon.launches
    got = neon_caller_cases()[name](b200_neon)
    assert b200_neon.launches > before
    b200_neon.check_status()
    if name in GPU_ONLY:
        return _check_shift_adamax(name, got)
    want = _reference(name)
    _compare(name, got, want, callers_golden, exact_reference=False)


def _check_shift_adamax(name, got):
    """ShiftAdaMax multiplies by powers of two picked by rounding a base-2 logarithm
    (optimizers/optimizer.py:933-991): a float64 and a float32 evaluation may round a few
    borderline elements to neighbouring powers, so compare with NervanaCPU allowing a small
    fraction of elements to differ (and no element by more than the step size allows)."""
    want = _reference(name)
    for k in want:
        g, w = np.asarray(got[k], np.float64), np.asarray(want[k], np.float64)
        assert g.shape == w.shape and np.all(np.isfinite(g)), k
        off = np.abs(g - w) > 1e-5 * np.abs(w) + 1e-7
        assert off.mean() < 0.02, "%s/%s: %.2f%% of elements differ" % (name, k, 100 * off.mean())


@pytest.mark.gpu
def test_array_iterator_on_b200(b200_neon):
    from tests.neon_cases import NUMPY_CHECKED
    run = NUMPY_CHECKED["array_iterator"]
    got, want = run(b200_neon), run.expected()
    assert sorted(got) == sorted(want)
    for k in want:
        assert np.array_equal(got[k], want[k]), k


@pytest.mark.gpu
def test_dropout_layer_on_b200(b200_neon):
    """Dropout (layers/layer.py:1968-2066): the mask is Bernoulli(keep), a new one per fprop,
    outputs are mask * inputs * scaling, bprop applies the same mask, inference only scales."""
    from tests.neon_cases import STATISTICAL
    r = STATISTICAL["dropout_layer"](b200_neon)
    keep = float(r["keep"][0, 0])
    mask, n = r["mask"], r["mask"].size
    assert set(np.unique(mask)) <= {0.0, 1.0}
    assert abs(mask.mean() - keep) < 4 * np.sqrt(keep * (1 - keep) / n)
    assert not np.array_equal(mask, r["mask_second"])
    np.testing.assert_allclose(r["y"], mask * r["x"], rtol=1e-6)
    np.testing.assert_allclose(r["y_second"], r["mask_second"] * r["x"], rtol=1e-6)
    np.testing.assert_allclose(r["deltas"], r["mask_second"], rtol=1e-6)
    np.testing.assert_allclose(r["y_inference"], keep * r["x"], rtol=1e-6)
