"""CPU tests pinning the numpy checker (oracle/) to neon's NervanaCPU."""
import os

import numpy as np
import pytest

from oracle.numpy_backend import OracleBackend
from tests.cases import run_case, standard_cases, summarize

CASES = standard_cases()
from oracle import neon_ref

REFERENCE = neon_ref.find_reference() or ""


def _check(fingerprint, golden, prefix):
    for field, val in fingerprint.items():
        want = golden["%s/%s" % (prefix, field)]
        if np.asarray(val).dtype.kind in "iub":
            assert np.array_equal(val, want), prefix
        else:
            # same numpy calls in the same order: identical bits expected; the
            # tolerance only absorbs a different numpy build's libm
            np.testing.assert_allclose(val, want, rtol=1e-6, atol=1e-7, err_msg=prefix)


@pytest.mark.parametrize("case", CASES, ids=lambda c: c.name)
def test_oracle_reproduces_reference_golden(case, golden):
    for dt in (np.float32, np.float64):
        be = OracleBackend(default_dtype=dt)
        with np.errstate(all="ignore"):
            res = run_case(be, case, compute_dtype=dt)
        for k, arr in res.items():
            if k.startswith("grad"):
                continue
            _check(summarize(arr), golden, "%s/%s/%s" % (case.name, np.dtype(dt).name, k))


@pytest.mark.skipif(not REFERENCE, reason="no neon source tree on this machine")
def test_oracle_matches_live_reference_bit_for_bit():
    from tests.golden.make_golden import import_reference_cpu
    NervanaCPU = import_reference_cpu(REFERENCE)
    for case in CASES:
        for dt in (np.float32, np.float64):
            with np.errstate(all="ignore"):
                ref = run_case(NervanaCPU(default_dtype=dt), case, compute_dtype=dt)
                got = run_case(OracleBackend(default_dtype=dt), case, compute_dtype=dt)
            for k in ref:
                assert ref[k].dtype == got[k].dtype, (case.name, k)
                assert np.array_equal(ref[k], got[k], equal_nan=True), (case.name, k)


def test_onehot_assignment_matches_reference_rule():
    be = OracleBackend()
    idx = be.array(np.array([[2, 0, 3, 1, 1]], dtype=np.int32), dtype=np.int32)
    out = be.zeros((4, 5))
    out[:] = be.onehot(idx, axis=0)
    want = np.zeros((4, 5), np.float32)
    want[[2, 0, 3, 1, 1], np.arange(5)] = 1
    assert np.array_equal(out.get(), want)


def test_log2_histogram_known_answers():
    """float_ew.py:1086-1100: bin = clamp(round(log2|x|) - offset, 0, nbins - 1); with offset -48,
    1.0 is bin 48, 1.5 and 2.0 bin 49, 2.9 and 3.0 bin 50; zero, NaN and anything at or below
    2^-48 fall into bin 0, infinity and anything from 2^15 up into bin 63."""
    v = np.array([1.0, 2.0, 3.0, 0.0, np.inf, np.nan, 2.0 ** -48, 2.0 ** -60, 1.5, 2.9, 2.0 ** 15, 2.0 ** 20],
                 np.float32)
    h = OracleBackend.log2_hist(v, 64, -48)
    assert {i: int(c) for i, c in enumerate(h) if c} == {0: 4, 48: 1, 49: 2, 50: 2, 63: 3}
    assert h.dtype == np.int32 and h.sum() == v.size
    # negative logs round away from zero too: 2^-1.6 -> -2, 2^-1.4 -> -1
    h = OracleBackend.log2_hist(np.array([2.0 ** -1.6, 2.0 ** -1.4], np.float32), 8, -4)
    assert {i: int(c) for i, c in enumerate(h) if c} == {2: 1, 3: 1}


def _reference_test_hist(inp, nbins=64, offset=-48):
    """The numpy formulation neon's own histogram test compares backends with
    (tests/test_backend_hist.py:25-43): np.histogram of rint(log2|x|) over unit bins."""
    bins = np.arange(nbins + 1) + float(offset)
    bins[0] = -float("Inf")
    with np.errstate(divide="ignore"):
        v = np.rint(np.log2(np.abs(inp.astype(np.float32))))
    return np.histogram(v, density=False, bins=bins)[0]


HIST_EDGE_INPUTS = [                                  # tests/test_backend_hist.py:101-108
    ("edges", np.array([2 ** -48, 2 ** 15], dtype=np.float32)),
    ("rounding", np.array([2 ** 5, 63.99998856, 2 ** 6, 2 ** -3, 2 ** -4, 0.11262291, 92.22483826], dtype=np.float32)),
    ("fp16 rounding", np.array([45.21875], dtype=np.float16)),
]


def test_log2_histogram_agrees_with_the_reference_tests_formulation():
    """Edge-case inputs of neon's histogram test, and its parametrised sweep (normal(64, 4) data
    as float32 and uint8, bins (64, -48) and (32, 0)): the restated kernel gives the counts of the
    test's np.histogram formulation."""
    for tag, inp in HIST_EDGE_INPUTS:
        assert np.array_equal(OracleBackend.log2_hist(inp), _reference_test_hist(inp)), tag
    rng = np.random.RandomState(0)
    for nbins, offset in ((64, -48), (32, 0)):
        for dim in ((64, 32768), (64, 1)):
            for dtype in (np.float32, np.uint8):
                inp = rng.normal(64, 4, dim[0] * dim[1]).reshape(dim).astype(dtype)
                assert np.array_equal(OracleBackend.log2_hist(inp, nbins, offset),
                                      _reference_test_hist(inp, nbins, offset)), (nbins, offset, dim, dtype)
