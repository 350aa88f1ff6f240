"""
Symbolic gradients of op-trees (neon_b200/autodiff.py).

Three checks, all on the CPU: against central differences of a numpy version of
the same function (the method of neon's tests/test_backend_autodiff.py:38-68,
whose function families -- basic arithmetic, abs/square, dot, reductions mixed
with dot, scalar broadcast, transposes -- are covered by the functions below);
bit for bit against neon's own ``Autodiff`` run on its NervanaCPU backend when a
neon checkout is present; and that every gradient tree lowers and compiles for
the GPU backend.
"""
import os

import numpy as np
import pytest

from neon_b200.autodiff import Autodiff, autodiff
from oracle.numpy_backend import OracleBackend

REFERENCE = os.environ.get("NEON_REFERENCE") or os.path.join(
    os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference")


# name -> (function of (be, x0..x4) for op-trees, the same for numpy arrays)
def _arith(be, a, b, c, d, e):
    return (a + c) + a * e + b * d - a / (c + 2.0)


def _real(be, a, b, c, d, e):
    return b + be.absolute(c + d) + e - (b + be.square(c + d) + e) + be.sqrt(be.absolute(a) + 1.0)


def _dot(be, a, b, c, d, e):
    return (a + d) + be.dot(b, c) - (b - c) - be.dot(d, e)


def _dot_reductions(be, a, b, c, d, e):
    return be.max(a, axis=1) + be.min(b, axis=0) + be.dot(1. / d, c + e) + be.min(d, axis=0)


def _scalar_broadcast(be, a, b, c, d, e):
    return 0.2 * a - b * c / 3 * 4 * b + a * a / a / d + e


def _transposes(be, a, b, c, d, e):
    f1 = ((a.T.T.T + b).T + (c - d.T.T + e).T).T
    f2 = (a + a.T - f1.T.T - b.T).T.T.T - e
    return f1 + f2


def _turned_products(be, a, b, c, d, e):
    # products with transposed views and transposed sub-trees: wrong unless the gradient is turned back
    return a * b.T + be.dot(c.T, d) * (a * e).T + be.sum(be.square(d - e.T), axis=0)


def _activations(be, a, b, c, d, e):
    return be.tanh(a) * be.sig(b) + be.exp(-c) * be.log(be.absolute(d) + 1.5) + be.maximum(a, e) - be.minimum(b, c) \
        + (be.absolute(e) + 0.5) ** 1.5


def _statistics(be, a, b, c, d, e):
    mean = be.mean(a, axis=1)
    var = be.var(a, axis=1)
    return (a - mean) / be.sqrt(var + 1e-3) * be.sum(b, axis=1) + be.sum(c * d) * e


class _NP(object):
    """numpy stand-in for the backend calls used above (keepdims reductions, as op-trees do)."""
    absolute, square, sqrt, exp, log, tanh, maximum, minimum, dot = (
        np.abs, np.square, np.sqrt, np.exp, np.log, np.tanh, np.maximum, np.minimum, np.dot)

    @staticmethod
    def sig(x):
        return 1.0 / (1.0 + np.exp(-x))

    @staticmethod
    def sum(x, axis=None):
        return np.sum(x, axis=axis, keepdims=True)

    @staticmethod
    def max(x, axis=None):
        return np.max(x, axis=axis, keepdims=True)

    @staticmethod
    def min(x, axis=None):
        return np.min(x, axis=axis, keepdims=True)

    @staticmethod
    def mean(x, axis=None):
        return np.mean(x, axis=axis, keepdims=True)

    @staticmethod
    def var(x, axis=None):
        return np.var(x, axis=axis, keepdims=True)


FUNCS = [_arith, _real, _dot, _dot_reductions, _scalar_broadcast, _transposes, _turned_products,
         _activations, _statistics]
FLAGS = ["pos_rand", "neg_rand", "rand"]


def _inputs(flag, dim, seed):
    rng = np.random.RandomState(seed)
    out = []
    for _ in range(5):
        x = rng.uniform(0.25, 1.25, (dim, dim))
        if flag == "neg_rand":
            x = -x
        elif flag == "rand":
            x = x * rng.choice([-1.0, 1.0], (dim, dim))
        out.append(x)
    return out


def _numerical(f, arrays, delta=1e-6):
    grads = []
    for x in arrays:
        g = np.zeros_like(x)
        for idx in np.ndindex(*x.shape):
            keep = x[idx]
            x[idx] = keep + delta
            up = np.sum(f(_NP, *arrays))
            x[idx] = keep - delta
            down = np.sum(f(_NP, *arrays))
            x[idx] = keep
            g[idx] = (up - down) / (2.0 * delta)
        grads.append(g)
    return grads


@pytest.mark.parametrize("flag", FLAGS)
@pytest.mark.parametrize("f", FUNCS, ids=[f.__name__ for f in FUNCS])
def test_gradients_match_central_differences(f, flag):
    if f is _real and flag != "pos_rand":
        pytest.skip("|c + d| has a kink where c + d changes sign")
    arrays = _inputs(flag, 3, seed=FUNCS.index(f))
    be = OracleBackend(rng_seed=0, default_dtype=np.float64)
    tensors = [be.array(x, dtype=np.float64) for x in arrays]
    tree = f(be, *tensors)
    val = be.empty(tree.shape, dtype=np.float64)
    val[:] = tree
    assert np.allclose(val.get(), f(_NP, *arrays), rtol=1e-12, atol=1e-12)
    ad = Autodiff(tree, be)
    got = ad.get_grad_asnumpyarray(tensors)
    want = _numerical(f, arrays)
    for i, (g, w) in enumerate(zip(got, want)):
        assert g.shape == w.shape
        assert np.allclose(g, w, rtol=1e-5, atol=1e-6), (f.__name__, flag, i, np.abs(g - w).max())


def test_next_error_scales_the_gradient_and_unused_tensors_get_zeros():
    be = OracleBackend(rng_seed=0, default_dtype=np.float64)
    rng = np.random.RandomState(1)
    xh, yh, eh = rng.rand(4, 6), rng.rand(4, 1), rng.rand(4, 6)
    x, y, unused = be.array(xh, dtype=np.float64), be.array(yh, dtype=np.float64), be.array(xh, dtype=np.float64)
    err = be.array(eh, dtype=np.float64)
    ad = Autodiff(x * y + be.exp(x), be, next_error=err)
    gx, gy, gu = ad.get_grad_asnumpyarray([x, y, unused])
    assert np.allclose(gx, eh * (yh + np.exp(xh)))
    assert np.allclose(gy, (eh * xh).sum(1, keepdims=True))          # folded back to the (4, 1) operand
    assert not gu.any()
    with pytest.raises(AssertionError):
        Autodiff(x * y, be, next_error=be.array(rng.rand(6, 4), dtype=np.float64))


def test_back_prop_grad_may_overwrite_the_error_buffer():
    """A layer hands its deltas in as next_error and as the buffer for the input gradient
    (neon/layers/layer.py:2646-2650): that buffer is written last."""
    be = OracleBackend(rng_seed=0, default_dtype=np.float64)
    rng = np.random.RandomState(2)
    xh, gh, eh = rng.rand(3, 8), rng.rand(3, 1), rng.rand(3, 8)
    x, gamma = be.array(xh, dtype=np.float64), be.array(gh, dtype=np.float64)
    deltas = be.array(eh, dtype=np.float64)
    ggamma = be.empty((3, 1), dtype=np.float64)
    ad = Autodiff(be.tanh(x) * gamma, be, next_error=deltas)
    ad.back_prop_grad([x, gamma], [deltas, ggamma])
    assert np.allclose(ggamma.get(), (eh * np.tanh(xh)).sum(1, keepdims=True))
    assert np.allclose(deltas.get(), eh * gh * (1 - np.tanh(xh) ** 2))
    with pytest.raises(AssertionError):
        ad.back_prop_grad([gamma], [x])              # a differentiated tensor cannot be a buffer


def test_views_reshapes_keep_their_shape_slices_are_refused():
    be = OracleBackend(rng_seed=0, default_dtype=np.float64)
    xh = np.random.RandomState(3).rand(4, 6)
    x = be.array(xh, dtype=np.float64)
    flat = x.reshape((2, 12))
    (g,) = Autodiff(be.square(flat), be).get_grad_asnumpyarray([flat])
    assert g.shape == (2, 12) and np.allclose(g, 2 * xh.reshape(2, 12))
    with pytest.raises(NotImplementedError):
        Autodiff(be.square(x[:, 0:3]), be)


def test_memoised_constructor_reuses_the_object_for_the_same_tree():
    be = OracleBackend(rng_seed=0)
    x, y = be.array(np.ones((2, 2), np.float32)), be.array(np.ones((2, 2), np.float32))
    tree = x * y + x
    first = autodiff(tree, be)
    assert autodiff(tree, be) is first
    assert autodiff(x * y + x, be) is first             # same structure over the same tensors
    assert autodiff(x * y + y, be) is not first
    err = be.array(np.ones((2, 2), np.float32))
    assert autodiff(tree, be, err) is not first and autodiff(tree, be, err) is autodiff(tree, be, err)


def test_gradient_trees_lower_and_compile_for_the_gpu_backend():
    from tests.dryrun import DryRunBackend
    be = DryRunBackend()
    tensors = [be.empty((64, 48)) for _ in range(5)]
    square = [be.empty((48, 48)) for _ in range(5)]
    for f in FUNCS:
        ts = square if f in (_dot, _dot_reductions, _transposes, _turned_products, _scalar_broadcast, _arith, _real) else tensors
        tree = f(be, *ts)
        ad = Autodiff(tree, be)
        before = be.launches
        grads = [be.empty(t.shape) for t in ts]
        ad.back_prop_grad(ts, grads)
        assert be.launches - before >= len(ts), f.__name__


@pytest.mark.skipif(not os.path.isdir(os.path.join(REFERENCE, "neon", "backends")),
                    reason="no neon checkout on this machine")
@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_same_gradients_as_neons_autodiff_on_its_cpu_backend(dtype):
    """Same trees, same accumulation order: the values are those of neon's class, bit for bit.
    (Functions that multiply by a transposed *view* are left out: there neon adds the view's
    gradient to the tensor's without turning it.)"""
    from tests.golden.make_golden import import_reference_cpu
    NervanaCPU = import_reference_cpu(REFERENCE)
    added = [n for n in ("float", "int") if not hasattr(np, n)]
    for n in added:
        setattr(np, n, {"float": float, "int": int}[n])
    try:
        from neon.backends.autodiff import Autodiff as NeonAutodiff
        theirs_be = NervanaCPU(default_dtype=dtype)
        mine_be = OracleBackend(rng_seed=0, default_dtype=dtype)
        for f in (_arith, _real, _dot, _dot_reductions, _scalar_broadcast, _transposes, _activations, _statistics):
            for flag in FLAGS:
                arrays = [x.astype(dtype) for x in _inputs(flag, 4, seed=7)]
                theirs = [theirs_be.array(x, dtype=dtype) for x in arrays]
                mine = [mine_be.array(x, dtype=dtype) for x in arrays]
                with np.errstate(all="ignore"):
                    want = NeonAutodiff(f(theirs_be, *theirs), theirs_be).get_grad_asnumpyarray(theirs)
                    got = Autodiff(f(mine_be, *mine), mine_be).get_grad_asnumpyarray(mine)
                for i, (g, w) in enumerate(zip(got, want)):
                    assert np.array_equal(g, w, equal_nan=True), (f.__name__, flag, i, np.abs(g - w).max())
    finally:
        for n in added:
            delattr(np, n)
