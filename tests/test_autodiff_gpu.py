"""
Gradient op-trees evaluated on the B200 backend against the same trees on the
float64 oracle backend: they are ordinary statements (fused element-wise,
reductions, dot, transposes), so the parity bounds are those of the other tests.
"""
import numpy as np
import pytest

from neon_b200.autodiff import Autodiff
from oracle.numpy_backend import OracleBackend
from tests import test_autodiff as cpu

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("f", cpu.FUNCS, ids=[f.__name__ for f in cpu.FUNCS])
def test_gradients_on_the_gpu_match_the_oracle(b200, f):
    be = b200
    oracle = OracleBackend(rng_seed=0, default_dtype=np.float64)
    arrays = [x.astype(np.float32) for x in cpu._inputs("pos_rand" if f is cpu._real else "rand", 64, seed=11)]
    mine = [be.array(x) for x in arrays]
    theirs = [oracle.array(x.astype(np.float64), dtype=np.float64) for x in arrays]
    got = Autodiff(f(be, *mine), be).get_grad_asnumpyarray(mine)
    want = Autodiff(f(oracle, *theirs), oracle).get_grad_asnumpyarray(theirs)
    for i, (g, w) in enumerate(zip(got, want)):
        scale = max(1.0, float(np.abs(w).max()))
        assert np.allclose(g, w, rtol=2e-4, atol=2e-4 * scale), (f.__name__, i, np.abs(g - w).max())


def test_batchnorm_gradients_through_back_prop_grad(b200):
    """The statement of cfg4 differentiated: deltas, grad_gamma and grad_beta of
    y = (x - mean) / sqrt(var + eps) * gamma + beta, written into the layer's buffers with the
    error buffer reused for the input gradient."""
    be = b200
    rng = np.random.RandomState(5)
    nfm, n = 32, 4096
    xh = (1 + 2 * rng.randn(nfm, n)).astype(np.float32)
    gh, bh = rng.uniform(.5, 1.5, (nfm, 1)).astype(np.float32), rng.uniform(.5, 1.5, (nfm, 1)).astype(np.float32)
    eh = rng.randn(nfm, n).astype(np.float32)
    x, gamma, beta, deltas = be.array(xh), be.array(gh), be.array(bh), be.array(eh)
    ggamma, gbeta = be.empty((nfm, 1)), be.empty((nfm, 1))
    tree = (x - be.mean(x, axis=1)) / be.sqrt(be.var(x, axis=1) + 1e-3) * gamma + beta
    ad = Autodiff(tree, be, next_error=deltas)
    ad.back_prop_grad([x, gamma, beta], [deltas, ggamma, gbeta])
    x64, e64 = xh.astype(np.float64), eh.astype(np.float64)
    mu, var = x64.mean(1, keepdims=True), x64.var(1, keepdims=True)
    rstd = 1.0 / np.sqrt(var + 1e-3)
    xhat = (x64 - mu) * rstd
    want_gbeta = e64.sum(1, keepdims=True)
    want_ggamma = (e64 * xhat).sum(1, keepdims=True)
    want_dx = gh * rstd * (e64 - want_gbeta / n - xhat * want_ggamma / n)
    assert np.allclose(gbeta.get(), want_gbeta, rtol=1e-4, atol=1e-3)
    assert np.allclose(ggamma.get(), want_ggamma, rtol=1e-4, atol=1e-3)
    assert np.allclose(deltas.get(), want_dx, rtol=1e-3, atol=1e-4)
