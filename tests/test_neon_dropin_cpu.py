"""
Drop-in check against an unmodified neon checkout (skipped where there is none):
neon's own optimizer, activation and cost code drives this package's backend
object.  No device is needed -- the dry-run backend lowers every statement and
compiles its kernels -- so this pins the interface (names, argument meaning,
lazy scalar op-trees such as ``be.sqrt(float)``), not the numerics, which the
GPU parity tests cover with the same statements.
"""
import os

import numpy as np
import pytest

from oracle import neon_ref

REFERENCE = neon_ref.find_reference() or ""
pytestmark = pytest.mark.skipif(not REFERENCE, reason="no neon source tree on this machine")


@pytest.fixture(scope="module")
def neon_env():
    from tests.golden.make_golden import import_reference_cpu
    import_reference_cpu(REFERENCE)
    from neon import NervanaObject
    from tests.dryrun import DryRunBackend
    be = DryRunBackend()
    be.bsz = 64
    old = NervanaObject.be
    NervanaObject.be = be
    # neon predates numpy 1.20: a few constructors still say np.float / np.int
    added = [n for n in ("float", "int") if not hasattr(np, n)]
    for n in added:
        setattr(np, n, {"float": float, "int": int}[n])
    yield be
    for n in added:
        delattr(np, n)
    NervanaObject.be = old


def test_backend_registers_under_its_name(neon_env):
    import neon_b200.neon_plugin as plugin
    from neon.backends.backend import Backend
    cls = plugin.register()
    assert "b200" in Backend.backend_choices() and Backend.backends["b200"] is cls
    # keywords gen_backend forwards (neon/backends/__init__.py:107-114)
    import inspect
    params = inspect.signature(cls.__init__).parameters
    for kw in ("rng_seed", "default_dtype", "stochastic_round", "device_id", "num_devices",
               "compat_mode", "deterministic"):
        assert kw in params, kw


def test_neon_optimizers_run_unmodified(neon_env):
    """tests/test_optimizer.py:43-66 pattern: a dummy layer, one optimize() call per optimizer."""
    be = neon_env
    from neon.optimizers import Adam, GradientDescentMomentum, RMSProp, Adagrad, Adadelta

    for opt in (Adam(), GradientDescentMomentum(0.1, 0.9), RMSProp(), Adagrad(), Adadelta(),
                Adam(gradient_clip_norm=1.0, gradient_clip_value=0.5)):
        before = len(be.passes)
        param, grad = be.empty((200, 128)), be.empty((200, 128))
        opt.optimize([_Layer(((param, grad), []))], epoch=0)
        assert len(be.passes) > before, type(opt).__name__


class _Layer(object):
    """What get_param_list expects of a layer (neon/optimizers/optimizer.py:30-41)."""

    def __init__(self, params):
        self.params = params

    def get_params(self):
        return self.params


def test_neon_transforms_and_costs_run_unmodified(neon_env):
    be = neon_env
    from neon.transforms import (Rectlin, Tanh, Logistic, Softmax, Explin, Normalizer,
                                 CrossEntropyBinary, CrossEntropyMulti, SumSquared, MeanSquared)
    x, t = be.empty((10, 64)), be.empty((10, 64))
    out = be.empty((10, 64))
    for act in (Rectlin(), Rectlin(slope=0.1), Tanh(), Logistic(), Softmax(), Explin(), Normalizer(divisor=4)):
        before = len(be.passes)
        out[:] = act(x)
        out[:] = act.bprop(x)
        assert len(be.passes) > before, type(act).__name__
    cost_out = be.empty((1, 64))
    for cost in (CrossEntropyBinary(), CrossEntropyMulti(), SumSquared(), MeanSquared()):
        before = len(be.passes)
        cost_out[:] = cost(x, t)
        out[:] = cost.bprop(x, t)
        assert len(be.passes) > before, type(cost).__name__


def test_neon_layers_run_unmodified(neon_env):
    """Bias, Activation, Dropout and BatchNorm layers (neon/layers/layer.py:1376-1530, 1939-2040,
    2352-2580) fprop + bprop through this backend, set up the way neon's layer tests do."""
    be = neon_env
    from neon.initializers import Constant
    from neon.layers import Activation, BatchNorm, Bias, Dropout
    from neon.transforms import Rectlin, Softmax, Tanh
    nin = 10
    x, err = be.empty((nin, be.bsz)), be.empty((nin, be.bsz))
    expected = {"Bias": 2, "Activation": 2, "Dropout": 2, "BatchNorm": 6}
    for make in (lambda: Bias(init=Constant(0.1)), lambda: Activation(Rectlin()), lambda: Activation(Tanh()),
                 lambda: Activation(Softmax()), lambda: Dropout(0.5), lambda: BatchNorm()):
        layer = make()
        layer.configure((nin,))
        layer.prev_layer = True
        layer.allocate()
        layer.set_deltas(type("Deltas", (), {"buffers": [be.iobuf(nin), be.iobuf(nin)]})())
        before = len(be.passes)
        layer.fprop(x)
        layer.bprop(err)
        assert len(be.passes) - before >= expected[type(layer).__name__], type(layer).__name__


def test_neon_array_iterator_runs_unmodified(neon_env):
    """ArrayIterator (neon/data/dataiterator.py:86-202): the dataset sits on the device as
    (examples, features); every minibatch is one copy_transpose of a row slice into the
    (features, batch) buffer plus one onehot statement for the labels, and the last, short
    minibatch wraps around to the first examples."""
    be = neon_env
    # the module file itself: the neon.data package also pulls in readers that need h5py
    import importlib.util
    spec = importlib.util.spec_from_file_location(
        "neon_dataiterator_unmodified", os.path.join(REFERENCE, "neon", "data", "dataiterator.py"))
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    ArrayIterator = module.ArrayIterator
    rng = np.random.RandomState(0)
    ndata, nfeat, nclass = 200, 12, 5
    X = rng.rand(ndata, nfeat).astype(np.float32)
    y = rng.randint(0, nclass, ndata)
    it = ArrayIterator(X, y, nclass=nclass)
    expected = -(-ndata // be.bsz)
    assert it.nbatches == expected
    shuffles, passes, batches = getattr(be, "shuffles", 0), len(be.passes), 0
    for xb, yb in it:
        assert tuple(xb.shape) == (nfeat, be.bsz) and tuple(yb.shape) == (nclass, be.bsz)
        batches += 1
    assert batches == expected          # (the iterator now starts its next epoch after the wrapped part)
    # one transpose + one onehot per minibatch, one more of each for the wrapped part
    assert be.shuffles - shuffles == batches + 1
    assert len(be.passes) - passes == batches + 1


def test_neon_batchnorm_autodiff_layer_uses_the_routed_autodiff(neon_env):
    """BatchNormAutodiff (neon/layers/layer.py:2583-2651) builds its fprop as one op-tree and asks
    ``Autodiff`` for the three gradients on every bprop.  neon's class refuses foreign op-tree
    nodes; after ``register()`` the name the layer module sees dispatches on the backend.  (The
    layer's own ``fprop`` calls ``init_buffers``, which its base class no longer has in this neon
    version, so the test takes the layer's op-tree builder and repeats the three lines of its
    ``bprop``.)"""
    be = neon_env
    import neon_b200.neon_plugin as plugin
    plugin.register()
    import neon.layers.layer as layer_module
    from neon.layers.layer import BatchNormAutodiff
    assert getattr(layer_module.Autodiff, "_b200_router", False)
    nfm = 10
    layer = BatchNormAutodiff()
    layer.x = be.empty((nfm, be.bsz))
    layer.gamma, layer.beta = be.empty((nfm, 1)), be.empty((nfm, 1))
    layer.grad_gamma, layer.grad_beta = be.empty((nfm, 1)), be.empty((nfm, 1))
    layer.deltas = be.empty((nfm, be.bsz))
    layer.fprop_op_tree = layer.get_forward_optree()
    y = be.empty((nfm, be.bsz))
    y[:] = layer.fprop_op_tree
    before = len(be.passes)
    ad = layer_module.Autodiff(layer.fprop_op_tree, be, next_error=layer.deltas)
    ad.back_prop_grad([layer.x, layer.gamma, layer.beta], [layer.deltas, layer.grad_gamma, layer.grad_beta])
    assert len(be.passes) - before >= 3          # grad_gamma, grad_beta, deltas
    assert layer_module.Autodiff(layer.fprop_op_tree, be, next_error=layer.deltas) is ad      # memoised
    # neon's own backends still get neon's class
    from neon.backends.nervanacpu import NervanaCPU
    cpu = NervanaCPU()
    t = cpu.array(np.ones((2, 2), np.float32))
    assert type(layer_module.Autodiff(t * t, cpu)).__module__ == "neon.backends.autodiff"
