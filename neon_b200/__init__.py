"""
neon_b200 -- a B200-native backend for neon's compound op-tree tensor engine.

    from neon_b200 import gen_backend
    be = gen_backend(backend="b200", rng_seed=0)
    x = be.array(host_array)
    out = be.empty((1, x.shape[1]))
    out[:] = be.sum(be.exp(x - be.max(x, axis=0)), axis=0)     # fused kernels on the GPU
"""

from .optree import OpCollection, OpTreeNode, Tensor          # noqa: F401


def gen_backend(*args, **kwargs):
    from .backend import gen_backend as _gen
    return _gen(*args, **kwargs)


def Autodiff(op_tree, be, next_error=None):
    """Symbolic gradients of an op-tree (see neon_b200/autodiff.py)."""
    from .autodiff import Autodiff as _Autodiff
    return _Autodiff(op_tree, be, next_error)


def __getattr__(name):
    if name in ("B200Backend", "B200Tensor"):
        from . import backend, tensor
        return {"B200Backend": backend.B200Backend, "B200Tensor": tensor.B200Tensor}[name]
    raise AttributeError(name)
