"""
Registers the b200 backend with an installed neon, so that
``neon.backends.gen_backend(backend='b200', ...)`` and the ``-b b200`` command
line choice work (neon keeps its backends in a name -> class registry filled by
``Backend_ABC_Meta``, neon/backends/abstract_backend.py:23-35, and
``gen_backend`` instantiates through it, neon/backends/__init__.py:107-120).

    import neon_b200.neon_plugin as plugin
    plugin.register()
    be = neon.backends.gen_backend(backend='b200', rng_seed=0, batch_size=128)

What ``register`` does besides the registry entry:

* neon code tests ``isinstance(x, neon.backends.backend.Tensor)`` in a few places
  (layer configuration, initializers, the helpers of neon's tests), so this
  package's tensor base class is re-parented onto neon's ``Tensor``;
* ``Autodiff`` as neon's layers see it (``BatchNormAutodiff``,
  neon/layers/layer.py:2583-2651) is routed to this package's implementation when
  the backend is this one: neon's class only accepts neon's own op-tree node type;
* with ``as_gpu=True`` the backend also answers to the name ``'gpu'`` and, where
  neon's own ``nervanagpu`` module cannot be imported (it needs pycuda), a module
  of that name is provided whose ``NervanaGPU`` / ``GPUTensor`` are this package's
  classes, and neon's device queries (``neon.backends.util.check_gpu``, pycuda based) are
  answered by this package's runtime.  That is how neon's own test files, which ask for
  ``'gpu'``, are run against this backend.
"""

import sys
import types


def register(as_gpu=False, backend_cls=None):
    from neon.backends.backend import Backend
    if backend_cls is None:
        from .backend import B200Backend as backend_cls
    _adopt_tensor_base()
    Backend.backends["b200"] = backend_cls
    _route_autodiff()
    if as_gpu:
        Backend.backends["gpu"] = backend_cls
        try:
            from neon.backends import nervanagpu                      # noqa: F401
        except ImportError:
            mod = types.ModuleType("neon.backends.nervanagpu")
            mod.NervanaGPU = backend_cls
            mod.GPUTensor = getattr(backend_cls, "tensor_cls", None)
            sys.modules["neon.backends.nervanagpu"] = mod
            import neon.backends
            neon.backends.nervanagpu = mod
        _answer_device_queries()
    return backend_cls


def _answer_device_queries():
    """neon asks pycuda for the device count and compute capability
    (neon/backends/util/check_gpu.py:20-100; its tests call these before touching a GPU
    backend).  Without pycuda both answer 0; let them ask this package's runtime instead."""
    from neon.backends.util import check_gpu
    from . import runtime as rt

    def get_device_count(verbose=False):
        return rt.device_count()

    def get_compute_capability(device_id=None, verbose=False):
        ids = range(rt.device_count()) if device_id is None else \
            ([device_id] if isinstance(device_id, int) else list(device_id))
        caps = []
        for i in ids:
            props = rt.device_props(i)
            caps.append(props.cc_major + props.cc_minor / 10.0)
        return max(caps) if caps else 0

    check_gpu.get_device_count = get_device_count
    check_gpu.get_compute_capability = get_compute_capability


def _adopt_tensor_base():
    """Make neon's Tensor a base class of this package's Tensor (after its own operator
    mix-in, so arithmetic keeps building this package's op-tree nodes)."""
    from neon.backends.backend import Tensor as NeonTensor
    from .optree import Tensor, _Operators
    if NeonTensor not in Tensor.__mro__:
        Tensor.__bases__ = (_Operators, NeonTensor)


def _route_autodiff():
    import neon.backends
    import neon.backends.autodiff
    import neon.layers.layer as layer_module
    from .autodiff import autodiff
    from .optree import OpTreeBackend
    theirs = neon.backends.Autodiff
    if getattr(theirs, "_b200_router", False):
        return

    def Autodiff(op_tree, be, next_error=None):
        if isinstance(be, OpTreeBackend):
            return autodiff(op_tree, be, next_error)
        return theirs(op_tree, be, next_error)
    Autodiff._b200_router = True
    neon.backends.Autodiff = Autodiff
    neon.backends.autodiff.Autodiff = Autodiff
    layer_module.Autodiff = Autodiff
