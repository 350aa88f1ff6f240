"""
Registers the b200 backend with an installed neon, so that
``neon.backends.gen_backend(backend='b200', ...)`` and the ``-b b200`` command
line choice work (neon keeps its backends in a name -> class registry filled by
``Backend_ABC_Meta``, neon/backends/abstract_backend.py:23-35, and
``gen_backend`` instantiates through it, neon/backends/__init__.py:107-120).

    import neon_b200.neon_plugin as plugin
    plugin.register()
    be = neon.backends.gen_backend(backend='b200', rng_seed=0, batch_size=128)

``register`` also routes ``Autodiff`` as neon's layers see it (``BatchNormAutodiff``,
neon/layers/layer.py:2583-2651) to this package's implementation when the backend is
this one: neon's class only accepts neon's own op-tree node type.
"""


def register():
    from neon.backends.backend import Backend
    from .backend import B200Backend
    Backend.backends["b200"] = B200Backend
    _route_autodiff()
    return B200Backend


def _route_autodiff():
    import neon.backends
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
    layer_module.Autodiff = Autodiff
