"""
Registers the b200 backend with an installed neon, so that
``neon.backends.gen_backend(backend='b200', ...)`` and the ``-b b200`` command
line choice work (neon keeps its backends in a name -> class registry filled by
``Backend_ABC_Meta``, neon/backends/abstract_backend.py:23-35, and
``gen_backend`` instantiates through it, neon/backends/__init__.py:107-120).

    import neon_b200.neon_plugin as plugin
    plugin.register()
    be = neon.backends.gen_backend(backend='b200', rng_seed=0, batch_size=128)
"""


def register():
    from neon.backends.backend import Backend
    from .backend import B200Backend
    Backend.backends["b200"] = B200Backend
    return B200Backend
