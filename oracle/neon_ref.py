"""
Locate and import an unmodified neon source tree.  TEST INFRASTRUCTURE: used by
the tests, the golden-vector generator and the CPU-baseline leg of bench.py;
nothing under neon_b200/ imports it.

Where neon is looked for, in order:

1. ``$NEON_REFERENCE`` (a checkout: the directory that holds ``neon/`` and ``tests/``);
2. ``oracle/_ref/`` -- a copy made by ``python oracle/make_ref.py`` (kept out of
   version control; it travels with the working tree to machines that have no
   checkout);
3. a directory named ``reference`` beside this repository.

neon targets python 2.7/3.5 and numpy 1.13.  Three modules it imports are not
installed here and have nothing to do with its numpy backend, so stand-ins go
into ``sys.modules`` before the import: ``future`` (py2/3 helpers), ``appdirs``
(cache-directory lookup) and the build-generated ``neon.version``.  A few of
its constructors still say ``np.float`` / ``np.int``, removed in numpy 1.24;
``numpy_compat()`` puts the aliases back for the duration of a test.
"""

import contextlib
import os
import sys
import types

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


def _is_checkout(path):
    return bool(path) and os.path.isdir(os.path.join(path, "neon", "backends"))


def find_reference():
    """Path of the neon tree to use, or None."""
    for cand in (os.environ.get("NEON_REFERENCE"), os.path.join(HERE, "_ref"),
                 os.path.join(os.path.dirname(ROOT), "reference")):
        if _is_checkout(cand):
            return cand
    return None


def install_shims():
    def mod(name, **attrs):
        m = types.ModuleType(name)
        m.__dict__.update(attrs)
        sys.modules[name] = m
        return m

    def with_metaclass(meta, *bases):
        return meta("_with_metaclass_base", bases or (object,), {})

    if "future" not in sys.modules:
        fut = mod("future")
        fut.utils = mod("future.utils", with_metaclass=with_metaclass, native_str=str,
                        native=lambda x: x)
        fut.standard_library = mod("future.standard_library", install_aliases=lambda: None)
        fut.builtins = mod("future.builtins")
    if "appdirs" not in sys.modules:
        mod("appdirs", user_cache_dir=lambda *a, **k: "/tmp/neon_cache",
            user_data_dir=lambda *a, **k: "/tmp/neon_data")
    if "neon.version" not in sys.modules:
        mod("neon.version", VERSION="reference-checkout", SHORT_VERSION="ref")


def import_neon(path=None):
    """Make ``import neon`` resolve to the tree at ``path`` (default: ``find_reference()``);
    returns the path.  Raises ImportError when there is no tree."""
    path = path or find_reference()
    if not _is_checkout(path):
        raise ImportError("no neon source tree found (set NEON_REFERENCE or run oracle/make_ref.py)")
    install_shims()
    if path not in sys.path:
        sys.path.insert(0, path)
    import neon                                                    # noqa: F401
    return path


def import_reference_cpu(path=None):
    """neon's NervanaCPU class from the tree at ``path``."""
    import_neon(path)
    from neon.backends.nervanacpu import NervanaCPU
    return NervanaCPU


@contextlib.contextmanager
def numpy_compat():
    """``np.float`` / ``np.int`` as neon's older code expects them."""
    added = [n for n in ("float", "int", "bool") if not hasattr(np, n)]
    for n in added:
        setattr(np, n, {"float": float, "int": int, "bool": bool}[n])
    try:
        yield
    finally:
        for n in added:
            delattr(np, n)
