"""
pytest plugin that lets neon's own test files run against this package:

    python -m pytest -p tests.neon_conformance <neon tree>/tests/test_backend_reduction.py -m hasgpu

Loaded (``-p``) before neon's ``tests/conftest.py`` is imported, it makes
``import neon`` work on this interpreter (see oracle/neon_ref.py) and registers
this package's backend under the names ``'b200'`` and ``'gpu'``, so neon's
fixtures -- ``gen_backend(backend='gpu', ...)`` and
``neon.backends.nervanagpu.NervanaGPU(...)`` -- hand its tests a b200 backend
where they expect NervanaGPU.  neon's files are used as they are.

``B200_CONFORMANCE_EXECUTOR=oracle`` registers the numpy checker instead (it
shares this package's op-tree front end); that is how the harness itself is
tested on machines without a GPU.
"""

import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from oracle import neon_ref                                            # noqa: E402

neon_ref.import_neon()
for _name, _type in (("float", float), ("int", int), ("bool", bool)):
    if not hasattr(np, _name):                       # neon predates numpy 1.24
        setattr(np, _name, _type)

import neon_b200.neon_plugin as _plugin                                 # noqa: E402

if os.environ.get("B200_CONFORMANCE_EXECUTOR", "b200") == "oracle":
    from oracle.numpy_backend import OracleBackend, OracleTensor

    class _CheckerAsBackend(OracleBackend):
        """The numpy checker with the few attributes neon's fixtures touch on a GPU backend."""
        tensor_cls = OracleTensor
        enable_winograd = False

        def cleanup_backend(self):
            pass

    _plugin.register(as_gpu=True, backend_cls=_CheckerAsBackend)
else:
    _plugin.register(as_gpu=True)


def pytest_configure(config):
    for m in ("hasgpu", "unsupported"):
        config.addinivalue_line("markers", "%s: marker used by neon's tests" % m)


def _backend_of(value):
    if isinstance(value, str):
        return value
    if isinstance(value, tuple) and value and isinstance(value[0], str):
        return value[0]
    return None


def pytest_collection_modifyitems(config, items):
    """Keep the tests that exercise the GPU backend: those whose backend fixture is
    parametrised with 'gpu', and those neon marks ``hasgpu``; drop the runs of the same
    tests on neon's own cpu / mkl backends (the mkl engine is not built here)."""
    keep, drop = [], []
    for item in items:
        names = set(getattr(item, "fixturenames", ()))
        params = getattr(getattr(item, "callspec", None), "params", {})
        backends = set(b for b in (_backend_of(v) for v in params.values()) if b in ("gpu", "cpu", "mkl"))
        on_gpu = "gpu" in backends or (item.get_closest_marker("hasgpu") is not None and not backends)
        other = backends - {"gpu"} or any("mkl" in n or n.startswith("backend_cpu") for n in names)
        (keep if on_gpu and not other else drop).append(item)
    if drop:
        config.hook.pytest_deselected(items=drop)
        items[:] = keep


@pytest.hookimpl(trylast=True)
def pytest_runtest_setup(item):
    """neon's older test classes prepare themselves in a plain ``setup`` method (the nose
    convention), which current pytest no longer calls: call it once the fixtures are up."""
    inst = getattr(item, "instance", None)
    prepare = getattr(inst, "setup", None)
    if inst is not None and callable(prepare) and not hasattr(inst, "setup_method"):
        prepare()

