"""
Generate tests/golden/optree_golden.npz from the real neon NervanaCPU backend.

Run where a neon source checkout is available (it cannot run on a machine
without one, which is why the outputs are committed):

    python tests/golden/make_golden.py [/path/to/neon/checkout]

(default: $NEON_REFERENCE, else a directory named "reference" beside this repository)

neon is imported unmodified from the checkout.  Three modules it wants are not
installed and have nothing to do with the numpy backend, so stand-ins are put in
``sys.modules`` before the import: ``future`` (py2/3 helpers), ``appdirs``
(cache-directory lookup) and the build-generated ``neon.version``.

For every case of ``tests/cases.py::standard_cases`` the script runs the case on
``NervanaCPU`` with float32 and with float64 tensors and stores a fingerprint of
each resulting tensor (the whole array when small, else a strided sample plus
float64 sum and abs-sum) under ``<case>/<dtype>/<tensor>/<field>``.
"""

import os
import sys
import types

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))


def import_reference_cpu(path):
    """Import neon's NervanaCPU from the checkout at ``path``."""
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
    mod("neon.version", VERSION="reference-checkout", SHORT_VERSION="ref")
    if path not in sys.path:
        sys.path.insert(0, path)
    from neon.backends.nervanacpu import NervanaCPU
    return NervanaCPU


def main():
    default = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(HERE))), "reference")
    path = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("NEON_REFERENCE", default)
    NervanaCPU = import_reference_cpu(path)
    from tests.cases import run_case, standard_cases, summarize

    store = {}
    for case in standard_cases():
        for dt in (np.float32, np.float64):
            be = NervanaCPU(default_dtype=dt)
            with np.errstate(all="ignore"):
                res = run_case(be, case, compute_dtype=dt)
            for k, arr in res.items():
                if k.startswith("grad"):
                    continue
                for field, val in summarize(arr).items():
                    store["%s/%s/%s/%s" % (case.name, np.dtype(dt).name, k, field)] = val
    out = os.path.join(HERE, "optree_golden.npz")
    np.savez_compressed(out, **store)
    print("wrote %s: %d entries, %.1f KiB" % (out, len(store), os.path.getsize(out) / 1024.))


if __name__ == "__main__":
    main()
