"""
Generate tests/golden/optree_golden.npz from the real neon NervanaCPU backend.

Run where a neon source checkout is available (the outputs are committed so that
the comparisons also work on a machine without one):

    python tests/golden/make_golden.py [/path/to/neon/checkout]

(default: $NEON_REFERENCE, else a directory named "reference" beside this repository)

neon is imported unmodified from the checkout (oracle/neon_ref.py supplies stand-ins
for three modules it wants that are not installed and have nothing to do with the
numpy backend).

For every case of ``tests/cases.py::standard_cases`` the script runs the case on
``NervanaCPU`` with float32 and with float64 tensors and stores a fingerprint of
each resulting tensor (the whole array when small, else a strided sample plus
float64 sum and abs-sum) under ``<case>/<dtype>/<tensor>/<field>``.

A second file, ``neon_callers_golden.npz``, holds the float64 NervanaCPU results of
``tests/neon_cases.py`` -- neon's own optimizers, layers, costs and
``compound_fprop_bn`` / ``compound_bprop_bn`` run on seeded inputs -- under
``<case>/<array>/<field>``.
"""

import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))


def import_reference_cpu(path=None):
    """Import neon's NervanaCPU from the checkout at ``path`` (see oracle/neon_ref.py)."""
    from oracle import neon_ref
    return neon_ref.import_reference_cpu(path)


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

    # neon's own optimizers, layers, costs and batch-norm entry points driving NervanaCPU (float64)
    from oracle.neon_ref import numpy_compat
    from tests.neon_cases import neon_caller_cases
    store = {}
    with numpy_compat():
        for name, run in neon_caller_cases().items():
            with np.errstate(all="ignore"):
                res = run(NervanaCPU(default_dtype=np.float64, rng_seed=0))
            for k, arr in res.items():
                for field, val in summarize(arr).items():
                    store["%s/%s/%s" % (name, k, field)] = val
    out = os.path.join(HERE, "neon_callers_golden.npz")
    np.savez_compressed(out, **store)
    print("wrote %s: %d entries, %.1f KiB" % (out, len(store), os.path.getsize(out) / 1024.))


if __name__ == "__main__":
    main()
