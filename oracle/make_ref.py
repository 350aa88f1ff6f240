"""
Copy the python sources of a neon checkout into ``oracle/_ref/`` so that the
unmodified reference (its NervanaCPU backend, optimizers, layers, and its own
test files for the op-tree path) can be imported on machines that have this
working tree but no checkout.  TEST INFRASTRUCTURE; ``oracle/_ref/`` is not
version controlled and nothing under ``neon_b200/`` reads it.

    python oracle/make_ref.py [/path/to/neon/checkout]

(default: $NEON_REFERENCE, else a directory named "reference" beside this
repository).  Only ``*.py`` files are copied, byte for byte; neon's test
directory keeps its own ``conftest.py`` and ``utils.py``.
"""

import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
DEST = os.path.join(HERE, "_ref")

# neon's tests of the op-tree path and of its direct callers (plus what they import)
TEST_FILES = [
    "conftest.py", "utils.py",
    "test_backend_reduction.py", "test_backend_compound_optree.py", "test_backend_tensor.py",
    "test_backend_sr.py", "test_backend_randomstate.py", "test_backend_copy_transpose.py",
    "test_backend_hist.py", "test_backend_autodiff.py", "test_backend_autodiff_extra.py",
    "test_optimizer.py", "test_activations.py", "test_costs.py", "test_schedule.py",
    "test_initializers.py", "test_misc.py", "test_gradient_bias.py", "test_gradient_batchnorm.py", "grad_funcs.py",
]


def copy_py_tree(src, dst):
    n = 0
    for base, dirs, files in os.walk(src):
        dirs[:] = [d for d in dirs if d != "__pycache__"]
        rel = os.path.relpath(base, src)
        for f in files:
            if f.endswith(".py"):
                os.makedirs(os.path.join(dst, rel), exist_ok=True)
                shutil.copyfile(os.path.join(base, f), os.path.join(dst, rel, f))
                n += 1
    return n


def make_ref(src=None):
    src = src or os.environ.get("NEON_REFERENCE") or os.path.join(os.path.dirname(ROOT), "reference")
    if not os.path.isdir(os.path.join(src, "neon", "backends")):
        raise SystemExit("no neon checkout at %s" % src)
    if os.path.isdir(DEST):
        shutil.rmtree(DEST)
    n = copy_py_tree(os.path.join(src, "neon"), os.path.join(DEST, "neon"))
    os.makedirs(os.path.join(DEST, "tests"), exist_ok=True)
    for f in TEST_FILES:
        p = os.path.join(src, "tests", f)
        if os.path.isfile(p):
            shutil.copyfile(p, os.path.join(DEST, "tests", f))
            n += 1
    return n


if __name__ == "__main__":
    count = make_ref(sys.argv[1] if len(sys.argv) > 1 else None)
    print("copied %d python files into %s" % (count, DEST))
