"""
neon's own test files, unmodified, run against this package.

Each file of neon's ``tests/`` directory that exercises the op-tree path or its
direct callers is handed to a pytest child process with ``-p tests.neon_conformance``
(see that module): neon's ``conftest.py`` then builds its 'gpu' backends from this
package, and the plugin keeps the GPU-backend runs of every test while dropping the
runs on neon's own cpu / mkl backends.

* GPU tests: executor = the b200 backend.
* CPU tests: executor = the numpy checker, which shares this package's op-tree
  front end -- a check of the front end (shape inference, operators, views, the
  lazy scalar trees optimizers build) and of this harness.

``test_backend_autodiff_extra.py`` prepares its test class in a nose-style ``setup`` method,
which current pytest no longer calls; the plugin calls it.  Files not run: everything about
GEMM / convolution / pooling / recurrent layers (outside the op-tree path).
"""
import os
import re
import subprocess
import sys

import pytest

from oracle import neon_ref

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = neon_ref.find_reference()
pytestmark = pytest.mark.skipif(REF is None or not os.path.isfile(os.path.join(REF or "", "tests", "conftest.py")),
                                reason="no neon source tree with its tests on this machine")

# file -> (least number of tests that must run and pass on the b200 backend, pytest -k filter or None)
GPU_FILES = {
    "test_backend_reduction.py": (48, None),
    "test_backend_compound_optree.py": (12, None),
    "test_backend_tensor.py": (32, None),
    "test_backend_sr.py": (1, None),
    "test_backend_randomstate.py": (2, None),
    "test_backend_copy_transpose.py": (8, None),
    "test_backend_hist.py": (9, None),
    "test_backend_autodiff.py": (36, None),
    "test_backend_autodiff_extra.py": (7, None),
    "test_optimizer.py": (12, None),
    "test_activations.py": (24, None),
    "test_costs.py": (25, None),
    "test_initializers.py": (20, None),
    "test_misc.py": (1, None),                      # dropout masks from the device generator
    "test_schedule.py": (5, None),
}
# what the numpy checker can execute (no random numbers, histograms, rounding modes, eager shift)
CPU_FILES = {
    "test_backend_reduction.py": (48, None),
    "test_backend_compound_optree.py": (12, None),
    "test_backend_tensor.py": (32, None),
    "test_backend_copy_transpose.py": (8, None),
    "test_backend_autodiff.py": (36, None),
    "test_backend_autodiff_extra.py": (7, None),
    "test_optimizer.py": (12, None),
    "test_activations.py": (23, "not sign"),
    "test_costs.py": (25, None),
    "test_initializers.py": (20, None),
    "test_schedule.py": (4, "not shift"),
}


def run_neon_test_file(name, executor, keyword=None, timeout=1500):
    """Returns (passed, failed + errors, tail of the child's output)."""
    cmd = [sys.executable, "-m", "pytest", "-p", "tests.neon_conformance", os.path.join(REF, "tests", name),
           "-q", "--rootdir", REF, "-p", "no:cacheprovider", "-W", "ignore", "--tb=short"]
    if keyword:
        cmd += ["-k", keyword]
    env = dict(os.environ, B200_CONFORMANCE_EXECUTOR=executor, NEON_REFERENCE=REF)
    proc = subprocess.run(cmd, cwd=ROOT, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                          text=True, timeout=timeout)
    out = proc.stdout
    summary = [ln for ln in out.splitlines() if re.search(r"\d+ (passed|failed|error)", ln)]
    last = summary[-1] if summary else ""

    def count(word):
        m = re.search(r"(\d+) %s" % word, last)
        return int(m.group(1)) if m else 0
    return count("passed"), count("failed") + count("error"), out[-6000:]


@pytest.mark.parametrize("name", sorted(CPU_FILES))
def test_neon_test_file_on_the_front_end_with_the_checker(name):
    least, keyword = CPU_FILES[name]
    passed, bad, tail = run_neon_test_file(name, "oracle", keyword)
    assert bad == 0 and passed >= least, tail


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(GPU_FILES))
def test_neon_test_file_on_b200(name):
    least, keyword = GPU_FILES[name]
    passed, bad, tail = run_neon_test_file(name, "b200", keyword)
    assert bad == 0 and passed >= least, tail
