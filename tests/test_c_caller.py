"""The C ABI from a C program (tests/c_abi_example.c), built with gcc against libb200ew.so."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "neon_b200")


@pytest.fixture(scope="module")
def c_program(tmp_path_factory):
    exe = str(tmp_path_factory.mktemp("cabi") / "c_abi_example")
    subprocess.check_call(["gcc", "-std=c99", "-Wall", "-Werror", "-O1", "-I", os.path.join(ROOT, "include"),
                           os.path.join(ROOT, "tests", "c_abi_example.c"), "-o", exe,
                           "-L", PKG, "-l:libb200ew.so", "-lm", "-Wl,-rpath," + PKG])
    return exe


def test_c_program_links_and_reports_errors_without_a_gpu(c_program):
    res = subprocess.run([c_program, "nogpu"], capture_output=True, text=True, timeout=60)
    assert res.returncode == 0 and "C-ABI-NOGPU-OK" in res.stdout, res.stdout + res.stderr


@pytest.mark.gpu
def test_c_program_runs_reductions_and_a_runtime_compiled_kernel(c_program):
    res = subprocess.run([c_program], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0 and "C-ABI-OK" in res.stdout, res.stdout + res.stderr
