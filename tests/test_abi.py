"""CPU tests of the C-ABI boundary: the library loads without a driver, exports
every symbol include/b200ew.h declares, and reports errors instead of crashing."""
import os
import re

import pytest

from neon_b200 import runtime as rt

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "b200ew.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_agree():
    declared = _declared()
    assert declared, "no declarations found"
    assert sorted(rt.SIGNATURES) == declared


def test_library_exports_every_declared_symbol():
    lib = rt.lib()
    for name in _declared():
        assert hasattr(lib, name), name
    assert lib.b200_version() >= 100


def test_errors_are_reported_not_raised_in_c():
    lib = rt.lib()
    assert lib.b200_device_count(None) == -1            # B200_ERR_INVALID
    assert "null" in rt.last_error()
    assert lib.b200_free(0) == 0
    with pytest.raises(rt.B200Error):
        rt.check(lib.b200_launch(0, 1, 1, 1, 1, 1, 1, 0, 0, None, 0, 1, 0))


def test_rng_state_round_trip_and_key_schedule():
    from oracle import sround
    rt.rng_seed(1234)
    keys = [rt.rng_next_key() for _ in range(4)]
    assert keys == [sround.launch_key(1234, i) for i in range(4)]
    assert rt.rng_get_state() == (1234, 4)
    rt.rng_set_state((1234, 1))
    assert rt.rng_next_key() == keys[1]


def test_nvrtc_reports_compile_errors():
    with pytest.raises(rt.B200Error) as e:
        rt.nvrtc_compile('#include "optree_templates.cuh"\nthis is not CUDA\n')
    assert e.value.status == -3
