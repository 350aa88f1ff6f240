"""GPU test of the fixed-function whole-tensor reduction of the C ABI
(b200_reduce_full): sum / max / min, optionally of |x|, over fp32 and fp16."""
import numpy as np
import pytest

from neon_b200 import runtime as rt

pytestmark = pytest.mark.gpu


def _reduce(values, op, absolute):
    rt.init(0)
    dt = rt.F32 if values.dtype == np.float32 else rt.F16
    src = rt.malloc(values.nbytes)
    out = rt.malloc(4)
    scratch = rt.malloc(rt.reduce_scratch_bytes())
    try:
        rt.memset(scratch, 0, 1, rt.reduce_scratch_bytes())
        rt.memcpy_h2d(src, values.ctypes.data, values.nbytes)
        res = np.zeros(1, np.float32)
        for _ in range(2):                      # second call reuses the scratch as the first left it
            rt.reduce_full(src, dt, values.size, op, absolute, out, scratch)
            rt.memcpy_d2h(res.ctypes.data, out, 4)
        return float(res[0])
    finally:
        for p in (src, out, scratch):
            rt.free(p)


@pytest.mark.parametrize("n", [1, 7, 1000, 4096 * 9 + 3, 1 << 22, (1 << 24) + 5])
@pytest.mark.parametrize("dtype", [np.float32, np.float16])
def test_reduce_full_matches_numpy(n, dtype):
    rng = np.random.RandomState(n % 1000)
    v = rng.uniform(-1, 1, n).astype(dtype)
    v64 = v.astype(np.float64)
    assert abs(_reduce(v, rt.SUM, False) - v64.sum()) <= 1e-5 * np.abs(v64).sum()
    assert _reduce(v, rt.MAX, False) == float(v.max())
    assert _reduce(v, rt.MIN, False) == float(v.min())
    assert _reduce(v, rt.MAX, True) == float(np.abs(v).max())
    assert abs(_reduce(v, rt.SUM, True) - np.abs(v64).sum()) <= 1e-5 * np.abs(v64).sum()


def test_reduce_full_rejects_bad_arguments():
    rt.init(0)
    lib = rt.lib()
    assert lib.b200_reduce_full(0, rt.F32, 10, rt.SUM, 0, 0, 0, 0) == -1
    p = rt.malloc(1024)
    try:
        assert lib.b200_reduce_full(p, rt.I32, 10, rt.SUM, 0, p, p, 0) == -7
        assert lib.b200_reduce_full(p, rt.F32, 0, rt.SUM, 0, p, p, 0) == -1
    finally:
        rt.free(p)
