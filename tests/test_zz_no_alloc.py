"""
GPU test of b200_reduce_full_noalloc, the reduction entry point for callers that
are not allowed to allocate device memory (its scratch is a static array inside
the library).  Collected last on purpose: if it fails under `pytest -x`, every
other test has already run.

The test itself may allocate -- it plays the caller that owns the input and the
4-byte output.  It calls the no-alloc entry point twice in a row through the C
ABI and requires both results to equal what the ordinary entry point
(b200_reduce_full, caller-provided scratch) returns for the same input: the two
run the same kernel with the same launch geometry, so the comparison is exact.
"""
import numpy as np
import pytest

from neon_b200 import runtime as rt

pytestmark = pytest.mark.gpu


def _both(values, op, absolute):
    rt.init(0)
    dt = rt.F32 if values.dtype == np.float32 else rt.F16
    src, out_a, out_b = rt.malloc(values.nbytes), rt.malloc(4), rt.malloc(4)
    scratch = rt.malloc(rt.reduce_scratch_bytes())
    try:
        rt.memset(scratch, 0, 1, rt.reduce_scratch_bytes())
        rt.memcpy_h2d(src, values.ctypes.data, values.nbytes)
        ref = np.zeros(1, np.float32)
        rt.reduce_full(src, dt, values.size, op, absolute, out_a, scratch)
        rt.memcpy_d2h(ref.ctypes.data, out_a, 4)
        got = []
        for i in range(2):                               # two calls in a row share the static scratch
            res = np.full(1, np.nan, np.float32)
            rt.memset(out_b, 0xFF, 1, 4)
            rt.stream_sync()
            allocs_before, free_before = rt.mem_stats()["device_allocs"], rt.mem_info()[0]
            rt.reduce_full_noalloc(src, dt, values.size, op, absolute, out_b)
            rt.stream_sync()
            # the call itself allocated nothing: neither through this library's arena nor,
            # as far as the driver's free-memory figure shows, any other way (after the first
            # call, which may load the library's device code on this GPU)
            assert rt.mem_stats()["device_allocs"] == allocs_before
            if i == 1:
                assert rt.mem_info()[0] == free_before
            rt.memcpy_d2h(res.ctypes.data, out_b, 4)
            got.append(float(res[0]))
        return float(ref[0]), got
    finally:
        for p in (src, out_a, out_b, scratch):
            rt.free(p)


@pytest.mark.parametrize("n", [5, 4096 * 9 + 3, (1 << 24) + 5])
@pytest.mark.parametrize("dtype", [np.float32, np.float16])
def test_noalloc_reduction_equals_ordinary_entry_point_twice(n, dtype):
    v = np.random.RandomState(n % 997).uniform(-1, 1, n).astype(dtype)
    for op, absolute in ((rt.SUM, False), (rt.MAX, True), (rt.MIN, False)):
        ref, got = _both(v, op, absolute)
        assert got[0] == ref and got[1] == ref, (op, absolute, ref, got)
    # and the values are right, not merely consistent
    v64 = v.astype(np.float64)
    ref, got = _both(v, rt.SUM, False)
    assert abs(got[1] - v64.sum()) <= 1e-5 * np.abs(v64).sum()
    assert _both(v, rt.MAX, True)[1][1] == float(np.abs(v).max().astype(np.float32))
    assert _both(v, rt.MIN, False)[1][1] == float(v.min().astype(np.float32))
    assert _both(v, rt.MAX, False)[1][1] == float(v.max().astype(np.float32))


def test_noalloc_refuses_inputs_beyond_its_maximum():
    rt.init(0)
    lib = rt.lib()
    limit = int(lib.b200_reduce_full_noalloc_max_count())
    assert limit == 1 << 32
    p = rt.malloc(64)
    try:
        assert lib.b200_reduce_full_noalloc(p, rt.F32, limit + 1, rt.SUM, 0, p, 0) == -1
        assert "maximum" in rt.last_error()
        assert lib.b200_reduce_full_noalloc(p, rt.I32, 8, rt.SUM, 0, p, 0) == -7
    finally:
        rt.free(p)
