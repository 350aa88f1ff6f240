"""The caching arena next to a caller's own stream: a freed block is handed out again only after
the work queued on every stream at the time of the free has run."""
import ctypes

import pytest

from neon_b200 import runtime as rt

pytestmark = pytest.mark.gpu


def test_a_block_freed_under_a_second_stream_waits_for_that_stream(b200):
    lib = rt.lib()
    nbytes = (1 << 28) + (6 << 20)            # a size no other test leaves cached blocks of
    # without other streams, reuse is immediate (ordered by the library's stream)
    a = rt.malloc(nbytes)
    rt.free(a)
    again = rt.malloc(nbytes)
    assert again == a
    rt.free(again)

    stream = ctypes.c_uint64(0)
    rt.check(lib.b200_stream_create(ctypes.byref(stream)))
    try:
        a = rt.malloc(nbytes)
        for _ in range(400):                       # ~20 ms of fills queued on the caller's stream
            rt.memset(a, 1, 1, nbytes, stream.value)
        rt.free(a)
        cached = rt.mem_stats()["cached"]
        b = rt.malloc(nbytes)                      # the fills are still running: a must stay parked
        assert b != a and rt.mem_stats()["cached"] == cached
        rt.check(lib.b200_stream_sync(stream.value))
        rt.free(b)
        rt.stream_sync(0)
        c = rt.malloc(nbytes)                      # both parked blocks have become free by now
        assert c in (a, b)
        rt.free(c)
    finally:
        rt.check(lib.b200_stream_destroy(stream.value))
    # the stream is gone: a freed block is on the free list at once again
    d = rt.malloc(nbytes)
    cached = rt.mem_stats()["cached"]
    rt.free(d)
    assert rt.mem_stats()["cached"] == cached + nbytes
