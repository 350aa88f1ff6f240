"""
ctypes binding of libb200ew.so (declared in include/b200ew.h).

The Python backend reaches the GPU only through this module -- the role pycuda
plays for neon's NervanaGPU.  A missing library or a failing call raises; there
is no CPU fallback.
"""

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libb200ew.so")
TEMPLATE_PATH = os.path.join(_HERE, "csrc", "optree_templates.cuh")

F32, F16, BF16, I32, U32, I16, U16, I8, U8 = range(9)
SUM, MAX, MIN = range(3)

u64, i32, u32 = C.c_uint64, C.c_int32, C.c_uint32
P = C.POINTER


class DeviceProps(C.Structure):
    _fields_ = [("sm_count", i32), ("cc_major", i32), ("cc_minor", i32),
                ("max_smem_per_block", i32), ("max_threads_per_sm", i32),
                ("l2_bytes", i32), ("clock_khz", i32), ("reserved", i32),
                ("total_mem", u64), ("name", C.c_char * 64)]


# name -> (restype, argtypes); everything include/b200ew.h declares
SIGNATURES = {
    "b200_version": (i32, []),
    "b200_last_error": (C.c_size_t, [C.c_char_p, C.c_size_t]),
    "b200_device_count": (i32, [P(i32)]),
    "b200_init": (i32, [i32]),
    "b200_shutdown": (i32, []),
    "b200_device_props_get": (i32, [i32, P(DeviceProps)]),
    "b200_mem_info": (i32, [P(u64), P(u64)]),
    "b200_malloc": (i32, [u64, P(u64)]),
    "b200_free": (i32, [u64]),
    "b200_mem_trim": (i32, []),
    "b200_mem_stats": (i32, [P(u64), P(u64), P(u64), P(u64)]),
    "b200_host_alloc": (i32, [u64, P(C.c_void_p)]),
    "b200_host_free": (i32, [C.c_void_p]),
    "b200_memcpy_h2d": (i32, [u64, C.c_void_p, u64, u64, i32]),
    "b200_memcpy_d2h": (i32, [C.c_void_p, u64, u64, u64, i32]),
    "b200_memcpy_d2d": (i32, [u64, u64, u64, u64]),
    "b200_memset": (i32, [u64, u32, i32, u64, u64]),
    "b200_stream_create": (i32, [P(u64)]),
    "b200_stream_destroy": (i32, [u64]),
    "b200_stream_sync": (i32, [u64]),
    "b200_stream_wait_event": (i32, [u64, u64]),
    "b200_default_stream": (i32, [P(u64)]),
    "b200_event_create": (i32, [P(u64)]),
    "b200_event_destroy": (i32, [u64]),
    "b200_event_record": (i32, [u64, u64]),
    "b200_event_sync": (i32, [u64]),
    "b200_event_elapsed_ms": (i32, [u64, u64, P(C.c_float)]),
    "b200_register_header": (i32, [C.c_char_p, C.c_char_p]),
    "b200_nvrtc_compile": (i32, [C.c_char_p, P(C.c_char_p), i32, P(C.c_void_p), P(u64), P(i32)]),
    "b200_buffer_free": (i32, [C.c_void_p]),
    "b200_kernel_get": (i32, [C.c_char_p, C.c_char_p, P(C.c_char_p), i32, P(u64)]),
    "b200_kernel_max_smem": (i32, [u64, i32]),
    "b200_kernel_occupancy": (i32, [u64, i32, i32, P(i32)]),
    "b200_kernel_max_clusters": (i32, [u64, i32, i32, i32, i32, P(i32)]),
    "b200_cache_stats": (i32, [P(u64), P(u64), P(u64)]),
    "b200_launch": (i32, [u64, u32, u32, u32, u32, u32, u32, u32, u64, C.c_void_p, u32, u32, i32]),
    "b200_graph_begin": (i32, [u64]),
    "b200_graph_end": (i32, [u64, P(u64)]),
    "b200_graph_launch": (i32, [u64, u64]),
    "b200_graph_destroy": (i32, [u64]),
    "b200_rng_seed": (i32, [u64]),
    "b200_rng_next_key": (i32, [P(u32)]),
    "b200_rng_get_state": (i32, [P(u64)]),
    "b200_rng_set_state": (i32, [P(u64)]),
    "b200_reduce_scratch_bytes": (u64, []),
    "b200_reduce_full": (i32, [u64, i32, u64, i32, i32, u64, u64, u64]),
    "b200_gemm": (i32, [u64, i32, C.c_int64, C.c_int64, u64, i32, C.c_int64, C.c_int64,
                        u64, i32, C.c_int64, C.c_int64, i32, i32, i32, C.c_float, C.c_float, u64]),
    "b200_dimshuffle": (i32, [u64, u64, i32, i32, P(C.c_int64), P(C.c_int64), P(C.c_int64), u64]),
    "b200_compensated_sum": (i32, [u64, u64, u64, i32, u64, C.c_float, C.c_float, i32, u64]),
    "b200_log2_hist": (i32, [u64, i32, u64, u64, i32, i32, u64]),
    "b200_reduce_full_noalloc_max_count": (u64, []),
    "b200_reduce_full_noalloc": (i32, [u64, i32, u64, i32, i32, u64, u64]),
    "b200_comm_unique_id": (i32, [P(C.c_uint8)]),
    "b200_comm_init": (i32, [P(C.c_uint8), i32, i32, P(u64)]),
    "b200_comm_destroy": (i32, [u64]),
    "b200_allreduce": (i32, [u64, u64, u64, u64, i32, i32, u64]),
    "b200_allgather": (i32, [u64, u64, u64, u64, u64]),
    "b200_xchg_create": (i32, [u64, i32, i32, u64, P(u64), P(u64)]),
    "b200_xchg_destroy": (i32, [u64]),
}

_lib = None
_header_registered = False


class B200Error(RuntimeError):
    def __init__(self, status, message):
        RuntimeError.__init__(self, "b200ew status %d: %s" % (status, message))
        self.status = status


def lib():
    """The loaded shared library (raises if it has not been built)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError("%s is missing: build it with `make -C neon_b200/csrc` "
                               "(or `python -c 'import __graft_entry__ as g; g.build()'`)" % LIB_PATH)
        _lib = C.CDLL(LIB_PATH, mode=C.RTLD_GLOBAL)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(_lib, name)
            fn.restype = res
            fn.argtypes = args
    return _lib


def last_error():
    buf = C.create_string_buffer(4096)
    lib().b200_last_error(buf, len(buf))
    return buf.value.decode("utf-8", "replace")


def check(status):
    if status != 0:
        raise B200Error(status, last_error())


def device_count():
    n = i32(0)
    check(lib().b200_device_count(C.byref(n)))
    return n.value


def init(device=0):
    _point_nccl_at_torch()
    check(lib().b200_init(device))
    register_templates()


def _point_nccl_at_torch():
    """Prefer the NCCL that ships with the python environment (newer than the
    system one) unless the user chose a library."""
    if os.environ.get("B200EW_NCCL_LIB"):
        return
    try:
        import importlib.util
        spec = importlib.util.find_spec("nvidia.nccl")
        if spec and spec.submodule_search_locations:
            cand = os.path.join(list(spec.submodule_search_locations)[0], "lib", "libnccl.so.2")
            if os.path.exists(cand):
                os.environ["B200EW_NCCL_LIB"] = cand
    except Exception:
        pass


def register_templates():
    global _header_registered
    if not _header_registered:
        with open(TEMPLATE_PATH, "rb") as f:
            check(lib().b200_register_header(b"optree_templates.cuh", f.read()))
        _header_registered = True


def device_props(device=0):
    p = DeviceProps()
    check(lib().b200_device_props_get(device, C.byref(p)))
    return p


def malloc(nbytes):
    ptr = u64(0)
    check(lib().b200_malloc(nbytes, C.byref(ptr)))
    return ptr.value


def free(ptr):
    check(lib().b200_free(ptr))


def mem_stats():
    a, b, c, d = u64(0), u64(0), u64(0), u64(0)
    check(lib().b200_mem_stats(C.byref(a), C.byref(b), C.byref(c), C.byref(d)))
    return {"in_use": a.value, "cached": b.value, "peak": c.value, "device_allocs": d.value}


def mem_info():
    """(free, total) device memory in bytes, as the driver reports it."""
    f, t = u64(0), u64(0)
    check(lib().b200_mem_info(C.byref(f), C.byref(t)))
    return f.value, t.value


def host_alloc(nbytes):
    p = C.c_void_p(0)
    check(lib().b200_host_alloc(nbytes, C.byref(p)))
    return p.value


def host_free(ptr):
    check(lib().b200_host_free(C.c_void_p(ptr)))


def memcpy_h2d(dst, host_ptr, nbytes, stream=0, sync=True):
    check(lib().b200_memcpy_h2d(dst, C.c_void_p(host_ptr), nbytes, stream, 1 if sync else 0))


def memcpy_d2h(host_ptr, src, nbytes, stream=0, sync=True):
    check(lib().b200_memcpy_d2h(C.c_void_p(host_ptr), src, nbytes, stream, 1 if sync else 0))


def memcpy_d2d(dst, src, nbytes, stream=0):
    check(lib().b200_memcpy_d2d(dst, src, nbytes, stream))


def memset(dst, value, width, count, stream=0):
    check(lib().b200_memset(dst, value, width, count, stream))


def stream_sync(stream=0):
    check(lib().b200_stream_sync(stream))


def default_stream():
    s = u64(0)
    check(lib().b200_default_stream(C.byref(s)))
    return s.value


def event_create():
    e = u64(0)
    check(lib().b200_event_create(C.byref(e)))
    return e.value


def event_record(ev, stream=0):
    check(lib().b200_event_record(ev, stream))


def event_sync(ev):
    check(lib().b200_event_sync(ev))


def event_elapsed_ms(start, end):
    ms = C.c_float(0)
    check(lib().b200_event_elapsed_ms(start, end, C.byref(ms)))
    return ms.value


def event_destroy(ev):
    check(lib().b200_event_destroy(ev))


def _opts(options):
    options = [o.encode() if isinstance(o, str) else o for o in (options or [])]
    arr = (C.c_char_p * max(1, len(options)))(*options)
    return arr, len(options)


def nvrtc_compile(source, options=None):
    """Compile to an sm_100a image without needing a device; returns (bytes, from_cache)."""
    register_templates()
    arr, n = _opts(options)
    img, size, cached = C.c_void_p(0), u64(0), i32(0)
    check(lib().b200_nvrtc_compile(source.encode(), arr, n, C.byref(img), C.byref(size), C.byref(cached)))
    data = C.string_at(img.value, size.value)
    lib().b200_buffer_free(img)
    return data, bool(cached.value)


def kernel_get(source, name="optree_kernel", options=None):
    arr, n = _opts(options)
    k = u64(0)
    check(lib().b200_kernel_get(source.encode(), name.encode(), arr, n, C.byref(k)))
    return k.value


def kernel_max_smem(kernel, nbytes):
    check(lib().b200_kernel_max_smem(kernel, nbytes))


def kernel_occupancy(kernel, threads, smem):
    n = i32(0)
    check(lib().b200_kernel_occupancy(kernel, threads, smem, C.byref(n)))
    return n.value


def kernel_max_clusters(kernel, threads, smem, cluster, grid_blocks):
    n = i32(0)
    check(lib().b200_kernel_max_clusters(kernel, threads, smem, cluster, grid_blocks, C.byref(n)))
    return n.value


def launch(kernel, grid, block, params, smem=0, stream=0, cluster=1, cooperative=False, dependent=False):
    check(lib().b200_launch(kernel, grid[0], grid[1], grid[2], block[0], block[1], block[2],
                            smem, stream, params, len(params), cluster, (1 if cooperative else 0) | (2 if dependent else 0)))


def graph_begin(stream=0):
    check(lib().b200_graph_begin(stream))


def graph_end(stream=0):
    g = u64(0)
    check(lib().b200_graph_end(stream, C.byref(g)))
    return g.value


def graph_launch(graph, stream=0):
    check(lib().b200_graph_launch(graph, stream))


def graph_destroy(graph):
    check(lib().b200_graph_destroy(graph))


def cache_stats():
    a, b, c = u64(0), u64(0), u64(0)
    check(lib().b200_cache_stats(C.byref(a), C.byref(b), C.byref(c)))
    return {"compiled": a.value, "disk_hits": b.value, "memory_hits": c.value}


def rng_seed(seed):
    check(lib().b200_rng_seed(seed & 0xFFFFFFFFFFFFFFFF))


def rng_next_key():
    k = (u32 * 2)()
    check(lib().b200_rng_next_key(k))
    return int(k[0]), int(k[1])


def rng_get_state():
    s = (u64 * 2)()
    check(lib().b200_rng_get_state(s))
    return int(s[0]), int(s[1])


def rng_set_state(state):
    s = (u64 * 2)(int(state[0]), int(state[1]))
    check(lib().b200_rng_set_state(s))


def reduce_scratch_bytes():
    return int(lib().b200_reduce_scratch_bytes())


def reduce_full(src, dtype, count, op, absolute, out, scratch, stream=0):
    check(lib().b200_reduce_full(src, dtype, count, op, 1 if absolute else 0, out, scratch, stream))


def gemm(a, a_dt, a_strides, b, b_dt, b_strides, c, c_dt, c_strides, m, n, k, alpha=1.0, beta=0.0, stream=0):
    check(lib().b200_gemm(a, a_dt, a_strides[0], a_strides[1], b, b_dt, b_strides[0], b_strides[1],
                          c, c_dt, c_strides[0], c_strides[1], m, n, k, alpha, beta, stream))


def dimshuffle(dst, src, elem_bytes, shape, dst_strides, src_strides, stream=0):
    """Permuted copy; all three lists are in output dimension order, strides in elements."""
    n = len(shape)
    arr = C.c_int64 * n
    check(lib().b200_dimshuffle(dst, src, elem_bytes, n, arr(*shape), arr(*dst_strides), arr(*src_strides), stream))


def compensated_sum(sum_ptr, cmp_ptr, add_ptr, dtype, count, cmp_scale, add_scale, rounding_bits, stream=0):
    check(lib().b200_compensated_sum(sum_ptr, cmp_ptr, add_ptr, dtype, count, cmp_scale, add_scale,
                                     rounding_bits, stream))


def log2_hist(src, dtype, count, hist, nbins, offset, stream=0):
    check(lib().b200_log2_hist(src, dtype, count, hist, nbins, offset, stream))


def reduce_full_noalloc(src, dtype, count, op, absolute, out, stream=0):
    """Whole-tensor reduction that allocates nothing (scratch is a static device array)."""
    check(lib().b200_reduce_full_noalloc(src, dtype, count, op, 1 if absolute else 0, out, stream))


def comm_unique_id():
    buf = (C.c_uint8 * 128)()
    check(lib().b200_comm_unique_id(buf))
    return bytes(buf)


def comm_init(uid, n_ranks, rank):
    buf = (C.c_uint8 * 128)(*uid)
    c = u64(0)
    check(lib().b200_comm_init(buf, n_ranks, rank, C.byref(c)))
    return c.value


def comm_destroy(comm):
    check(lib().b200_comm_destroy(comm))


def allreduce(comm, send, recv, count, dtype=F32, op=SUM, stream=0):
    check(lib().b200_allreduce(comm, send, recv, count, dtype, op, stream))


def allgather(comm, send, recv, send_bytes, stream=0):
    check(lib().b200_allgather(comm, send, recv, send_bytes, stream))


def xchg_create(comm, n_ranks, rank, nbytes):
    """Collective: (this rank's exchange area, device table of every rank's area)."""
    local, table = u64(0), u64(0)
    check(lib().b200_xchg_create(comm, n_ranks, rank, nbytes, C.byref(local), C.byref(table)))
    return local.value, table.value


def xchg_destroy(local):
    check(lib().b200_xchg_destroy(local))
