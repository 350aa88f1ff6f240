"""
The ``b200`` backend: executes op-trees on one B200 through libb200ew.so.

Stands where neon's ``NervanaGPU`` stands for the op-tree path
(neon/backends/nervanagpu.py:694-1439, 1825-1861, 3138-3231): same constructor
keywords as ``gen_backend`` forwards (neon/backends/__init__.py:107-114), same
tensor factories, ``execute``, RNG state functions and timing marks.  Methods
of the abstract backend that are not op-tree work (GEMM, convolution, pooling,
lookup tables) raise ``NotImplementedError``.
"""

import numpy as np

from . import runtime as rt
from .lowering import BoundPlan, MixedExtents, Planner, Statement, dtype_code, program_key
from .optree import OpCollection, OpTreeBackend, OpTreeNode, Tensor
from .tensor import B200Tensor

_COUNTER_BYTES = 1 << 20          # zero-initialised arrival counters, reset by the kernels
_SCRATCH_BYTES = 64 << 20


class _Scratch(object):
    """Bump allocator over two persistent device buffers: reduction results and
    partials (reused by every statement; the stream orders the reuse) and the
    arrival counters of split reductions (zeroed once, left zero by every kernel)."""

    def __init__(self):
        self.data = rt.malloc(_SCRATCH_BYTES)
        self.data_size = _SCRATCH_BYTES
        self.counters = rt.malloc(_COUNTER_BYTES)
        rt.memset(self.counters, 0, 1, _COUNTER_BYTES)
        self.reset()

    def reset(self):
        self.off = 0
        self.coff = 0

    def __call__(self, nbytes, zero):
        nbytes = (nbytes + 255) & ~255
        if zero:
            if self.coff + nbytes > _COUNTER_BYTES:
                raise MemoryError("split-reduction counters exceed %d bytes" % _COUNTER_BYTES)
            p = self.counters + self.coff
            self.coff += nbytes
            return p
        if self.off + nbytes > self.data_size:
            raise MemoryError("statement needs more than %d bytes of reduction scratch" % self.data_size)
        p = self.data + self.off
        self.off += nbytes
        return p

    def release(self):
        for p in (self.data, self.counters):
            try:
                rt.free(p)
            except Exception:
                pass


class _PlanCache(object):
    """Least-recently-used cache of statement plans.  Keys hold shapes, strides and
    alignments, so a workload that keeps cutting new views would otherwise grow it
    without bound (every entry keeps its generated source alive)."""

    def __init__(self, capacity=4096):
        import collections
        self.capacity = capacity
        self._d = collections.OrderedDict()

    def get(self, key):
        plan = self._d.get(key)
        if plan is not None:
            self._d.move_to_end(key)
        return plan

    def __setitem__(self, key, plan):
        self._d[key] = plan
        if len(self._d) > self.capacity:
            self._d.popitem(last=False)

    def __len__(self):
        return len(self._d)

    def clear(self):
        self._d.clear()


class CapturedGraph(object):
    """A recorded statement sequence (see ``B200Backend.capture``)."""

    def __init__(self, backend, handle, launches, rng_table=0, rng_count=0):
        self.backend, self.handle, self.launches = backend, handle, launches
        # recorded launches that draw random numbers read their keys from this device table
        self.rng_table, self.rng_count = rng_table, rng_count
        self._keys = np.empty((max(rng_count, 1), 2), np.uint32)

    def replay(self):
        if self.rng_count:
            # the keys the same launches would be given now, in the recorded order: a replay
            # draws exactly the random words eager execution would draw at this point
            keys = self._keys
            for i in range(self.rng_count):
                keys[i] = rt.rng_next_key()
            rt.memcpy_h2d(self.rng_table, keys.ctypes.data, keys.nbytes, self.backend.stream, sync=False)
        rt.graph_launch(self.handle, self.backend.stream)
        self.backend.launches += self.launches

    def __del__(self):
        try:
            if self.handle:
                rt.graph_destroy(self.handle)
                self.handle = 0
            if self.rng_table:
                rt.free(self.rng_table)
                self.rng_table = 0
        except Exception:
            pass


class B200Backend(OpTreeBackend):
    backend_name = "b200"
    tensor_cls = B200Tensor

    def __init__(self, rng_seed=None, default_dtype=np.float32, stochastic_round=False,
                 deterministic_update=False, deterministic=None, device_id=0, bench=False,
                 scratch_size=0, hist_bins=64, hist_offset=-48, compat_mode=None,
                 enable_winograd=True, cache_dir=None, num_devices=None, max_devices=None,
                 precise_math=False, check_bounds=None):
        self.enable_winograd = enable_winograd        # read by neon's fixtures; no convolutions here
        import os
        self.check_bounds = bool(int(os.environ.get("B200EW_CHECK", "0"))) if check_bounds is None else bool(check_bounds)
        if default_dtype not in (np.float16, np.float32) and np.dtype(default_dtype).name != "bfloat16":
            raise ValueError("Default data type for the b200 backend must be float16 or 32")
        if rt.device_count() <= int(device_id):
            raise RuntimeError("b200 backend needs CUDA device %d; none is visible" % int(device_id))
        rt.init(int(device_id))
        self.device_id = int(device_id)
        props = rt.device_props(self.device_id)
        self.sm_count = props.sm_count
        self.compute_capability = (props.cc_major, props.cc_minor)
        self.device_name = props.name.decode()
        self.stream = rt.default_stream()
        self.bench = bench
        self.use_pinned_mem = True
        self.round_mode = None
        self.set_stochastic_round(stochastic_round)
        self._scratch = _Scratch()
        self._planner = Planner(self.sm_count, precise_math=precise_math)
        # generated kernels wait for the previous kernel of the stream themselves (first instruction),
        # so the next launch's blocks can be placed while this one drains
        self.dependent_launch = os.environ.get("B200EW_DEPENDENT_LAUNCH", "1") != "0"
        self._rng_rec = None                   # set while a sequence is being recorded (see _record)
        self._status = rt.malloc(256)          # kernels set it when a bounded wait gives up
        rt.memset(self._status, 0, 1, 256)
        self._planner.status_ptr = self._status
        self._kernels = {}
        self._plans = _PlanCache()         # program_key -> BoundPlan
        self._temps = {}
        self._temps_used = {}
        self._marks = []
        self.launches = 0                  # kernels launched so far (statements may take several)
        self.launch_log = None             # set to a list to record (kind, desc) per launch
        self.trace = []                    # with bench=True: one record per launch (name, geometry, ms)
        self._trace_events = None
        self._timeline, self._timeline_pool = None, []
        self.hist_bins, self.hist_offset = None, None
        self.set_hist_buffers(hist_bins, hist_offset)
        super(B200Backend, self).__init__(rng_seed, default_dtype, compat_mode=compat_mode,
                                          deterministic=deterministic)

    # ------------------------------------------------------------------ lifecycle
    def cleanup_backend(self):
        sc = getattr(self, "_scratch", None)
        if sc is not None:
            sc.release()
            self._scratch = None

    def __del__(self):
        try:
            self.cleanup_backend()
        except Exception:
            pass

    def set_stochastic_round(self, rounding):
        """True -> 10 mantissa bits; an int -> that many; False/0 -> nearest
        (neon/backends/nervanagpu.py:892-899)."""
        if rounding is True:
            self.round_mode = 10
        elif rounding:
            self.round_mode = int(rounding)
        else:
            self.round_mode = 0

    # ------------------------------------------------------------------ RNG (nervanagpu.py:901-1049)
    def gen_rng(self, seed=None):
        self.rng = np.random.RandomState(seed)
        self.init_rng_state = self.rng.get_state()
        # device generator: counter based, keyed by a seed drawn without
        # advancing the host generator
        save = self.rng.get_state()
        dev_seed = int(self.rng.randint(0, 2 ** 31 - 1)) | (int(self.rng.randint(0, 2 ** 31 - 1)) << 31)
        self.rng.set_state(save)
        self.init_rng_state_dev = (dev_seed, 0)
        rt.rng_set_state(self.init_rng_state_dev)
        # one device context per backend, its generator always live: the bookkeeping NervanaGPU
        # exposes per CUDA context (nervanagpu.py:901-941), which neon's RNG tests look at
        self.context_rand_state_map = {self.device_id: self.init_rng_state_dev}
        self.context_rand_state_alive = {self.device_id: True}
        return self.rng

    def rng_reset(self):
        self.rng_set_state((self.init_rng_state, self.init_rng_state_dev))

    def rng_set_state(self, rng_states):
        if len(rng_states) != 2:
            self.rng_reset()
            self.rng.set_state(rng_states)
            return
        rt.rng_set_state(rng_states[1])
        self.rng.set_state(rng_states[0])

    def rng_get_state(self):
        return (self.rng.get_state(), np.array(rt.rng_get_state(), dtype=np.uint64))

    # ------------------------------------------------------------------ execute
    def execute(self, optree):
        """
        Run one assignment.  A tree whose reductions share an axis is one
        statement; otherwise inner results are first materialised into pooled
        temporaries, as ``_split_to_stacks`` does (nervanagpu.py:1099-1283).
        Whole-tensor reductions of contiguous operands become a single flat pass.
        """
        assert optree[0]["op"] == "assign"
        out, rhs = optree[1], optree[2]
        # common case first (nervanagpu.py:1239-1270): no dot / transpose node and all
        # reductions along one axis -> the program is one statement as it stands
        stack = optree.traverse([])
        axis, simple = None, True
        for s in stack:
            if type(s) is dict:
                op = s["op"]
                if op in OpCollection.reduction_ops:
                    if axis is not None and s.get("axis") != axis:
                        simple = False
                        break
                    axis = s.get("axis")
                elif op == "dot" or op == "transpose":
                    simple = False
                    break
        if simple:
            try:
                self._run_stack(out, stack)
                return out
            except MixedExtents:
                pass                            # same axis, different lengths: split below
        stmts = []
        self._temps_used = {}
        expr, tag = self._split(rhs, stmts)
        if tag == "flat" and tuple(out.shape) != (1, 1):
            expr = self._materialise(expr, (1, 1), stmts)
        if type(expr) is tuple:                 # the whole right-hand side is a dot
            stmts.append((out,) + expr[1:])
            expr = None
        for stmt in stmts:
            if len(stmt) == 3:
                self.compound_dot(stmt[1], stmt[2], stmt[0])
            else:
                self._run(stmt[0], stmt[1])
        if expr is not None:
            self._run(out, expr)
        return out

    # -- splitting ----------------------------------------------------------------
    def _temp(self, shape):
        """Pooled temporary of the default dtype, keyed by shape and by how many
        of that shape this statement already holds (nervanagpu.py:1051-1075)."""
        shape = tuple(shape)
        used = self._temps_used.get(shape, 0)
        self._temps_used[shape] = used + 1
        pool = self._temps.setdefault(shape, [])
        while len(pool) <= used:
            pool.append(self.empty(shape, dtype=self.default_dtype))
        return pool[used]

    def _materialise(self, expr, shape, stmts):
        if type(expr) is tuple:
            return self._finish_dot(expr, stmts)
        buf = self._temp(shape)
        stmts.append((buf, expr))
        return buf

    def _finish_dot(self, dot, stmts):
        buf = self._temp((dot[1].shape[0], dot[2].shape[1]))
        stmts.append((buf, dot[1], dot[2]))
        return buf

    @staticmethod
    def _flat_leaves_ok(node, shape_box):
        """True when every tensor under ``node`` is contiguous with one common shape
        (or is a (1,1) scalar) and there is no reduction or addressing op inside."""
        if isinstance(node, OpTreeNode):
            op = node[0]["op"]
            if op in OpCollection.reduction_ops or op in ("dot", "transpose", "onehot", "rand"):
                return False
            return all(B200Backend._flat_leaves_ok(c, shape_box) for c in node[1:] if c is not None)
        if isinstance(node, Tensor):
            if tuple(node.shape) == (1, 1):
                return True
            if not node.is_contiguous or node.take_array or len(node.shape) != 2:
                return False
            if shape_box[0] is None:
                shape_box[0] = tuple(node.shape)
            return shape_box[0] == tuple(node.shape)
        return True

    @staticmethod
    def _flatten(node, size):
        if isinstance(node, OpTreeNode):
            info = dict(node[0])
            info["shape"] = (1, size)
            return OpTreeNode(info, *[B200Backend._flatten(c, size) if c is not None else None
                                      for c in node[1:]])
        if isinstance(node, Tensor) and tuple(node.shape) != (1, 1):
            return node.reshape(1, size)
        return node

    @staticmethod
    def _flat_extent(node):
        """Number of elements the fused whole-tensor reduction(s) under ``node`` run over."""
        todo = [node]
        while todo:
            n = todo.pop()
            if isinstance(n, OpTreeNode):
                if n[0]["op"] in OpCollection.reduction_ops:
                    child = n[1]
                    return int(child.shape[1]) if hasattr(child, "shape") else 1
                todo.extend(c for c in n[1:] if c is not None)
        return None

    @staticmethod
    def _red_extent(node, axis):
        """Elements per result of the outermost reduction(s) along ``axis`` under ``node``."""
        todo = [node]
        while todo:
            n = todo.pop()
            if isinstance(n, OpTreeNode):
                if n[0]["op"] in OpCollection.reduction_ops and n[0].get("axis") == axis:
                    child = n[1]
                    return int(child.shape[axis]) if hasattr(child, "shape") else 1
                todo.extend(c for c in n[1:] if c is not None)
        return None

    def _split(self, node, stmts):
        """Returns (expression, tag): tag is None (no reduction inside), 0/1 (reduces
        along that axis) or 'flat' (contains a fused whole-tensor reduction and only
        (1,1)-shaped values around it)."""
        if not isinstance(node, OpTreeNode):
            return node, None
        info = node[0]
        op = info["op"]
        if op in OpCollection.reduction_ops:
            axis = info["axis"]
            child = node[1]
            if (op in ("sum", "max", "min") and isinstance(child, OpTreeNode) and child[0]["op"] == op
                    and child[0].get("axis") == 1 - axis):
                inner, itag = self._split(child[1], stmts)
                box = [None]
                if itag is None and self._flat_leaves_ok(inner, box) and box[0] is not None:
                    size = box[0][0] * box[0][1]
                    flat = self._flatten(inner, size)
                    return OpTreeNode({"op": op, "axis": 1, "shape": (1, 1)}, flat, None), "flat"
                # not fusable: reduce along the inner axis, then along this one
                if itag is not None and itag != 1 - axis:
                    inner = self._materialise(inner, (1, 1) if itag == "flat" else inner.shape, stmts)
                operand = self._materialise(OpTreeNode(child[0], inner, None), child[0]["shape"], stmts)
                return OpTreeNode(info, operand, None), axis
            operand, prev = self._split(child, stmts)
            if type(operand) is tuple:
                operand = self._finish_dot(operand, stmts)
            if prev is not None and prev != axis:
                shape = (1, 1) if prev == "flat" else operand.shape
                operand = self._materialise(operand, shape, stmts)
            return OpTreeNode(info, operand, None), axis
        if op == "transpose":
            operand, _ = self._split(node[1], stmts)
            if type(operand) is tuple:
                operand = self._finish_dot(operand, stmts)
            if isinstance(operand, Tensor):
                return operand.T, None
            return self._materialise(operand, operand.shape, stmts).T, None
        if op == "dot":
            # operands and result live in tensors; the product is its own launch
            # (nervanagpu.py:1123-1146)
            sides = []
            for child in (node[1], node[2]):
                operand, tag = self._split(child, stmts)
                if type(operand) is tuple:
                    operand = self._finish_dot(operand, stmts)
                if not isinstance(operand, Tensor):
                    operand = self._materialise(operand, (1, 1) if tag == "flat" else operand.shape, stmts)
                sides.append(operand)
            return ("dot", sides[0], sides[1]), None
        if op in OpCollection.unary_ops or node[2] is None:
            operand, tag = self._split(node[1], stmts)
            if type(operand) is tuple:
                operand = self._finish_dot(operand, stmts)
            return OpTreeNode(info, operand, None), tag
        left, lt = self._split(node[1], stmts)
        right, rt_ = self._split(node[2], stmts)
        if type(left) is tuple:
            left = self._finish_dot(left, stmts)
        if type(right) is tuple:
            right = self._finish_dot(right, stmts)
        if lt == "flat" and rt_ == "flat" and self._flat_extent(left) != self._flat_extent(right):
            # whole-tensor reductions of tensors of different sizes (the squared-gradient norm
            # over all layers, optimizers/optimizer.py:72-96): they cannot share a pass
            left, lt = self._materialise(left, (1, 1), stmts), None
        if lt in (0, 1) and rt_ == lt and self._red_extent(left, lt) != self._red_extent(right, lt):
            # both sides reduce along the same axis but over different numbers of elements
            left, lt = self._materialise(left, left.shape, stmts), None
        if lt is not None and rt_ is not None and lt != rt_:
            # two sides reduce differently: evaluate one of them first.  A flat side
            # is a (1,1) value; otherwise the side reducing along axis 0 goes first
            # unless axis 0 is the more frequent one (nervanagpu.py:1112-1118,1188-1206)
            if lt == "flat" or (rt_ != "flat" and lt == 0):
                left = self._materialise(left, (1, 1) if lt == "flat" else left.shape, stmts)
                lt = None
            else:
                right = self._materialise(right, (1, 1) if rt_ == "flat" else right.shape, stmts)
                rt_ = None
        tag = lt if lt is not None else rt_
        if tag == "flat":
            other = right if lt is not None else left
            if lt is not None and rt_ is not None:
                other = None
            if isinstance(other, (Tensor, OpTreeNode)) and tuple(other.shape) != (1, 1):
                # a whole-tensor reduction meets a full-size operand
                if lt == "flat":
                    left, tag = self._materialise(left, (1, 1), stmts), None
                else:
                    right, tag = self._materialise(right, (1, 1), stmts), None
        return OpTreeNode(info, left, right), tag

    # -- one statement ------------------------------------------------------------
    def _run(self, out, expr):
        self._run_stack(out, OpTreeNode({"op": "assign"}, out, expr).traverse([]))

    # ------------------------------------------------------------------ checked mode
    def check_operands(self, stack):
        """Checked mode (``check_bounds=True`` or B200EW_CHECK=1): before a statement is launched,
        every tensor's addressed span -- lowest to highest element its shape and strides reach --
        must lie inside the allocation it views, and every index vector of a fancy-indexed
        operand is read back and must stay inside the indexed axis.  A violation raises
        B200Error(B200_ERR_INVALID) and nothing is launched.  Costs a host loop per statement and
        a device-to-host copy per index vector, so it is a debugging aid, off by default."""
        for s in stack:
            if type(s) is dict:
                s = s.get("idx")
            if not isinstance(s, B200Tensor):
                continue
            block = s._block
            taken = s.take_array[1] if s.take_array else None
            if block is not None:
                lo = hi = 0
                for axis, (d, st) in enumerate(zip(s.shape, s.strides)):
                    if axis == taken:
                        continue                     # addressed through the index vector, checked below
                    if d == 0:
                        lo = hi = None
                        break
                    if st >= 0:
                        hi += (d - 1) * st
                    else:
                        lo += (d - 1) * st
                if lo is not None:
                    isz = s.dtype.itemsize
                    first, last = s.gpudata + lo * isz, s.gpudata + (hi + 1) * isz
                    if first < block.ptr or last > block.ptr + block.nbytes:
                        raise rt.B200Error(-1, "tensor %s (shape %s, strides %s) reaches bytes [%d, %d) of an "
                                           "allocation of %d bytes" % (s.name, s.shape, s.strides,
                                                                       first - block.ptr, last - block.ptr, block.nbytes))
            if s.take_array:
                vec, axis = s.take_array
                base = s.base if s.base is not None else s
                extent = base.shape[axis] if axis < len(base.shape) else 0
                idx = vec.get().reshape(-1)
                if idx.size and (int(idx.min()) < 0 or int(idx.max()) >= extent):
                    raise rt.B200Error(-1, "index vector of %s holds %d..%d for an axis of %d entries"
                                       % (s.name, int(idx.min()), int(idx.max()), extent))

    def _run_stack(self, out, stack):
        if self.check_bounds:
            self.check_operands(stack)
        rounding = self._rounding_bits(out)
        key = (program_key(stack), rounding)
        plan = self._plans.get(key)
        if plan is None:
            st = Statement(stack)
            self._scratch.reset()
            plan = self._plans[key] = BoundPlan(st, self._planner.plan(st, self._scratch, rounding=rounding))
        else:
            plan.rebind(stack)
        for pz in plan.passes:
            self._launch(pz)

    def _launch(self, pz):
        kernel = pz.kernel
        if kernel is None:
            kernel = self._kernels.get(pz.source)
            if kernel is None:
                kernel = self._kernels[pz.source] = rt.kernel_get(pz.source, pz.name)
            pz.kernel = kernel
            if pz.setup is not None:
                pz.setup(rt, kernel, pz)
        if pz.uses_rng:
            rec = self._rng_rec
            vals = pz.fields.values
            if rec is None:
                vals["rk0"], vals["rk1"] = rt.rng_next_key()
                vals["rk_tab"] = 0
            else:                               # being recorded: the key comes from the graph's table at replay
                if rec["count"] >= rec["capacity"]:
                    raise RuntimeError("more than %d launches with random numbers in one recorded sequence" % rec["capacity"])
                vals["rk_tab"] = rec["table"] + 8 * rec["count"]
                rec["count"] += 1
        if self.bench:
            if self._trace_events is None:
                self._trace_events = (rt.event_create(), rt.event_create())
            rt.event_record(self._trace_events[0], self.stream)
        mark = self._timeline_begin("kernel", pz.name) if self._timeline is not None else None
        rt.launch(kernel, pz.grid, pz.block, pz.fields.pack(), smem=pz.smem, stream=self.stream,
                  cluster=pz.cluster, dependent=self.dependent_launch)
        if mark is not None:
            rt.event_record(mark, self.stream)
        if self.bench:
            # per-launch timing, as be.bench does in the reference (float_ew.py:917-938); the
            # records stay in self.trace (newest last, bounded) and dump_trace() writes them out
            rt.event_record(self._trace_events[1], self.stream)
            rt.event_sync(self._trace_events[1])
            self.trace.append({"kernel": pz.name, "kind": pz.kind, "desc": pz.desc,
                               "ms": rt.event_elapsed_ms(*self._trace_events)})
            if len(self.trace) > 4096:
                del self.trace[:1024]
        self.launches += 1
        if self.launch_log is not None:
            self.launch_log.append((pz.kind, pz.desc))

    def _rounding_bits(self, out):
        """Mantissa bits for a stochastic store, 0 for nearest (float_ew.py:827-844)."""
        rounding = out.rounding
        if not rounding:
            return 0
        if rounding is True:
            rounding = 10
        if out.dtype.type is np.float32:
            rounding = min(int(rounding), 15)
        elif out.dtype.type is np.float16:
            rounding = min(int(rounding), 10)
        elif out.dtype.name == "bfloat16":
            rounding = min(int(rounding), 7)
        elif out.dtype.kind != "f":
            rounding = 1                       # integer stores: on/off only
        return max(int(rounding), 1)

    # ------------------------------------------------------------------ factories (nervanagpu.py:1285-1439)
    def empty(self, shape, dtype=None, name=None, persist_values=True,
              parallel=False, distributed=False, allocator=None):
        dtype = self.default_dtype if dtype is None else dtype
        return B200Tensor(self, shape, dtype=dtype, name=name, persist_values=persist_values,
                          rounding=self.round_mode)

    def array(self, ary, dtype=None, name=None, persist_values=True,
              parallel=False, distributed=False, allocator=None):
        dtype = self.default_dtype if dtype is None else dtype
        ary = np.asarray(ary)
        if ary.ndim < self._min_dims:
            ary = ary.reshape(ary.size, 1)
        if ary.dtype != np.dtype(dtype):
            ary = ary.astype(dtype)
        return B200Tensor(self, ary.shape, dtype=dtype, name=name, persist_values=persist_values,
                          rounding=self.round_mode).set(ary)

    def zeros(self, shape, dtype=None, name=None, persist_values=True,
              parallel=False, distributed=False, allocator=None):
        t = self.empty(shape, dtype=dtype, name=name, persist_values=persist_values)
        return t._assign(0)

    def ones(self, shape, dtype=None, name=None, persist_values=True,
             parallel=False, distributed=False, allocator=None):
        t = self.empty(shape, dtype=dtype, name=name, persist_values=persist_values)
        return t._assign(1)

    def empty_like(self, other, name=None, persist_values=True):
        return B200Tensor(self, other.shape, dtype=other.dtype, name=name,
                          persist_values=persist_values, rounding=self.round_mode)

    def zeros_like(self, other, name=None, persist_values=True):
        return self.empty_like(other, name=name, persist_values=persist_values)._assign(0)

    # ------------------------------------------------------------------ random ops (nervanagpu.py:1825-1861)
    def rand(self, out=None):
        return OpTreeNode.build("rand", None, None, out=out)

    def dropout(self, keep=0.5, out=None):
        return self.less_equal(self.rand(), keep, out=out)

    def make_binary_mask(self, out, keepthresh=0.5):
        self.dropout(keep=keepthresh, out=out)

    def binarize(self, ary, out, stochastic=True):
        """out = +1 / -1 from ary (neon/backends/nervanagpu.py:3120-3136): the sign of ary, or,
        stochastically, +1 with probability clip((ary + 1) / 2, 0, 1).  One fused statement."""
        if stochastic:
            p = self.clip((ary + 1) / 2.0, 0, 1)
            out[:] = 2 * self.less_equal(self.rand(), p) - 1
        else:
            out[:] = 2 * self.greater_equal(ary, 0) - 1
        return out

    def shift(self, ary, shift_ary, value=True, out=None):
        """out = ary scaled by a power of two taken from shift_ary (nervanagpu.py:1863-1894,
        kernel text backends/kernels/cuda/binary.py:174-227): with ``value`` the power of two
        nearest to |shift_ary| in the log domain, carrying its sign (0 gives 0); otherwise
        2**shift_ary for integer-valued shift_ary.  shift_ary broadcasts like any operand."""
        if not hasattr(ary, "shape"):
            ary = self.array(np.array(ary))
        if not hasattr(shift_ary, "shape"):
            shift_ary = self.array(np.array(shift_ary))
        if out is None:
            out = self.empty_like(ary)
        if value:
            e = OpTreeNode.build("round", self.log2(self.absolute(shift_ary)), None)
            out[:] = ary * self.sgn(shift_ary) * self.exp2(e)
        else:
            out[:] = ary * self.exp2(shift_ary)
        return out

    def fill_normal(self, ary, mean=0, stdv=1):
        ary[:] = (self.rng.standard_normal(ary.shape) * stdv + mean).astype(ary.dtype)

    def capture(self, fn):
        """
        Record the device work of ``fn()`` -- a sequence of assignments -- as a CUDA
        graph and return it; ``graph.replay()`` then issues the whole sequence with one
        call, which is what makes small, launch-bound statements (a few MB per tensor)
        run at the speed of their kernels instead of the speed of the host.  ``fn`` runs
        twice here: once eagerly (compiles, allocates temporaries), once recorded.
        Tensor addresses and python numbers are frozen as recorded; ``fn`` must not read
        tensors back or create them.  Statements that draw random numbers (``rand``,
        dropout masks, stochastic rounding) draw fresh ones in every replay -- the words
        eager execution would draw at that point, bit for bit: their launches read the
        key of their random stream from a small device table that ``replay`` refills.
        (``compensated_sum`` is not an op-tree statement: its rounding repeats.)
        """
        handle, launches, table, count = self._record(fn)
        return CapturedGraph(self, handle, launches, table, count)

    def _record(self, fn):
        """Run ``fn`` once, then record it: (graph handle, launches, key table, keys)."""
        fn()
        self.synchronize()
        before = self.launches
        rec = self._rng_rec = {"table": rt.malloc(8 * 1024), "capacity": 1024, "count": 0}
        try:
            rt.graph_begin(self.stream)
            try:
                fn()
            finally:
                handle = rt.graph_end(self.stream)
        finally:
            self._rng_rec = None
            if rec["count"] == 0:
                rt.free(rec["table"])
                rec["table"] = 0
        return handle, self.launches - before, rec["table"], rec["count"]

    def copy_transpose(self, a, out, axes=None, repeat=1):
        """out = numpy.transpose(a, axes) for tensors of any rank, views included
        (neon/backends/nervanagpu.py:3077-3118): one shared-memory tiled shuffle kernel."""
        assert a.dtype == out.dtype
        assert a.size == out.size
        assert a.gpudata != out.gpudata
        if axes is None:
            axes = tuple(range(len(a.shape) - 1, -1, -1))
        elif type(axes) is not tuple:
            axes = tuple(axes)
        assert all(out.shape[i] == a.shape[x] for i, x in enumerate(axes))
        if a.take_array is not None or out.take_array is not None:
            raise NotImplementedError("copy_transpose of a tensor indexed with an array")
        for _ in range(max(int(repeat), 1)):
            rt.dimshuffle(out.gpudata, a.gpudata, a.dtype.itemsize, out.shape, out.strides,
                          [a.strides[x] for x in axes], self.stream)
        self.launches += max(int(repeat), 1)
        return out

    # ------------------------------------------------------------------ log2 histograms (nervanagpu.py:826-834, 1077-1097)
    def set_hist_buffers(self, hist_bins, hist_offset):
        """Bins (one per power of two) and the power of two of bin 0 for ``tensor.hist(tag)``."""
        if hist_bins != self.hist_bins or hist_offset != self.hist_offset:
            if not 0 < int(hist_bins) <= 128:
                raise ValueError("between 1 and 128 histogram bins")
            self.hist_bins, self.hist_offset = int(hist_bins), int(hist_offset)
            self.hist_map = dict()
            self.hist_idx = 0
            self.hist_max = 4 * 4096
            self._hist_block = None          # hist_max rows of hist_bins counters, allocated at first use

    def _hist_tensor(self, tag):
        """The next free row of the histogram buffer as a (1, hist_bins) int32 tensor, remembered by tag."""
        assert self.hist_idx < self.hist_max
        if self._hist_block is None:
            self._hist_block = self.zeros((self.hist_max, self.hist_bins), dtype=np.int32)
        row = self._hist_block[self.hist_idx:self.hist_idx + 1]
        row.name = tag
        self.hist_map[tag] = self.hist_idx
        self.hist_idx += 1
        return row

    def dump_hist_data(self):
        """(tensor of all histograms taken so far, {tag: row}); starts a new collection."""
        if self._hist_block is None:
            self._hist_block = self.zeros((self.hist_max, self.hist_bins), dtype=np.int32)
        hist_data = self._hist_block[0:self.hist_idx] if self.hist_idx else self._hist_block[0:0]
        hist_map = self.hist_map
        self.hist_map = dict()
        self.hist_idx = 0
        return hist_data, hist_map

    def _compute_hist(self, tensor, hist_tensor):
        """hist_tensor[b] = number of elements of tensor with round(log2|x|) - hist_offset == b,
        clamped to the first and last bin (neon/backends/float_ew.py:1069-1158)."""
        if not tensor.is_contiguous or tensor.take_array is not None:
            raise ValueError("histogram of a contiguous tensor only")
        rt.log2_hist(tensor.gpudata, dtype_code(tensor.dtype), tensor.size, hist_tensor.gpudata,
                     self.hist_bins, self.hist_offset, self.stream)
        self.launches += 1

    def compensated_sum(self, sum_tensor, cmp_tensor, add_tensor, cmp_scale=1.0, add_scale=1.0):
        """Kahan-compensated ``sum_tensor += add_tensor*add_scale`` with the lost low-order
        bits kept in ``cmp_tensor`` (neon/backends/nervanagpu.py:1896-1917); the new sum is
        rounded stochastically when ``sum_tensor.rounding`` is set.  Contiguous tensors of
        one floating-point dtype."""
        if cmp_tensor.kahan_reset and cmp_tensor.kahan_count > cmp_tensor.kahan_reset:
            cmp_scale = 0
            cmp_tensor.kahan_count = 0
        assert sum_tensor.dtype.type == cmp_tensor.dtype.type == add_tensor.dtype.type
        assert sum_tensor.size == cmp_tensor.size == add_tensor.size
        for t in (sum_tensor, cmp_tensor, add_tensor):
            if not t.is_contiguous or t.take_array is not None:
                raise ValueError("compensated_sum needs contiguous tensors")
        cmp_tensor.kahan_count += 1
        rounding = sum_tensor.rounding
        bits = 10 if rounding is True else int(rounding or 0)
        rt.compensated_sum(sum_tensor.gpudata, cmp_tensor.gpudata, add_tensor.gpudata,
                           dtype_code(sum_tensor.dtype), sum_tensor.size, float(cmp_scale), float(add_scale),
                           bits, self.stream)
        self.launches += 1

    # ------------------------------------------------------------------ timing marks (nervanagpu.py:3138-3177)
    def init_mark(self):
        ev = rt.event_create()
        self._marks.append(ev)
        return ev

    def record_mark(self, marker):
        rt.event_record(marker, self.stream)

    def synchronize_mark(self, marker):
        rt.event_sync(marker)

    def get_time(self, start, end):
        return rt.event_elapsed_ms(start, end)

    # a timeline is lighter than bench=True: events around every launch (and, in the sharded
    # backend, every collective), read back only when it is stopped
    def start_timeline(self):
        self._timeline = []

    def _timeline_begin(self, kind, name):
        """Record the start event of an interval; returns the event to record at its end."""
        pool = self._timeline_pool
        ev0 = pool.pop() if pool else rt.event_create()
        ev1 = pool.pop() if pool else rt.event_create()
        rt.event_record(ev0, self.stream)
        self._timeline.append((kind, name, ev0, ev1))
        return ev1

    def stop_timeline(self):
        """[(kind, name, ms)] of everything issued since start_timeline()."""
        self.synchronize()
        out = []
        for kind, name, ev0, ev1 in self._timeline:
            out.append((kind, name, rt.event_elapsed_ms(ev0, ev1)))
            self._timeline_pool.extend((ev0, ev1))
        self._timeline = None
        return out

    def dump_trace(self, path):
        """Write the per-launch records collected with ``bench=True`` as JSON."""
        import json
        with open(path, "w") as f:
            json.dump(self.trace, f, indent=1)

    def synchronize(self):
        rt.stream_sync(self.stream)
        self.check_status()

    def check_status(self):
        """Raise if a kernel reported that one of its bounded waits ran out."""
        flag = np.zeros(1, np.int32)
        rt.memcpy_d2h(flag.ctypes.data, self._status, 4, self.stream, sync=True)
        if flag[0]:
            rt.memset(self._status, 0, 1, 4, self.stream)
            what = [msg for bit, msg in ((1, "its shared-memory staging copy"),
                                         (4, "the results of another GPU (exchange area)")) if flag[0] & bit]
            raise rt.B200Error(-6, "a kernel gave up waiting for " + " and ".join(what or ["(unknown)"]))

    # ------------------------------------------------------------------ not on the op-tree path
    def _off_path(self, *a, **k):
        raise NotImplementedError("outside the compound op-tree path of the b200 backend")

    def compound_dot(self, A, B, C, alpha=1.0, beta=0.0, relu=False, bsum=None):
        """C = alpha * A.B + beta * C for `dot` nodes of op-trees (plain tiled kernel;
        the reference's SASS GEMM path, nervanagpu.py:1441-1622, is not rebuilt)."""
        if relu or bsum is not None:
            raise NotImplementedError("fused relu / batch-sum epilogues of the GEMM path")
        assert A.shape[1] == B.shape[0] and C.shape == (A.shape[0], B.shape[1])
        from .lowering import dtype_code
        rt.gemm(A.ptr, dtype_code(A.dtype), A.strides, B.ptr, dtype_code(B.dtype), B.strides,
                C.ptr, dtype_code(C.dtype), C.strides, A.shape[0], B.shape[1], A.shape[1],
                float(alpha), float(beta), self.stream)
        self.launches += 1
        return C

    batched_dot = conv_layer = deconv_layer = fprop_conv = bprop_conv = _off_path
    update_conv = pool_layer = fprop_pool = bprop_pool = compound_bprop_lut = _off_path


def gen_backend(backend="b200", rng_seed=None, datatype=np.float32, batch_size=0,
                stochastic_round=False, device_id=0, max_devices=None, compat_mode=None,
                deterministic_update=None, deterministic=None):
    """Same call as ``neon.backends.gen_backend`` (neon/backends/__init__.py:49-120)
    for the one backend this package provides."""
    if backend != "b200":
        raise ValueError("backend must be one of ('b200')")
    be = B200Backend(rng_seed=rng_seed, default_dtype=datatype, stochastic_round=stochastic_round,
                     device_id=device_id, compat_mode=compat_mode, deterministic=deterministic)
    be.bsz = batch_size
    return be
