"""
Multi-GPU layer of the b200 backend: tensors sharded along the batch (column)
axis, one process per GPU.

neon's tree has no multi-device code (the multi-GPU backend was a closed
package: neon/backends/__init__.py:42-46); what remains are inert hooks --
the ``parallel=`` / ``distributed=`` keywords of the tensor factories
(neon/backends/abstract_backend.py:96-126) and per-layer parallelism tags.  This
module gives ``parallel=True`` a meaning:

* ``be.empty(shape, parallel=True)`` makes a ``ShardedTensor``: it reports the
  global shape (rows, cols) to the op-tree front end (so ``be.mean`` divides by
  the global count) and stores columns ``[c0, c1)`` on this rank.  Tensors made
  without the keyword are replicated.
* element-wise statements and reductions along axis 0 are shard-local;
* reductions along axis 1 (and over a whole tensor) reduce the local shard and
  finish across the GPUs inside the reduction kernel: the thread that holds a
  row's local result stores it into every rank's peer-mapped exchange area over
  NVLink, waits (time-bounded) for the other ranks' results and merges them in
  rank order (``xchg_rows`` in the kernel header), so a statement is planned as
  on one GPU and no collective is launched between its passes.  Statements the
  exchange area cannot carry (more than 16384 results, reductions down a transposed
  view) reduce locally and all-reduce the per-row results over NCCL instead;
* random numbers and stochastic rounding use the element index in the global
  tensor, so stored values do not depend on how many GPUs share the work.

Host plumbing (the NCCL unique id, barriers, max-over-ranks of timings) goes
over a small TCP star (``HostGroup``); ranks are told who they are by whatever
launched them (``RANK`` / ``WORLD_SIZE`` / ``MASTER_ADDR`` / ``MASTER_PORT``).
"""

import numpy as np

from . import runtime as rt
from .backend import B200Backend, CapturedGraph
from .lowering import BoundPlan, Statement, XchgUnsupported, program_key
from .optree import OpTreeNode, Tensor

_none_slice = slice(None, None, None)
_NCCL_OP = {"sum": rt.SUM, "max": rt.MAX, "min": rt.MIN}


def shard_columns(cols, world_size, rank):
    """Contiguous, equal column ranges; the global column count must divide."""
    if cols % world_size:
        raise ValueError("%d columns do not divide over %d devices" % (cols, world_size))
    per = cols // world_size
    return rank * per, (rank + 1) * per


class ShardedTensor(Tensor):
    """Column shard of a (rows, cols) tensor.  ``shape`` is global; ``local`` is the
    device tensor holding this rank's columns."""

    def __init__(self, backend, gshape, local, c0, name=None, flat_of=None):
        super(ShardedTensor, self).__init__(backend, tuple(gshape), local.dtype, name)
        self.local = local
        self.c0 = c0
        self.size = int(np.prod(gshape))
        self.take_array = None
        self.is_trans = False
        self.flat_of = flat_of            # (global cols, col0) when this is a flattened view

    rounding = property(lambda self: self.local.rounding,
                        lambda self, v: setattr(self.local, "rounding", v))
    ptr = property(lambda self: self.local.ptr)
    is_contiguous = property(lambda self: self.local.is_contiguous)
    strides = property(lambda self: self.local.strides)

    def __len__(self):
        return self.shape[0]

    def __getitem__(self, index):
        if isinstance(index, slice) and index == _none_slice:
            return self
        raise NotImplementedError("views of sharded tensors")

    def _assign(self, value):
        if isinstance(value, (int, float)):
            self.local._assign(value)
        elif isinstance(value, np.ndarray):
            self.set(value)
        elif isinstance(value, (Tensor, OpTreeNode)):
            OpTreeNode.build("assign", self, value)
        else:
            raise TypeError("Invalid type for assignment: %s" % type(value))
        return self

    def set(self, ary):
        """Takes the global array; keeps this rank's columns."""
        ary = np.asarray(ary).reshape(self.shape)
        lc = self.local.shape[1]
        self.local.set(np.ascontiguousarray(ary[:, self.c0:self.c0 + lc]))
        return self

    def get_local(self):
        return self.local.get()

    def get(self):
        """Global array, gathered over NCCL (every rank gets all of it)."""
        be = self.backend
        nbytes = self.local.nbytes
        buf = rt.malloc(nbytes * be.world_size)
        try:
            rt.allgather(be.comm, self.local.ptr, buf, nbytes, be.stream)
            host = np.empty((be.world_size,) + tuple(self.local.shape), self.dtype)
            rt.memcpy_d2h(host.ctypes.data, buf, nbytes * be.world_size, be.stream, sync=True)
        finally:
            rt.free(buf)
        return np.concatenate(list(host), axis=1)

    def reshape(self, *shape):
        if isinstance(shape[0], (tuple, list)):
            shape = tuple(shape[0])
        if tuple(shape) == self.shape:
            return self
        if tuple(shape) != (1, self.size):
            raise NotImplementedError("sharded tensors reshape only to (1, size)")
        return ShardedTensor(self.backend, shape, self.local.reshape(1, self.local.size), self.c0,
                             self.name, flat_of=(self.shape[1], self.c0, self.local.shape[1]))


class ShardedBackend(B200Backend):
    """B200Backend of one rank of a column-sharded job."""

    def __init__(self, rank, world_size, comm, host_barrier=None, host_max=None, use_exchange=True, **kw):
        super(ShardedBackend, self).__init__(**kw)
        self.rank, self.world_size, self.comm = rank, world_size, comm
        self.host_barrier = host_barrier or (lambda: None)
        self.host_max = host_max or (lambda v: v)
        self.collectives = 0                 # all-reduces issued so far
        self.exchanges = 0                   # reduction kernels that finished across the GPUs by themselves
        # peer-mapped exchange area
        self._xchg, self._xchg_local, self._xepoch = None, 0, 0
        if world_size > 1 and comm and use_exchange:
            cap = 16384                      # (rows x reductions) one launch can exchange
            nbytes = 2 * world_size * cap * 16
            self._xchg_local, table = rt.xchg_create(comm, world_size, rank, nbytes)
            # launch number of an exchange = its kernel parameter + this device word; the word
            # only changes when a recorded sequence is replayed (see capture)
            self._xbase_word, self._xbase = rt.malloc(256), 0
            rt.memset(self._xbase_word, 0, 4, 1, self.stream)
            self._xchg = {"table": table, "base": self._xbase_word, "rank": rank, "world": world_size, "cap": cap}

    # ---- factories: parallel=True -> column shard
    def _make(self, factory, shape, dtype, name, parallel, fill=None):
        if not parallel:
            return factory(shape, dtype=dtype, name=name)
        shape = tuple(shape) if isinstance(shape, (tuple, list)) else (int(shape), 1)
        if len(shape) != 2:
            raise ValueError("sharded tensors are 2-d (features, batch)")
        c0, c1 = shard_columns(shape[1], self.world_size, self.rank)
        local = factory((shape[0], c1 - c0), dtype=dtype, name=name)
        return ShardedTensor(self, shape, local, c0, name)

    def empty(self, shape, dtype=None, name=None, persist_values=True,
              parallel=False, distributed=False, allocator=None):
        return self._make(super(ShardedBackend, self).empty, shape, dtype, name, parallel)

    def zeros(self, shape, dtype=None, name=None, persist_values=True,
              parallel=False, distributed=False, allocator=None):
        return self._make(super(ShardedBackend, self).zeros, shape, dtype, name, parallel)

    def ones(self, shape, dtype=None, name=None, persist_values=True,
             parallel=False, distributed=False, allocator=None):
        return self._make(super(ShardedBackend, self).ones, shape, dtype, name, parallel)

    def array(self, ary, dtype=None, name=None, persist_values=True,
              parallel=False, distributed=False, allocator=None):
        if not parallel:
            return super(ShardedBackend, self).array(ary, dtype=dtype, name=name)
        ary = np.asarray(ary)
        t = self.empty(ary.shape, dtype=dtype, name=name, parallel=True)
        return t.set(ary.astype(t.dtype))

    # ---- temporaries of split statements: a part that spans the sharded columns is itself a shard
    @staticmethod
    def _sharded_columns(expr):
        """Global column count of the sharded tensors under ``expr`` (None when there are none)."""
        todo = [expr]
        while todo:
            node = todo.pop()
            if isinstance(node, ShardedTensor):
                return node.shape[1]
            if type(node) is OpTreeNode:
                todo.extend(n for n in (node[1], node[2]) if n is not None)
        return None

    def _materialise(self, expr, shape, stmts):
        shape = tuple(shape)
        if type(expr) is not tuple:
            g = self._sharded_columns(expr)
            if g is not None and g > 1 and len(shape) == 2 and shape[1] == g:
                key = ("sharded",) + shape
                used = self._temps_used.get(key, 0)
                self._temps_used[key] = used + 1
                pool = self._temps.setdefault(key, [])
                while len(pool) <= used:
                    pool.append(self.empty(shape, dtype=self.default_dtype, parallel=True))
                stmts.append((pool[used], expr))
                return pool[used]
        return super(ShardedBackend, self)._materialise(expr, shape, stmts)

    # ---- one statement
    def _run_stack(self, out, stack):
        sharded, local_stack = [], []
        for s in stack:                         # one walk: which operands are shards, and the rank's view of the program
            if type(s) is ShardedTensor:
                sharded.append(s)
                local_stack.append(s.local)
            else:
                local_stack.append(s)
        if not sharded:
            return super(ShardedBackend, self)._run_stack(out, stack)
        lin = None
        if type(out) is ShardedTensor:
            lin = out.flat_of if out.flat_of else (out.shape[1], out.c0, out.local.shape[1])
        if self.check_bounds:
            self.check_operands(local_stack)
        rounding = self._rounding_bits(local_stack[0])
        key = (program_key(local_stack), rounding, lin)
        cached = self._plans.get(key)
        if cached is None:
            uses_rng = bool(rounding) or any(type(s) is dict and s["op"] == "rand" for s in stack)
            # random words need element coordinates: a flat pass can supply them only when
            # no block straddles a row of the shard (the pass shrinks its blocks to 2048 elements if it has to)
            row_ok = lin is not None and out.flat_of is None and lin[2] % 2048 == 0
            st = Statement(local_stack, allow_flat=(not uses_rng) or row_ok)
            crosses = st.has_red and st.axis == 1
            local_ids = set(id(s.local) for s in sharded)
            shard_ops = set(i for i, o in enumerate(st.operands) if id(o.tensor) in local_ids)
            passes = None
            if crosses and self._xchg is not None:
                # reductions along the sharded axis finish across the GPUs inside their kernels
                flat = sharded[0].flat_of is not None
                has_arg = any(type(s) is dict and s["op"] in ("argmax", "argmin") for s in stack)
                if not (flat and has_arg):
                    xchg = dict(self._xchg, col0=0 if flat else sharded[0].c0)
                    try:
                        self._scratch.reset()
                        passes = self._planner.plan(st, self._scratch, rounding=rounding, lin=lin,
                                                    xchg=xchg, sharded=shard_ops)
                        crosses = False              # nothing left to do between the passes
                    except XchgUnsupported:
                        passes = None
                        st = Statement(local_stack, allow_flat=(not uses_rng) or row_ok)
            if passes is None:
                self._scratch.reset()
                passes = self._planner.plan(st, self._scratch, rounding=rounding, fuse_final=not crosses,
                                            lin=lin, sharded=shard_ops)
            cached = self._plans[key] = (BoundPlan(st, passes), crosses)
        else:
            cached[0].rebind(local_stack)
        plan, crosses = cached
        for pz in plan.passes:
            if pz.uses_xchg:
                self._xepoch += 1
                pz.fields.values["x_epoch"] = (self._xepoch - self._xbase) & 0xFFFFFFFF
                self.exchanges += 1
            self._launch(pz)
            if crosses:
                # one collective per run of results that share the operation and sit next to each
                # other in scratch (results of one pass are allocated back to back, each padded to
                # 256 bytes: the padding is reduced along with them and never read)
                run = None                       # [op, first address, end address]
                for op, addr_v, addr_i, count in pz.results:
                    if op not in _NCCL_OP:
                        if run is not None:
                            self._allreduce(run[1], (run[2] - run[1]) // 4, _NCCL_OP[run[0]])
                            run = None
                        self._merge_arg(op, addr_v, addr_i, count, sharded[0])
                        continue
                    if run is not None and run[0] == op and addr_v == ((run[2] + 255) & ~255):
                        run[2] = addr_v + 4 * count
                        continue
                    if run is not None:
                        self._allreduce(run[1], (run[2] - run[1]) // 4, _NCCL_OP[run[0]])
                    run = [op, addr_v, addr_v + 4 * count]
                if run is not None:
                    self._allreduce(run[1], (run[2] - run[1]) // 4, _NCCL_OP[run[0]])

    # ---- recorded sequences
    def capture(self, fn):
        """As ``B200Backend.capture``, for statements over sharded tensors: every rank records
        the same sequence and replays it at the same point of its program.  Reductions that
        finish across the GPUs number their launches; a replay gives the recorded launches
        fresh numbers by moving the device word their parameters are relative to, so recorded
        and eager statements can be mixed freely."""
        state = {}

        def run():
            # _record calls this twice: eagerly, then while recording
            if "runs" in state:
                state["first"] = self._xepoch
            state["runs"] = True
            fn()
        handle, launches, table, keys = self._record(run)
        first = state["first"]
        count = self._xepoch - first
        self._xepoch = first                      # nothing was launched while recording
        self.exchanges -= count
        return ShardedGraph(self, handle, launches, first, count, self._xbase, table, keys)

    def _merge_arg(self, op, addr_v, addr_i, count, like):
        """argmax / argmin across the shards on the path without the exchange area: every rank
        contributes (extreme value, local index) per row, all ranks gather the pairs, and the
        host of each rank -- all with the same data, so all with the same answer -- turns the
        indices into global ones in integer arithmetic and keeps, per row, the smallest global
        index among the ranks that hold the extreme value: the first occurrence, as
        numpy.argmax gives it.  (Synchronous, a few hundred bytes per row: this is the
        fallback; the exchange area does the same inside the reduction kernel.)"""
        W = self.world_size
        vals, idxs = rt.malloc(4 * count * W), rt.malloc(4 * count * W)
        try:
            rt.allgather(self.comm, addr_v, vals, 4 * count, self.stream)
            rt.allgather(self.comm, addr_i, idxs, 4 * count, self.stream)
            self.collectives += 2
            hv, hi = np.empty((W, count), np.float32), np.empty((W, count), np.int32)
            rt.memcpy_d2h(hv.ctypes.data, vals, hv.nbytes, self.stream, sync=True)
            rt.memcpy_d2h(hi.ctypes.data, idxs, hi.nbytes, self.stream, sync=True)
        finally:
            rt.free(vals)
            rt.free(idxs)
        glob = hi.astype(np.int64)
        if like.flat_of is None:
            per = like.shape[1] // W
            glob += (np.arange(W, dtype=np.int64) * per)[:, None]
        else:                                   # index into the flattened shard -> into the flattened tensor
            gcols, _, lcols = like.flat_of
            glob = (glob // lcols) * gcols + (np.arange(W, dtype=np.int64) * lcols)[:, None] + glob % lcols
        best = hv.max(axis=0) if op == "argmax" else hv.min(axis=0)
        glob[hv != best[None, :]] = np.iinfo(np.int64).max
        winner = glob.min(axis=0).astype(np.int32)
        rt.memcpy_h2d(addr_i, winner.ctypes.data, winner.nbytes, self.stream, sync=True)

    def _allreduce(self, addr, count, op):
        mark = self._timeline_begin("collective", "allreduce") if self._timeline is not None else None
        rt.allreduce(self.comm, addr, addr, count, rt.F32, op, self.stream)
        if mark is not None:
            rt.event_record(mark, self.stream)
        self.collectives += 1

    def allreduce_tensor(self, tensor, op="sum"):
        """In-place all-reduce of a replicated fp32 tensor (e.g. shard-local totals)."""
        assert tensor.dtype == np.float32 and tensor.is_contiguous
        self._allreduce(tensor.ptr, tensor.size, _NCCL_OP[op])


class ShardedGraph(CapturedGraph):
    """A recorded statement sequence of a ShardedBackend (see ``ShardedBackend.capture``)."""

    def __init__(self, backend, handle, launches, first, count, base, rng_table=0, rng_count=0):
        super(ShardedGraph, self).__init__(backend, handle, launches, rng_table, rng_count)
        # the recorded exchange launches carry parameters first + 1 - base .. first + count - base
        self.first, self.count, self.base = first, count, base

    def replay(self):
        be = self.backend
        if self.count:
            # the launches must get the numbers be._xepoch + 1 ..: parameter + word = number
            be._xbase = (be._xepoch - self.first + self.base) & 0xFFFFFFFF
            rt.memset(be._xbase_word, be._xbase, 4, 1, be.stream)
            be._xepoch += self.count
            be.exchanges += self.count
        super(ShardedGraph, self).replay()


class HostGroup(object):
    """The few host-side collectives the job needs -- hand out the communicator id, a barrier,
    a maximum over ranks (for timings) -- over plain TCP: rank 0 listens on ``MASTER_ADDR`` at
    ``MASTER_PORT + 1`` (the port itself belongs to whatever launched the ranks) and is the hub
    of a star.  Messages are fixed-size; nothing here touches tensor data."""

    def __init__(self, rank, world_size, addr=None, port=None, timeout=120.0):
        import os
        import socket
        import time
        self.rank, self.world_size = rank, world_size
        self.peers, self.hub = [], None
        if world_size == 1:
            return
        addr = addr or os.environ.get("MASTER_ADDR", "127.0.0.1")
        port = int(port or int(os.environ.get("MASTER_PORT", "29500")) + 1)
        if rank == 0:
            srv = socket.socket(socket.AF_INET, socket.SOCK_STREAM)
            srv.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
            srv.bind((addr, port))
            srv.listen(world_size)
            srv.settimeout(timeout)
            by_rank = {}
            while len(by_rank) < world_size - 1:
                conn, _ = srv.accept()
                conn.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)
                conn.settimeout(timeout)
                by_rank[int.from_bytes(self._recv(conn, 4), "little")] = conn
            srv.close()
            self.peers = [by_rank[r] for r in range(1, world_size)]
        else:
            deadline = time.time() + timeout
            while True:
                try:
                    self.hub = socket.create_connection((addr, port), timeout=timeout)
                    break
                except OSError:
                    if time.time() > deadline:
                        raise
                    time.sleep(0.05)
            self.hub.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)
            self.hub.sendall(int(rank).to_bytes(4, "little"))

    @staticmethod
    def _recv(conn, n):
        buf = b""
        while len(buf) < n:
            part = conn.recv(n - len(buf))
            if not part:
                raise ConnectionError("peer closed the rendezvous connection")
            buf += part
        return buf

    def broadcast(self, payload, nbytes):
        """``payload`` (bytes of length nbytes) of rank 0, on every rank."""
        if self.world_size == 1:
            return payload
        if self.rank == 0:
            for c in self.peers:
                c.sendall(payload)
            return payload
        return self._recv(self.hub, nbytes)

    def max(self, value):
        import struct
        if self.world_size == 1:
            return float(value)
        if self.rank == 0:
            vals = [float(value)] + [struct.unpack("<d", self._recv(c, 8))[0] for c in self.peers]
            out = max(vals)
            for c in self.peers:
                c.sendall(struct.pack("<d", out))
            return out
        self.hub.sendall(struct.pack("<d", float(value)))
        return struct.unpack("<d", self._recv(self.hub, 8))[0]

    def barrier(self):
        self.max(0.0)

    def close(self):
        for c in self.peers + ([self.hub] if self.hub else []):
            try:
                c.close()
            except OSError:
                pass
        self.peers, self.hub = [], None


def bootstrap(rank, world_size, make_id=None, init_comm=None, addr=None, port=None):
    """Host-side rendezvous: rank 0 creates the NCCL unique id, everybody receives it and joins
    the communicator.  Returns (comm, barrier, max_over_ranks).  The two callables default to
    the library's NCCL bridge; tests pass stand-ins."""
    make_id = make_id or rt.comm_unique_id
    init_comm = init_comm or rt.comm_init
    group = HostGroup(rank, world_size, addr, port)
    uid = bytes(make_id()) if rank == 0 else None
    uid = group.broadcast(uid, 128)
    comm = init_comm(uid, world_size, rank)
    return comm, group.barrier, group.max


def gen_sharded_backend(rank, world_size, device_id=0, rng_seed=None, datatype=np.float32, **kw):
    """One rank's backend of a ``world_size``-GPU job (launch one process per GPU,
    e.g. with ``python -m torch.distributed.run``)."""
    rt.init(int(device_id))
    comm, barrier, host_max = bootstrap(rank, world_size)
    return ShardedBackend(rank, world_size, comm, barrier, host_max, rng_seed=rng_seed,
                          default_dtype=datatype, device_id=device_id, **kw)
