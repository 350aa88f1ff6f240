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
* ``sum`` / ``max`` / ``min`` along axis 1 (and over a whole tensor) reduce the
  local shard, then the per-row fp32 results are all-reduced over NCCL before
  the next pass reads them (so a variance needs two all-reduces, of the sum and
  of the centred squares);
* random numbers and stochastic rounding use the element index in the global
  tensor, so stored values do not depend on how many GPUs share the work.

Host plumbing (rank discovery, the NCCL unique id, barriers, max-over-ranks of
timings) rides on a gloo ``torch.distributed`` group; no torch tensor touches
the data path.
"""

import numpy as np

from . import runtime as rt
from .backend import B200Backend
from .lowering import BoundPlan, Statement, program_key
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

    def __init__(self, rank, world_size, comm, host_barrier=None, host_max=None, **kw):
        super(ShardedBackend, self).__init__(**kw)
        self.rank, self.world_size, self.comm = rank, world_size, comm
        self.host_barrier = host_barrier or (lambda: None)
        self.host_max = host_max or (lambda v: v)
        self.collectives = 0                 # all-reduces issued so far

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
        sharded = [s for s in stack if isinstance(s, ShardedTensor)]
        if not sharded:
            return super(ShardedBackend, self)._run_stack(out, stack)
        lin = None
        if isinstance(out, ShardedTensor):
            lin = out.flat_of if out.flat_of else (out.shape[1], out.c0, out.local.shape[1])
        local_stack = [s.local if isinstance(s, ShardedTensor) else s for s in stack]
        rounding = self._rounding_bits(local_stack[0])
        key = (program_key(local_stack), rounding, lin)
        cached = self._plans.get(key)
        if cached is None:
            uses_rng = bool(rounding) or any(type(s) is dict and s["op"] == "rand" for s in stack)
            # random words need element coordinates: a flat pass can supply them only when
            # no block straddles a row of the shard (8192 elements per block at most)
            row_ok = lin is not None and out.flat_of is None and lin[2] % 8192 == 0
            st = Statement(local_stack, allow_flat=(not uses_rng) or row_ok)
            crosses = st.has_red and st.axis == 1
            self._scratch.reset()
            passes = self._planner.plan(st, self._scratch, rounding=rounding, fuse_final=not crosses, lin=lin)
            cached = self._plans[key] = (BoundPlan(st, passes), crosses)
        else:
            cached[0].rebind(local_stack)
        plan, crosses = cached
        for pz in plan.passes:
            self._launch(pz)
            if crosses:
                for op, addr_v, addr_i, count in pz.results:
                    if op in _NCCL_OP:
                        self._allreduce(addr_v, count, _NCCL_OP[op])
                    else:
                        self._merge_arg(op, addr_v, addr_i, count, sharded[0])

    def _merge_arg(self, op, addr_v, addr_i, count, like):
        """argmax / argmin across the shards: every rank contributes (extreme value,
        global column index) per row, all ranks gather the pairs and keep, per row,
        the index of the first rank that holds the extreme value -- columns grow with
        the rank, so that is the first occurrence, as numpy.argmax gives it."""
        from .tensor import B200Tensor
        W = self.world_size
        idx = B200Tensor(self, (1, count), np.int32, gpudata=addr_i)
        c0 = like.c0 if like.flat_of is None else 0
        idx[:] = idx + float(c0)                                   # local -> global column
        vals = self.empty((W, count), dtype=np.float32)
        idxs = self.empty((W, count), dtype=np.int32)
        rt.allgather(self.comm, addr_v, vals.ptr, 4 * count, self.stream)
        rt.allgather(self.comm, addr_i, idxs.ptr, 4 * count, self.stream)
        self.collectives += 2
        winner = self.empty((1, count), dtype=np.int32)
        winner[:] = self.argmax(vals, axis=0) if op == "argmax" else self.argmin(vals, axis=0)
        idx[:] = self.sum(self.onehot(winner, axis=0) * idxs, axis=0)

    def _allreduce(self, addr, count, op):
        rt.allreduce(self.comm, addr, addr, count, rt.F32, op, self.stream)
        self.collectives += 1

    def allreduce_tensor(self, tensor, op="sum"):
        """In-place all-reduce of a replicated fp32 tensor (e.g. shard-local totals)."""
        assert tensor.dtype == np.float32 and tensor.is_contiguous
        self._allreduce(tensor.ptr, tensor.size, _NCCL_OP[op])


def bootstrap(rank, world_size, make_id=None, init_comm=None):
    """Host-side rendezvous over a gloo process group: rank 0 creates the NCCL
    unique id, everybody receives it and joins the communicator.  Returns
    (comm, barrier, max_over_ranks).  The two callables default to the library's
    NCCL bridge; tests pass stand-ins."""
    import torch
    import torch.distributed as dist
    if not dist.is_initialized():
        dist.init_process_group(backend="gloo", rank=rank, world_size=world_size)
    make_id = make_id or rt.comm_unique_id
    init_comm = init_comm or rt.comm_init
    box = [make_id() if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    comm = init_comm(box[0], world_size, rank)

    def barrier():
        dist.barrier()

    def max_over_ranks(value):
        t = torch.tensor([float(value)], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0])

    return comm, barrier, max_over_ranks


def gen_sharded_backend(rank, world_size, device_id=0, rng_seed=None, datatype=np.float32, **kw):
    """One rank's backend of a ``world_size``-GPU job (launch one process per GPU,
    e.g. with ``python -m torch.distributed.run``)."""
    rt.init(int(device_id))
    comm, barrier, host_max = bootstrap(rank, world_size)
    return ShardedBackend(rank, world_size, comm, barrier, host_max, rng_seed=rng_seed,
                          default_dtype=datatype, device_id=device_id, **kw)
