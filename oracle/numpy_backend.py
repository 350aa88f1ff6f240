"""
TEST INFRASTRUCTURE ONLY -- the CPU checker for the compound-optree path.

A numpy restatement of how neon's NervanaCPU backend evaluates an op-tree
(``neon/backends/nervanacpu.py``): the tree is flattened to a postfix program
and interpreted with one numpy call per op.  Only ``tests/``, the smoke check
and the CPU-baseline leg of the benchmark may import this module; the product
(``neon_b200``) never does.

Parity status: PINNED.  ``tests/golden/make_golden.py`` imports the real
``NervanaCPU`` from a neon checkout, runs the five benchmark configurations
(at sizes numpy finishes in seconds) and the cases of neon's own backend tests,
and stores seeds + outputs in ``tests/golden/*.npz``; ``tests/test_oracle.py``
requires this restatement to reproduce those files bit for bit (same numpy
calls in the same order), and to match the live reference when one is present.

What follows which reference lines
  * op table ``NUMPY_OPS``       -- nervanacpu.py:480-522 (numpy_call_dict_cpu)
  * ``OracleBackend.execute``    -- nervanacpu.py:652-715
  * bare one-hot assignment      -- nervanacpu.py:660-683
  * ``OracleTensor``             -- nervanacpu.py:37-330 (CPUTensor), trimmed to
                                    what op-tree execution and the tests touch
  * assignment casts with numpy  -- nervanacpu.py:476-477 (``left[:] = right``)
"""

import numpy as np

from neon_b200.optree import OpCollection, OpTreeBackend, OpTreeNode, Tensor

_none_slice = slice(None, None, None)


def _argred(fn):
    def f(info, x):
        shape = list(x.shape)
        shape[info["axis"]] = 1
        return fn(x, axis=info["axis"]).reshape(shape)
    return f


def _assign(left, right):
    left[:] = right


# nervanacpu.py:480-522, entry for entry
NUMPY_OPS = {
    "assign": _assign,
    "neg": lambda x: -x,
    "abs": lambda x: np.abs(x),
    "sgn": lambda x: np.sign(x),
    "sqrt": lambda x: np.sqrt(x),
    "sqr": lambda x: np.square(x),
    "exp": lambda x: np.exp(x),
    "log": lambda x: np.log(x),
    "safelog": lambda x: np.log(np.maximum(x, np.exp(-50.))),
    "exp2": lambda x: np.exp2(x),
    "log2": lambda x: np.log2(x),
    "sig": lambda x: 1. / (1. + np.exp(-x)),
    "sig2": lambda x: 1. / (1. + np.exp2(-x)),
    "tanh": lambda x: np.tanh(x),
    "tanh2": lambda x: (np.exp2(2. * x) - 1.) / (np.exp2(2. * x) + 1.),
    "transpose": lambda x: np.transpose(x),
    "rint": lambda x: np.rint(x),
    "add": lambda a, b: a + b,
    "sub": lambda a, b: a - b,
    "mul": lambda a, b: a * b,
    "div": lambda a, b: a / b,
    "eq": lambda a, b: a == b,
    "ne": lambda a, b: a != b,
    "lt": lambda a, b: a < b,
    "le": lambda a, b: a <= b,
    "gt": lambda a, b: a > b,
    "ge": lambda a, b: a >= b,
    "pow": lambda a, b: np.power(a, b),
    "minimum": lambda a, b: np.minimum(a, b),
    "maximum": lambda a, b: np.maximum(a, b),
    "dot": lambda a, b: np.dot(a, b),
    "sum": lambda info, x: np.sum(x, axis=info["axis"], keepdims=True),
    "max": lambda info, x: np.max(x, axis=info["axis"], keepdims=True),
    "min": lambda info, x: np.min(x, axis=info["axis"], keepdims=True),
    "argmax": _argred(np.argmax),
    "argmin": _argred(np.argmin),
}

# The GPU kernel vocabulary has one op the CPU table lacks and that does not
# consume random bits (cuda_templates.py:531-538, testp.finite): restated here
# so finite() can be checked too.  Not part of nervanacpu.py.
GPU_ONLY_OPS = {
    "finite": lambda x: np.isfinite(x).astype(np.float32),
    # C's roundf as the GPU shift kernel uses it (kernels/cuda/binary.py:184)
    "round": lambda x: np.where(x >= 0, np.floor(x + 0.5), np.ceil(x - 0.5)),
}


class OracleTensor(Tensor):
    """numpy-backed tensor with the CPUTensor surface (nervanacpu.py:37-330)."""

    def __init__(self, backend, shape=None, dtype=np.float32, ary=None,
                 name=None, persist_values=True, base=None):
        super(OracleTensor, self).__init__(backend, shape, dtype, name, persist_values)
        dtype = np.dtype(dtype)
        if type(ary) is not np.ndarray:
            t = np.array(ary, dtype)
        elif ary.dtype != dtype:
            t = ary.astype(dtype)
        else:
            t = ary
        while t.ndim < self._min_dims:
            t = t.reshape(t.shape + (1,))
        self._tensor = t
        self.shape = tuple(int(d) for d in t.shape)
        self.size = int(t.size)
        self.dtype = dtype
        self.base = base
        self.rounding = 0
        self.is_trans = False

    @property
    def is_contiguous(self):
        return self._tensor.flags.c_contiguous

    def __len__(self):
        return self.shape[0] if len(self.shape) else 0

    def __getitem__(self, key):
        if not isinstance(key, tuple):
            if isinstance(key, slice) and key == _none_slice:
                return self
            key = (key,)
        key = tuple(slice(k % self.shape[i], k % self.shape[i] + 1)
                    if isinstance(k, (int, np.integer)) else k
                    for i, k in enumerate(key))
        sub = self._tensor[key]
        shape = list(sub.shape)
        while len(shape) > 2 and 1 in shape:
            shape.remove(1)
        view = OracleTensor(self.backend, ary=sub.reshape(shape),
                            dtype=sub.dtype, base=self)
        view.is_trans = self.is_trans
        return view

    def _assign(self, value):
        if isinstance(value, (OracleTensor, OpTreeNode)):
            OpTreeNode.build("assign", self, value)
        elif isinstance(value, (int, float, np.ndarray)):
            self.set(value)
        else:
            raise TypeError("Invalid type for assignment: %s" % type(value))
        return self

    def set(self, value):
        if isinstance(value, np.ndarray):
            if value.dtype != self.dtype:
                value = value.astype(self.dtype)
            assert value.size == self.size
            if value.ndim < self._min_dims:
                value = value.reshape(self.shape)
        self._tensor[:] = value
        return self

    def get(self):
        return self._tensor.copy()

    def raw(self):
        return self._tensor.ctypes.data

    def take(self, indices, axis=None, out=None):
        if isinstance(indices, OracleTensor):
            indices = indices._tensor
        indices = np.asarray(indices).squeeze()
        shape = list(self.shape)
        shape[axis] = indices.size
        view = OracleTensor(self.backend,
                            ary=self._tensor.take(indices, axis).reshape(shape),
                            dtype=self._tensor.dtype, base=self)
        if out is not None:
            return out._assign(view)
        return view

    def reshape(self, *shape):
        if isinstance(shape[0], (tuple, list)):
            shape = tuple(shape[0])
        if shape == self.shape:
            return self
        return OracleTensor(self.backend, ary=self._tensor.reshape(shape),
                            dtype=self._tensor.dtype, base=self)

    @property
    def T(self):
        view = OracleTensor(self.backend, ary=self._tensor.transpose(),
                            dtype=self._tensor.dtype, base=self)
        view.is_trans = not self.is_trans
        return view

    def transpose(self, out=None):
        if out:
            return OpTreeNode.build("assign", out, self.T)
        return self.T

    def share(self, shape, dtype=None, name=None):
        size = int(np.prod(shape))
        if size > self.size:
            raise ValueError("total size of new array must <= size of parent")
        dtype = self.dtype if dtype is None else np.dtype(dtype)
        raw = self._tensor.reshape(-1).view(np.uint8)
        ary = raw[:size * dtype.itemsize].view(dtype).reshape(shape)
        return OracleTensor(self.backend, ary=ary, dtype=ary.dtype, name=name,
                            base=self if self.base is None else self.base)


class OracleBackend(OpTreeBackend):
    """numpy interpreter of postfix op-tree programs (nervanacpu.py:524-715)."""
    backend_name = "oracle"

    def __init__(self, rng_seed=None, default_dtype=np.float32, **ignored):
        if default_dtype not in (np.float16, np.float32, np.float64):
            raise ValueError("default dtype must be float16, 32 or 64")
        super(OracleBackend, self).__init__(rng_seed, default_dtype)

    def gen_rng(self, seed=None):
        self.rng = np.random.RandomState(seed)
        self.init_rng_state = self.rng.get_state()
        return self.rng

    def execute(self, optree, ops=NUMPY_OPS):
        rhs = optree[2]
        if isinstance(rhs, OpTreeNode) and rhs[0]["op"] == "onehot":
            # nervanacpu.py:660-683: a bare one-hot assignment is scattered
            out = optree[1]._tensor
            axis = rhs[0]["axis"]
            hot = np.asarray(rhs[0]["idx"]._tensor).squeeze().reshape(-1)
            ind = [None, None]
            ind[axis] = hot
            ind[1 - axis] = np.arange(hot.size)
            out[:] = 0
            out[tuple(ind)] = 1
            return optree[1]

        program = optree.traverse([])
        stack = []
        for p in program:
            if isinstance(p, dict):
                op = p["op"]
                if op in OpCollection.reduction_ops:
                    stack.append(ops[op](p, stack.pop()))
                elif op in OpCollection.unary_ops:
                    fn = ops.get(op) or GPU_ONLY_OPS.get(op)
                    if fn is None:
                        raise NotImplementedError(op)
                    stack.append(fn(stack.pop()))
                elif op in OpCollection.binary_ops:
                    right = stack.pop()
                    left = stack.pop()
                    stack.append(ops[op](left, right))
                else:
                    raise NotImplementedError(op)
            elif isinstance(p, OracleTensor):
                stack.append(p._tensor)
            else:
                stack.append(p)
        assert len(stack) == 1
        return program[0]

    # ---- factories (nervanacpu.py:717-930)
    def _dt(self, dtype):
        return self.default_dtype if dtype is None else dtype

    def empty(self, shape, dtype=None, name=None, persist_values=True,
              parallel=False, distributed=False):
        dtype = self._dt(dtype)
        return OracleTensor(self, ary=np.zeros(shape, dtype), dtype=dtype, name=name)

    zeros = empty

    def ones(self, shape, dtype=None, name=None, persist_values=True,
             parallel=False, distributed=False):
        dtype = self._dt(dtype)
        return OracleTensor(self, ary=np.ones(shape, dtype), dtype=dtype, name=name)

    def array(self, ary, dtype=None, name=None, persist_values=True,
              parallel=False, distributed=False):
        dtype = self._dt(dtype)
        return OracleTensor(self, ary=np.array(ary, dtype), dtype=dtype, name=name)

    def empty_like(self, other, name=None, persist_values=True):
        return self.empty(other.shape, dtype=self.default_dtype, name=name)

    def zeros_like(self, other, name=None, persist_values=True):
        return self.zeros(other.shape, dtype=self.default_dtype, name=name)

    @staticmethod
    def log2_hist(values, nbins=64, offset=-48):
        """Counts per bin of clamp(round(log2|x|) - offset, 0, nbins - 1), with C's round (halves
        away from zero), zero and NaN in bin 0 and infinity in the last bin: what the kernel text
        of float_ew.py:1086-1100 computes in fp32 (GPU only in the reference)."""
        a = np.abs(np.asarray(values).astype(np.float32)).ravel()
        with np.errstate(divide="ignore", invalid="ignore"):
            lg = np.log2(a).astype(np.float32)
            t = np.where(lg >= 0, np.floor(lg + np.float32(0.5)), np.ceil(lg - np.float32(0.5))) - np.float32(offset)
        bins = np.where(~(t > 0), 0, np.where(t < nbins - 1, t, nbins - 1))
        bins = np.nan_to_num(bins, nan=0.0).astype(np.int64)
        return np.bincount(bins, minlength=nbins).astype(np.int32)

    def copy_transpose(self, a, out, axes=None, repeat=1):
        """numpy.transpose into ``out`` (nervanacpu.py:1046-1051)."""
        out._tensor[:] = np.transpose(a._tensor, axes).copy()

    def rng_reset(self):
        self.rng.set_state(self.init_rng_state)

    def rng_get_state(self):
        return self.rng.get_state()

    def rng_set_state(self, state):
        self.rng.set_state(state)
