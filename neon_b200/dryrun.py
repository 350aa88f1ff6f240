"""
A b200 backend that lowers and compiles but never touches a device: tensors get
made-up (aligned) addresses and every kernel a statement needs is compiled to an
sm_100a image with NVRTC instead of being launched.  Used at build time to
instantiate the kernel templates on a machine without a GPU (NVRTC cross-compiles)
and by the CPU-only tests of the host lowering.  It computes nothing: ``get()``
returns zeros.
"""
import numpy as np

from neon_b200 import runtime as rt
from neon_b200.backend import B200Backend
from neon_b200.lowering import Planner, Statement
from neon_b200.optree import OpTreeNode
from neon_b200.tensor import B200Tensor


class DryTensor(B200Tensor):
    """No device behind it: fills and copies go through the op-tree path too."""

    def _assign(self, value):
        if isinstance(value, np.ndarray):
            return self
        OpTreeNode.build("assign", self, value)
        return self

    def set(self, ary):
        return self

    def get(self, stream=None):
        return np.zeros(self.shape, self.dtype)


class DryRunBackend(B200Backend):

    def __init__(self, default_dtype=np.float32, sm_count=148):
        self.default_dtype = default_dtype
        self.device_id = 0
        self.sm_count = sm_count
        self.stream = 0
        self.round_mode = 0
        self.bsz = None
        self._min_dims = 2
        self._planner = Planner(sm_count)
        self._temps, self._temps_used = {}, {}
        from .backend import _PlanCache
        self._plans = _PlanCache()
        self.compat_mode = None
        self.bench = False
        self.trace = []
        self._next = 0x7F0000000000
        self.launches = 0
        self.passes = []            # every Pass planned so far
        self.sources = {}           # source -> image size
        self.compile = True
        self.check_bounds = False
        self._scratch = None
        self.rng = np.random.RandomState(0)

    def cleanup_backend(self):
        pass

    def _fake(self, nbytes):
        p = self._next
        self._next += (nbytes + 255) & ~255
        return p

    def _scratch_alloc(self, nbytes, zero):
        return self._fake(nbytes)

    def empty(self, shape, dtype=None, name=None, persist_values=True, **kw):
        dtype = self.default_dtype if dtype is None else dtype
        if not isinstance(shape, (tuple, list)):
            shape = (int(shape),)
        size = int(np.prod(shape)) * np.dtype(dtype).itemsize
        return DryTensor(self, shape, dtype=dtype, name=name, gpudata=self._fake(max(size, 1)),
                         rounding=self.round_mode)

    def array(self, ary, dtype=None, **kw):
        return self.empty(np.asarray(ary).shape, dtype=dtype or self.default_dtype)

    def zeros(self, shape, dtype=None, **kw):
        return self.empty(shape, dtype=dtype)

    ones = zeros

    def empty_like(self, other, name=None, persist_values=True):
        return self.empty(other.shape, dtype=other.dtype)

    zeros_like = empty_like

    def compound_dot(self, A, B, C, alpha=1.0, beta=0.0, relu=False, bsum=None):
        assert A.shape[1] == B.shape[0] and C.shape == (A.shape[0], B.shape[1])
        self.launches += 1
        self.dots = getattr(self, "dots", 0) + 1
        return C

    def copy_transpose(self, a, out, axes=None, repeat=1):
        axes = tuple(range(len(a.shape) - 1, -1, -1)) if axes is None else tuple(axes)
        assert a.dtype == out.dtype and a.size == out.size and a.gpudata != out.gpudata
        assert all(out.shape[i] == a.shape[x] for i, x in enumerate(axes))
        self.launches += 1
        self.shuffles = getattr(self, "shuffles", 0) + 1
        return out

    def _run_stack(self, out, stack):
        st = Statement(stack)
        passes = self._planner.plan(st, self._scratch_alloc, rounding=self._rounding_bits(out))
        for pz in passes:
            pz.fields.pack()
            self.passes.append(pz)
            self.launches += 1
            if self.compile and pz.source not in self.sources:
                img, _ = rt.nvrtc_compile(pz.source)
                self.sources[pz.source] = len(img)
