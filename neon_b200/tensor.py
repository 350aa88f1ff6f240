"""
Device tensor of the b200 backend.

Same surface and behaviour as neon's ``GPUTensor``
(neon/backends/nervanagpu.py:48-659): at least two dimensions, row-major,
strides counted in elements, views made by pointer arithmetic that keep their
base alive, fancy indexing recorded as ``take_array``, per-tensor ``rounding``
bits, and the three assignment fast paths (fill -> memset, same-layout tensor
-> device copy, anything else -> op-tree kernel).  Memory comes from the
library's caching arena instead of ``pycuda.driver.mem_alloc``.
"""

import numpy as np

from . import runtime as rt
from .optree import OpTreeNode, Tensor

_none_slice = slice(None, None, None)

SUPPORTED = (np.float16, np.float32, np.uint8, np.int8, np.uint16, np.int16, np.uint32, np.int32)
try:                                    # bfloat16 storage when the numpy extension type is installed
    import ml_dtypes
    bfloat16 = ml_dtypes.bfloat16
    SUPPORTED = SUPPORTED + (bfloat16,)
except ImportError:                     # pragma: no cover
    bfloat16 = None


def _contiguous_strides(shape):
    if not shape:
        return ()
    strides = [1]
    for s in shape[:0:-1]:
        strides.append(strides[-1] * max(1, s))
    return tuple(strides[::-1])


def _reshape_strides(strides, shape, new_shape):
    """Strides of a reshaped view (nervanagpu.py:3243-3263): leading dimensions
    that do not change keep their strides; everything after them must be laid
    out contiguously so that it can be re-cut freely."""
    keep = 0
    for a, b in zip(shape, new_shape):
        if a != b:
            break
        keep += 1
    tail_shape, tail_strides = tuple(shape[keep:]), tuple(strides[keep:])
    if tail_shape and tail_strides != _contiguous_strides(tail_shape):
        raise ValueError("Reshaping of non-contiguous dimensions unsupported.")
    return tuple(strides[:keep]) + _contiguous_strides(tuple(new_shape[keep:]))


class _Block(object):
    """Owner of one arena allocation; returns it when the last tensor lets go."""
    __slots__ = ("ptr", "nbytes")

    def __init__(self, nbytes):
        self.nbytes = nbytes
        self.ptr = rt.malloc(nbytes)

    def __del__(self):
        try:
            if self.ptr:
                rt.free(self.ptr)
                self.ptr = 0
        except Exception:
            pass


class B200Tensor(Tensor):

    def __init__(self, backend, shape=None, dtype=np.float32, name=None, persist_values=True,
                 allocator=None, base=None, gpudata=None, strides=None, take_array=None,
                 is_trans=False, rounding=0, _block=None):
        super(B200Tensor, self).__init__(backend, shape, dtype, name, persist_values)
        dtype = np.dtype(dtype)
        assert dtype.type in SUPPORTED, "unsupported dtype %s" % dtype
        if not isinstance(shape, (tuple, list)):
            assert isinstance(shape, (int, np.integer))
            shape = (int(shape),)
        shape = tuple(shape)
        if len(shape) < self._min_dims:
            shape = shape + (1,) * (self._min_dims - len(shape))
        dims, size = [], 1
        for d in shape:
            if int(d) != d:
                raise TypeError("shape dims must be integer values [%s]" % str(d))
            dims.append(int(d))
            size *= int(d)
        self.shape = tuple(dims)
        self.size = size
        self.dtype = dtype
        self.nbytes = dtype.itemsize * size
        if strides is None:
            self.strides = _contiguous_strides(self.shape)
        else:                                    # a view of fewer than two axes was padded with unit axes
            self.strides = tuple(int(s) for s in strides) + (1,) * (len(self.shape) - len(strides))
        self.base = base
        self.allocator = allocator
        self.take_array = take_array
        self.is_trans = is_trans
        self.rounding = rounding
        self.kahan_count = 0
        self.kahan_reset = 0
        if gpudata is None:
            assert base is None
            self._block = _Block(self.nbytes) if size else None
            self.gpudata = self._block.ptr if self._block else 0
        else:
            self._block = _block
            self.gpudata = int(gpudata)
        # what the plan cache needs to know about this tensor (none of it changes afterwards)
        self._plan_key = (dtype.str, self.shape, self.strides, self.gpudata & 15,
                          take_array[1] if take_array else None)

    # ---- description
    def __str__(self):
        return ("B200Tensor(base 0x%x) name:%s shape:%s dtype:%s strides:%s is_trans:%s is_contiguous:%s"
                % (self.gpudata, self.name, self.shape, self.dtype, self.strides, self.is_trans,
                   self.is_contiguous))

    __repr__ = __str__

    def __len__(self):
        return self.shape[0] if len(self.shape) else 0

    def __int__(self):
        return int(self.gpudata)

    @property
    def ptr(self):
        return int(self.gpudata)

    def raw(self):
        return self.gpudata

    @property
    def is_contiguous(self):
        return not self.take_array and self.strides == _contiguous_strides(self.shape)

    def _view(self, shape, strides, offset_bytes=0, take_array=None, is_trans=None, name=None, dtype=None):
        return self.__class__(backend=self.backend, shape=shape, dtype=dtype or self.dtype,
                              allocator=self.allocator, base=self, gpudata=self.gpudata + offset_bytes,
                              strides=strides, take_array=take_array,
                              is_trans=self.is_trans if is_trans is None else is_trans,
                              name=self.name if name is None else name, rounding=self.rounding,
                              _block=self._block)

    # ---- indexing: same views, limits and messages as GPUTensor.__getitem__ (nervanagpu.py:193-323)
    def _index_records(self, index):
        """One record per axis of this tensor for the subscript ``index`` (a tuple):
        ("slice", first, step, count), ("at", position), ("take", int32 index tensor)."""
        ndim = len(self.shape)
        plain = [e for e in index if e is not Ellipsis]
        if len(index) - len(plain) > 1:
            raise IndexError("more than one ellipsis not allowed in index")
        if len(plain) > ndim:
            raise IndexError("invalid use of ellipsis in index" if len(plain) < len(index)
                             else "too many axes in index")
        everything = slice(None, None, None)
        expanded = []
        for e in index:
            if e is Ellipsis:
                expanded.extend([everything] * (ndim - len(plain)))
            else:
                expanded.append(e)
        expanded.extend([everything] * (ndim - len(expanded)))
        records = []
        for axis, e in enumerate(expanded):
            extent = self.shape[axis]
            if isinstance(e, slice):
                first, stop, step = e.indices(extent)
                records.append(("slice", first, step, max(0, -((first - stop) // step))))
            elif isinstance(e, (B200Tensor, np.ndarray, list, tuple)):
                if isinstance(e, (list, tuple)):
                    e = np.array(e, dtype=np.int32)
                if isinstance(e, np.ndarray):
                    e = self.__class__(self.backend, e.shape, dtype=np.int32).set(e)
                if max(e.shape) != e.size:
                    raise IndexError("Fancy indexing only currently supported dim > 1 in a single dimension.")
                if any(r[0] == "take" for r in records):
                    raise IndexError("Fancy indexing only currently supported one axis at a time.")
                if e.dtype.type is not np.int32:
                    raise IndexError("Fancy indexing only currently supported with int32 types.")
                records.append(("take", e))
            elif isinstance(e, (int, np.integer)):
                position = int(e) + extent if e < 0 else int(e)
                if not 0 <= position < extent:
                    raise IndexError("subindex in axis %d out of range" % axis)
                records.append(("at", position))
            else:
                raise IndexError("invalid subindex in axis %d" % axis)
        return records

    def __getitem__(self, index):
        if not isinstance(index, tuple):
            if isinstance(index, slice) and index == _none_slice:
                return self
            index = (index,)
        shape, strides, offset, take_array = [], [], 0, None
        keep_unit_axes = len(self.shape) < 3          # a matrix stays a matrix: x[3] is a (1, n) row
        for axis, record in enumerate(self._index_records(index)):
            pitch = self.strides[axis]
            if record[0] == "slice":
                _, first, step, count = record
                offset += first * pitch
                shape.append(count)
                strides.append(step * pitch)
            elif record[0] == "at":
                offset += record[1] * pitch
                if keep_unit_axes:
                    shape.append(1)
                    strides.append(pitch)
            else:
                take_array = (record[1], axis)
                shape.append(record[1].size)
                strides.append(pitch)
        return self._view(tuple(shape), strides, offset * self.dtype.itemsize, take_array=take_array)

    # ---- assignment (nervanagpu.py:334-383)
    def _assign(self, value):
        stream = self.backend.stream
        if isinstance(value, (int, float)):
            if self.is_contiguous:
                bits = np.array(value).astype(self.dtype)
                isz = self.dtype.itemsize
                pattern = int(bits.view({1: np.uint8, 2: np.uint16, 4: np.uint32}[isz]))
                rt.memset(self.gpudata, pattern, isz, self.size, stream)
            else:
                OpTreeNode.build("assign", self, value)
        elif isinstance(value, B200Tensor):
            if (self.is_contiguous and value.is_contiguous and self.dtype == value.dtype
                    and self.shape == value.shape):
                rt.memcpy_d2d(self.gpudata, value.gpudata, self.nbytes, stream)
            else:
                OpTreeNode.build("assign", self, value)
        elif isinstance(value, OpTreeNode):
            OpTreeNode.build("assign", self, value)
        elif isinstance(value, np.ndarray):
            self.set(value)
        else:
            raise TypeError("Invalid type for assignment: %s" % type(value))
        return self

    # ---- host transfer (nervanagpu.py:385-435)
    def set(self, ary):
        ary = np.asarray(ary)
        if ary.size != self.size:
            raise TypeError("ary.size {} != self.size {}".format(ary.size, self.size))
        assert self.is_contiguous, "Array in set() must be contiguous"
        if ary.dtype != self.dtype:
            ary = ary.astype(self.dtype)
        if ary.ndim < self._min_dims:
            ary = ary.reshape(ary.size, 1)
        want = tuple(self.dtype.itemsize * s for s in self.strides)
        if ary.shape == self.shape and ary.strides != want and self.size > 1 \
                and any(d > 1 and a != w for d, a, w in zip(ary.shape, ary.strides, want)):
            raise TypeError("ary.strides != self.strides * self.dtype.itemsize : {} != {} * {}".format(
                ary.strides, self.strides, self.dtype.itemsize))
        ary = np.ascontiguousarray(ary)
        rt.memcpy_h2d(self.gpudata, ary.ctypes.data, self.nbytes, self.backend.stream, sync=True)
        return self

    def get(self, stream=None):
        if self.is_contiguous:
            src = self
        else:
            src = self.backend.empty(self.shape, self.dtype)
            src.copy(self)
        ary = np.empty(self.shape, self.dtype)
        rt.memcpy_d2h(ary.ctypes.data, src.gpudata, self.nbytes, self.backend.stream, sync=True)
        return ary

    def asbuffer(self):
        raise NotImplementedError("host buffer interface to device memory")

    # ---- views (nervanagpu.py:437-610)
    def take(self, indices, axis, out=None):
        if axis == 1:
            view = self.__getitem__((_none_slice, indices))
        else:
            view = self.__getitem__((indices, _none_slice))
        if out:
            return out._assign(view)
        return view

    def reshape(self, *shape):
        if isinstance(shape[0], (tuple, list)):
            shape = tuple(shape[0])
        if len(shape) < self._min_dims:
            shape = shape + (1,)
        if -1 in shape:
            missing = -self.size // int(np.prod(shape))
            shape = tuple(missing if x == -1 else x for x in shape)
        shape = tuple(int(x) for x in shape)
        if shape == self.shape:
            return self
        if int(np.prod(shape)) != self.size:
            raise ValueError("total size of new array must be unchanged")
        if self.take_array:
            raise TypeError("reshaping of non-contiguous arrays is not yet supported")
        return self._view(shape, _reshape_strides(self.strides, self.shape, shape))

    @property
    def T(self):
        if len(self.shape) <= 2:
            shape, strides = self.shape[::-1], self.strides[::-1]
        else:
            shape, strides = list(self.shape[::-1]), list(self.strides[::-1])
            shape = tuple(shape[-1:] + shape[:-1])
            strides = tuple(strides[-1:] + strides[:-1])
        return self._view(shape, strides, is_trans=not self.is_trans)

    def transpose(self, out=None):
        if out:
            return OpTreeNode.build("assign", out, self.T)
        return self.T

    def share(self, shape, dtype=None, name=None):
        if not isinstance(shape, (tuple, list)):
            shape = (int(shape),)
        size = int(np.prod(shape))
        if size > self.size:
            raise ValueError("total size of new array must <= size of parent")
        if not self.is_contiguous:
            raise TypeError("sharing of non-contigous arrays is not yet supported")
        dtype = self.dtype if dtype is None else np.dtype(dtype)
        base = self if self.base is None else self.base
        shape = tuple(shape)
        full = shape + (1,) * max(0, self._min_dims - len(shape))
        return self.__class__(backend=self.backend, shape=shape, dtype=dtype, allocator=self.allocator,
                              base=base, gpudata=self.gpudata, strides=_contiguous_strides(full),
                              name=name, rounding=self.rounding, _block=self._block)

    def hist(self, tag):
        """Histogram of round(log2|x|) of the tensor's values in the backend's bins
        (nervanagpu.py:619-637); ``tag`` names the histogram in ``dump_hist_data``."""
        if not self.is_contiguous or self.take_array is not None:
            raise ValueError("histogram of a contiguous tensor only")
        hist_tensor = self.backend._hist_tensor(tag)
        self.backend._compute_hist(self, hist_tensor)
        return hist_tensor
