"""
Op-tree front end: lazy expression nodes, the tensor base class whose operators
build them, and the backend mix-in with the `be.<op>(...)` builder functions.

This is the host-side boundary of the compound-optree engine.  It restates, API
for API, the part of neon's ``neon/backends/backend.py`` that layers, optimizers
and tests talk to:

* ``OpCollection``  (backend.py:30-42)   -- op-name sets
* ``Tensor``        (backend.py:45-435)  -- operator overloads return op-trees
* ``OpTreeNode``    (backend.py:1682-2073) -- tuple ``(op_dict, left, right)``,
  shape inference in ``build``, execute-on-assign, post-order ``traverse``
* ``Backend`` builder functions (backend.py:711-1537) -- ``add`` ... ``onehot``,
  ``sum/max/min(axis=None)`` as axis-0-then-axis-1 nesting, ``mean/var/std``
  composed from ``sum``.

Nothing in here touches a device; the same trees are executed by the CUDA
backend (``neon_b200.backend``) and by the numpy checker used in the tests.
"""

import numpy as np


class OpCollection(object):
    """Names of the operations an op-tree may hold (backend.py:30-42), plus ``round``
    (C's roundf, halves away from zero): the rounding neon's GPU ``shift`` kernel applies
    to log2|b| (backends/kernels/cuda/binary.py:184), used by ``B200Backend.shift``."""
    zero_operand_ops = {"rand", "onehot"}
    unary_ops = {"finite", "neg", "abs", "sgn", "sqrt", "sqr", "exp", "log",
                 "exp2", "log2", "sig", "sig2", "tanh", "tanh2", "transpose",
                 "safelog", "rint", "binarize", "round"}
    binary_ops = {"assign", "add", "sub", "mul", "div", "eq", "ne", "lt", "le",
                  "gt", "ge", "pow", "minimum", "maximum", "dot", "shift"}
    reduction_ops = {"sum", "max", "min", "argmax", "argmin"}
    float_ops = zero_operand_ops | unary_ops | binary_ops
    ew_ops = float_ops - {"dot", "transpose"}


_EW_NOT_ASSIGN = frozenset(OpCollection.ew_ops - {"assign"})


def _binary(op, swap=False):
    if swap:
        def f(self, other):
            return OpTreeNode.build(op, other, self)
    else:
        def f(self, other):
            return OpTreeNode.build(op, self, other)
    f.__name__ = "__%s__" % op
    return f


def _unary(op):
    def f(self):
        return OpTreeNode.build(op, self, None)
    return f


class _Operators(object):
    """Python operators -> lazy op-tree nodes; shared by Tensor and OpTreeNode
    (backend.py:365-435 and backend.py:2015-2073)."""
    __add__ = _binary("add")
    __sub__ = _binary("sub")
    __mul__ = _binary("mul")
    __div__ = _binary("div")
    __truediv__ = _binary("div")
    __pow__ = _binary("pow")
    __radd__ = _binary("add", True)
    __rsub__ = _binary("sub", True)
    __rmul__ = _binary("mul", True)
    __rdiv__ = _binary("div", True)
    __rtruediv__ = _binary("div", True)
    __rpow__ = _binary("pow", True)
    __eq__ = _binary("eq")
    __ne__ = _binary("ne")
    __lt__ = _binary("lt")
    __le__ = _binary("le")
    __gt__ = _binary("gt")
    __ge__ = _binary("ge")
    __abs__ = _unary("abs")
    __neg__ = _unary("neg")


class Tensor(_Operators):
    """
    Base of every backend tensor.  Never fewer than two dimensions: a wrapped
    scalar is (1, 1) (backend.py:45-86).  Concrete tensors implement storage,
    views and host transfer; arithmetic on them only builds op-trees.
    """
    _min_dims = 2

    def __init__(self, backend, shape=None, dtype=np.float32, name=None,
                 persist_values=True):
        self.backend = backend
        self.shape = shape
        self.dtype = dtype
        self.name = name
        self.persist_values = persist_values
        self.base = None

    def __hash__(self):           # __eq__ builds a tree, so hash by identity
        return id(self)

    def _original_base(self):
        t = self
        while t.base is not None:
            t = t.base
        return t

    def __setitem__(self, index, value):
        self.__getitem__(index)._assign(value)

    # the rest is backend specific
    def __getitem__(self, index):
        raise NotImplementedError()

    def _assign(self, value):
        raise NotImplementedError()

    def set(self, ary):
        raise NotImplementedError()

    def get(self):
        raise NotImplementedError()

    def asnumpyarray(self):
        return self.get()

    def fill(self, value):
        return self._assign(value)

    def copy(self, a):
        return self._assign(a)

    def copy_from(self, a):
        return self.set(a)


_ONE, _NONE = (1, 1), (0, 0)


def _shape2(x):
    """2-d shape used for inference: tensors/nodes their own, numbers (1,1),
    None (0,0) (backend.py:1793-1812); False for anything that cannot be an operand."""
    t = type(x)
    if t is OpTreeNode:
        return x[0]["shape"]
    if t is float or t is int:
        return _ONE
    if x is None:
        return _NONE
    if isinstance(x, Tensor):
        s = x.shape
        return s if len(s) == 2 else (tuple(s) + (1,) if len(s) == 1 else tuple(s))
    if isinstance(x, (int, float)):
        return _ONE
    return False


class OpTreeNode(_Operators, tuple):
    """
    One node of a lazy expression: ``(op_dict, left, right)``.  ``op_dict``
    carries ``"op"``, the inferred ``"shape"`` and op arguments such as
    ``"axis"``.  Operands are nodes, tensors, python numbers or None
    (backend.py:1682-1691).
    """

    def __new__(cls, *args):
        return tuple.__new__(cls, args)

    def __hash__(self):
        return id(self)

    def __str__(self):
        def nm(x):
            if isinstance(x, Tensor):
                return x.name if x.name else "tensor-" + hex(id(x))
            return str(x)
        return "(%s, %s, %s)" % (self[0], nm(self[1]), nm(self[2]))

    __repr__ = __str__

    @staticmethod
    def build(op, a, b, out=None, **kwargs):
        """
        Make a node for ``op(a, b)``, inferring its 2-d shape; an ``assign``
        (or a non-None ``out``) executes the tree at once through the backend
        of the destination tensor (backend.py:1776-1850).
        """
        sa, sb = _shape2(a), _shape2(b)
        if sa is False or sb is False:
            return NotImplemented
        if op in _EW_NOT_ASSIGN:
            s0, s1 = sa[0], sa[1]
            if sb[0] > s0:
                s0 = sb[0]
            if sb[1] > s1:
                s1 = sb[1]
            shape = (s0, s1)
        elif op in OpCollection.reduction_ops:
            if "axis" in kwargs:
                shape = list(sa)
                shape[kwargs["axis"]] = 1
                shape = tuple(shape)
            else:
                shape = (1, 1)
        elif op == "assign":
            shape = tuple(sa)
        elif op == "dot":
            assert len(sa) == len(sb) == 2 and sa[1] == sb[0]
            shape = (sa[0], sb[1])
        elif op == "transpose":
            assert b is None
            shape = tuple(reversed(sa))
        else:
            raise TypeError("%s is not a valid operation" % op)

        info = {"op": op, "shape": shape}
        info.update(kwargs)
        node = OpTreeNode(info, a, b)
        if op == "assign":
            return node.execute()
        if out is not None:
            return OpTreeNode({"op": "assign"}, out, node).execute()
        return node

    def execute(self):
        """Run a tree whose root is ``assign`` on the destination's backend
        (backend.py:1852-1866)."""
        assert self[0]["op"] == "assign"
        backend = self[1].backend
        if not hasattr(backend, "execute"):
            raise NotImplementedError()
        return backend.execute(self)

    def traverse(self, stack):
        """Post-order walk appending operands then the op dict: the postfix
        program ``[out, leaves..., ops..., assign]`` (backend.py:1868-1890)."""
        for child in (self[1], self[2]):
            if isinstance(child, OpTreeNode):
                child.traverse(stack)
            elif child is not None:
                stack.append(child)
        stack.append(self[0])
        return stack

    @property
    def shape(self):
        return self[0]["shape"]

    @property
    def T(self):
        return OpTreeNode.build("transpose", self, None)

    def transpose(self, out=None):
        return OpTreeNode.build("transpose", self, None, out=out)

    def key(self):
        """Hashable identity of the tree: ops (+axis) and tensor objects
        (backend.py:1717-1734)."""
        items = []
        for s in self.traverse([]):
            if type(s) is dict:
                s = (s["op"], s["axis"]) if "axis" in s else s["op"]
            items.append(s)
        return tuple(items)

    def intrinsic_key_maps(self):
        """Structure key with tensors replaced by (first-seen index, shape),
        plus the two index<->tensor maps (backend.py:1736-1774)."""
        items, t2i, i2t = [], {}, {}
        for s in self.traverse([]):
            if type(s) is dict:
                s = (s["op"], s["axis"]) if "axis" in s else s["op"]
            elif isinstance(s, Tensor):
                if s not in t2i:
                    i2t[len(t2i)] = s
                    t2i[s] = len(t2i)
                s = (t2i[s], s.shape)
            items.append(s)
        return tuple(items), t2i, i2t

    def astensor(self):
        """Evaluate into a freshly allocated tensor (backend.py:1993-2013)."""
        be = None
        for s in self.traverse([]):
            if isinstance(s, Tensor):
                be = s.backend
                break
        if be is None:
            raise ValueError("No tensor object in op_tree")
        buf = be.empty(self.shape)
        buf[:] = self
        return buf

    def asnumpyarray(self):
        return self.astensor().get()


def _ew2(op):
    def f(self, a, b, out=None):
        return OpTreeNode.build(op, a, b, out=out)
    f.__name__ = op
    return f


def _ew1(op):
    def f(self, a, out=None):
        return OpTreeNode.build(op, a, None, out=out)
    f.__name__ = op
    return f


class OpTreeBackend(object):
    """
    The ``be.<op>`` builder functions of neon's ``Backend`` (backend.py:711-1537)
    plus its constructor state (backend.py:474-498).  Concrete backends add
    ``execute``, tensor factories and the RNG.
    """

    def __init__(self, rng_seed=None, default_dtype=np.float32,
                 compat_mode=None, deterministic=None):
        self.default_dtype = default_dtype
        self.rng_seed = rng_seed
        self.rng = self.gen_rng(rng_seed)
        self.bsz = None
        self._min_dims = 2
        if compat_mode is not None and compat_mode != "caffe":
            raise ValueError("%s mode not supported currently" % compat_mode)
        self.compat_mode = compat_mode
        self.deterministic = self.rng_seed is not None

    def gen_rng(self, seed=None):
        raise NotImplementedError()

    def execute(self, node):
        raise NotImplementedError()

    # ---- element-wise builders (backend.py:740-1294)
    add = _ew2("add")
    subtract = _ew2("sub")
    multiply = _ew2("mul")
    divide = _ew2("div")
    true_divide = _ew2("div")
    power = _ew2("pow")
    equal = _ew2("eq")
    not_equal = _ew2("ne")
    less = _ew2("lt")
    less_equal = _ew2("le")
    greater = _ew2("gt")
    greater_equal = _ew2("ge")
    maximum = _ew2("maximum")
    minimum = _ew2("minimum")
    negative = _ew1("neg")
    sgn = _ew1("sgn")
    absolute = _ew1("abs")
    fabs = _ew1("abs")
    sqrt = _ew1("sqrt")
    square = _ew1("sqr")
    exp = _ew1("exp")
    exp2 = _ew1("exp2")
    safelog = _ew1("safelog")
    log = _ew1("log")
    log2 = _ew1("log2")
    sig = _ew1("sig")
    sig2 = _ew1("sig2")
    tanh = _ew1("tanh")
    tanh2 = _ew1("tanh2")
    finite = _ew1("finite")
    rint = _ew1("rint")

    def reciprocal(self, a, out=None):
        return self.divide(1., a, out=out)

    def binarize(self, a, stochastic=True, out=None):
        return OpTreeNode.build("binarize", a, None, stochastic=stochastic, out=out)

    def shift(self, a, b, value=True, out=None):
        return OpTreeNode.build("shift", a, b, value=value, out=out)

    def clip(self, a, a_min, a_max, out=None):
        return self.minimum(self.maximum(a, a_min), a_max, out=out)

    def dot(self, a, b, out=None):
        return OpTreeNode.build("dot", a, b, out=out)

    # ---- reductions (backend.py:1313-1424): axis=None nests axis 0 then 1
    def _reduce(self, op, a, axis, out):
        if axis is None:
            inner = OpTreeNode.build(op, a, None, axis=0)
            return OpTreeNode.build(op, inner, None, axis=1, out=out)
        return OpTreeNode.build(op, a, None, axis=axis, out=out)

    def sum(self, a, axis=None, out=None, keepdims=True):
        return self._reduce("sum", a, axis, out)

    def max(self, a, axis=None, out=None, keepdims=True):
        return self._reduce("max", a, axis, out)

    def min(self, a, axis=None, out=None, keepdims=True):
        return self._reduce("min", a, axis, out)

    def argmax(self, a, axis=1, out=None, keepdims=True):
        return OpTreeNode.build("argmax", a, None, axis=axis, out=out)

    def argmin(self, a, axis=1, out=None, keepdims=True):
        return OpTreeNode.build("argmin", a, None, axis=axis, out=out)

    # ---- statistics composed from sum (backend.py:1426-1502)
    def mean(self, a, axis=None, partial=None, out=None, keepdims=True):
        shape = a.shape
        if axis is None:
            return self.multiply(self.sum(a), 1.0 / (shape[0] * shape[1]), out=out)
        return self.multiply(self.sum(a, axis=axis), 1.0 / shape[axis], out=out)

    def var(self, a, axis=None, partial=None, out=None, keepdims=True, binary=False):
        if binary:
            def op(x):
                return self.shift(x, x)
        else:
            op = self.square
        if axis is None:
            return self.mean(op(a - self.mean(a)), out=out)
        return self.mean(op(a - self.mean(a, axis=axis)), axis=axis, out=out)

    def std(self, a, axis=None, partial=None, out=None, keepdims=True):
        return self.sqrt(self.var(a, axis=axis, partial=partial, out=out))

    # ---- addressing ops (backend.py:1504-1537)
    def take(self, a, indices, axis, out=None):
        return a.take(indices, axis, out)

    def onehot(self, indices, axis, out=None):
        if axis not in (0, 1):
            raise ValueError("bad axis for onehot")
        assert indices.dtype in [np.dtype(np.int32), np.dtype(np.uint32)], \
            "onehot indices should be int32 or uint32, got " + str(indices.dtype)
        return OpTreeNode.build("onehot", None, None, idx=indices, axis=axis, out=out)

    # ---- layer helpers that are pure op-trees
    def iobuf(self, dim0, x=None, dtype=None, name=None, persist_values=True,
              shared=None, parallelism=None):
        """Zeroed (features, batch) buffer sized by ``self.bsz`` (backend.py:546-594)."""
        if x is not None:
            return x
        if isinstance(dim0, tuple):
            if len(dim0) == 2:
                bufshape = (dim0[0], dim0[1] * self.bsz)
            else:
                bufshape = (int(np.prod(dim0)), self.bsz)
        else:
            bufshape = (dim0, self.bsz)
        if shared is not None:
            t = shared if shared.shape == bufshape else shared.share(bufshape)
        else:
            t = self.empty(bufshape, dtype=dtype, name=name, persist_values=persist_values)
        t[:] = 0
        return t

    # ---- plumbing the layer classes call on every backend (backend.py:533-700);
    #      single-device backends answer with the neutral values
    def set_caffe_compat(self):
        self.compat_mode = "caffe"

    def check_caffe_compat(self):
        return self.compat_mode == "caffe"

    def shared_iobuf_size(self, shape, parallelism):
        num_dev = 1 if parallelism in ("Data", "Model") else getattr(self, "num_dev", 1)
        return num_dev * int(np.prod(shape))

    def distribute_data(self, tensor, layer_parallelism):
        return None

    def convert_data(self, tensor, layer_mkl):
        return None

    def clean_data(self, tensor, layer_mkl):
        return None

    def allocate_new_deltas(self, delta, in_shape, parallelism):
        return delta

    def allocate_new_outputs(self, layer, share_output):
        layer.allocate(shared_outputs=share_output)

    def is_mkl(self):
        return False

    def revert_tensor(self, tensor):
        pass

    def begin(self, block, identifier):
        pass

    def end(self, block, identifier):
        pass

    # ---- layer entry points that are op-trees on the GPU backend
    #      (nervanagpu.py:3179-3231)
    def relu_layer(self):
        return None

    def batchnorm_layer(self, in_shape):
        return None

    def mergesum_layer(self, layer_num):
        return None

    def mergebroadcast_layer(self, layer_num):
        return None

    def fprop_relu(self, layer, x, slope):
        return self.maximum(x, 0) + slope * self.minimum(0, x)

    def bprop_relu(self, layer, x, error, deltas, slope):
        return self.greater(x, 0) + slope * self.less(x, 0)

    def fprop_softmax(self, x, axis):
        return (self.reciprocal(self.sum(self.exp(x - self.max(x, axis=axis)), axis=axis)) *
                self.exp(x - self.max(x, axis=axis)))

    def fprop_transform(self, ngLayer, transform, inputs, outputs, relu=False):
        outputs[:] = transform(inputs)

    def bprop_transform(self, ngLayer, transform, outputs, error, deltas, relu):
        deltas[:] = transform.bprop(outputs) * error

    def fprop_skipnode(self, x, y, beta):
        y[:] = y * beta + x

    def bprop_skipnode(self, error, deltas, alpha, beta):
        deltas[:] = deltas * beta + alpha * error

    def fprop_mergesum(self, ngLayer, inputs, inference, layers, outputs, out_shape):
        for l in layers:
            l.fprop(inputs, inference, beta=0 if l is layers[0] else 1)

    def bprop_mergesum(self, ngLayer, alpha, beta, layers, error, deltas):
        for l in reversed(layers):
            l.bprop(error, alpha=alpha, beta=beta if l is layers[-1] else 1)

    def fprop_mergebroadcast(self, ngLayer, inputs, inference, outputs, layers, out_shape):
        for l in layers:
            l.fprop(inputs, inference)

    def bprop_mergebroadcast(self, ngLayer, layers, error_views, error, delta, out_shape,
                             alpha, beta, alphas, betas):
        betas[-1] = beta
        for l, e, a, b in reversed(list(zip(layers, error_views, alphas, betas))):
            l.bprop(e, alpha=a * alpha, beta=b)

    # ---- batch normalisation as the BatchNorm layer calls it (layers/layer.py:2483-2520).
    #      Semantics of the fused GPU kernels (cuda_batchnorm.py:27-219 and 222-431,
    #      nervanagpu.py:2463-2547), expressed as op-tree statements: xsum stays the
    #      batch *sum*, the variance is the centred second moment, xhat multiplies by
    #      the reciprocal root.
    def compound_fprop_bn(self, x, xsum, xvar, gmean, gvar, gamma, beta, y, eps, rho,
                          compute_batch_sum, accumbeta=0.0, relu=False, threads=None, repeat=1,
                          binary=False, inference=False, outputs=None, layer=None):
        if binary:
            raise NotImplementedError("binary (shift based) batch normalisation")
        if inference:
            xhat = (x - gmean) / self.sqrt(gvar + eps)
            y[:] = y * accumbeta + xhat * gamma + beta
            return
        if compute_batch_sum:
            xsum[:] = self.sum(x, axis=1)
        rcp_n = 1.0 / x.shape[1]
        xmean = xsum * rcp_n
        xvar[:] = self.sum(self.square(x - xmean), axis=1) * rcp_n
        gmean[:] = gmean * rho + (1.0 - rho) * xmean
        gvar[:] = gvar * rho + (1.0 - rho) * xvar
        val = (x - xmean) * self.reciprocal(self.sqrt(xvar + eps)) * gamma + beta
        if relu:
            val = self.maximum(val, 0)
        out = y.reshape(x.shape)
        if accumbeta != 0.0:
            val = out * accumbeta + val
        out[:] = val

    def compound_bprop_bn(self, delta_out, grad_gamma, grad_beta, delta_in, x, xsum, xvar,
                          gamma, eps, threads=None, repeat=1, binary=False, layer=None):
        if binary:
            raise NotImplementedError("binary (shift based) batch normalisation")
        rcp_n = 1.0 / x.shape[1]
        rstd = self.reciprocal(self.sqrt(xvar + eps))
        xhat = (x - xsum * rcp_n) * rstd
        grad_gamma[:] = self.sum(xhat * delta_in, axis=1)
        grad_beta[:] = self.sum(delta_in, axis=1)
        xtmp = (xhat * grad_gamma + grad_beta) * rcp_n
        delta_out.reshape(delta_in.shape)[:] = (delta_in - xtmp) * gamma * rstd

    def update_fc_bias(self, err, out):
        """out = sum(err, axis=1) (backend.py:1539-1547)."""
        self.sum(err, axis=1, out=out)

    def add_fc_bias(self, inputs, bias):
        """inputs += bias, bias broadcast along the batch (backend.py:1549-1557)."""
        self.add(inputs, bias, out=inputs)
