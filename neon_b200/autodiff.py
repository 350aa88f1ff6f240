"""
Symbolic gradients of op-trees.

Same interface and results as neon's ``Autodiff`` (neon/backends/autodiff.py:
338-465): given a lazy expression ``f`` built from tensors of a backend, it
builds, again as lazy op-trees, the gradient of ``sum(f * next_error)`` with
respect to every tensor in it; assigning one of these trees to a tensor runs it
through the same fused kernels as any other statement.  neon's own class cannot
be used on this package's trees (it tests ``type(tree) == OpTreeNode`` against
neon's node class), which is why the algorithm is restated here:

  * reverse sweep over the tree, left operand first; a tensor that occurs more
    than once collects ``g = g + increment`` in the order of the sweep
    (autodiff.py:546-587);
  * one local rule per operation (autodiff.py:163-264), e.g. ``z = x / y`` gives
    ``(dz / y, -dz * x / y^2)``, ``max``/``min`` along an axis pass ``dz`` to the
    positions that equal the result;
  * after each rule the increment is folded back to the operand's shape
    (autodiff.py:75-118): broadcast operands get the sum over the broadcast
    axes, operands of a reduction get ``dz`` stretched with ``0 * x + dz``.

Tensors are identified by the allocation they view, as neon does with
``_original_base``, so a gradient asked for a view is the gradient collected
for its base; a transposed view contributes its gradient transposed.
"""

import collections

import numpy as np

from .optree import OpTreeNode, Tensor

_SCALARS = (int, float, np.float16, np.float32, np.float64, np.uint8, np.int8, np.uint16, np.int16,
            np.uint32, np.int32)


def _is_scalar(x):
    return isinstance(x, _SCALARS) and not isinstance(x, bool)


# ---------------------------------------------------------------- local rules
# rule(x, y, z, dz, op_dict, be) -> (increment for x, increment for y or None)
def _zero1(x, y, z, dz, op, be):
    return dz * 0., None


def _zero2(x, y, z, dz, op, be):
    return dz * 0., dz * 0.


def _sum_rule(x, y, z, dz, op, be):
    assert op.get("axis") in (0, 1)
    return dz, None                      # stretched to x's shape afterwards


RULES = {
    "eq": _zero2, "ne": _zero2, "lt": _zero2, "le": _zero2, "gt": _zero2, "ge": _zero2,
    "sgn": _zero1, "finite": _zero1, "argmax": _zero1, "argmin": _zero1, "rint": _zero1,
    "add": lambda x, y, z, dz, op, be: (dz, dz),
    "sub": lambda x, y, z, dz, op, be: (dz, -dz),
    "mul": lambda x, y, z, dz, op, be: (dz * y, dz * x),
    "div": lambda x, y, z, dz, op, be: (dz / y, -dz * x / be.square(y)),
    "pow": lambda x, y, z, dz, op, be: (dz * y * x ** (y - 1.), dz * z * be.log(x)),
    "dot": lambda x, y, z, dz, op, be: (be.dot(dz, y.T), be.dot(x.T, dz)),
    "neg": lambda x, y, z, dz, op, be: (-dz, None),
    "abs": lambda x, y, z, dz, op, be: (dz * be.sgn(x), None),
    "sqrt": lambda x, y, z, dz, op, be: (dz * 0.5 / z, None),
    "sqr": lambda x, y, z, dz, op, be: (dz * 2. * x, None),
    "exp": lambda x, y, z, dz, op, be: (dz * z, None),
    "exp2": lambda x, y, z, dz, op, be: (dz * z * be.log(2.), None),
    "log": lambda x, y, z, dz, op, be: (dz / x, None),
    "safelog": lambda x, y, z, dz, op, be: (dz / x, None),
    "log2": lambda x, y, z, dz, op, be: (dz / x / be.log(2.), None),
    "sig": lambda x, y, z, dz, op, be: (dz * z * (1. - z), None),
    "sig2": lambda x, y, z, dz, op, be: (dz * z * (1. - z) * be.log(2.), None),
    "tanh": lambda x, y, z, dz, op, be: (dz * (1. - be.square(z)), None),
    "tanh2": lambda x, y, z, dz, op, be: (dz * (1. - be.square(z)) * be.log(2.), None),
    "max": lambda x, y, z, dz, op, be: (dz * (x == z), None),
    "min": lambda x, y, z, dz, op, be: (dz * (x == z), None),
    "maximum": lambda x, y, z, dz, op, be: (dz * be.greater_equal(x, y), dz * be.greater_equal(y, x)),
    "minimum": lambda x, y, z, dz, op, be: (dz * be.less_equal(x, y), dz * be.less_equal(y, x)),
    "sum": _sum_rule,
    "transpose": lambda x, y, z, dz, op, be: (dz.T, None),
}


def _fold(inc, x, be):
    """Increment ``inc`` (shape of the node's result) -> shape of operand ``x``."""
    if inc is None or x is None:
        return inc
    if _is_scalar(x):
        return 0.
    want, have = tuple(x.shape), tuple(inc.shape)
    if want == have:
        return inc
    if len(want) != 2 or len(have) != 2:
        raise NotImplementedError("gradients of tensors with more than two dimensions")
    if want == (1, 1):
        return be.sum(inc)                               # scalar tensor broadcast everywhere
    if want[0] == have[0] and want[1] == 1:
        return be.sum(inc, axis=1)                       # column broadcast along the rows
    if want[0] == 1 and want[1] == have[1]:
        return be.sum(inc, axis=0)                       # row broadcast down the columns
    if (have[0] == want[0] and have[1] == 1) or (have[0] == 1 and have[1] == want[1]):
        return 0 * x + inc                               # operand of a reduction: stretch dz
    raise NotImplementedError("cannot fold a gradient of shape %s to %s" % (have, want))


def _base(t):
    b = t._original_base
    return b() if callable(b) else b


def _to_base(dz, view, base):
    """Gradient with respect to ``view`` -> gradient kept for the allocation it views.  A view of
    the whole allocation keeps its own shape (layers differentiate with respect to a reshaped
    input and hand in a buffer of that shape, neon/layers/layer.py:2632-2651); a transposed view
    contributes its gradient transposed (neon adds the gradient of ``x.T`` to that of ``x`` without
    turning it, which only additive expressions survive); a view of part of the allocation is
    refused rather than given a gradient of the wrong extent."""
    if view is base:
        return dz
    if int(np.prod(view.shape)) != int(np.prod(base.shape)):
        raise NotImplementedError("gradient with respect to a slice of a tensor")
    turned = bool(getattr(view, "is_trans", False)) != bool(getattr(base, "is_trans", False))
    if not turned:
        return dz
    if tuple(view.shape) == tuple(base.shape)[::-1]:
        return dz if _is_scalar(dz) else dz.T
    raise NotImplementedError("gradient with respect to a reshaped transpose")


class Autodiff(object):
    """Gradients of ``op_tree`` with respect to the tensors in it, as op-trees.

    Arguments:
        op_tree: OpTreeNode, Tensor or python number to differentiate
        be: the backend its tensors belong to
        next_error: tensor or op-tree of ``op_tree``'s shape holding the incoming
            gradient (a layer's deltas); ones of that shape when omitted
    """

    def __init__(self, op_tree, be, next_error=None):
        assert _is_scalar(op_tree) or type(op_tree) is OpTreeNode or isinstance(op_tree, Tensor), \
            "op_tree type not supported"
        assert be is not None
        self.op_tree = op_tree
        self.be = be
        self.dtype = be.default_dtype
        if next_error is not None:
            assert next_error.shape == op_tree.shape, (
                "next_error.shape %s must be consistant with op_tree.shape %s"
                % (next_error.shape, op_tree.shape))
            self.next_error = next_error
        else:
            self.next_error = be.ones(op_tree.shape)
        self.map_tensor_grad_op_tree = {}      # allocation -> gradient op-tree
        self._sweep(op_tree, self.next_error)

    # ---- the reverse sweep
    def _sweep(self, node, dz):
        stack = [(node, dz)]
        while stack:
            node, dz = stack.pop()
            if isinstance(node, Tensor):
                key = _base(node)
                dz = _to_base(dz, node, key)
                have = self.map_tensor_grad_op_tree.get(key)
                self.map_tensor_grad_op_tree[key] = dz if have is None else have + dz
            elif type(node) is OpTreeNode:
                op, x, y = node[0], node[1], node[2]
                if op["op"] not in RULES:
                    raise NotImplementedError("no gradient rule for %s" % op["op"])
                dx, dy = RULES[op["op"]](x, y, node, dz, op, self.be)
                dx, dy = _fold(dx, x, self.be), _fold(dy, y, self.be)
                # left operand first: push the right one below it
                if dy is not None and y is not None:
                    stack.append((y, dy))
                if x is not None:
                    stack.append((x, dx))
            # python numbers take no gradient

    def cleanup(self):
        self.map_tensor_grad_op_tree = {}
        self.op_tree = self.next_error = self.be = self.dtype = None

    # ---- results
    def _zero_like(self, tensor):
        return tensor * 0.

    def get_grad_op_tree(self, tensors):
        """Gradient op-trees for ``tensors`` (zeros for a tensor the expression does not use)."""
        return [self.map_tensor_grad_op_tree.get(_base(t), self._zero_like(t)) for t in tensors]

    def get_grad_tensor(self, tensors):
        out = []
        for tree in self.get_grad_op_tree(tensors):
            val = self.be.empty(tree.shape)
            val[:] = tree
            out.append(val)
        return out

    def get_grad_asnumpyarray(self, tensors):
        return [v.get().astype(self.dtype) for v in self.get_grad_tensor(tensors)]

    def back_prop_grad(self, tensors, gradients):
        """Evaluate the gradients of ``tensors`` into the buffers ``gradients``.  A buffer may be
        ``next_error`` itself (a layer overwriting its deltas): it is written last, after every
        gradient that still reads it."""
        for buf in gradients:
            assert _base(buf) not in self.map_tensor_grad_op_tree, "a differentiated tensor used as gradient buffer"
        deferred = None
        for tensor, buf in zip(tensors, gradients):
            if buf is self.next_error:
                deferred = tensor
            else:
                buf[:] = self.map_tensor_grad_op_tree.get(_base(tensor), buf * 0.)
        if deferred is not None:
            self.next_error[:] = self.map_tensor_grad_op_tree.get(_base(deferred), self.next_error * 0.)


# Layers differentiate the same tree on every minibatch; building the gradient trees again
# each time would cost more than running them (neon memoises without bound on
# (op_tree.key(), be, next_error), autodiff.py:312-335; here the most recent 64 are kept).
_CACHE = collections.OrderedDict()
_CACHE_SIZE = 64


def autodiff(op_tree, be, next_error=None):
    """``Autodiff(op_tree, be, next_error)``, reusing the object built for the same tree, backend
    and error tensor (cached objects keep all three alive, so their identities stay unique)."""
    key = (op_tree.key() if type(op_tree) is OpTreeNode else id(op_tree), id(be), id(next_error))
    ad = _CACHE.get(key)
    if ad is None:
        ad = Autodiff(op_tree, be, next_error)
        _CACHE[key] = ad
        while len(_CACHE) > _CACHE_SIZE:
            _CACHE.popitem(last=False)
    else:
        _CACHE.move_to_end(key)
    return ad
