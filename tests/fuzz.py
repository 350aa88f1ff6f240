"""
Seeded random op-tree statements for differential testing: the same statement is
built on two backends from the same description.  Shapes include odd sizes,
(n,1)/(1,n)/(1,1) broadcast operands, sliced and transposed views, fp16 and fp32
storage, reductions along either axis or over the whole tensor followed by more
element-wise work, and outputs that are views.  Values stay in (0.1, 1.1) so that
sums do not cancel and every function is well conditioned.
"""
import numpy as np

DIMS = (1, 3, 8, 17, 32, 64, 100, 257, 1024)

UNARY = ("neg", "abs", "sqr", "tanh", "sig", "exp", "sqrt", "log", "recip")
BINARY = ("add", "sub", "mul", "div", "maximum", "minimum")
REDUCE = ("sum", "max", "min", "mean")


class Spec(object):
    """Description of one statement, independent of any backend."""

    def __init__(self, seed):
        rng = np.random.RandomState(seed)
        self.seed = seed
        self.shape = (int(rng.choice(DIMS)), int(rng.choice(DIMS)))
        self.leaves = []                       # (kind, shape, dtype, view)
        self.tree = self._expr(rng, depth=int(rng.randint(1, 5)))
        self.red = None
        if rng.rand() < 0.6:
            self.red = (str(rng.choice(REDUCE)), [0, 1, None][int(rng.randint(0, 3))])
            self.post = self._post(rng) if rng.rand() < 0.5 else None
            if rng.rand() < 0.15:
                self.red = (str(rng.choice(("argmax", "argmin"))), int(rng.randint(0, 2)))
                self.post = None
        self.out_dtype = np.float16 if rng.rand() < 0.3 else np.float32
        self.out_view = rng.rand() < 0.25

    def _leaf(self, rng):
        r = rng.rand()
        R, C = self.shape
        if r < 0.15:
            return ("const", float(np.round(rng.uniform(0.25, 2.0), 3)))
        shape = (R, C) if r < 0.6 else ((R, 1) if r < 0.75 else ((1, C) if r < 0.9 else (1, 1)))
        dtype = np.float16 if rng.rand() < 0.3 else np.float32
        view = "none"
        if shape == (R, C):
            v = rng.rand()
            view = "slice" if v < 0.2 else ("trans" if v < 0.3 else "none")
        self.leaves.append((shape, dtype, view))
        return ("leaf", len(self.leaves) - 1)

    def _expr(self, rng, depth):
        if depth == 0:
            return self._leaf(rng)
        if rng.rand() < 0.35:
            return ("u", str(rng.choice(UNARY)), self._expr(rng, depth - 1))
        return ("b", str(rng.choice(BINARY)), self._expr(rng, depth - 1), self._expr(rng, int(rng.randint(0, depth))))

    def _post(self, rng):
        # element-wise work on the reduction result, possibly against a full-size leaf
        return (str(rng.choice(("add", "mul", "sub"))), self._leaf(rng), rng.rand() < 0.4)

    def out_shape(self):
        if self.red is None:
            return self.shape
        op, axis = self.red
        if axis is None:
            shape = (1, 1)
        else:
            shape = list(self.shape)
            shape[axis] = 1
            shape = tuple(shape)
        if self.post is not None and self.post[1][0] == "leaf":
            ls = self.leaves[self.post[1][1]][0]
            shape = (max(shape[0], ls[0]), max(shape[1], ls[1]))
        return shape


def host_arrays(spec):
    rng = np.random.RandomState(spec.seed + 7919)
    arrays = []
    for shape, dtype, view in spec.leaves:
        if view == "slice":
            base = rng.uniform(0.1, 1.1, (shape[0] + 3, shape[1] + 5))
        elif view == "trans":
            base = rng.uniform(0.1, 1.1, (shape[1], shape[0]))
        else:
            base = rng.uniform(0.1, 1.1, shape)
        arrays.append(base.astype(dtype))
    return arrays


def shardable(spec, world):
    """Statements a column-sharded backend can take as they are: no views, a column count the
    ranks can share evenly."""
    return (spec.shape[1] > 1 and spec.shape[1] % world == 0 and not spec.out_view
            and all(view == "none" for _, _, view in spec.leaves))


def build(be, spec, arrays, compute_dtype=None, full_kw=None):
    """Create the tensors on ``be`` and run the statement; returns the output tensor (full base).
    ``full_kw``: extra keywords for tensors that span all columns (e.g. parallel=True)."""
    full_kw = full_kw or {}
    leaves = []
    for (shape, dtype, view), a in zip(spec.leaves, arrays):
        dt = compute_dtype if compute_dtype is not None else dtype
        kw = full_kw if shape[1] == spec.shape[1] else {}
        t = be.array(a, dtype=dt, **kw)
        if view == "slice":
            t = t[2:2 + shape[0], 1:1 + shape[1]]
        elif view == "trans":
            t = t.T
        leaves.append(t)

    def ev(node):
        if node[0] == "const":
            return node[1]
        if node[0] == "leaf":
            return leaves[node[1]]
        if node[0] == "u":
            x = ev(node[2])
            op = node[1]
            if isinstance(x, float):
                x = leaves[0] * 0.0 + x if leaves else x
            if op == "neg":
                return -x
            if op == "abs":
                return be.absolute(x)
            if op == "sqr":
                return be.square(x)
            if op == "tanh":
                return be.tanh(x)
            if op == "sig":
                return be.sig(x)
            if op == "exp":
                return be.exp(be.minimum(x, 3.0))
            if op == "sqrt":
                return be.sqrt(be.absolute(x) + 0.1)
            if op == "log":
                return be.log(be.absolute(x) + 0.5)
            return be.reciprocal(be.absolute(x) + 0.5)
        a, b = ev(node[2]), ev(node[3])
        op = node[1]
        if isinstance(a, float) and isinstance(b, float):
            return a + b
        if op == "add":
            return a + b
        if op == "sub":
            return a - b
        if op == "mul":
            return a * b
        if op == "div":
            return a / (be.absolute(b) + 0.5)
        if op == "maximum":
            return be.maximum(a, b)
        return be.minimum(a, b)

    if not leaves:
        return None                      # a tree of constants only: nothing to compare
    tree = ev(spec.tree)
    if isinstance(tree, float):
        tree = leaves[0] * 0.0 + tree if leaves else None
    if tree is None:
        return None
    if spec.red is not None:
        op, axis = spec.red
        # keep magnitudes bounded before reducing
        tree = be.minimum(be.absolute(tree), 50.0) if not op.startswith("arg") else tree
        fn = getattr(be, op)
        tree = fn(tree, axis=axis)
        if spec.post is not None:
            pop, leaf, swap = spec.post
            other = ev(leaf)
            if pop == "add":
                tree = other + tree if swap else tree + other
            elif pop == "mul":
                tree = other * tree if swap else tree * other
            else:
                tree = other - tree if swap else tree - other
    oshape = tuple(tree.shape) if hasattr(tree, "shape") else spec.out_shape()
    odt = spec.out_dtype if compute_dtype is None else compute_dtype
    if spec.red is not None and spec.red[0].startswith("arg"):
        odt = np.int32
    if spec.out_view:
        base = be.zeros((oshape[0] + 2, oshape[1] + 4), dtype=odt)
        base[1:1 + oshape[0], 3:3 + oshape[1]] = tree
        return base
    out = be.zeros(oshape, dtype=odt, **(full_kw if oshape[1] == spec.shape[1] else {}))
    out[:] = tree
    return out
