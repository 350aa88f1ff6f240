"""
Host lowering of one op-tree assignment into kernel passes.

Takes the postfix program an ``OpTreeNode`` flattens to
(``[out, operands..., op dicts..., {'op': 'assign'}]``) and produces a list of
``Pass`` objects: which skeleton of ``csrc/optree_templates.cuh`` runs, the
generated ``S<V>`` struct that plugs into it, the launch geometry and the
parameter block.  This is the job ``call_compound_kernel`` and
``_get_compound_kernel`` do in neon (neon/backends/float_ew.py:644-940 and
:268-617, with the stage split of :59-257); the semantics kept from there:

* one reduction axis per statement, 0 or 1 (:682-693); stride-0 broadcast of
  (n,1)/(1,n)/(1,1) operands (:751-763); operand de-duplication by tensor
  identity and constants by value (:735-749, :788-800); shape algebra and the
  ``TypeError``/``ValueError`` it raises (:810-825, :682-690, :724-726, :899-906);
* identical reduction sub-trees are evaluated once (:147-190);
* python numbers reach the kernel as fp32 run-time arguments, so changing a
  learning rate does not compile a new kernel (:788-800);
* rounding on store follows the output tensor's ``rounding`` attribute (:827-844).

What is different by design: a reduction level is a grid-wide pass (its result
is stored in fp32 scratch and re-read by later passes) instead of a loop inside
a single block per row, so every pass can use all SMs and coalesced loads
whichever axis is reduced; sub-trees made of constants only are folded on the
host in fp32.
"""

import struct

import numpy as np

from .optree import OpCollection, Tensor

DT_CODES = {"f4": 0, "f2": 1, "bf2": 2, "i4": 3, "u4": 4, "i2": 5, "u2": 6, "i1": 7, "u1": 8}
DT_NAMES = ["F32", "F16", "BF16", "I32", "U32", "I16", "U16", "I8", "U8"]
DT_SIZE = [4, 2, 2, 4, 4, 2, 2, 1, 1]
RED_CODE = {"sum": "OP_SUM", "max": "OP_MAX", "min": "OP_MIN", "argmax": "OP_ARGMAX", "argmin": "OP_ARGMIN"}

BLOCK = 256

# fp32 expressions of the element-wise vocabulary (neon/backends/cuda_templates.py:542-574)
UNARY_C = {
    "neg": "-{0}",
    "abs": "fabsf({0})",
    "sgn": "(({0} == 0.0f) ? 0.0f : copysignf(1.0f, {0}))",
    "sqrt": "sqrtf({0})",
    "sqr": "({0} * {0})",
    "exp": "expf({0})",
    "log": "logf({0})",
    "safelog": "(({0} > 0.0f) ? logf({0}) : -50.0f)",
    "exp2": "exp2f({0})",
    "log2": "log2f({0})",
    "sig": "(1.0f / (1.0f + expf(-{0})))",
    "sig2": "(1.0f / (1.0f + exp2f(-{0})))",
    "tanh": "tanhf({0})",
    "tanh2": "((exp2f(2.0f * {0}) - 1.0f) / (exp2f(2.0f * {0}) + 1.0f))",
    "finite": "(isfinite({0}) ? 1.0f : 0.0f)",
    "round": "roundf({0})",
}
BINARY_C = {
    "add": "({0} + {1})", "sub": "({0} - {1})", "mul": "({0} * {1})", "div": "({0} / {1})",
    "eq": "(({0} == {1}) ? 1.0f : 0.0f)", "ne": "(({0} != {1}) ? 1.0f : 0.0f)",
    "lt": "(({0} < {1}) ? 1.0f : 0.0f)", "le": "(({0} <= {1}) ? 1.0f : 0.0f)",
    "gt": "(({0} > {1}) ? 1.0f : 0.0f)", "ge": "(({0} >= {1}) ? 1.0f : 0.0f)",
    "minimum": "fminf({0}, {1})", "maximum": "fmaxf({0}, {1})", "pow": "powf({0}, {1})",
}
# cheaper versions (a few ulp, see csrc/optree_templates.cuh) used unless precise math is asked for
UNARY_FAST = dict(UNARY_C)
UNARY_FAST.update({
    "sqrt": "fast_sqrt({0})",
    "tanh": "fast_tanh({0})",
    "exp": "fast_exp({0})",
    "exp2": "ex2_approx({0})",
    "sig": "rcp_approx(1.0f + fast_exp(-{0}))",
    "sig2": "rcp_approx(1.0f + ex2_approx(-{0}))",
    "tanh2": "fast_div(ex2_approx(2.0f * {0}) - 1.0f, ex2_approx(2.0f * {0}) + 1.0f)",
})
BINARY_FAST = dict(BINARY_C)
BINARY_FAST.update({"div": "fast_div({0}, {1})"})
# the same ops on host fp32 scalars, for folding constant-only sub-trees
_f = np.float32
UNARY_HOST = {
    "neg": lambda a: -a, "abs": np.abs, "sgn": np.sign, "sqrt": np.sqrt, "sqr": lambda a: a * a,
    "exp": np.exp, "log": np.log, "safelog": lambda a: np.log(a) if a > 0 else _f(-50.0),
    "exp2": np.exp2, "log2": np.log2, "sig": lambda a: _f(1) / (_f(1) + np.exp(-a)),
    "sig2": lambda a: _f(1) / (_f(1) + np.exp2(-a)), "tanh": np.tanh,
    "tanh2": lambda a: (np.exp2(_f(2) * a) - _f(1)) / (np.exp2(_f(2) * a) + _f(1)),
    "finite": lambda a: _f(np.isfinite(a)),
    "round": lambda a: np.where(a >= 0, np.floor(a + _f(0.5)), np.ceil(a - _f(0.5))).astype(np.float32),
}
BINARY_HOST = {
    "add": lambda a, b: a + b, "sub": lambda a, b: a - b, "mul": lambda a, b: a * b,
    "div": lambda a, b: a / b, "eq": lambda a, b: _f(a == b), "ne": lambda a, b: _f(a != b),
    "lt": lambda a, b: _f(a < b), "le": lambda a, b: _f(a <= b), "gt": lambda a, b: _f(a > b),
    "ge": lambda a, b: _f(a >= b), "minimum": min, "maximum": max, "pow": np.power,
}


def dtype_code(dtype):
    dtype = np.dtype(dtype)
    key = "bf2" if dtype.name == "bfloat16" else dtype.str[1:]
    if key not in DT_CODES:
        raise TypeError("unsupported tensor dtype %s" % dtype)
    return DT_CODES[key]


# --------------------------------------------------------------------------- DAG
class Node(object):
    __slots__ = ("kind", "op", "args", "shape", "tix", "value", "axis", "level", "nid", "extra")

    def __init__(self, kind, op=None, args=(), shape=(1, 1), tix=None, value=None, axis=None, extra=None):
        self.kind = kind        # 't' tensor, 'c' const, 'u' unary, 'b' binary, 'r' reduction, 'z' zero-operand
        self.op = op
        self.args = args
        self.shape = shape
        self.tix = tix
        self.value = value
        self.axis = axis
        self.level = 0
        self.nid = -1
        self.extra = extra


class Operand(object):
    """A distinct tensor of the statement: pointer, dtype, 2-d shape, element strides."""
    __slots__ = ("tensor", "ptr", "dt", "shape", "strides", "alias_out", "span", "_frame_strides", "take")

    def __init__(self, tensor, shape, strides):
        self.tensor = tensor
        # fancy-indexed view: (address of the int32 index vector, tensor axis it replaces)
        self.take = (int(tensor.take_array[0].ptr), tensor.take_array[1]) if tensor.take_array else None
        self.ptr = int(tensor.ptr)
        self.dt = dtype_code(tensor.dtype)
        self.shape = tuple(shape)
        self.strides = tuple(int(s) for s in strides)
        lo = hi = 0
        for d, s in zip(self.shape, self.strides):
            if d > 1:
                if s >= 0:
                    hi += (d - 1) * s
                else:
                    lo += (d - 1) * s
        isz = DT_SIZE[self.dt]
        self.span = (self.ptr + lo * isz, self.ptr + (hi + 1) * isz)
        self.alias_out = False


class _Pseudo(object):
    """Operand-like view of a reduction result held in scratch."""
    __slots__ = ("ptr", "dt", "shape", "strides", "alias_out", "_frame_strides", "take")

    def __init__(self, ptr, dt, shape):
        self.ptr, self.dt, self.shape = ptr, dt, tuple(shape)
        self.take = None
        self.strides = (1, 1)           # a vector: the extent-1 axis is zeroed by the frame
        self.alias_out = True           # written by an earlier launch: plain loads


def shares_memory(a, b):
    """Conservative aliasing test: two tensors that live in the same allocation may
    overlap, so reads of one must not use the read-only data path while the other
    is written."""
    ba, bb = getattr(a, "_block", None), getattr(b, "_block", None)
    if ba is None or bb is None:
        return a._original_base() is b._original_base()
    return ba is bb


def eval_recipe(recipe, stack):
    """fp32 value of a folded constant (the caller silences numpy's floating-point warnings)."""
    kind = recipe[0]
    if kind == "l":
        return np.float32(float(stack[recipe[1]]))
    if kind == "k":
        return np.float32(recipe[1])
    if kind == "u":
        return np.float32(UNARY_HOST[recipe[1]](eval_recipe(recipe[2], stack)))
    return np.float32(BINARY_HOST[recipe[1]](eval_recipe(recipe[2], stack), eval_recipe(recipe[3], stack)))


def _recipe_reads_stack(recipe):
    """Does a folded constant depend on a python number of the program (which a later call with
    the same program_key may change)?"""
    kind = recipe[0]
    if kind == "l":
        return True
    if kind == "k":
        return False
    return any(_recipe_reads_stack(r) for r in recipe[2:])


def program_key(stack):
    """Hashable description of a postfix program with everything that shapes the
    generated kernels and their geometry -- dtypes, shapes, strides, pointer
    alignment, which operands are the same tensor or share the output's
    allocation, ops and axes -- and nothing that is a run-time argument
    (addresses, values of python numbers)."""
    out = stack[0]
    out_block = getattr(out, "_block", None)
    seen = {}
    key = []
    add = key.append
    for s in stack:
        t = type(s)
        if t is dict:
            idx = s.get("idx")
            add((s["op"], s.get("axis"), None if idx is None else seen.setdefault(id(idx), len(seen))))
        elif t is float or t is int:
            add(None)
        elif isinstance(s, Tensor):
            ix = seen.setdefault(id(s), len(seen))
            pk = getattr(s, "_plan_key", None)
            if pk is None:
                pk = (s.dtype.str, s.shape, s.strides, s.ptr & 15, s.take_array[1] if s.take_array else None)
            if s is out:
                alias = False
            elif out_block is not None and getattr(s, "_block", None) is not None:
                alias = s._block is out_block
            else:
                alias = shares_memory(s, out)
            add((ix, pk, alias))
        else:
            add(None)
    return tuple(key)


class BoundPlan(object):
    """Passes of a statement plus the recipe to re-aim them at new tensors and
    numbers of a program with the same ``program_key``."""

    def __init__(self, st, passes):
        self.passes = passes
        self.binds = []
        for pz in passes:
            ptrs, consts, takes = [], [], []
            for name in pz.fields.names():
                if name == "o":
                    ptrs.append((name, 0))
                elif name == "o_take":
                    takes.append((name, 0))
                elif name[0] == "t" and name.endswith("_take"):
                    takes.append((name, st.tensor_pos[int(name[1:-5])]))
                elif name[0] == "t" and name[1:].isdigit():
                    ptrs.append((name, st.tensor_pos[int(name[1:])]))
                elif name[0] == "c" and name[1:].isdigit():
                    recipe = st.nodes[int(name[1:])].extra
                    if _recipe_reads_stack(recipe):
                        consts.append((name, recipe))
                    # else: folded from literals of the expression's structure only; the planner
                    # has stored its value and it cannot change between calls
            self.binds.append((ptrs, consts, takes))

    def rebind(self, stack):
        for pz, (ptrs, consts, takes) in zip(self.passes, self.binds):
            vals = pz.fields.values
            for name, pos in takes:
                vals[name] = stack[pos].take_array[0].ptr
            for name, pos in ptrs:
                obj = stack[pos]
                vals[name] = (obj["idx"] if type(obj) is dict else obj).ptr
            if consts:
                # constants may overflow or divide by zero exactly as the kernel would
                with np.errstate(all="ignore"):
                    for name, recipe in consts:
                        vals[name] = float(eval_recipe(recipe, stack))


def _fast_flat_ok(t, out_shape):
    return len(t.shape) >= 1 and tuple(t.shape) == tuple(out_shape) and t.is_contiguous and not t.take_array


class Statement(object):
    """The DAG of one assignment plus everything ``plan`` needs to lower it."""

    def __init__(self, stack, allow_flat=True):
        self.nodes = []
        self._memo = {}
        self.operands = []          # Operand list (inputs)
        self._tensor_ix = {}
        out = stack[0]
        if not isinstance(out, Tensor):
            raise TypeError("first element of the program must be the output tensor")
        self.out_tensor = out

        # ---- pass 1 (float_ew.py:672-707): reduction axis and simple-elementwise test
        axis = None
        has_red = False
        flat_ok = True
        for s in stack:
            if type(s) is dict:
                op = s["op"]
                if op in OpCollection.reduction_ops:
                    if s.get("axis", None) not in (0, 1):
                        raise ValueError("Only reduction along an axis currently supported")
                    if has_red and s["axis"] != axis:
                        raise ValueError("Reduction only allowed along one axis per kernel.")
                    has_red, axis = True, s["axis"]
                elif op in ("onehot", "rand"):
                    flat_ok = False
            elif isinstance(s, Tensor):
                if not _fast_flat_ok(s, out.shape):
                    if not (tuple(s.shape) == (1, 1) and s is not out):
                        flat_ok = False
        self.axis = 1 if axis is None else axis
        self.has_red = has_red
        self.flat = flat_ok and not has_red and allow_flat
        if not self.flat:
            for s in stack:
                if isinstance(s, Tensor) and len(s.shape) != 2:
                    raise ValueError("Operations that are not simple elementwise are only "
                                     "currently supported in 2 dimensions.")
        if self.flat:
            self.out_shape = (1, int(out.size))
        else:
            self.out_shape = tuple(out.shape)

        # ---- pass 2: postfix -> DAG with shape algebra (float_ew.py:713-906)
        st = []
        first = True
        self.tensor_pos = []        # operand index -> position in the program of its first use
        for pos, s in enumerate(stack):
            if isinstance(s, Tensor):
                if first:
                    first = False
                    st.append("OUT")
                    continue
                known = len(self.operands)
                st.append(self._tensor_node(s))
                if len(self.operands) > known:
                    self.tensor_pos.extend([pos] * (len(self.operands) - known))
            elif type(s) in (int, float) or isinstance(s, (np.floating, np.integer)):
                st.append(self._const(float(s), ("l", pos)))
            elif type(s) is dict:
                op = s["op"]
                if op == "assign":
                    rhs = st.pop()
                    dst = st.pop()
                    if dst != "OUT" or st:
                        raise TypeError("malformed program: assign must close it")
                    self._check_assign(rhs)
                    self.root = rhs
                elif op in OpCollection.reduction_ops:
                    st.append(self._reduce(op, st.pop()))
                elif op in ("rand", "onehot"):
                    known = len(self.operands)
                    st.append(self._zero_op(s))
                    if len(self.operands) > known:          # the index tensor of a one-hot
                        self.tensor_pos.extend([pos] * (len(self.operands) - known))
                elif op in UNARY_C:
                    st.append(self._unary(op, st.pop()))
                elif op in BINARY_C:
                    b = st.pop()
                    a = st.pop()
                    st.append(self._binary(op, a, b))
                else:
                    raise TypeError("%s is not a valid operation" % op)
            else:
                raise TypeError("args must be instance of Tensor, int, float, or dict (for operators)")
        self.out = Operand(out, self.out_shape,
                           (0, 1) if self.flat else out.strides)
        for o in self.operands:
            o.alias_out = shares_memory(o.tensor, out)

    # -- node constructors (hash-consed)
    def _intern(self, key, make):
        n = self._memo.get(key)
        if n is None:
            n = make()
            n.nid = len(self.nodes)
            self.nodes.append(n)
            self._memo[key] = n
        return n

    def _tensor_node(self, t):
        ix = self._tensor_ix.get(id(t))
        if ix is None:
            if self.flat:
                shape = (1, 1) if tuple(t.shape) == (1, 1) and t.size == 1 and self.out_shape != (1, 1) \
                    else (1, int(t.size))
                strides = (0, 1)
            else:
                shape, strides = tuple(t.shape), tuple(t.strides)
            ix = self._tensor_ix[id(t)] = len(self.operands)
            self.operands.append(Operand(t, shape, strides))
        shape = self.operands[ix].shape
        return self._intern(("t", ix), lambda: Node("t", tix=ix, shape=shape))

    def _const(self, v, recipe):
        """Constant node.  ``recipe`` says how to recompute the value from the numbers
        of a later program of the same structure: ("l", position), ("k", value),
        ("u", op, recipe) or ("b", op, recipe, recipe)."""
        v = float(np.float32(v))
        return self._intern(("c", recipe), lambda: Node("c", value=v, extra=recipe))

    @staticmethod
    def _bshape(shapes):
        out = [1, 1]
        for s in shapes:
            for i in range(2):
                if s[i] != out[i]:
                    if s[i] == 1 or out[i] == 1:
                        out[i] = max(out[i], s[i])
                    else:
                        raise TypeError("Input shape:%s not compatible" % (tuple(s),))
        return tuple(out)

    def _unary(self, op, a):
        if a.kind == "c":
            with np.errstate(all="ignore"):
                return self._const(UNARY_HOST[op](np.float32(a.value)), ("u", op, a.extra))
        return self._intern(("u", op, a.nid),
                            lambda: self._lvl(Node("u", op=op, args=(a,), shape=a.shape)))

    def _binary(self, op, a, b):
        if a.kind == "c" and b.kind == "c":
            with np.errstate(all="ignore"):
                return self._const(BINARY_HOST[op](np.float32(a.value), np.float32(b.value)),
                                   ("b", op, a.extra, b.extra))
        shape = self._bshape((b.shape, a.shape))
        return self._intern(("b", op, a.nid, b.nid),
                            lambda: self._lvl(Node("b", op=op, args=(a, b), shape=shape)))

    def _reduce(self, op, a):
        ax = self.axis
        if a.shape[ax] == 1:
            # reducing an extent of one: the value itself, or index 0
            return self._const(0.0, ("k", 0.0)) if op.startswith("arg") else a
        extent = getattr(self, "_red_extent", None)
        if extent is None:
            self._red_extent = a.shape[ax]
        elif extent != a.shape[ax]:
            raise MixedExtents("reductions over %d and %d elements cannot share one kernel"
                               % (extent, a.shape[ax]))
        shape = list(a.shape)
        shape[ax] = 1
        shape = tuple(shape)

        def make():
            n = Node("r", op=op, args=(a,), shape=shape, axis=ax)
            n.level = a.level + 1
            return n
        return self._intern(("r", op, a.nid), make)

    def _zero_op(self, info):
        if info["op"] == "rand":
            # every rand() in a tree is its own stream
            k = ("z", "rand", len(self.nodes))
            return self._intern(k, lambda: Node("z", op="rand", shape=self.out_shape, extra=len(self.nodes)))
        idx = info["idx"]
        ix_node = self._tensor_node(idx)
        hot = info["axis"]
        n_hot = self.out_shape[hot]
        count = max(idx.shape)
        shape = [0, 0]
        shape[hot] = n_hot
        shape[1 - hot] = count
        return self._intern(("z", "onehot", ix_node.tix, hot),
                            lambda: Node("z", op="onehot", shape=tuple(shape), tix=ix_node.tix, axis=hot))

    @staticmethod
    def _lvl(n):
        n.level = max(a.level for a in n.args)
        return n

    def _check_assign(self, rhs):
        self._bshape((rhs.shape, self.out_shape))
        for i in range(2):
            if rhs.shape[i] != 1 and rhs.shape[i] != self.out_shape[i]:
                raise TypeError("Input shape:%s not compatible" % (tuple(rhs.shape),))


# --------------------------------------------------------------------------- code generation
class _Fields(object):
    """Parameter-block layout: 8-byte members first, then 4-byte ones."""

    def __init__(self):
        self.f8 = []
        self.f4 = []
        self.values = {}

    def u64(self, name, v):
        self._add(self.f8, ("u64", "Q", name), v)

    def i64(self, name, v):
        self._add(self.f8, ("i64", "q", name), v)

    def i32(self, name, v):
        self._add(self.f4, ("int", "i", name), v)

    def u32(self, name, v):
        self._add(self.f4, ("u32", "I", name), v)

    def f32(self, name, v):
        self._add(self.f4, ("float", "f", name), v)

    def _add(self, lst, decl, v):
        if decl[2] not in self.values:
            lst.append(decl)
        self.values[decl[2]] = v

    def decl(self):
        lines = ["    %s %s;" % (c, n) for c, _, n in self.f8 + self.f4]
        if len(self.f4) % 2:
            lines.append("    int pad_;")
        return "struct P {\n%s\n};" % "\n".join(lines)

    def names(self):
        return [n for _, _, n in self.f8 + self.f4]

    def fmt(self):
        f = "<" + "".join(c for _, c, _ in self.f8 + self.f4)
        if len(self.f4) % 2:
            f += "i"
        return f

    def pack(self, values=None):
        """The kernel's parameter block.  The layout is frozen at the first call."""
        packer = getattr(self, "_packer", None)
        if packer is None:
            self._names = self.names()
            self._pad = len(self.f4) % 2
            packer = self._packer = struct.Struct(self.fmt())
        values = self.values if values is None else values
        vals = [values[n] for n in self._names]
        if self._pad:
            vals.append(0)
        return packer.pack(*vals)


class Pass(object):
    """One kernel launch of a statement."""
    __slots__ = ("source", "name", "grid", "block", "fields", "kernel", "uses_rng", "desc",
                 "results", "kind", "smem", "cluster", "setup", "uses_xchg")

    def __init__(self):
        self.kernel = None
        self.uses_rng = False
        self.smem = 0          # dynamic shared memory per block
        self.cluster = 1       # thread blocks per cluster
        self.setup = None      # callable(runtime, kernel, pass) run once after compilation
        self.results = []      # (reduction op, fp32 result address, int32 index address or 0, count)
        self.uses_xchg = False    # the launcher supplies the exchange launch number in field "x_epoch"


class MixedExtents(ValueError):
    """Reductions over different numbers of elements in one statement: the backend evaluates
    them as separate statements."""


class XchgUnsupported(Exception):
    """The statement cannot finish its reductions through the exchange area (too many results,
    or a kernel shape without that path): the caller falls back to collectives between passes."""


def _red_code(r):
    """Reduction slot code of node r: its op, or one half of a moments pair."""
    if r.extra is not None:
        return "OP_MOM_MEAN" if r.extra[0] == "mean" else "OP_MOM_M2"
    return RED_CODE[r.op]


def _has_index(r):
    """The slot carries an int beside its value (arg index, or the count of a moments pair)."""
    return r.op.startswith("arg") or r.extra is not None


def _pair_order(rs):
    """Reductions of one pass with every moments pair in neighbouring slots (mean, then M2)."""
    out = []
    for r in rs:
        if r.extra is not None and r.extra[0] == "m2":
            continue
        out.append(r)
        if r.extra is not None:
            out.append(r.extra[1])
    return out


def _pow2ceil(x):
    p = 1
    while p < x:
        p *= 2
    return p


class Planner(object):
    """
    Lowers a Statement to passes.  ``scratch(nbytes, zero)`` must return a device
    address valid until the statement's launches have been issued; ``sm_count``
    sizes the grids.
    """

    def __init__(self, sm_count=148, target_blocks_per_sm=8, precise_math=False):
        self.sm_count = sm_count
        self.target = sm_count * target_blocks_per_sm
        self.unary = UNARY_C if precise_math else UNARY_FAST
        self.binary = BINARY_C if precise_math else BINARY_FAST
        # launch tuning (measured on B200, see profiles/): vectors per thread and
        # minimum resident blocks per SM of the element-wise skeleton
        self.red_resident = 5              # blocks of a reduction kernel resident per SM (48 registers)
        self.rowres = True                 # keep rows in cluster shared memory across passes when they fit
        self.smem_cap = 200 * 1024         # dynamic shared memory a row-resident block may ask for
        self.rowres_slice_cap = 100 * 1024 # preferred largest slice of a row per block (two blocks per SM)
        self.rowres_unroll = 2             # vectors per thread and chunk in the row-resident kernel
        self.rowres_threads = None         # cap on its block size (None: as many as the registers allow)
        self.rowres_exchange_resident_only = True   # exchange inside the row-resident kernel only for few rows per cluster (see _rowres_pass)
        self.status_ptr = 0                # device int the kernels set when a bounded wait gives up
        self.wait_limit_ns = 2000000000    # how long a block waits for its staged row slice
        self.debug_starve_bytes = 0        # tests only: announce this many bytes that never arrive
        self.ew_unroll = 4
        self.ew_min_blocks = None          # None: 5 for instruction-heavy statements, else 4
        self.fuse_moments = True           # sum(e) and sum(sqr(e - m)) in one pass when m needs sum-level results

    # ---- helpers on the frame: K = kept axis, N = loop axis
    def plan(self, st, scratch, rounding=0, fuse_final=True, lin=None, xchg=None, sharded=None):
        """Return the list of Pass objects for Statement ``st``.  ``fuse_final=False``
        keeps every reduction result in scratch (for a caller that combines results
        of several devices between passes); ``lin=(ncols, col0, local cols)`` makes
        element indices for random numbers those of a wider tensor this one is a
        column slice of; ``sharded`` names the operands (by index) that are column shards, and
        ``xchg`` (a dict: table, base, rank, world, cap, col0) makes every reduction that spans
        them finish across the GPUs inside its kernel.
        Raises XchgUnsupported when the statement cannot use the exchange area."""
        self._lin = lin
        self._xchg = xchg           # reductions finish across GPUs inside the kernel (see _reduction_pass)
        self._sharded = sharded     # indices of the operands that are column shards of wider tensors
        ra = st.axis                # reduced / loop axis in tensor coordinates
        ka = 1 - ra
        reds = [n for n in st.nodes if n.kind == "r" and self._reachable(st, n)]
        if self.fuse_moments and fuse_final:
            reds = self._pair_moments(st, reds, ka, ra)
        levels = sorted(set(n.level for n in reds))
        passes = []
        res_buf = {}                # reduction nid -> (addr_val, addr_idx or 0)
        full_shape = self._full_shape(st)
        root_is_k = st.root.shape[ra] == 1
        out_is_k = st.out_shape[ra] == 1
        if fuse_final and levels and self.rowres:
            pz = self._rowres_pass(st, reds, levels, ka, ra, full_shape, rounding, root_is_k and out_is_k)
            if pz is not None:
                return [pz]
        for lv in levels:
            rs = _pair_order([n for n in reds if n.level == lv])
            final = fuse_final and (lv == levels[-1]) and root_is_k and out_is_k and st.root.level == lv
            K = full_shape[ka]
            if not final:
                for r in rs:
                    res_buf[r.nid] = (scratch(4 * K, False),
                                      scratch(4 * K, False) if r.op.startswith("arg") else 0)
            pz = self._reduction_pass(st, rs, res_buf, ka, ra, full_shape, scratch, final)
            if not final:
                # for a caller that combines results of several devices between the passes: the
                # reductions that span the column shards (all of them when it did not say which
                # operands are shards)
                pz.results = [(r.op,) + res_buf[r.nid] + (K,) for r in rs
                              if self._sharded is None or self._spans_shards(st, r, self._sharded)]
            passes.append(pz)
            if final:
                return passes
        passes.append(self._ew_pass(st, res_buf, ka, ra, rounding))
        return passes

    # ---- moments pairs ---------------------------------------------------------------
    def _pair_moments(self, st, reds, ka, ra):
        """Find reductions of the form sum(sqr(e - m)) (or sqr(m - e)) where e varies along the
        reduced axis and m is a per-row value that needs results of the pass e itself could be
        reduced in -- the variance pattern, m = sum(e) * c.  Evaluated as written, such a sum
        waits for another full pass over e.  Instead the pass that can reduce e accumulates the
        first two moments of e (see "moments" in the kernel header), and sum(sqr(e - m)) is
        M2 + n * (mean - m)^2 for whatever m turns out to be -- exact for any m, so nothing
        here depends on the value of a constant.  The reduction moves one level down; levels
        of everything above it are recomputed.  Only with lanes along the reduced axis (the row
        kernels).  Returns the reductions to schedule (a sum(e) node is added if the tree has
        none: it is the pair's mean slot)."""
        self._frame(st, ka, ra)
        if self._lanes_on_k(st, ka, ra, self._full_shape(st)[ka]):
            return reds
        found = []
        taken = set()
        for r2 in reds:
            if r2.op != "sum" or r2.extra is not None:
                continue
            sq = r2.args[0]
            if sq.kind != "u" or sq.op != "sqr":
                continue
            d = sq.args[0]
            if d.kind != "b" or d.op != "sub":
                continue
            for e, m in ((d.args[0], d.args[1]), (d.args[1], d.args[0])):
                if (e.shape[ra] > 1 and m.shape[ra] == 1 and m.kind != "c" and m.level == e.level + 1
                        and e.nid not in taken and not self._contains_zero_op(e)):
                    found.append((r2, e, m))
                    taken.add(e.nid)
                    break
        if not found:
            return reds
        reds = list(reds)
        for r2, e, m in found:
            r1 = st._reduce("sum", e)
            if r1.extra is not None:
                continue
            r1.extra = ("mean", r2)
            r2.extra = ("m2", r1, m, e)
            if r1 not in reds:
                reds.append(r1)
        # levels again, bottom up (nodes are in creation order, arguments first); a pair's M2
        # now sits at the level of the plain reduction of e
        for n in st.nodes:
            if n.kind in ("u", "b"):
                n.level = max(a.level for a in n.args)
            elif n.kind == "r":
                if n.extra is not None and n.extra[0] == "m2":
                    n.level = n.extra[3].level + 1
                else:
                    n.level = n.args[0].level + 1
        return reds

    @staticmethod
    def _spans_shards(st, red, sharded):
        """True when reduction ``red`` reduces something computed from a column-sharded tensor
        (``sharded``: operand indices), directly or through an earlier such reduction."""
        todo, seen = [Planner._red_operand(red)], set()
        while todo:
            n = todo.pop()
            if n.nid in seen:
                continue
            seen.add(n.nid)
            if n.kind == "t" and n.tix in sharded:
                return True
            if n.kind == "z" and n.op == "onehot" and n.tix in sharded:
                return True
            todo.extend(n.args)
        return False

    @staticmethod
    def _contains_zero_op(node):
        todo, seen = [node], set()
        while todo:
            n = todo.pop()
            if n.nid in seen:
                continue
            seen.add(n.nid)
            if n.kind == "z":
                return True
            if n.kind != "r":
                todo.extend(n.args)
        return False

    @staticmethod
    def _lanes_on_k(st, ka, ra, K):
        """True when a reduction pass of this statement runs its lanes along the kept axis
        (the reduced axis is the strided one of its full-size operands)."""
        def lanes_ok(axis_name):
            for o in st.operands:
                sk, sn = o._frame_strides
                if o.shape[ka] > 1 and o.shape[ra] > 1 and (sn if axis_name == "n" else sk) != 1:
                    return False
            return True
        return (not lanes_ok("n")) and lanes_ok("k") and K > 1

    def _fixup_lines(self, ep, rs, fresh):
        """Code that turns the M2 of every moments pair among ``rs`` into the sum the statement
        asked for, sum((e - m)^2) = M2 + n (mean - m)^2, with m evaluated by emitter ``ep`` from
        the finished results r[] of this pass (and earlier ones).  Returns (lines, {nid: name}):
        the lines to run first and the name under which each corrected sum is available."""
        lines, names = [], {}
        for r in rs:
            if r.extra is None or r.extra[0] != "m2":
                continue
            r1, m = r.extra[1], r.extra[2]
            i1, i2 = fresh[r1.nid], fresh[r.nid]
            before = len(ep.h_lines)
            mref = ep.hoist(m)
            lines.extend(ep.h_lines[before:])
            del ep.h_lines[before:]
            name = "m2c%d" % r.nid
            cnt = "(float)ri[%d]" % i1                       # elements the pair has seen (all shards)
            lines.append("float %s; { const int i = 0; (void)i; const float dm = r[%d] / %s - %s; "
                         "%s = __fmaf_rn(dm * dm, %s, r[%d]); }" % (name, i1, cnt, mref, name, cnt, i2))
            names[r.nid] = name
        return lines, names

    # ---- row-resident statement: all passes in one cluster kernel -------------------
    def _rowres_pass(self, st, reds, levels, ka, ra, full_shape, rounding, red_out):
        """One kernel for a statement whose passes all walk the same rows along the
        contiguous axis, when a row of its full-size inputs fits in the shared memory
        of a cluster of at most 8 blocks.  Returns None when that does not apply."""
        K, N = full_shape[ka], full_shape[ra]
        if rounding or any(n.kind == "z" for n in st.nodes):
            return None
        # rows that continue on other GPUs: each pass's results are exchanged in rr_combine
        xchg = self._xchg
        crossing = dict((r.nid, bool(xchg) and self._spans_shards(st, r, self._sharded or ())) for r in reds)
        if not any(crossing.values()):
            xchg = None
        elif len(reds) * K > xchg["cap"]:
            return None
        if st.out.take is not None or any(o.take is not None for o in st.operands):
            return None
        n_passes = len(levels) + (0 if red_out else 1)
        if n_passes < 2:
            return None
        self._frame(st, ka, ra)
        tables = (self.unary, self.binary)
        f = _Fields()
        ems, lane_ops, staged = [], [], {}
        res_buf = {}
        for r in reds:
            res_buf[r.nid] = (0, 0)
        for lv in levels:
            em = self._Emit(st, f, ka, ra, False, res_buf, lv - 1, tables)
            em.no_nc = True
            rs = _pair_order([n for n in reds if n.level == lv])
            outs = [em.elem(self._red_operand(r)) for r in rs]
            ems.append((em, rs, outs))
            lane_ops += em.lane_ops
            staged.update(em.full_inputs)
        # finished results of each pass are corrected in registers before rr_combine publishes them
        fixups = []
        for em, rs, outs in ems:
            fx = self._Emit(st, f, ka, ra, False, res_buf, rs[0].level - 1, tables)
            fx.no_nc = True
            fresh = {r.nid: j for j, r in enumerate(rs)}
            for r in rs:
                if r.extra is None or r.extra[0] != "m2":
                    fx.names[("h", r.nid)] = "(float)ri[%d]" % fresh[r.nid] if r.op.startswith("arg") else "r[%d]" % fresh[r.nid]
            fix_lines, fixed = self._fixup_lines(fx, rs, fresh)
            fixups.append(fix_lines + ["r[%d] = %s;" % (fresh[nid], name) for nid, name in fixed.items()])
        fin = self._Emit(st, f, ka, ra, False, res_buf, 1 << 30, tables)
        fin.no_nc = True
        if red_out:
            last_rs = ems[-1][1]
            for i, r in enumerate(last_rs):
                fin.names[("h", r.nid)] = "(float)ri[%d]" % i if r.op.startswith("arg") else "r[%d]" % i
            if st.root.kind == "r" and st.root.op.startswith("arg"):
                store = "st_index<%s>(p.o, k * p.o_sk, ri[%d]);" % (DT_NAMES[st.out.dt], last_rs.index(st.root))
            else:
                store = "{ const int i = 0; (void)i; st_one<%s>(p.o, k * p.o_sk, %s); }" % (
                    DT_NAMES[st.out.dt], fin.hoist(st.root))
            extra_ops = []
        else:
            val = fin.elem(st.root)
            lane_ops += fin.lane_ops
            staged.update(fin.full_inputs)
            extra_ops = [(st.out, "n")]
        if not staged:
            return None
        for o in staged.values():
            if o._frame_strides[1] != 1:
                return None
        V = self._pick_v(lane_ops, N, True, extra=extra_ops)
        if V == 1 or N % V:
            return None
        # the staging copies are cp.async.bulk: source, destination and byte count must be
        # multiples of 16.  Slices and chunks start and end on V-element boundaries, so every
        # staged operand needs V elements to be a whole number of 16-byte units, a 16-byte
        # aligned base and a row pitch that keeps rows 16-byte aligned.
        for o in staged.values():
            isz = DT_SIZE[o.dt]
            if (V * isz) % 16 or o.ptr % 16 or (o._frame_strides[0] * isz) % 16 or (N * isz) % 16:
                return None
        nvec = N // V
        row_bytes = sum(DT_SIZE[o.dt] for o in staged.values())          # per element
        C = None
        for c in (1, 2, 4, 8):
            per = (nvec + c - 1) // c * V
            need = sum(((per * DT_SIZE[o.dt] + 127) & ~127) for o in staged.values())
            if need <= self.rowres_slice_cap:
                C = c
                break
        if C is None:                         # does not fit in small slices: one big block per SM
            for c in (1, 2, 4, 8):
                per = (nvec + c - 1) // c * V
                need = sum(((per * DT_SIZE[o.dt] + 127) & ~127) for o in staged.values())
                if need <= self.smem_cap:
                    C = c
                    break
        if C is None:
            return None
        while C < 8 and K * C < self.sm_count and (nvec + 2 * C - 1) // (2 * C) >= 512:
            C *= 2                            # few rows: more blocks per row to fill the machine
        per = (nvec + C - 1) // C * V
        need = sum(((per * DT_SIZE[o.dt] + 127) & ~127) for o in staged.values())
        seg_vecs = per // V
        if seg_vecs < 256 or K * C * 2 < self.sm_count:
            return None                       # rows too short or too few: the multi-pass kernels do better
        # 64 registers per thread: at most 1024 threads resident per SM, shared by the
        # blocks that fit next to each other in shared memory
        fit = (self.smem_cap + 24 * 1024) // max(need, 1)
        blocks_per_sm = 4 if fit >= 4 else (2 if fit >= 2 else 1)
        threads = 1024 // blocks_per_sm
        while threads > 256 and seg_vecs < 2 * threads:
            threads //= 2
        if xchg and self.rowres_exchange_resident_only and K * C > 2 * self.sm_count * blocks_per_sm:
            # rows that also wait for other GPUs: only while a cluster has at most two rows to do.
            # A cluster that loops over rows pays one cross-GPU round trip per row in sequence, and
            # a shard of 1/N of the tensor is read from L2 by a second launch anyway.  Measured,
            # batch norm of (256, 401408) fp16, eager: 2 GPUs (3.5 rows per cluster) 68 us against
            # 62 us for statistics kernel + element-wise kernel; 4 GPUs (1.7 rows) 42 against 52 us
            return None
        unroll = self.rowres_unroll
        if self.rowres_threads:
            threads = min(threads, int(self.rowres_threads))
        if (seg_vecs + threads * unroll - 1) // (threads * unroll) > 32:      # RR_MAX_CHUNKS mbarriers
            return None
        nrmax = max(len(rs) for _, rs, _ in ems)
        nres = len(reds)
        slot_of = {}
        for _, rs, _ in ems:                      # results of one pass sit next to each other
            for r in rs:
                slot_of[r.nid] = len(slot_of)

        f.u64("o", st.out.ptr)
        f.i64("o_sk", st.out._frame_strides[0])
        f.i64("o_sn", st.out._frame_strides[1])
        f.i64("K", K)
        f.i64("N", N)
        f.i64("nvec", nvec)
        f.u64("status", self.status_ptr)
        f.u64("wait_ns", int(self.wait_limit_ns))
        f.u32("starve", int(self.debug_starve_bytes))
        if xchg:
            f.u64("x_table", xchg["table"])
            f.u32("x_epoch", 0)
            f.u64("x_base", xchg["base"])
            f.u32("x_rank", xchg["rank"])
            f.u32("x_world", xchg["world"])
            f.u32("x_cap", xchg["cap"])
            f.i32("x_col0", xchg["col0"])
        offs, off = {}, 0
        for pre, o in sorted(staged.items()):
            offs[pre] = off
            f.u32("off_" + pre, off)
            off += (per * DT_SIZE[o.dt] + 127) & ~127
        dyn_bytes = off

        parts = ['#include "optree_templates.cuh"', "using namespace b200;", f.decl()]
        for i, (em, rs, outs) in enumerate(ems):
            ops = " : ".join("r == %d ? %s" % (j, _red_code(r)) for j, r in enumerate(rs[:-1]))
            ops = (ops + " : " if ops else "") + _red_code(rs[-1])
            tail = ["out[%d][i] = %s;" % (j, e) for j, e in enumerate(outs)]
            xc = " || ".join("r == %d" % j for j, r in enumerate(rs) if crossing[r.nid])
            parts.append(self._struct("S%d" % i, em, tail, len(rs), ops, None, None,
                                      acc_tail=self._accum_tail(em, rs, outs), fix_lines=fixups[i], xc=xc))
        if red_out:
            parts.append(self._struct("SF", fin, [], 0, "OP_SUM", fin.h_lines + [store], None, epilogue_only=True))
        else:
            st_lines = ["SrCtx c; c.shift = 0; c.mask = 0;",
                        "st_f<%s, V, false>(p.o, k * p.o_sk + n, v, c, nullptr);" % DT_NAMES[st.out.dt]]
            parts.append(self._struct("SE", fin, ["out[0][i] = %s;" % val], 0, "OP_SUM", None, st_lines))

        # the generated staging struct: announce and start the copies of chunk c of row k
        issue = ["const u32 e0 = c * cx.cv * %du;" % V,
                 "const u32 seg = (cx.v1 - cx.v0) * %du;" % V,
                 "const u32 ne = seg - e0 < cx.cv * %du ? seg - e0 : cx.cv * %du;" % (V, V),
                 "const i64 n0 = (i64)cx.v0 * %d + e0;" % V,
                 "asm volatile(\"fence.proxy.async.shared::cta;\" ::: \"memory\");",
                 "mbar_expect_tx(bars + c, ne * %du + (c == 0 ? p.starve : 0u));" % row_bytes]
        for pre, o in sorted(staged.items()):
            isz = DT_SIZE[o.dt]
            issue.append("rr_copy(dyn + p.off_%s + e0 * %du, p.%s + (u64)((k * p.%s_sk + n0) * %d), ne * %du, bars + c);"
                         % (pre, isz, pre, pre, isz, isz))
        parts.append("struct ST {\n    static DEV void issue(const P& p, const RowCtx& cx, i64 k, u32 c, "
                     "unsigned char* dyn, u64* bars) {\n        " + "\n        ".join(issue) + "\n    }\n};")

        body = []
        body.append("extern __shared__ __align__(128) unsigned char dyn[];")
        body.append("__shared__ u64 bars[2 * RR_MAX_CHUNKS];")
        body.append("__shared__ float sv[%d][%d]; __shared__ int si[%d][%d];" % (nrmax, threads // 32, nrmax, threads // 32))
        body.append("__shared__ u32 slots[%d][2][%d][%d][2]; __shared__ u32 s_res[%d];" % (len(ems), nrmax, C, nres))
        body.append("RowCtx cx; rr_begin<%d, %d, %d>(cx, p.nvec, bars);" % (C, threads, unroll))
        body.append("const i64 n0 = (i64)cx.v0 * %d;" % V)
        body.append("const i64 kfirst = %s, kstep = %s;" % (("cluster_index()", "cluster_count()") if C > 1
                                                            else ("blockIdx.x", "gridDim.x")))
        body.append("if (kfirst < p.K) rr_issue_row<ST>(p, cx, kfirst, dyn, bars);")
        body.append("P q = p;")
        for pre, o in sorted(staged.items()):
            body.append("q.%s = (u64)(dyn + p.off_%s) - (u64)(n0 * %d); q.%s_sk = 0;" % (pre, pre, DT_SIZE[o.dt], pre))
        for r in reds:
            if ("r%d" % r.nid) in f.values:
                body.append("q.r%d = (u64)&s_res[%d]; q.r%d_sk = 0; q.r%d_sn = 0;" % (r.nid, slot_of[r.nid], r.nid, r.nid))
        body.append("for (i64 k = kfirst; k < p.K; k += kstep) {")
        body.append("    const i64 knext = k + kstep;")
        body.append("    float a[%d]; int ai[%d];" % (nrmax, nrmax))
        dyn_cur, bars_cur = "dyn", "bars"
        for i, (em, rs, outs) in enumerate(ems):
            last = red_out and i == len(ems) - 1
            body.append("    rr_pass<S%d, ST, P, %d, %d, %d, %s, %s>(q, p, k, knext, cx, %s, %s, a, ai, sv, si);"
                        % (i, V, threads, unroll, "true" if i == 0 else "false", "true" if last else "false",
                           dyn_cur, bars_cur))
            body.append("    rr_combine<S%d, P, %d, %d, %d, %d>(q, k, cx, a, ai, sv, si, &slots[%d][0][0][0][0], &s_res[%d]);"
                        % (i, V, C, threads, slot_of[rs[0].nid], i, slot_of[rs[0].nid]))
        if red_out:
            body.append("    if (threadIdx.x == 0 && cx.rank == 0) SF<%d>::epilogue(q, k, a, ai);" % V)
        else:
            body.append("    rr_pass<SE, ST, P, %d, %d, %d, false, true>(q, p, k, knext, cx, %s, %s, a, ai, sv, si);"
                        % (V, threads, unroll, dyn_cur, bars_cur))
        body.append("    rr_row_end(cx);")
        body.append("}")
        if C > 1:
            body.append("cluster_barrier();      // nobody leaves while a peer may still read its exchange slots")
        text = "\n".join(parts) + "\n"
        import zlib
        name = "ot_rowres_kernel_%08x" % (zlib.crc32((text + "\n".join(body)).encode()) & 0xFFFFFFFF)
        text += ('extern "C" __global__ void __launch_bounds__(%d, %d) %s(const __grid_constant__ P p) {\n    grid_enter();\n    %s\n}\n'
                 % (threads, blocks_per_sm, name, "\n    ".join(body)))
        pz = Pass()
        pz.kind = "rowres"
        pz.name, pz.source, pz.fields = name, text, f
        pz.block = (threads, 1, 1)
        pz.smem, pz.cluster = dyn_bytes, C
        pz.uses_xchg = bool(xchg)
        clusters = max(1, min(K, (self.sm_count * blocks_per_sm) // C))
        pz.grid = (clusters * C, 1, 1)
        pz.desc = "rowres V=%d K=%d N=%d cluster=%d threads=%d smem=%d passes=%d grid=%s" % (
            V, K, N, C, threads, dyn_bytes, n_passes, pz.grid)

        def setup(rt, kernel, pz, K=K, C=C, threads=threads, dyn=dyn_bytes):
            """Opt in to the dynamic shared memory and size the grid to the clusters the
            device can hold at once (they loop over the rows)."""
            rt.kernel_max_smem(kernel, dyn)
            fit = rt.kernel_max_clusters(kernel, threads, dyn, C, pz.grid[0]) if C > 1 else \
                rt.kernel_occupancy(kernel, threads, dyn) * self.sm_count
            fit = max(1, min(K, fit))
            pz.grid = (fit * C, 1, 1)
        pz.setup = setup
        return pz

    @staticmethod
    def _red_operand(r):
        """The expression a reduction slot accumulates: a pair's M2 slot accumulates e itself."""
        return r.extra[3] if (r.extra is not None and r.extra[0] == "m2") else r.args[0]

    @staticmethod
    def _accum_tail(em, rs, outs):
        """(per-lane lines, per-vector lines) of S::accum for a pass whose reductions are all sums
        or moments pairs and where the accumulation can absorb an operand's conversion (a stored
        16-bit float summed as it is) or is a moments pair; None when the generic eval +
        reduction step should be used."""
        if any(r.op != "sum" for r in rs):
            return None
        pre, lines, post, fused = [], [], [], False
        for j, (r, e) in enumerate(zip(rs, outs)):
            if r.extra is not None and r.extra[0] == "m2":
                continue                                   # written with its mean slot
            half = em.half_leaf(Planner._red_operand(r))
            if r.extra is not None:                        # mean slot j, M2 slot j + 1
                # a vector's deviations are summed in two registers and added to lane 0 of the
                # accumulators: the pair costs two live accumulators, not 2 V
                fused = True
                kexpr = "__int_as_float(acci[%d][0])" % (j + 1)
                if half is not None:
                    first = "mx_add<%s, V>(%s, 0, 0.0f)" % (DT_NAMES[half[1]], half[0])
                    dexpr = "mx_sub<%s, V>(%s, i, %s)" % (DT_NAMES[half[1]], half[0], kexpr)
                else:
                    first, dexpr = e, "(%s - %s)" % (e, kexpr)
                pre.append("float s1v%d = 0.0f, s2v%d = 0.0f;" % (j, j))
                lines.append("if (i == 0 && acci[%d][0] == 0) acci[%d][0] = __float_as_int(%s);" % (j, j + 1, first))
                lines.append("{ const float d = %s; s1v%d += d; s2v%d = __fmaf_rn(d, d, s2v%d); }" % (dexpr, j, j, j))
                post.append("acc[%d][0] += s1v%d; acc[%d][0] += s2v%d; acci[%d][0] += V;" % (j, j, j + 1, j, j))
            elif half is not None:
                fused = True
                lines.append("acc[%d][i] = mx_add<%s, V>(%s, i, acc[%d][i]);" % (j, DT_NAMES[half[1]], half[0], j))
            else:
                lines.append("acc[%d][i] += %s;" % (j, e))
        return (pre, lines, post) if fused else None

    @staticmethod
    def _accum_fn(em, acc_tail, nred, ind):
        if acc_tail is None:
            return ["    enum { FUSED = 0 };"]
        pre, lines, post = acc_tail
        body = list(em.e_pre) + list(pre)
        body.append("_Pragma(\"unroll\") for (int i = 0; i < V; ++i) {")
        body.extend("    " + x for x in em.e_lines)
        body.extend("    " + x for x in lines)
        body.append("}")
        body.extend(post)
        return ["    enum { FUSED = 1 };",
                "    static DEV void accum(const P& p, const H& h, const L& l, i64 k, i64 n, float (&acc)[%d][V], "
                "int (&acci)[%d][V]) {" % (nred, nred)
                + ind + ind.join(body) + "\n    }"]

    @staticmethod
    def _struct(name, em, eval_tail, nred, ops, ep_lines, st_lines, epilogue_only=False, acc_tail=None,
                fix_lines=None, xc=None):
        ind = "\n        "
        nout = max(nred, 1)
        parts = ["template <int V> struct %s {" % name]
        parts.append("    enum { NRED = %d, XCHG = %d };" % (nred, 1 if xc else 0))
        parts.append("    static DEV constexpr int op(int r) { return %s; }" % ops)
        if xc:
            parts.append("    static DEV constexpr bool xc(int r) { return %s; }" % xc)
        if not epilogue_only:
            parts.append("    struct H { %s int unused_; };" % " ".join(em.h_decl))
            parts.append("    struct L { %s int unused_; };" % " ".join(em.l_decl))
            parts.append("    static DEV void load_h(const P& p, i64 k, H& h) {" + ind + ind.join(em.h_lines) + "\n    }")
            parts.append("    static DEV void load_l(const P& p, i64 k, i64 n, L& l) {" + ind + ind.join(em.l_lines) + "\n    }")
            body = list(em.e_pre)
            body.append("_Pragma(\"unroll\") for (int i = 0; i < V; ++i) {")
            body.extend("    " + x for x in em.e_lines)
            body.extend("    " + x for x in eval_tail)
            body.append("}")
            parts.append("    static DEV void eval(const P& p, const H& h, const L& l, i64 k, i64 n, float (&out)[%d][V]) {" % nout
                         + ind + ind.join(body) + "\n    }")
            parts.extend(Planner._accum_fn(em, acc_tail, nout, ind))
        else:
            parts.append("    enum { FUSED = 0 };")
        if st_lines is not None:
            parts.append("    static DEV void store(const P& p, i64 k, i64 n, const float* v) {" + ind + ind.join(st_lines) + "\n    }")
        if ep_lines is not None:
            parts.append("    static DEV void epilogue(const P& p, i64 k, const float* r, const int* ri) {"
                         + ind + ind.join(ep_lines) + "\n    }")
        if fix_lines is not None:
            parts.append("    static DEV void fixup(const P& p, i64 k, float* r, const int* ri) {"
                         + ind + ind.join(fix_lines) + "\n    }")
        parts.append("};")
        return "\n".join(parts)

    def _pick_split(self, units, max_split):
        """How many blocks share one reduction unit (a row, or a tile of columns).
        Blocks run in rounds of sm_count * resident; a round that is nearly empty
        costs as much as a full one, and past ~60% occupancy the memory system is
        saturated.  So: as few rounds as possible with the last one at least 60%
        full, and within that the split that leaves about 80% of the slots used
        (measured best for the whole-tensor and the 256-row cases)."""
        slots = self.sm_count * self.red_resident
        max_split = max(1, int(max_split))
        best = None
        for sp in range(1, min(max_split, 4 * slots) + 1):
            ctas = units * sp
            rounds = (ctas + slots - 1) // slots
            last = ctas - (rounds - 1) * slots
            if last < 0.6 * slots and not (rounds == 1 and sp == max_split):
                continue
            score = (rounds, abs(last / float(slots) - 0.8))
            if best is None or score < best[0]:
                best = (score, sp)
            if ctas > 2 * slots:
                break
        if best is None:
            # no split fills a round: take the largest one that stays within one round
            return max(1, min(max_split, slots // max(units, 1)))
        return best[1]

    # rough instruction counts per element of the fast-math expansions
    _OP_COST = {"tanh": 15, "tanh2": 16, "exp": 8, "exp2": 3, "log": 10, "log2": 8, "safelog": 12, "sig": 12,
                "sig2": 7, "pow": 30, "div": 3, "sqrt": 2, "sgn": 3, "finite": 2, "rand": 12}

    def _issue_bound(self, st, bytes_per_element, rounding):
        """True when the statement's arithmetic, not its memory traffic, limits an
        element-wise pass: more than ~3 instructions per byte moved."""
        seen, cost, todo = set(), 0, [st.root]
        while todo:
            n = todo.pop()
            if n.nid in seen:
                continue
            seen.add(n.nid)
            if n.kind in ("u", "b", "z"):
                cost += self._OP_COST.get(n.op, 1)
            elif n.kind == "t":
                cost += 1
            if n.kind != "r":
                todo.extend(n.args)
        if rounding:
            cost += 9
        return cost > 3.0 * max(bytes_per_element, 1)

    @staticmethod
    def _reachable(st, node):
        seen = set()
        stack = [st.root]
        while stack:
            n = stack.pop()
            if n.nid in seen:
                continue
            seen.add(n.nid)
            if n is node:
                return True
            stack.extend(n.args)
        return False

    @staticmethod
    def _full_shape(st):
        shp = list(st.out_shape)
        for n in st.nodes:
            for i in range(2):
                shp[i] = max(shp[i], n.shape[i])
        return tuple(shp)

    # ---- expression emission ------------------------------------------------
    class _Emit(object):
        """Collects code for one pass in a given orientation."""

        def __init__(self, st, fields, ka, ra, lanes_on_k, res_buf, avail_level, tables):
            self.unary, self.binary = tables
            self.fast = self.binary is BINARY_FAST
            self.st = st
            self.f = fields
            self.ka, self.ra = ka, ra
            self.lk = lanes_on_k
            self.res_buf = res_buf
            self.avail = avail_level          # reductions of level <= avail come from scratch
            self.h_lines, self.h_decl = [], []
            self.l_lines, self.l_decl = [], []
            self.e_pre, self.e_lines = [], []
            self.names = {}                    # nid -> (expr string in eval scope, is hoisted)
            self.hoisted = {}                  # nid -> name in H
            self.loop_ops = {}                 # tix -> array name in eval
            self.uses_rng = False
            self.lane_ops = []                 # (operand, lane axis) of every vector access
            self.pseudo = {}
            self.no_nc = False                 # True: operands may point at shared memory, plain loads only
            self.full_inputs = {}              # prefix -> operand, tensors that vary along both axes

        def var_k(self, n):
            return n.shape[self.ka] > 1

        def var_n(self, n):
            return n.shape[self.ra] > 1

        def _leaf(self, n):
            """Operand record and parameter-field prefix of a tensor node, or of a
            reduction result an earlier pass left in scratch (a length-K fp32/int32
            vector, seen as a tensor of the node's shape)."""
            if n.kind == "t":
                o, pre = self.st.operands[n.tix], "t%d" % n.tix
            else:
                assert n.level <= self.avail, "reduction not yet available"
                pre = "r%d" % n.nid
                o = self.pseudo.get(n.nid)
                if o is None:
                    av, ai = self.res_buf[n.nid]
                    o = _Pseudo(ai if n.op.startswith("arg") else av,
                                DT_CODES["i4"] if n.op.startswith("arg") else DT_CODES["f4"], n.shape)
                    self.pseudo[n.nid] = o
            sk, sn = o.strides[self.ka], o.strides[self.ra]
            if o.shape[self.ka] == 1:
                sk = 0
            if o.shape[self.ra] == 1:
                sn = 0
            o._frame_strides = (sk, sn)
            self.f.u64(pre, o.ptr)
            self.f.i64(pre + "_sk", sk)
            self.f.i64(pre + "_sn", sn)
            if o.take is not None:
                self.f.u64(pre + "_take", o.take[0])
                if o.take[1] == (self.ka if self.lk else self.ra):
                    # gather along the lanes: no vector access for this operand
                    o._frame_strides = (sk, sn) if False else ((0x7fffffff, sn) if self.lk else (sk, 0x7fffffff))
            return o, pre

        def _off(self, o, pre, vec):
            """Element offset of (k, n) in operand ``pre``; ``vec``: a V-wide access
            (unit stride along the lanes when V > 1)."""
            kk, nn = "k * p.%s_sk" % pre, "n * p.%s_sn" % pre
            if vec and self.lk:
                kk = "(V > 1 ? k : k * p.%s_sk)" % pre
            elif vec:
                nn = "(V > 1 ? n : n * p.%s_sn)" % pre
            if o.take is not None:
                if o.take[1] == self.ka:
                    kk = "(i64)ld_idx(p.%s_take, k) * p.%s_sk" % (pre, pre)
                else:
                    nn = "(i64)ld_idx(p.%s_take, n) * p.%s_sn" % (pre, pre)
            if self.st.flat:
                return "n"
            return "%s + %s" % (kk, nn)

        # value of node for use in hoisted (per-k) code; scope 'h'
        def hoist(self, n):
            """Emit per-kept-index code for K-only node n; returns its name in load_h scope."""
            key = ("h", n.nid)
            if key in self.names:
                return self.names[key]
            if n.kind == "c":
                self.f.f32("c%d" % n.nid, n.value)
                name = "p.c%d" % n.nid
                self.names[key] = name
                return name
            name = "k%d" % n.nid
            if n.kind in ("t", "r"):
                o, pre = self._leaf(n)
                nc = "false" if (o.alias_out or self.no_nc) else "true"
                if self.lk and self.var_k(n):
                    self.lane_ops.append((o, "k"))
                    koff = "(i64)ld_idx(p.%s_take, k) * p.%s_sk" % (pre, pre) \
                        if (o.take is not None and o.take[1] == self.ka) else "k * p.%s_sk" % pre
                    self.h_lines.append("float %s[V]; ld_f<%s, V, %s>(p.%s, %s, %s);"
                                        % (name, DT_NAMES[o.dt], nc, pre, koff, name))
                    ref = name + "[i]"
                else:
                    koff = "(i64)ld_idx(p.%s_take, k) * p.%s_sk" % (pre, pre) \
                        if (o.take is not None and o.take[1] == self.ka) else "k * p.%s_sk" % pre
                    self.h_lines.append("float %s[1]; ld_f<%s, 1, %s>(p.%s, %s, %s);"
                                        % (name, DT_NAMES[o.dt], nc, pre, koff, name))
                    ref = name + "[0]"
                self.names[key] = ref
                return ref
            # computed K-only node
            args = [self.hoist(a) for a in n.args]
            expr = (self.unary[n.op] if n.kind == "u" else self.binary[n.op]).format(*args)
            if self.lk:
                self.h_lines.append("float %s[V];\n        _Pragma(\"unroll\") for (int i = 0; i < V; ++i) %s[i] = %s;"
                                    % (name, name, expr))
                ref = name + "[i]"
            else:
                self.h_lines.append("float %s[1]; { const int i = 0; (void)i; %s[0] = %s; }" % (name, name, expr))
                ref = name + "[0]"
            self.names[key] = ref
            return ref

        def elem(self, n):
            """Emit per-element code for node n; returns the expression naming its value in eval scope."""
            key = ("e", n.nid)
            if key in self.names:
                return self.names[key]
            if n.kind == "c":
                self.f.f32("c%d" % n.nid, n.value)
                self.names[key] = "p.c%d" % n.nid
                return self.names[key]
            if n.kind == "z":
                return self._zero(n, key)
            if not self.var_n(n):
                # K-only: computed in load_h, carried in H
                ref = self.hoist(n)
                if ref.startswith("p.c"):
                    self.names[key] = ref
                    return ref
                hname = "h%d" % n.nid
                if n.nid not in self.hoisted:
                    self.hoisted[n.nid] = hname
                    if self.lk:
                        self.h_decl.append("float %s[V];" % hname)
                        self.h_lines.append("_Pragma(\"unroll\") for (int i = 0; i < V; ++i) h.%s[i] = %s;" % (hname, ref))
                    else:
                        self.h_decl.append("float %s;" % hname)
                        self.h_lines.append("{ const int i = 0; (void)i; h.%s = %s; }" % (hname, ref))
                self.names[key] = ("h.%s[i]" % hname) if self.lk else ("h.%s" % hname)
                return self.names[key]
            if n.kind in ("t", "r"):
                o, pre = self._leaf(n)
                nc = "false" if (o.alias_out or self.no_nc) else "true"
                lane_var = self.var_k(n) if self.lk else True     # var_n holds here
                if n.kind == "t" and self.var_k(n):
                    self.full_inputs[pre] = o
                aname = "a_" + pre
                if lane_var:
                    self.lane_ops.append((o, "k" if self.lk else "n"))
                    self.l_decl.append("u32 %s[(%d * V + 3) / 4];" % (aname, DT_SIZE[o.dt]))
                    off = self._off(o, pre, True)
                    self.l_lines.append("ld_w<%s, V, %s>(p.%s, %s, l.%s);" % (DT_NAMES[o.dt], nc, pre, off, aname))
                    self.e_pre.append("float %s[V]; cvt_in<%s, V>(l.%s, %s);" % (aname, DT_NAMES[o.dt], aname, aname))
                    ref = aname + "[i]"
                else:
                    self.l_decl.append("u32 %s[1];" % aname)
                    self.l_lines.append("ld_w<%s, 1, %s>(p.%s, %s, l.%s);"
                                        % (DT_NAMES[o.dt], nc, pre, self._off(o, pre, False), aname))
                    self.e_pre.append("float %s[1]; cvt_in<%s, 1>(l.%s, %s);" % (aname, DT_NAMES[o.dt], aname, aname))
                    ref = aname + "[0]"
                self.names[key] = ref
                return ref
            if (n.kind == "b" and n.op == "div" and self.fast and not self.var_n(n.args[1])
                    and n.args[1].kind != "c"):
                # dividing every element by a per-row value: multiply by its reciprocal, taken
                # once per thread in the hoisted code (fast-math mode; within 2 ulp of the quotient)
                den = n.args[1]
                ref = self.hoist(den)
                hname = "q%d" % den.nid
                if hname not in self.hoisted:
                    self.hoisted[hname] = hname
                    if self.lk:
                        self.h_decl.append("float %s[V];" % hname)
                        self.h_lines.append("_Pragma(\"unroll\") for (int i = 0; i < V; ++i) h.%s[i] = 1.0f / %s;" % (hname, ref))
                    else:
                        self.h_decl.append("float %s;" % hname)
                        self.h_lines.append("{ const int i = 0; (void)i; h.%s = 1.0f / %s; }" % (hname, ref))
                rcp = ("h.%s[i]" % hname) if self.lk else ("h.%s" % hname)
                expr = "(%s * %s)" % (self.elem(n.args[0]), rcp)
            elif n.kind == "b" and n.op in ("add", "sub") and self.mixed_operand(n) is not None:
                # one operand is a stored 16-bit float: the add converts it on the fly
                j = self.mixed_operand(n)
                raw, dt = self.half_leaf(n.args[j])
                other = self.elem(n.args[1 - j])
                if n.op == "add":
                    expr = "mx_add<%s, V>(%s, i, %s)" % (DT_NAMES[dt], raw, other)
                elif j == 0:
                    expr = "mx_sub<%s, V>(%s, i, %s)" % (DT_NAMES[dt], raw, other)
                else:                                   # c - a = -(a - c), exactly
                    expr = "(-mx_sub<%s, V>(%s, i, %s))" % (DT_NAMES[dt], raw, other)
            else:
                args = [self.elem(a) for a in n.args]
                expr = (self.unary[n.op] if n.kind == "u" else self.binary[n.op]).format(*args)
            name = "x%d" % n.nid
            self.e_lines.append("const float %s = %s;" % (name, expr))
            self.names[key] = name
            return name

        def half_leaf(self, n):
            """(words of the loaded vector, dtype code) when n is a 16-bit float tensor read one
            element per lane, else None."""
            if n.kind != "t" or not self.var_n(n) or (self.lk and not self.var_k(n)):
                return None
            o, pre = self._leaf(n)
            if o.dt not in (DT_CODES["f2"], DT_CODES["bf2"]):
                return None
            self.elem(n)                                # declares the load
            return "l.a_" + pre, o.dt

        def mixed_operand(self, n):
            """Index of the operand of add/sub node n that a mixed-precision instruction can take
            in its stored form, or None."""
            for j in (0, 1):
                if self.half_leaf(n.args[j]) is not None and n.args[1 - j].kind != "c":
                    return j
            for j in (0, 1):
                if self.half_leaf(n.args[j]) is not None:
                    return j
            return None

        def coords(self):
            """(row, col) expressions of lane i in eval scope."""
            kk = "(k + i)" if self.lk else "k"
            nn = "n" if self.lk else "(n + i)"
            return (kk, nn) if self.ka == 0 else (nn, kk)

        def lin_index(self):
            row, col = self.coords()
            self.f.i64("lin_r", 0)
            self.f.i64("lin_c", 0)
            self.f.i64("lin_0", 0)
            return "(u64)(p.lin_0 + %s * p.lin_r + %s * p.lin_c)" % (row, col)

        def _zero(self, n, key):
            name = "x%d" % n.nid
            if n.op == "rand":
                self.uses_rng = True
                self.f.u32("rk0", 0)
                self.f.u32("rk1", 0)
                self.f.u64("rk_tab", 0)
                fetch = "const Rng rkey = rng_key(p.rk0, p.rk1, p.rk_tab);"
                if fetch not in self.e_pre:
                    self.e_pre.append(fetch)
                sid = 1 + sum(1 for m in self.st.nodes[:n.nid] if m.kind == "z" and m.op == "rand")
                self.e_lines.append("const float %s = frand(Rng{rkey.k0 + %uu, rkey.k1}, %s);"
                                    % (name, (sid * 0x68E31DA4) & 0xFFFFFFFF, self.lin_index()))
            else:
                o, _ = self._leaf(self.st._memo[("t", n.tix)])
                row, col = self.coords()
                hot, other = (row, col) if n.axis == 0 else (col, row)
                # index tensor is a vector: address it by its longer dimension
                step = "p.t%d_sk" % n.tix if o.shape[self.ka] > 1 else "p.t%d_sn" % n.tix
                self.e_lines.append("const float %s = (ld_idx(p.t%d, (i64)%s * %s) == (int)%s) ? 1.0f : 0.0f;"
                                    % (name, n.tix, other, step, hot))
            self.names[key] = name
            return name

    # ---- vector width ---------------------------------------------------------
    @staticmethod
    def _pick_v(lane_ops, lane_extent, need_divisible, extra=()):
        ops = list(lane_ops) + list(extra)
        if not ops:
            return 1
        vmax = min(8, 16 // min(DT_SIZE[o.dt] for o, _ in ops))
        v = vmax
        while v > 1:
            ok = (lane_extent % v == 0) if need_divisible else (lane_extent >= v)
            for o, lane_axis in ops:
                isz = DT_SIZE[o.dt]
                align = min(16, v * isz)
                sk, sn = o._frame_strides
                lane_stride, other_stride = (sk, sn) if lane_axis == "k" else (sn, sk)
                if lane_stride != 1:
                    ok = False
                if o.ptr % align or (other_stride * isz) % align:
                    ok = False
            if ok:
                return v
            v //= 2
        return 1

    def _frame(self, st, ka, ra):
        for o in st.operands + [st.out]:
            sk, sn = o.strides[ka], o.strides[ra]
            if o.shape[ka] == 1:
                sk = 0
            if o.shape[ra] == 1:
                sn = 0
            if o.take is not None and o.take[1] == ra:
                sn = 0x7fffffff                 # gathered along the loop axis: never a vector access
            o._frame_strides = (sk, sn)

    # ---- passes -----------------------------------------------------------------
    def _reduction_pass(self, st, reds, res_buf, ka, ra, full_shape, scratch, final):
        K, N = full_shape[ka], full_shape[ra]
        self._frame(st, ka, ra)
        # orientation: lanes along N when the loop axis is the contiguous one
        lanes_on_k = self._lanes_on_k(st, ka, ra, K)
        xchg = self._xchg
        crossing = [bool(xchg) and self._spans_shards(st, r, self._sharded or ()) for r in reds]
        if not any(crossing):
            xchg = None
        elif lanes_on_k or len(reds) * K > xchg["cap"]:
            raise XchgUnsupported("reduction of %d x %d results does not fit the exchange area" % (len(reds), K))
        f = _Fields()
        em = self._Emit(st, f, ka, ra, lanes_on_k, res_buf, reds[0].level - 1, (self.unary, self.binary))
        outs = []
        for r in reds:
            outs.append(em.elem(self._red_operand(r)))
        eval_tail = ["out[%d][i] = %s;" % (i, e) for i, e in enumerate(outs)]
        acc_tail = self._accum_tail(em, reds, outs)

        # epilogue: raw results to scratch, or the root expression into the output
        ep = self._Emit(st, f, ka, ra, False, res_buf, reds[0].level - 1, (self.unary, self.binary))
        ep_lines = []
        fresh = {r.nid: i for i, r in enumerate(reds)}
        # results of this pass as the epilogue names them; a moments pair's second slot is first
        # turned into the sum the statement asked for
        for r in reds:
            if r.extra is None or r.extra[0] != "m2":
                ep.names[("h", r.nid)] = "(float)ri[%d]" % fresh[r.nid] if r.op.startswith("arg") else "r[%d]" % fresh[r.nid]
        fix_lines, fixed = self._fixup_lines(ep, reds, fresh)
        for nid, name in fixed.items():
            ep.names[("h", nid)] = name
        if final:
            odt = st.out.dt
            f.u64("o", st.out.ptr)
            f.i64("o_sk", st.out._frame_strides[0])
            ko = "k * p.o_sk"
            if st.out.take is not None and st.out.take[1] == ka:
                f.u64("o_take", st.out.take[0])
                ko = "(i64)ld_idx(p.o_take, k) * p.o_sk"
            if st.root.kind == "r" and st.root.op.startswith("arg"):
                val = None
                store = "st_index<%s>(p.o, %s, ri[%d]);" % (DT_NAMES[odt], ko, fresh[st.root.nid])
            else:
                val = ep.hoist(st.root)
                store = "{ const int i = 0; (void)i; st_one<%s>(p.o, %s, %s); }" % (DT_NAMES[odt], ko, val)
            ep_lines = fix_lines + ep.h_lines + [store]
        else:
            ep_lines = list(fix_lines)
            for r in reds:
                av, ai = res_buf[r.nid]
                i = fresh[r.nid]
                if r.nid in fixed:
                    f.u64("r%dv" % r.nid, av)
                    ep_lines.append("reinterpret_cast<float*>(p.r%dv)[k] = %s;" % (r.nid, fixed[r.nid]))
                elif r.op.startswith("arg"):
                    f.u64("r%dv" % r.nid, ai)
                    ep_lines.append("reinterpret_cast<int*>(p.r%dv)[k] = ri[%d];" % (r.nid, i))
                    # the extreme value itself, for callers that merge results of several devices
                    f.u64("r%dx" % r.nid, av)
                    ep_lines.append("reinterpret_cast<float*>(p.r%dx)[k] = r[%d];" % (r.nid, i))
                else:
                    f.u64("r%dv" % r.nid, av)
                    ep_lines.append("reinterpret_cast<float*>(p.r%dv)[k] = r[%d];" % (r.nid, i))

        # geometry
        pz = Pass()
        if lanes_on_k:
            V = self._pick_v(em.lane_ops, K, True)
            # narrow tiles (8 lanes x V = one 128-byte line of fp32/fp16 per row) keep the
            # number of tiles up and the number of slices per tile -- which the last
            # block of a tile has to combine -- down
            CW = min(8, _pow2ceil((K + V - 1) // V))
            RH = BLOCK // CW
            tiles = (K + CW * V - 1) // (CW * V)
            split = self._pick_split(tiles, (N + RH * 4 - 1) // (RH * 4))
            seg = (N + split - 1) // split
            split = (N + seg - 1) // seg
            grid = (tiles, split, 1)
            unroll = 4 if seg >= RH * 8 else 1
            call = "red_cols_kernel<S, P, %d, %d, %d, %d>(p);" % (V, BLOCK, CW, unroll)
            ncount = tiles
            pz.kind = "red_cols"
        else:
            V = self._pick_v(em.lane_ops, N, False)
            nvec = N // V
            if nvec >= 2 * BLOCK or (K * 8 <= self.target and nvec > 32):
                TPR = BLOCK
                split = self._pick_split(K, nvec // (BLOCK * 4))
                seg = (nvec + split - 1) // split
                split = max(1, (nvec + seg - 1) // seg)
                grid = (K * split, 1, 1)
                unroll = 4 if seg >= BLOCK * 8 else (2 if seg >= BLOCK * 2 else 1)
            else:
                TPR = max(1, min(32, _pow2ceil(max(nvec, 1))))
                split, seg = 1, nvec
                grid = ((K + (BLOCK // TPR) - 1) // (BLOCK // TPR), 1, 1)
                unroll = 1
            call = "red_rows_kernel<S, P, %d, %d, %d, %d>(p);" % (V, BLOCK, TPR, unroll)
            f.i64("nvec", nvec)
            ncount = K
            pz.kind = "red_rows"
        f.i64("K", K)
        f.i64("N", N)
        f.i64("seg", seg)
        f.i32("split", split)
        nr = len(reds)
        has_arg = any(_has_index(r) for r in reds)
        if split > 1:
            f.u64("part_v", scratch(4 * nr * K * split, False))
            f.u64("part_i", scratch(4 * nr * K * split, False) if has_arg else 0)
            f.u64("counters", scratch(4 * ncount, True))
        else:
            f.u64("part_v", 0)
            f.u64("part_i", 0)
            f.u64("counters", 0)
        ops = " : ".join("r == %d ? %s" % (i, _red_code(r)) for i, r in enumerate(reds[:-1]))
        ops = (ops + " : " if ops else "") + _red_code(reds[-1])
        xc = None
        if xchg:
            f.u64("x_table", xchg["table"])
            f.u64("status", self.status_ptr)
            f.u64("wait_ns", int(self.wait_limit_ns))
            f.u32("x_epoch", 0)
            f.u64("x_base", xchg["base"])
            f.u32("x_rank", xchg["rank"])
            f.u32("x_world", xchg["world"])
            f.u32("x_cap", xchg["cap"])
            f.i32("x_col0", xchg["col0"])
            xc = " || ".join("r == %d" % i for i, c in enumerate(crossing) if c)
        src, pz.name = self._source(f, em, eval_tail, nr, ops, ep_lines, None, call, acc_tail=acc_tail, xc=xc)
        pz.uses_xchg = bool(xchg)
        pz.source, pz.fields, pz.grid, pz.block = src, f, grid, (BLOCK, 1, 1)
        pz.uses_rng = em.uses_rng
        pz.desc = "%s V=%d K=%d N=%d split=%d grid=%s" % (pz.kind, V, K, N, split, grid)
        return pz

    def _ew_pass(self, st, res_buf, ka0, ra0, rounding):
        # an element-wise pass is free to pick its frame: prefer the one whose loop axis is contiguous
        best = None
        for ka, ra in ((0, 1), (1, 0)):
            self._frame(st, ka, ra)
            f = _Fields()
            em = self._Emit(st, f, ka, ra, False, res_buf, 1 << 30, (self.unary, self.binary))
            val = em.elem(st.root)
            K, N = st.out_shape[ka], st.out_shape[ra]
            V = self._pick_v(em.lane_ops, N, not st.flat, extra=[(st.out, "n")])
            cand = (V, ka, ra, f, em, val, K, N)
            if best is None or V > best[0]:
                best = cand
            if st.flat:
                break
        V, ka, ra, f, em, val, K, N = best
        self._frame(st, ka, ra)
        odt = st.out.dt
        f.u64("o", st.out.ptr)
        f.i64("o_sk", st.out._frame_strides[0])
        f.i64("o_sn", st.out.strides[ra] if st.out.shape[ra] > 1 else 0)
        f.i64("K", K)
        f.i64("N", N)
        nvec = N // V
        f.i64("nvec", nvec)
        sr = bool(rounding)
        st_lines = []
        o_off = "n" if st.flat else "k * p.o_sk + (V > 1 ? n : n * p.o_sn)"
        if st.out.take is not None:
            f.u64("o_take", st.out.take[0])
            if st.out.take[1] == ka:
                o_off = "(i64)ld_idx(p.o_take, k) * p.o_sk + (V > 1 ? n : n * p.o_sn)"
            else:
                o_off = "k * p.o_sk + (i64)ld_idx(p.o_take, n) * p.o_sn"
        if sr:
            em.uses_rng = True
            f.u32("rk0", 0)
            f.u32("rk1", 0)
            f.u64("rk_tab", 0)
            f.i32("sr_mb", int(rounding))
            em.lin_index()
            # element index of lane i = idx0 + i*step; row-major index of the output tensor
            ncols = 0 if st.flat else st.out_shape[1]
            if self._lin is not None:
                ncols = self._lin[0] if self._lin[1] % V == 0 else 1      # 1: never aligned
                if st.flat:
                    aligned_flat = ncols % V == 0 and self._lin[2] % V == 0
            step = "p.lin_c" if ra == 1 else "p.lin_r"
            row, col = ("k", "n") if ka == 0 else ("n", "k")
            pair = "true" if odt in (DT_CODES["f2"], DT_CODES["bf2"]) else "false"
            aligned = "true" if (ra == 1 and (st.flat or ncols % V == 0)) else "false"
            if st.flat and self._lin is not None:
                aligned = "true" if aligned_flat else "false"
            # the bit count is a literal (plans are cached per rounding setting), so shifts and
            # masks fold; at the full mantissa width of a 16-bit float the mask is dropped, the
            # truncating conversion that follows clears the same bits
            full = (odt == DT_CODES["f2"] and int(rounding) == 10) or (odt == DT_CODES["bf2"] and int(rounding) == 7)
            st_lines.append("SrCtx c = sr_ctx(%d);%s const Rng g = rng_key(p.rk0, p.rk1, p.rk_tab); u32 ur[V];"
                            % (int(rounding), " c.mask = 0xffffffffu;" if full else ""))
            if st.flat and self._lin is None:
                lin_expr = "(u64)n"                       # one row: the element index is n itself
            elif st.flat:
                # the skeleton passes the row's index shift as k.  While the enclosing tensor has
                # fewer than 2^32 elements the sum fits 32 bits, and the upper word of the random
                # counter is a literal zero the hash can fold, as in the unsharded kernel
                shard_cols = self._lin[2]
                enclosing = (st.out_shape[1] // max(shard_cols, 1)) * self._lin[0]
                lin_expr = "(u64)((u32)n + (u32)k)" if enclosing < (1 << 32) else "(u64)(n + k)"
            elif ra == 1:
                lin_expr = "(u64)(p.lin_0 + %s * p.lin_r + %s)" % (row, col)     # lin_c is 1
            else:
                lin_expr = "(u64)(p.lin_0 + %s * p.lin_r + %s * p.lin_c)" % (row, col)
            top13 = "true" if (odt == DT_CODES["f2"] and int(rounding) == 10) else "false"
            st_lines.append("rng_lanes<V, %s, %s, %s>(g, %s, %s, ur);" % (pair, aligned, top13, lin_expr, step))
            st_lines.append("st_f<%s, V, true>(p.o, %s, v, c, ur);" % (DT_NAMES[odt], o_off))
        else:
            st_lines.append("SrCtx c; c.shift = 0; c.mask = 0;")
            st_lines.append("st_f<%s, V, false>(p.o, %s, v, c, nullptr);" % (DT_NAMES[odt], o_off))
        total = nvec if st.flat else K * nvec
        big = self.ew_unroll
        unroll = big if total >= self.target * BLOCK * big else (2 if total >= self.target * BLOCK else 1)
        unroll = min(unroll, big)
        block = BLOCK
        if not st.flat and nvec >= BLOCK * unroll and K <= 65535 * 65535:
            # long rows: blocks tile each row (block y/z = row), no index division
            mode = 2
            grid = ((nvec + BLOCK * unroll - 1) // (BLOCK * unroll), min(K, 65535), (K + 65534) // 65535)
        else:
            mode = 1 if st.flat else 0
            if st.flat and self._lin is not None and "lin_0" in f.values:
                # flat view of a column shard whose kernel needs element coordinates (random
                # words): blocks must not straddle rows
                cl = self._lin[2]
                # whole blocks per row; short rows: half-size blocks keep the vectors per thread up
                fits = [(u, b) for b in (BLOCK, BLOCK // 2) for u in (4, 2, 1)
                        if u <= unroll and cl % (b * u * V) == 0]
                assert fits and N % V == 0
                unroll, block = max(fits, key=lambda ub: (ub[0], -ub[1]))
                mode = 3
                bpr = cl // (block * unroll * V)
                shard_rows = N // cl
                f.u32("flat_bpr", bpr)
                f.u32("flat_rows", shard_rows)
            if mode == 3:                       # one grid row per tensor row: no index division
                grid = (bpr, min(shard_rows, 65535), (shard_rows + 65534) // 65535)
            else:
                grid = (max(1, (total + BLOCK * unroll - 1) // (BLOCK * unroll)), 1, 1)
        widest = max([DT_SIZE[odt]] + [DT_SIZE[o.dt] for o, _ in em.lane_ops])
        idx32 = mode != 0 and (N + BLOCK * unroll * V) * widest < (1 << 32)
        call = "ew_kernel<S, P, %d, %d, %d, %d, %s>(p);" % (V, block, unroll, mode, "true" if idx32 else "false")
        min_blocks = self.ew_min_blocks
        if min_blocks is None:
            moved = DT_SIZE[odt] + sum(DT_SIZE[o.dt] for o, _ in em.lane_ops)
            min_blocks = 5 if self._issue_bound(st, moved, rounding) else 4
        min_blocks *= BLOCK // block
        src, name = self._source(f, em, ["out[0][i] = %s;" % val], 0, "OP_SUM", None, st_lines, call,
                                 min_blocks=min_blocks, block=block)
        pz = Pass()
        pz.name = name
        pz.kind = "ew_flat" if st.flat else "ew_2d"
        pz.source, pz.fields, pz.grid, pz.block = src, f, grid, (block, 1, 1)
        pz.uses_rng = em.uses_rng
        pz.desc = "%s V=%d K=%d N=%d grid=%s" % (pz.kind, V, K, N, grid)
        if "lin_r" in f.values:
            # linear element index = row * ncols + col of the output tensor
            f.values["lin_r"] = st.out_shape[1] if not st.flat else 0
            f.values["lin_c"] = 1
            if self._lin is not None:
                f.values["lin_r"], f.values["lin_0"] = self._lin[0], self._lin[1]
                if st.flat:            # flat index n -> n + c0 + row * (global - local row length)
                    f.values["lin_r"] = self._lin[0] - self._lin[2]
        return pz

    @staticmethod
    def _source(f, em, eval_tail, nred, ops, ep_lines, st_lines, call, min_blocks=1, acc_tail=None, xc=None,
                block=BLOCK):
        ind = "\n        "
        nout = max(nred, 1)
        parts = ['#include "optree_templates.cuh"', "using namespace b200;", f.decl(), "template <int V> struct S {"]
        parts.append("    enum { NRED = %d, XCHG = %d };" % (nred, 1 if xc else 0))
        parts.append("    static DEV constexpr int op(int r) { return %s; }" % ops)
        if xc:
            parts.append("    static DEV constexpr bool xc(int r) { return %s; }" % xc)
        parts.append("    struct H { %s int unused_; };" % " ".join(em.h_decl))
        parts.append("    struct L { %s int unused_; };" % " ".join(em.l_decl))
        parts.append("    static DEV void load_h(const P& p, i64 k, H& h) {" + ind + ind.join(em.h_lines) + "\n    }")
        parts.append("    static DEV void load_l(const P& p, i64 k, i64 n, L& l) {" + ind + ind.join(em.l_lines) + "\n    }")
        body = list(em.e_pre)
        body.append("_Pragma(\"unroll\") for (int i = 0; i < V; ++i) {")
        body.extend("    " + s for s in em.e_lines)
        body.extend("    " + s for s in eval_tail)
        body.append("}")
        parts.append("    static DEV void eval(const P& p, const H& h, const L& l, i64 k, i64 n, float (&out)[%d][V]) {" % nout
                     + ind + ind.join(body) + "\n    }")
        parts.extend(Planner._accum_fn(em, acc_tail, nout, ind))
        if st_lines is not None:
            parts.append("    static DEV void store(const P& p, i64 k, i64 n, const float* v) {" + ind + ind.join(st_lines) + "\n    }")
        if ep_lines is not None:
            parts.append("    static DEV void epilogue(const P& p, i64 k, const float* r, const int* ri) {"
                         + ind + ind.join(ep_lines) + "\n    }")
        parts.append("};")
        body = "\n".join(parts) + "\n"
        # kernel name = skeleton + digest of the instance, so profiles can tell instances apart
        import zlib
        name = "ot_%s_%08x" % (call.split("<")[0], zlib.crc32(body.encode()) & 0xFFFFFFFF)
        body += ('extern "C" __global__ void __launch_bounds__(%d, %d) %s(const __grid_constant__ P p) { grid_enter(); %s }\n'
                 % (block, min_blocks, name, call))
        return body, name
