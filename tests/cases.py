"""
Backend-independent op-tree programs used by the parity tests, the golden
fixture generator and the smoke check.

Every case is a function ``run(be, t)`` written against the neon backend API
only (``be.<op>``, tensor operators, ``out[:] = tree``), so the very same code
runs on neon's NervanaCPU, on the numpy checker and on the CUDA backend -- the
pattern of neon's own tests (tests/utils.py:47-133, tests/conftest.py:244-320).

Inputs come from ``np.random.RandomState(seed)`` on the host.  Storage dtypes
are per tensor; for a CPU run float tensors are created in the requested
compute dtype instead (fp16 storage is upcast so numpy does not round every
intermediate to half precision -- tests/test_backend_tensor.py:89 does the same).
"""

import numpy as np


class Case(object):
    def __init__(self, name, inputs, outputs, run, tol=None, gpu_semantics=False, derived=None):
        self.name = name
        self.inputs = inputs      # callable(rng) -> {name: ndarray (storage dtype)}
        self.outputs = outputs    # {name: (shape, storage dtype)}
        self.run = run            # callable(be, t) -> None
        self.tol = tol or {}
        self.gpu_semantics = gpu_semantics   # True: result undefined on NervanaCPU
        # outputs that are functions of another (rounded) output of the same run:
        # {name: callable(results) -> (expected float64 array, magnitude for the tolerance)}
        self.derived = derived or {}

    def __repr__(self):
        return "Case(%s)" % self.name


def _is_float(dt):
    dt = np.dtype(dt)
    return dt.kind == "f" or dt.name == "bfloat16"


def run_case(be, case, compute_dtype=None, seed=0, rounding=None):
    """
    Run ``case`` on backend ``be``; returns {name: ndarray} for inputs that were
    updated in place and for all outputs.  ``compute_dtype`` (fp32/fp64) replaces
    every float storage dtype (CPU checker runs).
    """
    rng = np.random.RandomState(seed)
    arrays = case.inputs(rng)
    t = {}
    for k, a in arrays.items():
        dt = a.dtype
        if compute_dtype is not None and _is_float(dt):
            dt = compute_dtype
        t[k] = be.array(a, dtype=dt)
    for k, (shape, dt) in case.outputs.items():
        if compute_dtype is not None and _is_float(dt):
            dt = compute_dtype
        t[k] = be.zeros(shape, dtype=dt)
        if rounding and k in rounding:
            t[k].rounding = rounding[k]
    case.run(be, t)
    return {k: v.get() for k, v in t.items()}


def summarize(a, limit=1024):
    """Small fingerprint of an array for the golden files: whole array when it is
    small, else an evenly strided sample plus float64 sum and abs-sum."""
    a = np.asarray(a)
    flat = a.reshape(-1)
    if flat.size <= limit:
        return {"full": a}
    step = flat.size // limit
    f64 = flat.astype(np.float64)
    return {"sample": flat[::step].copy(), "step": np.int64(step),
            "sum": np.float64(f64.sum()), "abssum": np.float64(np.abs(f64).sum())}


# ----------------------------------------------------------------------------
# benchmark configurations (sizes are parameters; defaults = the quoted sizes)
# ----------------------------------------------------------------------------

def cfg1(rows=4096, cols=128):
    def inputs(rng):
        return {"a": rng.randn(rows, cols).astype(np.float32),
                "b": rng.randn(rows, cols).astype(np.float32),
                "c": rng.uniform(-0.5, 0.5, (rows, 1)).astype(np.float32)}

    def run(be, t):
        t["out"][:] = be.maximum(t["a"] * t["b"] + t["c"], 0)
        t["s"][:] = be.sum(t["out"], axis=0)
        t["m"][:] = be.argmax(t["out"], axis=0)

    return Case("cfg1_bias_relu_%dx%d" % (rows, cols), inputs,
                {"out": ((rows, cols), np.float32), "s": ((1, cols), np.float32),
                 "m": ((1, cols), np.int32)}, run)


def cfg2(rows=32000, cols=256):
    def inputs(rng):
        return {"x": (3.0 * rng.randn(rows, cols)).astype(np.float32)}

    def run(be, t):
        x = t["x"]
        mx = be.max(x, axis=0)
        e = be.exp(x - mx)
        t["y"][:] = e / be.sum(e, axis=0)
        t["idx"][:] = be.argmax(x, axis=0)

    return Case("cfg2_softmax_%dx%d" % (rows, cols), inputs,
                {"y": ((rows, cols), np.float32), "idx": ((1, cols), np.int32)}, run)


ADAM = dict(beta_1=0.9, beta_2=0.999, epsilon=1e-8, learning_rate=1e-3)


def adam_step(be, param, grad, m, v, t, beta_1=0.9, beta_2=0.999,
              epsilon=1e-8, learning_rate=1e-3, scale_factor=1.0, clip=None):
    """
    One parameter update as neon's Adam.optimize issues it
    (neon/optimizers/optimizer.py:898-930): three op-tree assignments, with the
    bias-corrected step size ``l`` itself a lazy scalar-only op-tree
    (``be.sqrt`` of a python float), exactly as the optimizer writes it.
    """
    l = learning_rate * be.sqrt(1 - beta_2 ** t) / (1 - beta_1 ** t)
    g = grad / be.bsz
    m[:] = m * beta_1 + (1. - beta_1) * g
    v[:] = v * beta_2 + (1. - beta_2) * g * g
    upd = (scale_factor * l * m) / (be.sqrt(v) + epsilon)
    if clip is not None:
        upd = be.clip(upd, -clip, clip)
    param[:] = param - upd


def cfg3(n=100000000, steps=100, shape=None):
    shape = shape or ((n // 1000, 1000) if n % 1000 == 0 else (n, 1))

    def inputs(rng):
        d = {"param": (0.02 * rng.randn(*shape)).astype(np.float32)}
        for s in range(steps):
            g = np.random.RandomState(1000 + s).randn(*shape) * 1e-3
            d["grad%d" % s] = g.astype(np.float16)
        return d

    def run(be, t):
        be.bsz = 1
        for s in range(steps):
            adam_step(be, t["param"], t["grad%d" % s], t["m"], t["v"], s + 1)

    return Case("cfg3_adam_%d_x%d" % (n, steps), inputs,
                {"m": (shape, np.float32), "v": (shape, np.float32)}, run)


def cfg4(chans=256, cols=56 * 56 * 128):
    def inputs(rng):
        return {"x": (1.0 + 2.0 * rng.randn(chans, cols)).astype(np.float16),
                "gamma": rng.uniform(0.5, 1.5, (chans, 1)).astype(np.float32),
                "beta": rng.uniform(0.5, 1.5, (chans, 1)).astype(np.float32)}

    def run(be, t):
        x = t["x"]
        mean = be.mean(x, axis=1)
        var = be.var(x, axis=1)
        t["y"][:] = (x - mean) / be.sqrt(var + 1e-5) * t["gamma"] + t["beta"]

    return Case("cfg4_batchnorm_%dx%d" % (chans, cols), inputs,
                {"y": ((chans, cols), np.float16)}, run)


def cfg5(rows=32768, cols=32768, rounding=False):
    def inputs(rng):
        return {"x": rng.uniform(-4, 4, (rows, cols)).astype(np.float16),
                "y": rng.uniform(-4, 4, (rows, cols)).astype(np.float16)}

    def run(be, t):
        x, y, z = t["x"], t["y"], t["z"]
        z[:] = be.tanh(x) * be.sqrt(be.absolute(y)) + 0.5 * x * y
        t["total"][:] = be.sum(z, axis=None)
        t["peak"][:] = be.max(be.absolute(z), axis=None)

    # total and peak are reductions of the *stored* fp16 z, and total cancels heavily:
    # they are checked against the float64 reduction of the z the same run produced,
    # relative to sum|z| (a 1-ulp difference in z between two backends moves total by
    # far more than 1e-5 of itself)
    def want_total(res):
        z64 = res["z"].astype(np.float64)
        return np.array([[z64.sum()]]), float(np.abs(z64).sum())

    def want_peak(res):
        return np.array([[np.abs(res["z"].astype(np.float64)).max()]]), None

    return Case("cfg5_chain_%dx%d" % (rows, cols), inputs,
                {"z": ((rows, cols), np.float16), "total": ((1, 1), np.float32),
                 "peak": ((1, 1), np.float32)}, run,
                derived={"total": want_total, "peak": want_peak})


# ----------------------------------------------------------------------------
# cases after neon's own backend tests
# ----------------------------------------------------------------------------

UNARY = {
    # name: (builder, input generator)  -- positive inputs where the op needs them
    "neg": (lambda be, a: -a, "rand"),
    "abs": (lambda be, a: be.absolute(a), "rand"),
    "sgn": (lambda be, a: be.sgn(a), "rand"),
    "sqrt": (lambda be, a: be.sqrt(a), "pos"),
    "sqr": (lambda be, a: be.square(a), "rand"),
    "exp": (lambda be, a: be.exp(a), "rand"),
    "log": (lambda be, a: be.log(a), "pos"),
    "safelog": (lambda be, a: be.safelog(a), "pos"),
    "exp2": (lambda be, a: be.exp2(a), "rand"),
    "log2": (lambda be, a: be.log2(a), "pos"),
    "sig": (lambda be, a: be.sig(a), "rand"),
    "sig2": (lambda be, a: be.sig2(a), "rand"),
    "tanh": (lambda be, a: be.tanh(a), "rand"),
    "tanh2": (lambda be, a: be.tanh2(a), "rand"),
    "reciprocal": (lambda be, a: be.reciprocal(a), "pos"),
}

BINARY = {
    "add": lambda be, a, b: a + b,
    "sub": lambda be, a, b: a - b,
    "mul": lambda be, a, b: a * b,
    "div": lambda be, a, b: a / b,
    "pow": lambda be, a, b: be.power(be.absolute(a) + 0.5, b),
    "minimum": lambda be, a, b: be.minimum(a, b),
    "maximum": lambda be, a, b: be.maximum(a, b),
    "eq": lambda be, a, b: be.equal(a, b),
    "ne": lambda be, a, b: be.not_equal(a, b),
    "lt": lambda be, a, b: a < b,
    "le": lambda be, a, b: a <= b,
    "gt": lambda be, a, b: a > b,
    "ge": lambda be, a, b: a >= b,
    "rsub_const": lambda be, a, b: 2.5 - a * b,
    "rdiv_const": lambda be, a, b: 1.5 / (be.absolute(a) + 1.0) + b,
    "clip": lambda be, a, b: be.clip(a + b, -0.5, 0.75),
}


def _gen(rng, kind, shape):
    if kind == "pos":
        return rng.uniform(0.05, 3.0, shape)
    return rng.uniform(-2.0, 2.0, shape)


def unary_case(op, shape=(64, 327), dtype=np.float32):
    build, kind = UNARY[op]

    def inputs(rng):
        return {"a": _gen(rng, kind, shape).astype(dtype)}

    def run(be, t):
        t["out"][:] = build(be, t["a"])

    return Case("unary_%s_%dx%d_%s" % (op, shape[0], shape[1], np.dtype(dtype).name),
                inputs, {"out": (shape, dtype)}, run)


def binary_case(op, shape_a=(64, 327), shape_b=None, dtype=np.float32):
    """Shapes follow tests/test_backend_tensor.py:233-315: full, (n,1) and (1,n) operands."""
    shape_b = shape_b or shape_a
    build = BINARY[op]
    oshape = (max(shape_a[0], shape_b[0]), max(shape_a[1], shape_b[1]))

    def inputs(rng):
        a = _gen(rng, "rand", shape_a)
        b = _gen(rng, "rand", shape_b)
        if op in ("eq", "ne", "le", "ge"):
            a = np.round(a * 2) / 2
            b = np.round(b * 2) / 2
        return {"a": a.astype(dtype), "b": b.astype(dtype)}

    def run(be, t):
        t["out"][:] = build(be, t["a"], t["b"])

    return Case("binary_%s_%s_%s_%s" % (op, "x".join(map(str, shape_a)),
                                        "x".join(map(str, shape_b)), np.dtype(dtype).name),
                inputs, {"out": (oshape, dtype)}, run)


REDUCE = {
    "sum": lambda be, x, ax: be.sum(x, axis=ax),
    "max": lambda be, x, ax: be.max(x, axis=ax),
    "min": lambda be, x, ax: be.min(x, axis=ax),
    "mean": lambda be, x, ax: be.mean(x, axis=ax),
    "var": lambda be, x, ax: be.var(x, axis=ax),
    "std": lambda be, x, ax: be.std(x, axis=ax),
    "argmax": lambda be, x, ax: be.argmax(x, axis=ax),
    "argmin": lambda be, x, ax: be.argmin(x, axis=ax),
    "sumsq": lambda be, x, ax: be.sum(be.square(x), axis=ax),
    "absmax": lambda be, x, ax: be.max(be.absolute(x), axis=ax),
}


def reduce_case(op, shape, axis, dtype=np.float32, ties=False):
    """After tests/test_backend_reduction.py:31-107 (axis 0/1) plus axis=None."""
    build = REDUCE[op]
    if axis is None:
        oshape = (1, 1)
    else:
        oshape = list(shape)
        oshape[axis] = 1
        oshape = tuple(oshape)
    odtype = np.int32 if op.startswith("arg") else np.float32

    def inputs(rng):
        x = rng.uniform(-1.0, 1.0, shape)
        if ties:
            x = np.round(x * 4) / 4          # many equal extrema: first index must win
        return {"x": x.astype(dtype)}

    def run(be, t):
        t["out"][:] = build(be, t["x"], axis)

    return Case("reduce_%s_%s_ax%s_%s%s" % (op, "x".join(map(str, shape)), axis,
                                            np.dtype(dtype).name, "_ties" if ties else ""),
                inputs, {"out": (oshape, odtype)}, run)


def compound_cases():
    """Multi-stage and mixed-axis trees (tests/test_backend_compound_optree.py:39-119,
    tests/test_activations.py:144-180, layers that compose broadcasts)."""
    cases = []

    def in1(shape, scale=1.0):
        return lambda rng: {"x": (scale * rng.uniform(-1, 1, shape)).astype(np.float32)}

    def softmax1(be, t):
        x = t["x"]
        t["out"][:] = be.reciprocal(be.sum(be.exp(x - be.max(x, axis=1)), axis=1)) * \
            be.exp(x - be.max(x, axis=1))
    cases.append(Case("softmax_axis1_50x128", in1((50, 128), 3.0),
                      {"out": ((50, 128), np.float32)}, softmax1))

    def softmax0(be, t):
        x = t["x"]
        t["out"][:] = be.exp(x - be.max(x, axis=0)) / be.sum(be.exp(x - be.max(x, axis=0)), axis=0)
    cases.append(Case("softmax_axis0_1000x64", in1((1000, 64), 3.0),
                      {"out": ((1000, 64), np.float32)}, softmax0))

    def stdvar(be, t):
        t["out"][:] = be.std(be.var(t["x"], axis=0), axis=1)
    cases.append(Case("std_of_var_mixed_axes_50x128", in1((50, 128)),
                      {"out": ((1, 1), np.float32)}, stdvar))

    def maxmin(be, t):
        x = t["x"]
        t["out"][:] = be.max(x, axis=1) - be.min(x, axis=1) + be.mean(x, axis=1) * 0.5
    cases.append(Case("max_minus_min_axis1_33x77", in1((33, 77)),
                      {"out": ((33, 1), np.float32)}, maxmin))

    def center(be, t):
        x = t["x"]
        t["out"][:] = (x - be.mean(x, axis=1)) / (be.std(x, axis=1) + 1e-3)
    cases.append(Case("standardize_rows_40x300", in1((40, 300)),
                      {"out": ((40, 300), np.float32)}, center))

    def bcast_red(be, t):
        x = t["x"]
        t["out"][:] = be.sum(x, axis=0)      # (1,n) result broadcast into a full tensor
    cases.append(Case("reduction_broadcast_into_full_20x48", in1((20, 48)),
                      {"out": ((20, 48), np.float32)}, bcast_red))

    def view_out(be, t):
        x = t["x"]
        t["out"][0, :] = be.mean(x, axis=0)
        t["out"][1, :] = be.max(x, axis=0)
        t["col"][:, 1] = be.sum(x, axis=1)
    cases.append(Case("reductions_into_row_and_column_views_50x128", in1((50, 128)),
                      {"out": ((4, 128), np.float32), "col": ((50, 3), np.float32)}, view_out))

    def inplace(be, t):
        x = t["x"]
        x[:] = x * 0.5 + 1.0
        x[:] = x - be.mean(x, axis=0)
        t["out"][:] = x
    cases.append(Case("inplace_updates_64x96", in1((64, 96)),
                      {"out": ((64, 96), np.float32)}, inplace))

    def sliced(be, t):
        x = t["x"]
        t["out"][:] = x[3:35, 5:69] * 2.0 + x[0:32, 0:64]
    cases.append(Case("sliced_operands_40x80", in1((40, 80)),
                      {"out": ((32, 64), np.float32)}, sliced))

    def transposed(be, t):
        x = t["x"]
        t["out"][:] = x.T * 3.0 - 1.0
    cases.append(Case("transposed_view_operand_24x56", in1((24, 56)),
                      {"out": ((56, 24), np.float32)}, transposed))

    def allred(be, t):
        x = t["x"]
        t["s"][:] = be.sum(x)
        t["mx"][:] = be.max(x)
        t["mn"][:] = be.min(x)
        t["mean"][:] = be.mean(x)
        t["var"][:] = be.var(x)
    cases.append(Case("full_reductions_257x129", in1((257, 129)),
                      {"s": ((1, 1), np.float32), "mx": ((1, 1), np.float32),
                       "mn": ((1, 1), np.float32), "mean": ((1, 1), np.float32),
                       "var": ((1, 1), np.float32)}, allred))

    def scalar_fill(be, t):
        t["out"][:] = 3.5
        t["out"][2:5, 1:7] = -1.25
        t["x"][:] = t["out"][0:6, 0:10]
    cases.append(Case("scalar_fills_and_copies", in1((6, 10)),
                      {"out": ((8, 12), np.float32)}, scalar_fill))

    def ce(be, t):
        y, tt = t["x"], t["t"]
        t["out"][:] = be.sum(-be.safelog(y) * tt, axis=0)
    cases.append(Case("cross_entropy_multi_10x64",
                      lambda rng: {"x": rng.uniform(0.01, 1, (10, 64)).astype(np.float32),
                                   "t": (rng.uniform(0, 1, (10, 64)) > 0.8).astype(np.float32)},
                      {"out": ((1, 64), np.float32)}, ce))
    return cases


def adam_small():
    return cfg3(n=6000, steps=3, shape=(60, 100))


def standard_cases():
    """The list the golden fixtures and the parity tests iterate over."""
    cases = [cfg1(), cfg2(2000, 96), adam_small(), cfg4(32, 4096), cfg5(128, 192)]
    for op in sorted(UNARY):
        cases.append(unary_case(op))
    cases.append(unary_case("tanh", (4, 3), np.float16))
    cases.append(unary_case("exp", (1, 1023), np.float16))
    for op in sorted(BINARY):
        cases.append(binary_case(op))
    for op in ("add", "mul", "sub", "div", "gt"):
        cases.append(binary_case(op, (64, 327), (64, 1)))
        cases.append(binary_case(op, (64, 327), (1, 327)))
        cases.append(binary_case(op, (64, 1), (1, 1023)))
    cases.append(binary_case("add", (4, 3), (4, 3), np.float16))
    cases.append(binary_case("mul", (64, 327), (64, 1), np.float16))
    for shape in ((2, 2), (10, 32), (50, 50), (50, 128), (33, 77), (1, 1), (1000, 513)):
        for axis in (0, 1, None):
            for op in ("sum", "max", "min", "mean"):
                cases.append(reduce_case(op, shape, axis))
        for axis in (0, 1):
            for op in ("var", "std", "argmax", "argmin", "sumsq", "absmax"):
                cases.append(reduce_case(op, shape, axis))
    cases.append(reduce_case("argmax", (300, 40), 0, ties=True))
    cases.append(reduce_case("argmin", (300, 40), 0, ties=True))
    cases.append(reduce_case("argmax", (40, 3000), 1, ties=True))
    cases.append(reduce_case("argmin", (40, 3000), 1, ties=True))
    cases.append(reduce_case("sum", (64, 4096), 1, np.float16))
    cases.append(reduce_case("sum", (4096, 64), 0, np.float16))
    cases.extend(compound_cases())
    return cases
