"""
Cases in which neon's OWN classes -- optimizers, layers, costs, activations, the
data iterator, and the backends' ``compound_fprop_bn`` / ``compound_bprop_bn``
entry points -- drive a backend object.  Each case is a function ``run(be)``
that sets ``NervanaObject.be = be``, builds the neon objects, feeds them seeded
inputs and returns the resulting arrays by name.

The same function runs on neon's NervanaCPU (float64 tensors: the reference
result) and on the b200 backend; ``tests/golden/make_golden.py`` stores the
NervanaCPU results in ``tests/golden/neon_callers_golden.npz`` so the comparison
can also be made against committed results.  Running a case always needs a neon
source tree, since the callers are neon's code.

neon sources followed: optimizers/optimizer.py:72-115, 416-991;
layers/layer.py:1376-1452 (Bias), 1455-1530 (Activation), 1968-2066 (Dropout),
2196-2262 (GeneralizedCost), 2352-2520 (BatchNorm); backends/nervanacpu.py:1688-1760;
tests/test_optimizer.py:43-66 (the dummy-layer harness).
"""

import numpy as np

BSZ = 64


class _ParamHolder(object):
    """What get_param_list expects of a layer (optimizers/optimizer.py:25-41)."""

    def __init__(self, plist):
        self.plist = plist

    def get_params(self):
        return self.plist


def _use(be, bsz=BSZ):
    from neon import NervanaObject
    NervanaObject.be = be
    be.bsz = bsz
    return be


def _fdt(be):
    """Floating dtype of host arrays handed to ``be`` (its default dtype)."""
    return np.dtype(be.default_dtype)


# --------------------------------------------------------------------------- optimizers
def _optimizer_case(make, steps=4, shapes=((96, 160), (50, 1)), grad_scale=1.0, epochs=None):
    def run(be):
        _use(be, bsz=4)
        rng = np.random.RandomState(11)
        opt = make()
        plist = []
        for shp in shapes:
            p = be.array((0.1 * rng.randn(*shp)).astype(_fdt(be)))
            g = be.empty(shp)
            plist.append(((p, g), []))
        holder = _ParamHolder(plist)
        for s in range(steps):
            for (p, g), _ in plist:
                g.set((grad_scale * rng.randn(*g.shape)).astype(_fdt(be)))
            opt.optimize([holder], epoch=(epochs[s] if epochs else s))
        out = {}
        for i, ((p, g), states) in enumerate(plist):
            out["param%d" % i] = p.get()
            for j, st in enumerate(states):
                out["param%d_state%d" % (i, j)] = st.get()
        return out
    return run


def _optimizers():
    from neon.optimizers import (Adadelta, Adagrad, Adam, ExpSchedule, GradientDescentMomentum, RMSProp,
                                 ShiftAdaMax, StepSchedule)
    return {
        "opt_gdm": lambda: GradientDescentMomentum(0.1, 0.9),
        "opt_gdm_plain_wdecay": lambda: GradientDescentMomentum(0.05, 0.0, wdecay=0.01),
        "opt_gdm_nesterov_wdecay_clip": lambda: GradientDescentMomentum(
            0.1, 0.9, wdecay=0.005, nesterov=True, gradient_clip_norm=2.0, gradient_clip_value=0.4,
            param_clip_value=0.25),
        "opt_gdm_step_schedule": lambda: GradientDescentMomentum(
            0.1, 0.8, schedule=StepSchedule([1, 3], [0.05, 0.01])),
        "opt_gdm_exp_schedule": lambda: GradientDescentMomentum(0.1, 0.8, schedule=ExpSchedule(0.5)),
        "opt_rmsprop": lambda: RMSProp(),
        "opt_rmsprop_clip": lambda: RMSProp(decay_rate=0.9, learning_rate=0.01, gradient_clip_norm=1.5,
                                            gradient_clip_value=0.3, param_clip_value=0.3),
        "opt_adagrad": lambda: Adagrad(),
        "opt_adagrad_clip": lambda: Adagrad(learning_rate=0.05, gradient_clip_norm=1.0, gradient_clip_value=0.5),
        "opt_adadelta": lambda: Adadelta(),
        "opt_adadelta_clip": lambda: Adadelta(decay=0.9, param_clip_value=0.2),
        "opt_adam": lambda: Adam(),
        "opt_adam_clip": lambda: Adam(learning_rate=0.01, gradient_clip_norm=1.0, gradient_clip_value=0.5,
                                      param_clip_value=0.3),
        "opt_shift_adamax": lambda: ShiftAdaMax(),
    }


# --------------------------------------------------------------------------- batch normalisation
def _bn_inputs(rng, nfm, n, dt):
    x = (1.0 + 2.0 * rng.randn(nfm, n)).astype(dt)
    gamma = rng.uniform(0.5, 1.5, (nfm, 1)).astype(dt)
    beta = rng.uniform(-0.5, 0.5, (nfm, 1)).astype(dt)
    err = rng.randn(nfm, n).astype(dt)
    return x, gamma, beta, err


def bn_compound(nfm=48, n=640, accumbeta=0.0, inference=False, rho=0.9, eps=1e-3):
    """The backend entry points as the BatchNorm layer calls them (layers/layer.py:2483-2520),
    two training steps (so the running statistics are a true blend) and a backward pass."""
    def run(be):
        _use(be)
        dt = _fdt(be)
        rng = np.random.RandomState(3)
        x_h, gamma_h, beta_h, err_h = _bn_inputs(rng, nfm, n, dt)
        x, gamma, beta, err = be.array(x_h), be.array(gamma_h), be.array(beta_h), be.array(err_h)
        xsum, xvar = be.zeros((nfm, 1)), be.zeros((nfm, 1))
        gmean = be.array(rng.randn(nfm, 1).astype(dt))
        gvar = be.array(rng.uniform(0.5, 2, (nfm, 1)).astype(dt))
        y = be.array(rng.randn(nfm, n).astype(dt))
        if inference:
            be.compound_fprop_bn(x, xsum, xvar, gmean, gvar, gamma, beta, y, eps, rho, True,
                                 accumbeta, False, inference=True)
            return {"y": y.get()}
        for _ in range(2):
            be.compound_fprop_bn(x, xsum, xvar, gmean, gvar, gamma, beta, y, eps, rho, True,
                                 accumbeta, False)
        dx, ggamma, gbeta = be.zeros((nfm, n)), be.zeros((nfm, 1)), be.zeros((nfm, 1))
        be.compound_bprop_bn(dx, ggamma, gbeta, err, x, xsum, xvar, gamma, eps)
        # NervanaCPU leaves the batch MEAN in xsum, the GPU kernels the batch SUM
        # (nervanacpu.py:1724 against cuda_batchnorm.py:27-219): compare the mean
        from neon.backends.nervanacpu import NervanaCPU
        mean = xsum.get() if isinstance(be, NervanaCPU) else xsum.get() / float(n)
        return {"xmean": mean, "xvar": xvar.get(), "gmean": gmean.get(), "gvar": gvar.get(), "y": y.get(),
                "dx": dx.get(), "grad_gamma": ggamma.get(), "grad_beta": gbeta.get()}
    return run


def bn_layer(nfm=40, bsz=BSZ):
    """neon's BatchNorm layer object, fprop (training), fprop (inference), bprop."""
    def run(be):
        _use(be, bsz)
        from neon.layers import BatchNorm
        dt = _fdt(be)
        rng = np.random.RandomState(4)
        x_h, gamma_h, beta_h, err_h = _bn_inputs(rng, nfm, bsz, dt)
        layer = BatchNorm(rho=0.8, eps=1e-4)
        _prepare(be, layer, nfm)
        layer.gamma.set(gamma_h.astype(layer.gamma.dtype))
        layer.beta.set(beta_h.astype(layer.beta.dtype))
        x, err = be.array(x_h), be.array(err_h)
        out = {"y": layer.fprop(x).get().copy()}
        out["deltas"] = layer.bprop(err).get().copy()
        out["grad_gamma"], out["grad_beta"] = layer.grad_gamma.get(), layer.grad_beta.get()
        out["gmean"], out["gvar"] = layer.gmean.get(), layer.gvar.get()
        out["y_inference"] = layer.fprop(x, inference=True).get().copy()
        return out
    return run


def _prepare(be, layer, nin):
    """configure / allocate / set_deltas the way neon's layer tests do."""
    layer.configure((nin,) if not isinstance(nin, tuple) else nin)
    layer.prev_layer = True
    layer.allocate()
    shape = layer.out_shape if isinstance(layer.out_shape, tuple) else (layer.out_shape,)
    size = int(np.prod(shape))
    layer.set_deltas(type("Deltas", (), {"buffers": [be.iobuf(size), be.iobuf(size)]})())
    return layer


# --------------------------------------------------------------------------- layers, costs
def bias_layer(nin=30, bsz=BSZ):
    def run(be):
        _use(be, bsz)
        from neon.initializers import Uniform
        from neon.layers import Bias
        rng = np.random.RandomState(6)
        dt = _fdt(be)
        layer = _prepare(be, Bias(init=Uniform(-1, 1)), nin)
        w = rng.uniform(-1, 1, (nin, 1)).astype(dt)
        layer.W.set(w.astype(layer.W.dtype))
        x = be.array(rng.randn(nin, bsz).astype(dt))
        err = be.array(rng.randn(nin, bsz).astype(dt))
        y = layer.fprop(x).get().copy()
        layer.bprop(err)
        return {"y": y, "dW": layer.dW.get()}
    return run


def activation_layers(nin=24, bsz=BSZ):
    def run(be):
        _use(be, bsz)
        from neon.layers import Activation
        from neon.transforms import Explin, Logistic, Normalizer, Rectlin, Softmax, Tanh
        rng = np.random.RandomState(7)
        dt = _fdt(be)
        x_h, err_h = (2 * rng.randn(nin, bsz)).astype(dt), rng.randn(nin, bsz).astype(dt)
        out = {}
        for name, act in (("rectlin", Rectlin()), ("leaky", Rectlin(slope=0.1)), ("tanh", Tanh()),
                          ("logistic", Logistic()), ("softmax", Softmax()), ("explin", Explin()),
                          ("normalizer", Normalizer(divisor=4))):
            layer = _prepare(be, Activation(act), nin)
            x, err = be.array(x_h), be.array(err_h)
            out[name + "_fprop"] = layer.fprop(x).get().copy()
            out[name + "_bprop"] = layer.bprop(err).get().copy()
        return out
    return run


def costs(nin=10, bsz=BSZ):
    def run(be):
        _use(be, bsz)
        from neon.layers import GeneralizedCost
        from neon.transforms import CrossEntropyBinary, CrossEntropyMulti, MeanSquared, SumSquared
        rng = np.random.RandomState(8)
        dt = _fdt(be)
        p = rng.uniform(0.05, 0.95, (nin, bsz))
        p /= p.sum(axis=0, keepdims=True)
        t = np.zeros((nin, bsz))
        t[rng.randint(0, nin, bsz), np.arange(bsz)] = 1
        y, tgt = be.array(p.astype(dt)), be.array(t.astype(dt))
        out = {}
        for name, cf in (("xent_binary", CrossEntropyBinary()), ("xent_multi", CrossEntropyMulti()),
                         ("sum_squared", SumSquared()), ("mean_squared", MeanSquared())):
            cost = GeneralizedCost(costfunc=cf)
            cost.outputs = be.iobuf((1, 1))            # (1, batch), as GeneralizedCost.initialize makes it
            cost.deltas = be.iobuf(nin)
            out[name + "_cost"] = np.array(cost.get_cost(y, tgt), dtype=np.float64).reshape(1, 1)
            out[name + "_errors"] = cost.get_errors(y, tgt).get().copy()
        return out
    return run


def dropout_layer(nin=200, bsz=128, keep=0.7):
    """Not compared element for element (each backend draws its own mask): returns the mask
    statistics and the identity outputs == mask * inputs * scaling that must hold on any backend."""
    def run(be):
        _use(be, bsz)
        from neon.layers import Dropout
        rng = np.random.RandomState(9)
        dt = _fdt(be)
        layer = _prepare(be, Dropout(keep=keep), nin)
        x_h = rng.randn(nin, bsz).astype(dt)
        # the layer works in place (outputs is inputs): a fresh input tensor per call
        y = layer.fprop(be.array(x_h)).get().copy()
        mask = layer.keep_mask.get().copy()
        y2 = layer.fprop(be.array(x_h)).get().copy()
        err = be.array(np.ones((nin, bsz), dt))
        d = layer.bprop(err).get().copy()
        mask2 = layer.keep_mask.get().copy()
        inf = layer.fprop(be.array(x_h), inference=True).get().copy()
        return {"y": y, "mask": mask, "x": x_h, "y_second": y2, "mask_second": mask2, "deltas": d,
                "y_inference": inf, "keep": np.array([[keep]])}
    return run


def array_iterator(ndata=200, nfeat=12, nclass=5, bsz=64):
    """ArrayIterator (neon/data/dataiterator.py:86-202): every minibatch as the layers see it."""
    def run(be):
        _use(be, bsz)
        import importlib.util
        import os
        import neon
        # the module file itself: the neon.data package also pulls in readers that need h5py
        path = os.path.join(os.path.dirname(neon.__file__), "data", "dataiterator.py")
        spec = importlib.util.spec_from_file_location("neon_dataiterator_unmodified", path)
        module = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(module)
        rng = np.random.RandomState(10)
        X = rng.rand(ndata, nfeat).astype(np.float32)
        y = rng.randint(0, nclass, ndata)
        it = module.ArrayIterator(X, y, nclass=nclass)
        out = {}
        for i, (xb, yb) in enumerate(it):
            out["x%d" % i] = xb.get().copy()
            out["y%d" % i] = yb.get().copy()
        return out

    def expected():
        """What the iterator must deliver, from numpy alone (NervanaCPU's own one-hot scatter,
        nervanacpu.py:660-683, indexes with a list of lists, which numpy >= 1.23 reads
        differently, so the reference side of this case cannot run on a current numpy)."""
        rng = np.random.RandomState(10)
        X = rng.rand(ndata, nfeat).astype(np.float32)
        y = rng.randint(0, nclass, ndata)
        out = {}
        for i in range(-(-ndata // bsz)):
            rows = np.arange(i * bsz, (i + 1) * bsz) % ndata       # the last batch wraps around
            out["x%d" % i] = X[rows].T
            out["y%d" % i] = (np.arange(nclass)[:, None] == y[rows][None, :]).astype(np.float32)
        return out
    run.expected = expected
    return run


def neon_caller_cases():
    """name -> run(be).  Importing neon happens inside (the caller has made it importable)."""
    cases = {}
    for name, make in _optimizers().items():
        cases[name] = _optimizer_case(make)
    cases["opt_adam_16_steps"] = _optimizer_case(_optimizers()["opt_adam"], steps=16)
    cases["bn_compound"] = bn_compound()
    cases["bn_compound_accumbeta"] = bn_compound(accumbeta=0.5)
    cases["bn_compound_inference"] = bn_compound(inference=True, accumbeta=0.25)
    cases["bn_compound_long_rows"] = bn_compound(nfm=160, n=8192)
    cases["bn_layer"] = bn_layer()
    cases["bias_layer"] = bias_layer()
    cases["activation_layers"] = activation_layers()
    cases["costs"] = costs()
    return cases


# not compared with NervanaCPU: random draws are backend specific (dropout: checked by
# properties); the iterator's reference is plain numpy (see array_iterator.expected)
STATISTICAL = {"dropout_layer": dropout_layer()}
NUMPY_CHECKED = {"array_iterator": array_iterator()}
# cases that need operations only the GPU backends of neon have (eager shift)
GPU_ONLY = ("opt_shift_adamax",)
