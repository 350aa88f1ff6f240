"""One rank of the multi-GPU parity run (started by tests/test_sharded_gpu.py through
torch.distributed.run).  Compares column-sharded execution with the float64 checker
on the global arrays and with unsharded execution on the same device."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    from neon_b200.sharded import gen_sharded_backend
    from oracle.numpy_backend import OracleBackend
    from tests.parity import check_output
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    exchange = os.environ.get("B200_SHARDED_EXCHANGE", "1") == "1"
    be = gen_sharded_backend(rank, world, device_id=int(os.environ.get("LOCAL_RANK", rank)), rng_seed=0,
                             use_exchange=exchange)
    if os.environ.get("B200_SHARDED_MODE") == "expiry":
        return expiry(be, rank, world)
    ob = OracleBackend(default_dtype=np.float64)
    rng = np.random.RandomState(0)

    # ---- batch-norm statistics + normalise (config 4 shape class), columns sharded
    rows, cols = 64, 8192 * world
    xh = (1.0 + 2.0 * rng.randn(rows, cols)).astype(np.float16)
    gh = rng.uniform(0.5, 1.5, (rows, 1)).astype(np.float32)
    bh = rng.uniform(0.5, 1.5, (rows, 1)).astype(np.float32)
    x = be.array(xh, dtype=np.float16, parallel=True)
    y = be.empty((rows, cols), dtype=np.float16, parallel=True)
    g, b = be.array(gh), be.array(bh)
    before, before_x, launches = be.collectives, be.exchanges, be.launches
    y[:] = (x - be.mean(x, axis=1)) / be.sqrt(be.var(x, axis=1) + 1e-5) * g + b
    if exchange:        # one kernel: rows stay in shared memory, the statistics finish across the GPUs inside it
        assert (be.collectives - before, be.exchanges - before_x, be.launches - launches) == (0, 1, 1)
    else:
        assert be.collectives - before == 2
    ox, og, obt = ob.array(xh, dtype=np.float64), ob.array(gh, dtype=np.float64), ob.array(bh, dtype=np.float64)
    oy = ob.zeros((rows, cols), dtype=np.float64)
    oy[:] = (ox - ob.mean(ox, axis=1)) / ob.sqrt(ob.var(ox, axis=1) + 1e-5) * og + obt
    check_output("sharded batchnorm y", y.get(), oy.get(), np.float16)
    mean = be.empty((rows, 1))
    mean[:] = be.mean(x, axis=1)
    check_output("sharded mean", mean.get(), xh.astype(np.float64).mean(axis=1, keepdims=True), np.float32)
    mx = be.empty((rows, 1))
    mx[:] = be.max(x, axis=1) - be.min(x, axis=1)
    x64 = xh.astype(np.float64)
    check_output("sharded max-min", mx.get(), x64.max(1, keepdims=True) - x64.min(1, keepdims=True), np.float32)
    am = be.empty((rows, 1), dtype=np.int32)
    am[:] = be.argmax(x, axis=1)
    assert np.array_equal(am.get(), x64.argmax(1).reshape(-1, 1)), "sharded argmax"
    am[:] = be.argmin(x, axis=1)
    assert np.array_equal(am.get(), x64.argmin(1).reshape(-1, 1)), "sharded argmin"
    # a reduction on top of a reduction whose result is the statement's output: the row-resident
    # kernel with clusters of two, both passes exchanged, the index finished by the cluster's first block
    before_x, launches = be.exchanges, be.launches
    am[:] = be.argmax(be.absolute(x - be.mean(x, axis=1)), axis=1)
    if exchange:
        assert (be.exchanges - before_x, be.launches - launches) == (1, 1)
    dev64 = np.abs(x64 - x64.mean(1, keepdims=True))
    picked = np.take_along_axis(dev64, am.get().astype(np.int64), axis=1)
    assert np.all(picked >= dev64.max(1, keepdims=True) * (1 - 1e-3)), "sharded argmax of deviations, short rows"
    tie = np.round(xh.astype(np.float32)).astype(np.float16)       # many equal maxima: first one wins
    xt = be.array(tie, dtype=np.float16, parallel=True)
    am[:] = be.argmax(xt, axis=1)
    assert np.array_equal(am.get(), tie.astype(np.float64).argmax(1).reshape(-1, 1)), "sharded argmax with ties"
    s0 = be.empty((1, cols), parallel=True)
    s0[:] = be.sum(x, axis=0)
    check_output("sharded axis-0 sum", s0.get(), x64.sum(0, keepdims=True), np.float32)

    # ---- three passes (softmax): one launch while every row has a resident block of its own,
    #      the multi-launch form beyond that (700 rows of 32 KB: more rows than resident blocks)
    for rows in (500, 700):
        cols = 16384 * world
        xh = (0.5 + rng.randn(rows, cols)).astype(np.float16)
        x = be.array(xh, dtype=np.float16, parallel=True)
        y = be.empty((rows, cols), dtype=np.float16, parallel=True)
        x64 = xh.astype(np.float64)
        before, before_x, launches = be.collectives, be.exchanges, be.launches
        e = be.exp(x - be.max(x, axis=1))
        y[:] = e / be.sum(e, axis=1)
        if exchange:
            assert be.collectives == before
            if rows == 500:
                assert (be.exchanges - before_x, be.launches - launches) == (1, 1)
        e64 = np.exp(x64 - x64.max(1, keepdims=True))
        check_output("sharded softmax", y.get(), e64 / e64.sum(1, keepdims=True), np.float16)
        y[:] = (x - be.mean(x, axis=1)) / be.sqrt(be.var(x, axis=1) + 1e-5)
        check_output("sharded standardise", y.get(),
                     (x64 - x64.mean(1, keepdims=True)) / np.sqrt(x64.var(1, keepdims=True) + 1e-5), np.float16)
        far = be.empty((rows, 1), dtype=np.int32)
        far[:] = be.argmax(be.absolute(x - be.mean(x, axis=1)), axis=1)
        dev = np.abs(x64 - x64.mean(1, keepdims=True))
        picked = np.take_along_axis(dev, far.get().astype(np.int64), axis=1)
        assert np.all(picked >= dev.max(1, keepdims=True) * (1 - 1e-3)), "sharded argmax of deviations"
        del x, y, e

    # ---- a recorded sequence of sharded statements, replayed between eager ones
    if exchange:
        rows, cols = 96, 4096 * world
        xh = rng.randn(rows, cols).astype(np.float32)
        x = be.array(xh, parallel=True)
        y = be.empty((rows, cols), parallel=True)
        top, low = be.empty((rows, 1)), be.empty((rows, 1))

        def sequence():
            y[:] = (x - be.mean(x, axis=1)) / be.sqrt(be.var(x, axis=1) + 1e-5)
            top[:] = be.max(y, axis=1)
            x[:] = y * 2.0 + 1.0

        graph = be.capture(sequence)               # runs it once eagerly, then records it
        want = xh.astype(np.float64)

        def expected(v):
            yy = (v - v.mean(1, keepdims=True)) / np.sqrt(v.var(1, keepdims=True) + 1e-5)
            return yy, yy.max(1, keepdims=True), yy * 2.0 + 1.0
        _, _, want = expected(want)
        for turn in range(5):
            before_x = be.exchanges
            graph.replay()
            assert be.exchanges - before_x == 2
            yy, tt, want = expected(want)
            low[:] = be.min(y, axis=1)             # an eager exchange between the replays
            check_output("replayed y, turn %d" % turn, y.get(), yy, np.float32)
            check_output("replayed max, turn %d" % turn, top.get(), tt, np.float32)
            check_output("eager min after replay %d" % turn, low.get(), yy.min(1, keepdims=True), np.float32)
        del graph
        # stochastic rounding inside a recorded sharded sequence: replays draw what eager steps would
        zq = be.empty((rows, cols), dtype=np.float16, parallel=True)
        zq.rounding = True

        def rounded():
            y[:] = (x - be.mean(x, axis=1)) * 3.0
            zq[:] = y * 1.0009765625 + top
            x[:] = x * 0.5 + 0.25
        x.local.set(np.ascontiguousarray(xh[:, x.c0:x.c0 + x.local.shape[1]]))
        be.rng_reset()
        eager_bits = []
        for _ in range(4):
            rounded()
            eager_bits.append(zq.local.get().view(np.uint16).copy())
        x.local.set(np.ascontiguousarray(xh[:, x.c0:x.c0 + x.local.shape[1]]))
        be.rng_reset()
        graph = be.capture(rounded)
        assert graph.rng_count == 1 and graph.count == 1
        assert np.array_equal(zq.local.get().view(np.uint16), eager_bits[0])
        for i in range(1, 4):
            graph.replay()
            assert np.array_equal(zq.local.get().view(np.uint16), eager_bits[i]), "replayed rounding, step %d" % i
        del x, y, graph

    # ---- fp16 chain with stochastic rounding + whole-tensor reductions (config 5 shape class)
    rows, cols = 256, 1024 * world
    xh = rng.uniform(-4, 4, (rows, cols)).astype(np.float16)
    yh = rng.uniform(-4, 4, (rows, cols)).astype(np.float16)
    xs, ys = be.array(xh, dtype=np.float16, parallel=True), be.array(yh, dtype=np.float16, parallel=True)
    zs = be.empty((rows, cols), dtype=np.float16, parallel=True)
    zs.rounding = True
    total, peak = be.empty((1, 1)), be.empty((1, 1))
    be.rng_reset()
    zs[:] = be.tanh(xs) * be.sqrt(be.absolute(ys)) + 0.5 * xs * ys
    total[:] = be.sum(zs)
    peak[:] = be.max(be.absolute(zs))
    z_sharded = zs.get()
    # the same statements unsharded on this device, same generator state: identical bits
    xf, yf = be.array(xh, dtype=np.float16), be.array(yh, dtype=np.float16)
    zf = be.empty((rows, cols), dtype=np.float16)
    zf.rounding = True
    be.rng_reset()
    zf[:] = be.tanh(xf) * be.sqrt(be.absolute(yf)) + 0.5 * xf * yf
    assert np.array_equal(z_sharded.view(np.uint16), zf.get().view(np.uint16)), "rounding depends on sharding"
    z64 = z_sharded.astype(np.float64)
    check_output("sharded total", total.get(), np.array([[z64.sum()]]), np.float32, scale=float(np.abs(z64).sum()))
    assert float(peak.get()[0, 0]) == float(np.abs(z_sharded).max())
    # ---- seeded random statements (tests/fuzz.py) over column-sharded tensors
    from tests import fuzz
    ran = 0
    for seed in range(400):
        spec = fuzz.Spec(seed)
        if not fuzz.shardable(spec, world):
            continue
        arrays = fuzz.host_arrays(spec)
        got = fuzz.build(be, spec, arrays, full_kw={"parallel": True})
        if got is None:
            continue
        with np.errstate(all="ignore"):
            want = fuzz.build(OracleBackend(default_dtype=np.float64), spec, arrays, compute_dtype=np.float64)
        g, w = got.get(), want.get()
        ran += 1
        if spec.red is not None and spec.red[0].startswith("arg"):
            continue                                   # near-ties of computed values may pick other positions
        if spec.red is not None and spec.red[0] == "min":
            continue                                   # minima of differences are ill-conditioned in fp32
        check_output("sharded fuzz seed %d" % seed, g, w, g.dtype)
    assert ran > 40, ran
    be.synchronize()
    be.host_barrier()
    if rank == 0:
        print("SHARDED-OK world=%d collectives=%d exchanges=%d" % (world, be.collectives, be.exchanges))


def expiry(be, rank, world):
    """A rank that leaves a statement out: the others' kernels wait for its results, give up
    after the time limit, report through the status word -- and the job carries on."""
    from neon_b200 import runtime as rt
    rng = np.random.RandomState(1)
    rows, cols = 48, 4096 * world
    xh = rng.randn(rows, cols).astype(np.float32)
    x = be.array(xh, parallel=True)
    m = be.empty((rows, 1))
    m[:] = be.max(x, axis=1)
    be.synchronize()
    assert np.array_equal(m.get(), xh.max(1, keepdims=True))
    be._planner.wait_limit_ns = 30 * 1000 * 1000
    be._plans.clear()
    be.host_barrier()
    if rank != world - 1:
        m[:] = be.max(x, axis=1)
        try:
            be.synchronize()
            raise AssertionError("the wait for the missing rank did not run out")
        except rt.B200Error as e:
            assert e.status == -6 and "another GPU" in str(e), str(e)
    else:
        be._xepoch += 1          # the launch number of the statement this rank leaves out
    be.host_barrier()
    be._planner.wait_limit_ns = 2000000000
    be._plans.clear()
    m[:] = be.min(x, axis=1)
    be.synchronize()
    assert np.array_equal(m.get(), xh.min(1, keepdims=True))
    be.host_barrier()
    if rank == 0:
        print("SHARDED-OK expiry world=%d" % world)


if __name__ == "__main__":
    main()
