#!/usr/bin/env python
"""
Benchmark of the compound-optree engine.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
                    [--workload cfg5|cfg3|cfg4|cfg1|cfg2|transpose|kahan] [--scaling strong|weak]

Headline workload (config 5 of the baseline list, the largest single-GPU one):
x, y fp16 of shape (32768, 32768) ~U(-4,4), one step =

    z[:]     = tanh(x) * sqrt(|y|) + 0.5 * x * y       stored as fp16 with stochastic rounding
    total[:] = sum(z)                                   over all elements
    peak[:]  = max(|z|)                                 over all elements

The metric is effective HBM bandwidth: algorithmic bytes (every distinct input of
a statement read once, its output written once: 6 + 2 + 2 bytes per element)
divided by device time.  With N > 1 the SAME (32768, 32768) problem is sharded by
columns over the N ranks (strong scaling: 32768/N columns each); the element-wise
statement is shard-local and the two whole-tensor reductions are combined across
the GPUs.  ``--scaling weak`` gives every rank a full (32768, 32768) shard instead.

Prints one JSON line.  ``value`` times the statements with inputs resident in HBM;
``e2e`` repeats them with the host->device copy of x and y (pinned memory) and the
device->host read of total and peak inside the timed region.  The default run adds,
under ``also``, the two other sharded configurations at their quoted global sizes
(config 3, the Adam update of 1e8 parameters; config 4, the batch-norm statement on
(256, 401408) fp16), each with its own per-step breakdown, and for N > 1 the
weak-scaling figure of the headline workload under ``weak``.
"""
import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

ROWS = COLS = 32768
BYTES_PER_ELEMENT = 6 + 2 + 2          # z statement, total, peak (algorithmic)
Z_BYTES_PER_ELEMENT = 6                # dominant kernel: read x, y (fp16), write z (fp16)
METRIC = "compound-optree effective HBM GB/s"
WORKLOAD = ("cfg5: z=tanh(x)*sqrt(|y|)+0.5*x*y (fp16, stochastic rounding), "
            "total=sum(z), peak=max|z|")
# DRAM traffic of the z kernel from ncu (profiles/ew_kernel_cfg5_fp16_chain.md, a 2^29-element
# launch: 2,147,534,592 bytes read, 1,041,722,112 written): reads scale with the element count
# (4.0001 bytes per element); writes are 2 bytes per element minus what is still in L2 when the
# kernel ends, a constant that does not grow with the launch (32.0 MB)
Z_DRAM_READ_PER_ELEMENT = 2147534592.0 / (1 << 29)
Z_DRAM_WRITE_L2_RESIDUE = 2.0 * (1 << 29) - 1041722112.0


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler(object):
    """nvidia-smi SM clock / throttle-reason samples while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device):
        self.device = device
        self.lines = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.device), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [s.strip() for s in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for n, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": float(np.median(sm)) if sm else None,
                "sm_max_mhz": float(max(mx)) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def fill_uniform_f16(dst, seed, lo=-4.0, hi=4.0, chunk=1 << 24):
    """Seeded U(lo,hi) into the fp16 array dst, chunked to bound host memory."""
    rng = np.random.default_rng(seed)
    flat = dst.reshape(-1)
    for s in range(0, flat.size, chunk):
        n = min(chunk, flat.size - s)
        flat[s:s + n] = (rng.random(n, dtype=np.float32) * np.float32(hi - lo) + np.float32(lo)).astype(np.float16)


def statements(be, x, y, z, total, peak):
    z[:] = be.tanh(x) * be.sqrt(be.absolute(y)) + 0.5 * x * y
    total[:] = be.sum(z)
    peak[:] = be.max(be.absolute(z))


def adam_step(be, param, grad, m, v, t, beta_1=0.9, beta_2=0.999, epsilon=1e-8, learning_rate=1e-3):
    """The three assignments neon's Adam.optimize issues per parameter tensor
    (neon/optimizers/optimizer.py:898-930), the bias-corrected step size a lazy scalar op-tree."""
    l = learning_rate * be.sqrt(1 - beta_2 ** t) / (1 - beta_1 ** t)
    g = grad / be.bsz
    m[:] = m * beta_1 + (1. - beta_1) * g
    v[:] = v * beta_2 + (1. - beta_2) * g * g
    param[:] = param - (1.0 * l * m) / (be.sqrt(v) + epsilon)


# --------------------------------------------------------------------------- CPU reference arm
def _cpu_worker(args):
    """One host process: neon's NervanaCPU (from a neon source tree) -- or, where there is no
    tree, the numpy restatement of it -- on its column block of the sample.  Returns
    (elements, wall-clock seconds of each pass, which implementation ran)."""
    elements, reps, seed = args
    sys.path.insert(0, ROOT)
    kind = "port"
    be = None
    try:
        from oracle import neon_ref
        if neon_ref.find_reference():
            NervanaCPU = neon_ref.import_reference_cpu()
            be = NervanaCPU(default_dtype=np.float32)
            kind = "reference"
    except Exception:
        be = None
    if be is None:
        from oracle.numpy_backend import OracleBackend
        be = OracleBackend(default_dtype=np.float32)
    cols = 4096
    rows = max(1, elements // cols)
    rng = np.random.default_rng(seed)
    xh = (rng.random((rows, cols), dtype=np.float32) * 8 - 4)
    yh = (rng.random((rows, cols), dtype=np.float32) * 8 - 4)
    x, y = be.array(xh), be.array(yh)          # fp16 storage is upcast for the CPU run
    z, total, peak = be.zeros((rows, cols)), be.zeros((1, 1)), be.zeros((1, 1))
    times = []
    for _ in range(reps):
        t0 = time.perf_counter()
        statements(be, x, y, z, total, peak)
        times.append(time.perf_counter() - t0)
    return rows * cols, times, kind


def cpu_rate(elements, reps, cores=None, skip=0):
    """The CPU implementation on a bounded sample.  NervanaCPU is single threaded (numpy
    ufuncs), but the path shards by columns, so the sample is split over ``cores`` processes
    that run at the same time -- the most the reference's CPU code can get out of this host.
    Returns (GB/s, seconds per pass, cores, implementation, elements, wall seconds)."""
    cores = cores or max(1, len(os.sched_getaffinity(0)))
    per = max(4096, elements // cores)
    t0 = time.perf_counter()
    if cores == 1:
        results = [_cpu_worker((per, reps, 0))]
    else:
        import multiprocessing as mp
        with mp.get_context("spawn").Pool(cores) as pool:
            results = pool.map(_cpu_worker, [(per, reps, i) for i in range(cores)])
    wall = time.perf_counter() - t0
    n = sum(r[0] for r in results)
    # pass i is over when the slowest process finishes it
    per_pass = [max(r[1][i] for r in results) for i in range(skip, reps)]
    sec = float(np.mean(per_pass)) if skip else min(per_pass)
    kind = "reference" if all(r[2] == "reference" for r in results) else "port"
    return n * BYTES_PER_ELEMENT / sec / 1e9, sec, cores, kind, n, wall


def _kind_text(kind):
    return ("neon's own NervanaCPU (unmodified sources)" if kind == "reference"
            else "numpy restatement of NervanaCPU (no neon source tree on this machine)")


def run_reference(args, rank, world):
    """Reference arm: the CPU implementation of the path on this box's host cores, one process
    per core, each step a bounded sample of the workload."""
    if rank != 0:
        return
    sample = 1 << 26
    reps = args.warmup + args.steps
    gbs, sec, cores, kind, n, wall = cpu_rate(sample, reps, skip=args.warmup)
    single = cpu_rate(1 << 23, 3, cores=1)
    line = {
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
        "scaling": args.scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "rows": args.rows, "cols": args.cols,
                   "sample_elements_per_step": n},
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": cores, "kind": kind,
                         "sample": "%d of 2^30 elements per step split over %d processes, %s, fp16 inputs "
                                   "upcast to fp32" % (n, cores, _kind_text(kind)),
                         "single_process": {"value": single[0], "unit": "GB/s", "cores": 1,
                                            "sample": "2^23 elements, best of 3 passes"}},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "host_cores": os.cpu_count(), "wall_s": wall,
    }
    print(json.dumps(line))


# --------------------------------------------------------------------------- timing helpers
class Job(object):
    """Backend plus the host-side collectives of this run."""

    def __init__(self, be, rank, world, barrier, host_max):
        self.be, self.rank, self.world = be, rank, world
        self.barrier, self.host_max = barrier, host_max
        self.kw = {"parallel": True} if world > 1 else {}

    def time_steps(self, step, steps):
        """Device time of ``steps`` calls of ``step`` in ms: CUDA events on the backend's stream,
        a host barrier and a device synchronize on both sides, the maximum over ranks."""
        be = self.be
        ev0, ev1 = be.init_mark(), be.init_mark()
        self.barrier()
        be.synchronize()
        launches0 = be.launches
        be.record_mark(ev0)
        for s in range(steps):
            step(s)
        be.record_mark(ev1)
        be.synchronize()
        self.barrier()
        return self.host_max(be.get_time(ev0, ev1)), be.launches - launches0

    def breakdown(self, step, steps=5):
        """Per-step split of device time into this package's kernels, collectives between the
        GPUs and the rest (gaps between launches: host issue time, event and launch latency),
        from events around every launch of a few extra, untimed steps."""
        be = self.be
        if not hasattr(be, "start_timeline"):
            return None
        for s in range(2):
            step(s)
        be.synchronize()
        self.barrier()
        ev0, ev1 = be.init_mark(), be.init_mark()
        be.start_timeline()
        be.record_mark(ev0)
        for s in range(steps):
            step(s)
        be.record_mark(ev1)
        be.synchronize()
        records = be.stop_timeline()
        total = be.get_time(ev0, ev1) / steps
        kern = sum(ms for kind, _, ms in records if kind == "kernel") / steps
        coll = sum(ms for kind, _, ms in records if kind == "collective") / steps
        out = {"step_ms": self.host_max(total), "kernel_ms": self.host_max(kern),
               "collective_ms": self.host_max(coll), "gap_ms": self.host_max(max(total - kern - coll, 0.0)),
               "launches_per_step": sum(1 for kind, _, _ in records if kind == "kernel") // steps,
               "collectives_per_step": sum(1 for kind, _, _ in records if kind == "collective") // steps,
               "note": "max over ranks of each term, medians not taken; events around every launch add a little gap"}
        return out


def shard_note(world, scaling):
    if world == 1:
        return "none"
    return "columns, %s scaling" % scaling


# --------------------------------------------------------------------------- the other configurations
def other_workloads(name, job, scaling):
    """The remaining baseline configurations as ([(label, statement, algorithmic bytes)], elements).
    Byte and element counts are those of the whole job.  Strong scaling: the quoted global size
    is sharded by columns; weak scaling: every rank gets the quoted size."""
    be, world, rank, kw = job.be, job.world, job.rank, job.kw
    mult = world if scaling == "weak" else 1
    rng = np.random.RandomState(7 + rank)

    def local(cols):          # columns of the global tensor this rank fills
        return cols * mult // world if world > 1 else cols

    def sharded(make_local, shape, dtype=np.float32):
        """Tensor of global ``shape`` whose local columns are filled from ``make_local``."""
        if world == 1:
            return be.array(make_local((shape[0], shape[1])).astype(dtype), dtype=dtype)
        t = be.empty(shape, dtype=dtype, **kw)
        t.local.set(make_local(t.local.shape).astype(dtype))
        return t

    if name == "cfg1":
        r, c = 4096, 128 * mult
        a = sharded(lambda s: rng.randn(*s), (r, c))
        b = sharded(lambda s: rng.randn(*s), (r, c))
        bias = be.array(rng.uniform(-.5, .5, (r, 1)).astype(np.float32))
        out = be.empty((r, c), **kw)
        s = be.empty((1, c), **kw)
        m = be.empty((1, c), dtype=np.int32, **kw)

        def st_out(): out[:] = be.maximum(a * b + bias, 0)
        def st_sum(): s[:] = be.sum(out, axis=0)
        def st_arg(): m[:] = be.argmax(out, axis=0)
        n = r * c
        return [("bias+relu", st_out, 12 * n + 4 * r), ("sum axis0", st_sum, 4 * n + 4 * c),
                ("argmax axis0", st_arg, 4 * n + 4 * c)], n
    if name == "cfg2":
        r, c = 32000, 256 * mult
        x = sharded(lambda s: 3.0 * rng.randn(*s), (r, c))
        y = be.empty((r, c), **kw)
        idx = be.empty((1, c), dtype=np.int32, **kw)

        def st_y():
            mx = be.max(x, axis=0)
            e = be.exp(x - mx)
            y[:] = e / be.sum(e, axis=0)
        def st_idx(): idx[:] = be.argmax(x, axis=0)
        n = r * c
        return [("softmax axis0", st_y, 8 * n), ("argmax axis0", st_idx, 4 * n + 4 * c)], n
    if name == "cfg3":
        shape = (100000, 1000 * mult)
        n = shape[0] * shape[1]
        param = sharded(lambda s: 0.02 * rng.randn(*s), shape)
        grad = sharded(lambda s: 1e-3 * rng.randn(*s), shape, np.float16)
        mm, vv = be.zeros(shape, **kw), be.zeros(shape, **kw)
        be.bsz = 1
        step = [0]

        def st_adam():
            step[0] += 1
            adam_step(be, param, grad, mm, vv, step[0])
        return [("adam step (3 statements)", st_adam, 36 * n)], n
    if name == "cfg4":
        r, c = 256, 56 * 56 * 128 * mult
        x = sharded(lambda s: 1.0 + 2.0 * rng.randn(*s), (r, c), np.float16)
        gamma = be.array(rng.uniform(.5, 1.5, (r, 1)).astype(np.float32))
        beta = be.array(rng.uniform(.5, 1.5, (r, 1)).astype(np.float32))
        y = be.empty((r, c), dtype=np.float16, **kw)

        def st_bn():
            y[:] = (x - be.mean(x, axis=1)) / be.sqrt(be.var(x, axis=1) + 1e-5) * gamma + beta
        n = r * c
        return [("batchnorm stats+normalise", st_bn, 4 * n + 2048)], n
    if name == "transpose":
        # the data-feed step in front of every fprop (ArrayIterator): (examples, features) rows
        # to (features, batch) columns; one 256 MiB matrix each of fp32, fp16 and uint8 (input and
        # output together are four times the L2)
        stmts = []
        for dt, (r, c) in ((np.float32, (8192, 8192)), (np.float16, (16384, 8192)), (np.uint8, (16384, 16384))):
            a = be.zeros((r, c), dtype=dt)
            out = be.empty((c, r), dtype=dt)
            stmts.append(("copy_transpose %s %dx%d" % (np.dtype(dt).name, r, c),
                          (lambda a=a, out=out: be.copy_transpose(a, out)), 2 * a.nbytes))
        return stmts, 8192 * 8192
    if name == "kahan":
        n = 100000000
        stmts = []
        for dt in (np.float32, np.float16):
            s_, c_, a_ = (be.zeros((n, 1), dtype=dt) for _ in range(3))
            s_.rounding = True
            stmts.append(("compensated_sum %s, stochastic rounding" % np.dtype(dt).name,
                          (lambda s_=s_, c_=c_, a_=a_: be.compensated_sum(s_, c_, a_)), 5 * s_.nbytes))
        return stmts, n
    raise SystemExit("unknown workload %s" % name)


def measure_other(name, job, steps, warmup, scaling, extras=True):
    """Timed run of one of the other configurations; returns the record for the JSON line."""
    be, world = job.be, job.world
    stmts, n_global = other_workloads(name, job, scaling)
    n_local = n_global // world

    def step(_):
        for _, fn, _ in stmts:
            fn()
    for s in range(max(warmup, 3)):
        step(s)
    be.synchronize()
    log = be.launch_log = []
    ms_total, launches = job.time_steps(step, steps)
    be.launch_log = None
    kinds = [k for k, _ in log[: max(launches // steps, 1)]]
    nbytes_step = sum(b for _, _, b in stmts)
    ms_step = ms_total / steps
    peak_gbs, peak_kind = measured_peak()
    value = nbytes_step / ms_step / 1e6
    rec = {"workload": name, "value": value, "unit": "GB/s", "ms_per_step": ms_step, "steps": steps,
           "elements": n_global, "elements_per_s": n_global / (ms_step * 1e-3),
           "algorithmic_bytes_per_step": nbytes_step,
           "pct_of_measured_peak_per_gpu": 100.0 * value / world / peak_gbs, "peak_kind": peak_kind,
           "pct_of_8TBps_per_gpu": 100.0 * value / world / 8000.0,
           "l2": "working set is L2-resident between steps" if n_local * 4 < 100e6 else "exceeds L2",
           "gpu_launches": launches, "launches_per_step": kinds,
           "breakdown": job.breakdown(step)}
    # the same sequence recorded once as a CUDA graph and replayed (every rank records and
    # replays its own; reductions across the GPUs number their launches relative to a device word)
    if hasattr(be, "capture"):
        graph = be.capture(lambda: step(0))
        for _ in range(3):
            graph.replay()
        graph_total, _ = job.time_steps(lambda s: graph.replay(), steps)
        graph_ms = graph_total / steps
        rec["graph_replay"] = {"ms_per_step": graph_ms, "GBps": nbytes_step / graph_ms / 1e6,
                               "note": "statement sequence recorded once with be.capture(), replayed with one call"}
        del graph
    if not extras:
        return rec
    # per statement, from events around each one (a few more steps)
    marks = [[(be.init_mark(), be.init_mark()) for _ in stmts] for _ in range(steps)]
    for s in range(steps):
        for i, (_, fn, _) in enumerate(stmts):
            be.record_mark(marks[s][i][0])
            fn()
            be.record_mark(marks[s][i][1])
    be.synchronize()
    rec["statements"] = []
    for i, (label, _, nbytes) in enumerate(stmts):
        ms = float(np.median([be.get_time(*marks[s][i]) for s in range(steps)]))
        rec["statements"].append({"statement": label, "ms": ms, "algorithmic_bytes": nbytes,
                                  "GBps": nbytes / ms / 1e6})
    # working sets that stay in L2 between steps: the same statements again with L2 flushed
    # (a 256 MiB fill) before each one, timed per statement so that the fill is not counted
    if world == 1 and n_local * 4 < 100e6:
        flush = be.empty((1 << 26, 1))
        cold_marks = [[(be.init_mark(), be.init_mark()) for _ in stmts] for _ in range(steps)]
        for s in range(steps):
            for i, (_, fn, _) in enumerate(stmts):
                flush.fill(0)
                be.record_mark(cold_marks[s][i][0])
                fn()
                be.record_mark(cold_marks[s][i][1])
        be.synchronize()
        cold_ms = sum(float(np.median([be.get_time(*cold_marks[s][i]) for s in range(steps)]))
                      for i in range(len(stmts)))
        rec["cold"] = {"ms_per_step": cold_ms, "GBps": nbytes_step / cold_ms / 1e6,
                       "note": "L2 flushed (256 MiB fill) before every statement; sum of per-statement medians"}
    return rec


def run_other(args, job):
    sampler = ClockSampler(int(os.environ.get("LOCAL_RANK", "0")))
    if job.rank == 0:
        sampler.start()
        time.sleep(0.2)
    rec = measure_other(args.workload, job, args.steps, args.warmup, args.scaling)
    clocks = sampler.stop() if job.rank == 0 else None
    if job.rank != 0:
        return
    line = {"metric": METRIC, "value": rec.pop("value"), "unit": "GB/s", "n_gpus": job.world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": rec.pop("ms_per_step"), "higher_is_better": True,
            "scaling": args.scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": args.workload, "elements": rec["elements"],
                       "sharding": shard_note(job.world, args.scaling), "l2": rec["l2"]},
            "clocks": clocks}
    line.update(rec)
    print(json.dumps(line))


# --------------------------------------------------------------------------- headline workload
def cfg5_tensors(job, rows, cols_global, seeds):
    """x, y, z, total, peak for a (rows, cols_global) problem, plus this rank's pinned host
    copies of x and y (the source of the end-to-end copies)."""
    from neon_b200 import runtime as rt
    be, world, rank, kw = job.be, job.world, job.rank, job.kw
    cols_local = cols_global // world
    n_local = rows * cols_local
    nbytes = n_local * 2
    hx_p, hy_p = rt.host_alloc(nbytes), rt.host_alloc(nbytes)
    hx = np.frombuffer((ctypes.c_char * nbytes).from_address(hx_p), dtype=np.float16).reshape(rows, cols_local)
    hy = np.frombuffer((ctypes.c_char * nbytes).from_address(hy_p), dtype=np.float16).reshape(rows, cols_local)
    fill_uniform_f16(hx, seeds[0] + rank)
    fill_uniform_f16(hy, seeds[1] + rank)
    gshape = (rows, cols_global)
    x = be.empty(gshape, dtype=np.float16, **kw)
    y = be.empty(gshape, dtype=np.float16, **kw)
    z = be.empty(gshape, dtype=np.float16, **kw)
    z.rounding = True
    total, peak = be.empty((1, 1)), be.empty((1, 1))
    rt.memcpy_h2d(x.ptr, hx_p, nbytes, be.stream, sync=True)
    rt.memcpy_h2d(y.ptr, hy_p, nbytes, be.stream, sync=True)
    return dict(x=x, y=y, z=z, total=total, peak=peak, hx_p=hx_p, hy_p=hy_p, nbytes=nbytes,
                n_local=n_local, n_global=rows * cols_global)


def free_host(t):
    from neon_b200 import runtime as rt
    rt.host_free(t["hx_p"])
    rt.host_free(t["hy_p"])


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--rows", type=int, default=ROWS)
    ap.add_argument("--cols", type=int, default=COLS, help="columns of the global tensor (strong) / of each shard (weak)")
    ap.add_argument("--e2e-steps", type=int, default=3)
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-also", action="store_true", help="skip the cfg3 / cfg4 / weak-scaling extras of the default run")
    ap.add_argument("--scaling", default="strong", choices=("strong", "weak"))
    ap.add_argument("--rowres", default="auto", choices=("auto", "always", "never"),
                    help="multi-pass statements over long rows (cfg4): let the planner choose between the one-launch "
                         "row-resident kernel and one launch per pass (auto), or force either form")
    ap.add_argument("--workload", default="cfg5", help="cfg5 (default, the reported metric), cfg1..cfg4, transpose (data-feed copy_transpose) or kahan (compensated_sum)")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        return run_reference(args, rank, world)
    if world != args.gpus:
        raise SystemExit("--gpus %d but WORLD_SIZE=%d: launch with torch.distributed.run" % (args.gpus, world))

    from neon_b200 import runtime as rt
    if world > 1:
        from neon_b200.sharded import gen_sharded_backend
        # stdout carries the JSON line only: whatever NCCL prints while the communicator
        # comes up (its version banner, debug lines) is sent to stderr
        sys.stdout.flush()
        saved = os.dup(1)
        os.dup2(2, 1)
        try:
            be = gen_sharded_backend(rank=rank, world_size=world, device_id=local_rank, rng_seed=0)
            warm = be.empty((1, 1))
            warm[:] = 0
            be.allreduce_tensor(warm)
            be.synchronize()
        finally:
            sys.stdout.flush()
            os.dup2(saved, 1)
            os.close(saved)
        job = Job(be, rank, world, be.host_barrier, be.host_max)
    else:
        from neon_b200 import gen_backend
        be = gen_backend(backend="b200", rng_seed=0, device_id=local_rank)
        job = Job(be, rank, world, (lambda: None), (lambda v: v))

    if args.rowres == "never":
        be._planner.rowres = False
    elif args.rowres == "always":
        be._planner.rowres_exchange_resident_only = False

    if args.workload != "cfg5":
        return run_other(args, job)

    rows = args.rows
    cols_global = args.cols * (world if args.scaling == "weak" else 1)
    t = cfg5_tensors(job, rows, cols_global, (100, 200))
    x, y, z, total, peak = t["x"], t["y"], t["z"], t["total"], t["peak"]
    n_local, n_global, nbytes = t["n_local"], t["n_global"], t["nbytes"]

    for _ in range(max(args.warmup, 3)):
        statements(be, x, y, z, total, peak)
    be.synchronize()

    # ---- timed region: K steps, inputs resident in HBM (per-rank inputs of a step exceed L2
    #      up to 8 ranks: 4 GiB / N)
    kz = [(be.init_mark(), be.init_mark()) for _ in range(args.steps)]
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)

    def step(s):
        be.record_mark(kz[s][0])
        z[:] = be.tanh(x) * be.sqrt(be.absolute(y)) + 0.5 * x * y
        be.record_mark(kz[s][1])
        total[:] = be.sum(z)
        peak[:] = be.max(be.absolute(z))
    ms_total, launches = job.time_steps(step, args.steps)
    z_ms = float(np.mean([be.get_time(a, b) for a, b in kz]))
    res_total, res_peak = float(total.get()[0, 0]), float(peak.get()[0, 0])

    # ---- end to end: host buffers in, host scalars out, every step
    e2e_steps = max(1, args.e2e_steps)

    def e2e_step(s):
        rt.memcpy_h2d(x.ptr, t["hx_p"], nbytes, be.stream, sync=False)
        rt.memcpy_h2d(y.ptr, t["hy_p"], nbytes, be.stream, sync=False)
        statements(be, x, y, z, total, peak)
        total.get()
        peak.get()
    e2e_ms, _ = job.time_steps(e2e_step, e2e_steps)
    clocks = sampler.stop() if rank == 0 else None      # sampled over both timed regions
    breakdown = job.breakdown(lambda s: statements(be, x, y, z, total, peak))
    # the step recorded once and replayed (fresh rounding bits in every replay, see be.capture)
    graph = be.capture(lambda: statements(be, x, y, z, total, peak))
    for _ in range(3):
        graph.replay()
    replay_total, _ = job.time_steps(lambda s: graph.replay(), args.steps)
    del graph

    # ---- the other sharded configurations and (N > 1) the weak-scaling figure
    also, weak = {}, None
    if not args.no_also:
        del x, y, z
        free_host(t)
        t = None
        for name in ("cfg3", "cfg4"):
            also[name] = measure_other(name, job, args.steps, args.warmup, args.scaling, extras=False)
        if world > 1 and args.scaling == "strong":
            tw = cfg5_tensors(job, rows, args.cols * world, (300, 400))

            def weak_step(s):
                statements(be, tw["x"], tw["y"], tw["z"], tw["total"], tw["peak"])
            for s in range(3):
                weak_step(s)
            be.synchronize()
            wms, _ = job.time_steps(weak_step, args.steps)
            wms /= args.steps
            weak = {"value": tw["n_global"] * BYTES_PER_ELEMENT / (wms * 1e-3) / 1e9, "unit": "GB/s",
                    "ms_per_step": wms, "elements": tw["n_global"],
                    "note": "every rank holds a (%d, %d) shard; the problem grows with the number of GPUs" % (rows, args.cols)}
            free_host(tw)

    if rank != 0:
        return
    ms_step = ms_total / args.steps
    value = n_global * BYTES_PER_ELEMENT / (ms_step * 1e-3) / 1e9
    e2e_value = n_global * BYTES_PER_ELEMENT / (e2e_ms / e2e_steps * 1e-3) / 1e9
    peak_gbs, peak_kind = measured_peak()
    z_gbs = n_local * Z_BYTES_PER_ELEMENT / (z_ms * 1e-3) / 1e9
    traffic = Z_DRAM_READ_PER_ELEMENT * n_local + max(2.0 * n_local - Z_DRAM_WRITE_L2_RESIDUE, 0.0)
    line = {
        "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": args.scaling, "vs_baseline": None, "dtype": "f32", "storage_dtype": "f16", "data": "synthetic",
        "config": {"workload": WORKLOAD,
                   "rows": rows, "cols": cols_global, "elements": n_global, "elements_per_gpu": n_local,
                   "sharding": shard_note(world, args.scaling),
                   "l2": "inputs of a step (%.0f MiB per GPU) exceed L2; no flush needed" % (2 * nbytes / 2 ** 20),
                   "algorithmic_bytes_per_element": BYTES_PER_ELEMENT},
        "elements_per_s": n_global / (ms_step * 1e-3),
        "pct_of_8TBps_per_gpu": 100.0 * value / world / 8000.0,
        "pct_of_measured_peak_per_gpu": 100.0 * value / world / peak_gbs,
        "roofline": {"bound": "hbm", "kernel": "ew_flat (z statement)", "achieved": z_gbs,
                     "peak": peak_gbs, "peak_kind": peak_kind, "unit": "GB/s",
                     "frac": z_gbs / peak_gbs, "frac_of_8TBps": z_gbs / 8000.0, "ms_per_launch": z_ms,
                     "algorithmic_bytes_per_launch": n_local * Z_BYTES_PER_ELEMENT, "traffic": traffic,
                     "traffic_source": "ncu capture of a 2^29-element launch: DRAM reads scaled by the element "
                                       "count, writes = 2 B/element minus the 32.0 MB still in L2 at kernel end"},
        "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": 2 * nbytes * world,
                "d2h_bytes_per_step": 8 * world, "steps": e2e_steps, "ms_per_step": e2e_ms / e2e_steps},
        "gpu_launches": launches, "clocks": clocks, "breakdown": breakdown,
        "graph_replay": {"ms_per_step": replay_total / args.steps,
                         "GBps": n_global * BYTES_PER_ELEMENT / (replay_total / args.steps * 1e-3) / 1e9,
                         "note": "the three statements recorded once with be.capture(), replayed with one call; "
                                 "every replay draws fresh rounding bits"},
        "results": {"total": res_total, "peak": res_peak},
    }
    if also:
        line["also"] = also
    if weak is not None:
        line["weak"] = weak
    if not args.no_cpu and world == 1:
        gbs, sec, cores, kind, n, _ = cpu_rate(1 << 26, 8)
        single = cpu_rate(1 << 23, 3, cores=1)
        line["cpu_baseline"] = {"value": gbs, "unit": "GB/s", "cores": cores, "kind": kind,
                                "sample": "2^26 of 2^30 elements split over %d processes, best of 8 passes "
                                          "(%.2f s each), %s, fp16 inputs upcast to fp32"
                                          % (cores, sec, _kind_text(kind)),
                                "single_process": {"value": single[0], "unit": "GB/s", "cores": 1,
                                                   "sample": "2^23 elements, best of 3 passes"}}
    print(json.dumps(line))


if __name__ == "__main__":
    main()
