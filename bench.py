#!/usr/bin/env python
"""
Benchmark of the compound-optree engine.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (config 5 of the baseline list, the largest single-GPU one): per GPU,
x, y fp16 of shape (32768, 32768) ~U(-4,4) and one step =

    z[:]     = tanh(x) * sqrt(|y|) + 0.5 * x * y       stored as fp16 with stochastic rounding
    total[:] = sum(z)                                   over all elements
    peak[:]  = max(|z|)                                 over all elements

The metric is effective HBM bandwidth: algorithmic bytes (every distinct input of
a statement read once, its output written once: 6 + 2 + 2 bytes per element)
divided by device time.  With N > 1 every rank holds a (32768, 32768) column
shard of a (32768, N*32768) tensor (weak scaling), the element-wise statement is
shard-local and the two whole-tensor reductions end with an NCCL all-reduce.

Prints one JSON line.  `value` times the statements with inputs resident in HBM;
`e2e` repeats them with the host->device copy of x and y (pinned memory) and the
device->host read of total and peak inside the timed region.
"""
import argparse
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
# dram__bytes_read.sum + dram__bytes_write.sum of the z kernel divided by its elements, from the
# ncu capture of a 2^26-element launch (profiles/ew_kernel_cfg5_fp16_chain.md: 268.5 MB + 102.6 MB);
# traffic grows in proportion to the elements, so a full launch is this times its element count
Z_DRAM_BYTES_PER_ELEMENT = (268.459264e6 + 102.589184e6) / (1 << 26)


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


def _cpu_worker(args):
    """One host process: the numpy checker (restatement of NervanaCPU) on its column shard.
    Returns the wall-clock seconds of each of `reps` passes."""
    elements, reps, seed = args
    sys.path.insert(0, ROOT)
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
    return rows * cols, times


def cpu_port_rate(elements, reps, cores=None):
    """CPU baseline on a bounded sample.  NervanaCPU is single threaded (numpy ufuncs), but
    the path shards by columns, so the sample is split over `cores` processes that run at
    the same time -- the most the reference's CPU code can get out of this host.
    Returns (GB/s, seconds per pass, cores)."""
    cores = cores or max(1, len(os.sched_getaffinity(0)))
    per = max(4096, elements // cores)
    if cores == 1:
        results = [_cpu_worker((per, reps, 0))]
    else:
        import multiprocessing as mp
        with mp.get_context("spawn").Pool(cores) as pool:
            results = pool.map(_cpu_worker, [(per, reps, i) for i in range(cores)])
    n = sum(r[0] for r in results)
    # pass i is over when the slowest process finishes it
    per_pass = [max(r[1][i] for r in results) for i in range(reps)]
    best = min(per_pass)
    return n * BYTES_PER_ELEMENT / best / 1e9, best, cores


def run_reference(args, rank, world):
    """Reference arm: the CPU implementation of the path (numpy restatement of neon's
    NervanaCPU) on this box's host cores, one process per core."""
    if rank != 0:
        return
    sample = 1 << 26
    reps = args.warmup + args.steps
    t0 = time.perf_counter()
    cores = max(1, len(os.sched_getaffinity(0)))
    per = max(4096, sample // cores)
    if cores == 1:
        results = [_cpu_worker((per, reps, 0))]
    else:
        import multiprocessing as mp
        with mp.get_context("spawn").Pool(cores) as pool:
            results = pool.map(_cpu_worker, [(per, reps, i) for i in range(cores)])
    wall = time.perf_counter() - t0
    n = sum(r[0] for r in results)
    per_pass = [max(r[1][i] for r in results) for i in range(args.warmup, reps)]
    sec = float(np.mean(per_pass))
    gbs = n * BYTES_PER_ELEMENT / sec / 1e9
    line = {
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "rows": args.rows, "cols_per_gpu": args.cols,
                   "sample_elements_per_step": n},
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": cores, "kind": "port",
                         "sample": "%d of 2^30 elements per step split over %d processes, numpy restatement "
                                   "of NervanaCPU, fp16 inputs upcast to fp32" % (n, cores)},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "host_cores": os.cpu_count(), "wall_s": wall,
    }
    print(json.dumps(line))


def other_workloads(name, be, world, rank):
    """The remaining baseline configurations as (tensors, [(label, statement, algorithmic bytes)]).
    Sizes per GPU; with world > 1 the column (batch) axis is sharded and grows with world."""
    kw = {"parallel": True} if world > 1 else {}
    rng = np.random.RandomState(7 + rank)
    if name == "cfg1":
        r, c = 4096, 128
        a = be.array(rng.randn(r, c * world).astype(np.float32), **kw)
        b = be.array(rng.randn(r, c * world).astype(np.float32), **kw)
        bias = be.array(rng.uniform(-.5, .5, (r, 1)).astype(np.float32))
        out = be.empty((r, c * world), **kw)
        s = be.empty((1, c * world), **kw)
        m = be.empty((1, c * world), dtype=np.int32, **kw)

        def st_out(): out[:] = be.maximum(a * b + bias, 0)
        def st_sum(): s[:] = be.sum(out, axis=0)
        def st_arg(): m[:] = be.argmax(out, axis=0)
        n = r * c
        return [("bias+relu", st_out, 12 * n + 4 * r), ("sum axis0", st_sum, 4 * n + 4 * c),
                ("argmax axis0", st_arg, 4 * n + 4 * c)], n
    if name == "cfg2":
        r, c = 32000, 256
        x = be.array((3.0 * rng.randn(r, c * world)).astype(np.float32), **kw)
        y = be.empty((r, c * world), **kw)
        idx = be.empty((1, c * world), dtype=np.int32, **kw)

        def st_y():
            mx = be.max(x, axis=0)
            e = be.exp(x - mx)
            y[:] = e / be.sum(e, axis=0)
        def st_idx(): idx[:] = be.argmax(x, axis=0)
        n = r * c
        return [("softmax axis0", st_y, 8 * n), ("argmax axis0", st_idx, 4 * n + 4 * c)], n
    if name == "cfg3":
        n = 100000000
        shape = (100000, 1000 * world)
        from tests.cases import adam_step
        param = be.array((0.02 * rng.randn(*shape)).astype(np.float32), **kw)
        grad = be.array((1e-3 * rng.randn(*shape)).astype(np.float16), dtype=np.float16, **kw)
        mm, vv = be.zeros(shape, **kw), be.zeros(shape, **kw)
        be.bsz = 1
        step = [0]

        def st_adam():
            step[0] += 1
            adam_step(be, param, grad, mm, vv, step[0])
        return [("adam step (3 statements)", st_adam, 36 * n)], n
    if name == "cfg4":
        r, c = 256, 56 * 56 * 128
        x = be.array((1.0 + 2.0 * rng.randn(r, c * world)).astype(np.float16), dtype=np.float16, **kw)
        gamma = be.array(rng.uniform(.5, 1.5, (r, 1)).astype(np.float32))
        beta = be.array(rng.uniform(.5, 1.5, (r, 1)).astype(np.float32))
        y = be.empty((r, c * world), dtype=np.float16, **kw)

        def st_bn():
            y[:] = (x - be.mean(x, axis=1)) / be.sqrt(be.var(x, axis=1) + 1e-5) * gamma + beta
        n = r * c
        return [("batchnorm stats+normalise", st_bn, 4 * n + 2048)], n
    if name == "transpose":
        # the data-feed step in front of every fprop (ArrayIterator): (examples, features) rows
        # to (features, batch) columns; one large matrix each of fp32, fp16 and uint8
        stmts = []
        r, c = 8192, 8192
        for dt in (np.float32, np.float16, np.uint8):
            a = be.zeros((r, c), dtype=dt)
            out = be.empty((c, r), dtype=dt)
            stmts.append(("copy_transpose %s" % np.dtype(dt).name,
                          (lambda a=a, out=out: be.copy_transpose(a, out)), 2 * a.nbytes))
        return stmts, r * c
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


def run_other(args, be, rank, world, barrier, max_over_ranks):
    stmts, n_local = other_workloads(args.workload, be, world, rank)
    for _ in range(max(args.warmup, 3)):
        for _, fn, _ in stmts:
            fn()
    be.synchronize()
    marks = [[(be.init_mark(), be.init_mark()) for _ in stmts] for _ in range(args.steps)]
    ev0, ev1 = be.init_mark(), be.init_mark()
    log = be.launch_log = []
    launches0 = be.launches
    barrier()
    be.synchronize()
    be.record_mark(ev0)
    for s in range(args.steps):
        for i, (_, fn, _) in enumerate(stmts):
            be.record_mark(marks[s][i][0])
            fn()
            be.record_mark(marks[s][i][1])
    be.record_mark(ev1)
    be.synchronize()
    barrier()
    ms_total = max_over_ranks(be.get_time(ev0, ev1))
    launches = be.launches - launches0
    # the same sequence recorded once as a CUDA graph and replayed (single GPU only)
    graph_ms = None
    if world == 1 and hasattr(be, "capture"):
        be.launch_log = None

        def sequence():
            for _, fn, _ in stmts:
                fn()
        graph = be.capture(sequence)
        for _ in range(3):
            graph.replay()
        be.synchronize()
        be.record_mark(ev0)
        for s in range(args.steps):
            graph.replay()
        be.record_mark(ev1)
        be.synchronize()
        graph_ms = be.get_time(ev0, ev1) / args.steps
    # working sets that stay in L2 between steps: the same statements again with L2 flushed
    # (a 256 MiB fill) before each one, timed per statement so that the fill is not counted
    cold = None
    if world == 1 and n_local * 4 < 100e6:
        flush = be.empty((1 << 26, 1))
        cold_marks = [[(be.init_mark(), be.init_mark()) for _ in stmts] for _ in range(args.steps)]
        for s in range(args.steps):
            for i, (_, fn, _) in enumerate(stmts):
                flush.fill(0)
                be.record_mark(cold_marks[s][i][0])
                fn()
                be.record_mark(cold_marks[s][i][1])
        be.synchronize()
        cold_ms = sum(float(np.median([be.get_time(*cold_marks[s][i]) for s in range(args.steps)]))
                      for i in range(len(stmts)))
        cold = {"ms_per_step": cold_ms, "GBps": sum(b for _, _, b in stmts) / cold_ms / 1e6,
                "note": "L2 flushed (256 MiB fill) before every statement; sum of per-statement medians"}
    if rank != 0:
        return
    per = []
    for i, (label, _, nbytes) in enumerate(stmts):
        ms = float(np.median([be.get_time(*marks[s][i]) for s in range(args.steps)]))
        per.append({"statement": label, "ms": ms, "algorithmic_bytes": nbytes, "GBps": nbytes / ms / 1e6})
    nbytes_step = sum(b for _, _, b in stmts) * world
    ms_step = ms_total / args.steps
    peak_gbs, peak_kind = measured_peak()
    value = nbytes_step / ms_step / 1e6
    kinds = log[: launches // args.steps]
    print(json.dumps({
        "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "elements_per_gpu": n_local,
                   "l2": "working set is L2-resident between steps" if n_local * 4 < 100e6 else "exceeds L2"},
        "pct_of_measured_peak_per_gpu": 100.0 * value / world / peak_gbs, "peak_kind": peak_kind,
        "statements": per, "gpu_launches": launches,
        "cold": cold,
        "graph_replay": None if graph_ms is None else {
            "ms_per_step": graph_ms, "GBps": nbytes_step / graph_ms / 1e6,
            "note": "statement sequence recorded once with be.capture(), replayed with one call"},
        "launches_per_step": [k for k, _ in kinds]}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--rows", type=int, default=ROWS)
    ap.add_argument("--cols", type=int, default=COLS)
    ap.add_argument("--e2e-steps", type=int, default=3)
    ap.add_argument("--no-cpu", action="store_true")
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
        barrier, max_over_ranks = be.host_barrier, be.host_max
    else:
        from neon_b200 import gen_backend
        be = gen_backend(backend="b200", rng_seed=0, device_id=local_rank)
        barrier, max_over_ranks = (lambda: None), (lambda v: v)

    if args.workload != "cfg5":
        return run_other(args, be, rank, world, barrier, max_over_ranks)

    rows, cols = args.rows, args.cols
    n_local = rows * cols
    # pinned host copies of this rank's shard (also the source of the e2e copies)
    nbytes = n_local * 2
    hx_p, hy_p = rt.host_alloc(nbytes), rt.host_alloc(nbytes)
    import ctypes
    hx = np.frombuffer((ctypes.c_char * nbytes).from_address(hx_p), dtype=np.float16).reshape(rows, cols)
    hy = np.frombuffer((ctypes.c_char * nbytes).from_address(hy_p), dtype=np.float16).reshape(rows, cols)
    fill_uniform_f16(hx, 100 + rank)
    fill_uniform_f16(hy, 200 + rank)

    kw = {"parallel": True} if world > 1 else {}
    gshape = (rows, cols * world)
    x = be.empty(gshape, dtype=np.float16, **kw)
    y = be.empty(gshape, dtype=np.float16, **kw)
    z = be.empty(gshape, dtype=np.float16, **kw)
    z.rounding = True
    total, peak = be.empty((1, 1)), be.empty((1, 1))
    rt.memcpy_h2d(x.ptr, hx_p, nbytes, be.stream, sync=True)
    rt.memcpy_h2d(y.ptr, hy_p, nbytes, be.stream, sync=True)

    for _ in range(max(args.warmup, 3)):
        statements(be, x, y, z, total, peak)
    be.synchronize()

    # ---- timed region: K steps, inputs resident in HBM (4 GiB of inputs per step >> L2)
    ev0, ev1 = be.init_mark(), be.init_mark()
    kz = [(be.init_mark(), be.init_mark()) for _ in range(args.steps)]
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    launches0 = be.launches
    barrier()
    be.synchronize()
    be.record_mark(ev0)
    for s in range(args.steps):
        be.record_mark(kz[s][0])
        z[:] = be.tanh(x) * be.sqrt(be.absolute(y)) + 0.5 * x * y
        be.record_mark(kz[s][1])
        total[:] = be.sum(z)
        peak[:] = be.max(be.absolute(z))
    be.record_mark(ev1)
    be.synchronize()
    barrier()
    ms_total = max_over_ranks(be.get_time(ev0, ev1))
    launches = be.launches - launches0
    z_ms = float(np.mean([be.get_time(a, b) for a, b in kz]))
    res_total, res_peak = float(total.get()[0, 0]), float(peak.get()[0, 0])

    # ---- end to end: host buffers in, host scalars out, every step
    e2e_steps = max(1, args.e2e_steps)
    barrier()
    be.synchronize()
    be.record_mark(ev0)
    for s in range(e2e_steps):
        rt.memcpy_h2d(x.ptr, hx_p, nbytes, be.stream, sync=False)
        rt.memcpy_h2d(y.ptr, hy_p, nbytes, be.stream, sync=False)
        statements(be, x, y, z, total, peak)
        total.get()
        peak.get()
    be.record_mark(ev1)
    be.synchronize()
    barrier()
    e2e_ms = max_over_ranks(be.get_time(ev0, ev1))
    clocks = sampler.stop() if rank == 0 else None      # sampled over both timed regions

    if rank != 0:
        return
    n_global = n_local * world
    ms_step = ms_total / args.steps
    value = n_global * BYTES_PER_ELEMENT / (ms_step * 1e-3) / 1e9
    e2e_value = n_global * BYTES_PER_ELEMENT / (e2e_ms / e2e_steps * 1e-3) / 1e9
    peak_gbs, peak_kind = measured_peak()
    z_gbs = n_local * Z_BYTES_PER_ELEMENT / (z_ms * 1e-3) / 1e9
    line = {
        "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD,
                   "rows": rows, "cols_per_gpu": cols, "elements_per_gpu": n_local,
                   "sharding": "columns" if world > 1 else "none",
                   "l2": "inputs (4 GiB per step) exceed L2; no flush needed",
                   "algorithmic_bytes_per_element": BYTES_PER_ELEMENT},
        "elements_per_s": n_global / (ms_step * 1e-3),
        "pct_of_8TBps_per_gpu": 100.0 * value / world / 8000.0,
        "roofline": {"bound": "hbm", "kernel": "ew_flat (z statement)", "achieved": z_gbs,
                     "peak": peak_gbs, "peak_kind": peak_kind, "unit": "GB/s",
                     "frac": z_gbs / peak_gbs, "ms_per_launch": z_ms,
                     "algorithmic_bytes_per_launch": n_local * Z_BYTES_PER_ELEMENT, "traffic": None},
        "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": 2 * nbytes,
                "d2h_bytes_per_step": 8, "steps": e2e_steps, "ms_per_step": e2e_ms / e2e_steps},
        "gpu_launches": launches, "clocks": clocks,
        "results": {"total": res_total, "peak": res_peak},
    }
    if Z_DRAM_BYTES_PER_ELEMENT is not None:
        line["roofline"]["traffic"] = Z_DRAM_BYTES_PER_ELEMENT * n_local
    if not args.no_cpu:
        gbs, sec, cores = cpu_port_rate(1 << 26, 8)
        line["cpu_baseline"] = {"value": gbs, "unit": "GB/s", "cores": cores, "kind": "port",
                                "sample": "2^26 of 2^30 elements split over %d processes, best of 8 passes "
                                          "(%.2f s each), numpy restatement of NervanaCPU, fp16 inputs "
                                          "upcast to fp32" % (cores, sec)}
    print(json.dumps(line))


if __name__ == "__main__":
    main()
