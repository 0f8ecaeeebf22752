#!/usr/bin/env python
"""Benchmark of the array hot path on B200.

A step is one pass of the sharded workload over one batch of synthetic input: every GPU holds a
contiguous shard of 2^30 Float32 elements of x, y, z (U[-1,1), counter-based generator, seed 4)
and runs  r .= x .* y .+ exp.(-abs.(z))  followed by  sum(abs2, r)  whose one-element partial is
all-reduced inside the reduction kernel.  With 8 GPUs that is the 2^33-element configuration;
per-GPU work is fixed as N grows (weak scaling; --scaling strong splits 2^33 over the GPUs
instead).  The metric is achieved HBM bandwidth in GB/s: algorithmic bytes (16 B/element for the
broadcast + 4 B/element for the reduction) over the device time of the step, maximum over ranks.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--no-suite]
                    [--scaling weak|strong] [--collective fused|nccl|none] [--transport host|vmm|ipc]

For N > 1 launch through torchrun (one rank per GPU); rank 0 prints ONE JSON line.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))
import __graft_entry__ as entry  # noqa: E402

BYTES_PER_ELEM = 16 + 4          # broadcast: 3 reads + 1 write; reduction: 1 read
# DRAM bytes per element of the broadcast kernel from its ncu capture on a 2^28-element launch
# (dram__bytes_read.sum 3221.3 MB + dram__bytes_write.sum 1043.6 MB for 2^28 elements; the reads are
# exactly the three inputs, 2.7 % of the output was still dirty in L2 when the kernel ended); traffic
# grows in proportion to the element count, so a launch over n elements moves this many bytes per
# element.
EW_TRAFFIC_BYTES_PER_ELEM = 4265.96e6 / (1 << 28)
NOMINAL_HBM_GBS = 8000.0


def measured_peak() -> tuple[float, str]:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()          # the exact process started above
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        sm, smax, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0])); smax.append(float(parts[1]))
            except ValueError:
                continue
            for nm, v in zip(names, parts[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "samples": len(sm), "reasons": sorted(reasons)}


class Dist:
    """Host-side plumbing between ranks (gloo): id exchange, barrier, max over ranks."""

    def __init__(self, rank, world):
        self.rank, self.world, self.dist = rank, world, None
        if world > 1:
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            import torch.distributed as dist
            dist.init_process_group("gloo", init_method="env://", rank=rank, world_size=world)
            self.dist = dist

    def exchange(self, payload):
        if self.dist is None:
            return payload
        box = [payload]
        self.dist.broadcast_object_list(box, src=0)
        return box[0]

    def barrier(self):
        if self.dist is not None:
            self.dist.barrier()

    def max(self, v: float) -> float:
        if self.dist is None:
            return v
        import torch
        t = torch.tensor([v], dtype=torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t[0])

    def allgather(self, payload):
        if self.dist is None:
            return [payload]
        out = [None] * self.world
        self.dist.all_gather_object(out, payload)
        return out

    def close(self):
        if self.dist is not None:
            self.dist.destroy_process_group()


def time_loop(pkg, stream, fn, reps: int) -> float:
    """Average milliseconds of `fn` over `reps` back-to-back calls, CUDA events on `stream`."""
    a, b = pkg.Event(stream.device, timing=True), pkg.Event(stream.device, timing=True)
    for _ in range(min(3, reps)):      # untimed: module load, scratch growth, clock ramp
        fn()
    stream.synchronize()
    a.record(stream)
    for _ in range(reps):
        fn()
    b.record(stream)
    b.synchronize()
    return pkg.elapsed_ms(a, b) / reps


def run_suite(pkg, peak: float, only: str | None = None, shrink: int = 0, reps_scale: float = 1.0) -> dict:
    """Single-GPU numbers for the other configurations (kernel time, inputs resident in HBM;
    64 MiB cases rotate over four buffer sets so that they cannot be served from L2).
    `only` selects the cases whose name starts with it; `shrink` divides every size by 2^shrink
    (small cases for profiler captures)."""
    R, st = pkg.random, pkg.current_stream()
    out = {}
    i = [0]

    def want(name):
        return only is None or name.startswith(only) or only.startswith(name)

    def reps(k):
        return max(1, int(k * reps_scale))

    def rec(name, bytes_, ms, extra=None):
        gbs = bytes_ / ms / 1e6
        out[name] = {"ms": round(ms, 4), "GB/s": round(gbs, 1), "frac_of_8TBs": round(gbs / NOMINAL_HBM_GBS, 3),
                     "frac_of_measured_copy": round(gbs / peak, 3)}
        if extra:
            out[name].update(extra)

    def rotate(calls):
        def go():
            calls[i[0] % len(calls)](); i[0] += 1
        return go

    # config 1: 2^24 Float32 vectors.  Descriptors are prepared once: these kernels run for
    # 10-30 us, a fresh flattening of the expression in Python would be timed instead of them.
    if want("c1"):
        n = (1 << 24) >> shrink
        sets = [[R.fill_random_(pkg.ROCArray(np.float32, n), R.UNIFORM01, seed=0, stream_id=4 * s + k) for k in range(2)]
                + [pkg.ROCArray(np.float32, n)] for s in range(4)]
        a = np.float32(2.5)
        if want("c1_axpy"):
            rec("c1_axpy_2p24_f32", 12 * n, time_loop(pkg, st, rotate([pkg.broadcast.prepared(z, a * x.dot + y.dot) for x, y, z in sets]), reps(200)))
        rs = pkg.ROCArray(np.float32, 1)
        if want("c1_sum"):
            rec("c1_sum_2p24_f32", 4 * n, time_loop(pkg, st, rotate([pkg.mapreduce_prepared("identity", "+", rs, x, init=np.float32(0)) for x, _, _ in sets]), reps(200)))
        if want("c1_cumsum"):
            rec("c1_cumsum_2p24_f32", 8 * n, time_loop(pkg, st, rotate([pkg.accumulate_prepared("+", z, x) for x, _, z in sets]), reps(200)))
        del sets
    # expressions the hard-wired kernels do not match: how fast an arbitrary fused broadcast runs,
    # with the evaluator specialised for the expression at run time (the default) and interpreted
    if want("gen"):
        n = (1 << 26) >> shrink
        xs = [R.fill_random_(pkg.ROCArray(np.float32, n), R.UNIFORM11, seed=4, stream_id=k) for k in range(3)]
        out_ = pkg.ROCArray(np.float32, n)
        bcm = pkg.broadcast
        xi = R.fill_random_(pkg.ROCArray(np.int32, n), R.INTEGERS, seed=2, lo=-100, hi=100)
        outd = pkg.ROCArray(np.float64, n)
        trees = (("x*y+exp(-abs(z))+c_2p26_f32", out_, lambda: xs[0].dot * xs[1].dot + bcm.exp(-bcm.abs_(xs[2])) + np.float32(0.25)),
                 ("max(x-y,2z)_2p26_f32", out_, lambda: bcm.maximum(xs[0].dot - xs[1].dot, xs[2].dot * np.float32(2))),
                 ("i32*f32->f64_2p26", outd, lambda: xi.dot * xs[0].dot * 1.5))
        for mode, on in (("specialised", True), ("interpreted", False)):
            bcm.jit_configure(on)
            try:
                for name, dest, tree in trees:
                    rec(f"gen_{mode}_{name}", 16 * n, time_loop(pkg, st, pkg.broadcast.prepared(dest, tree()), reps(20)))
            finally:
                bcm.jit_configure(True)
        # a reduction over a two-operand map expression (dot product): 8 B per element
        r1 = pkg.ROCArray(np.float32, 1)
        for mode, on in (("specialised", True), ("interpreted", False)):
            bcm.jit_configure(on)
            try:
                rec(f"gen_{mode}_sum(x.*y)_2p26_f32", 8 * n,
                    time_loop(pkg, st, pkg.mapreduce_prepared(None, "+", r1, xs[0].dot * xs[1].dot, init=np.float32(0)), reps(20)))
            finally:
                bcm.jit_configure(True)
        out["gen_runtime_compiler"] = bcm.jit_stats()
        del xs, out_, xi, outd
    # config 2: 8192 x 8192 matrices
    if want("c2"):
        m = 8192 >> (shrink // 2)
        import ml_dtypes
        for dt, tag in ((np.float32, "f32"), (np.float16, "f16"), (ml_dtypes.bfloat16, "bf16")):
            if not any(want(f"c2_{k}_8192_{tag}") for k in ("sum_dims1", "max_dims2", "sumsq")):
                continue
            mats = [R.fill_random_(pkg.ROCArray(dt, (m, m)), R.NORMAL, seed=1, stream_id=s) for s in range(2)]
            r1, r2, r0 = pkg.ROCArray(np.float32, (1, m)), pkg.ROCArray(dt, (m, 1)), pkg.ROCArray(np.float32, (1, 1))
            zero, ninf = np.float32(0), np.dtype(dt).type(-np.inf)
            nb = m * m * np.dtype(dt).itemsize
            if want(f"c2_sum_dims1_8192_{tag}"):
                rec(f"c2_sum_dims1_8192_{tag}", nb, time_loop(pkg, st, rotate([pkg.mapreduce_prepared("identity", "+", r1, A, init=zero) for A in mats]), reps(50)))
            if want(f"c2_max_dims2_8192_{tag}"):
                rec(f"c2_max_dims2_8192_{tag}", nb, time_loop(pkg, st, rotate([pkg.mapreduce_prepared("identity", "max", r2, A, init=ninf) for A in mats]), reps(50)))
            if want(f"c2_sumsq_8192_{tag}"):
                rec(f"c2_sumsq_8192_{tag}", nb, time_loop(pkg, st, rotate([pkg.mapreduce_prepared("abs2", "+", r0, A, init=zero) for A in mats]), reps(50)))
            del mats
    # scans along one dimension of a matrix (the shapes of the reference's own accumulate benchmarks,
    # perf/array.jl:70-85, at B200 size): 8 B per element
    if want("mat_cumsum"):
        m = 8192 >> (shrink // 2)
        A = R.fill_random_(pkg.ROCArray(np.float32, (m, m)), R.UNIFORM01, seed=2)
        Bm = pkg.ROCArray(np.float32, (m, m))
        for d in (1, 2):
            rec(f"mat_cumsum_dims{d}_8192_f32", 8 * m * m, time_loop(pkg, st, pkg.accumulate_prepared("+", Bm, A, dims=d), reps(10)))
        del A, Bm
    # the reference's own benchmark shapes (perf/array.jl:1-17,67-120,144-145): 512 x 1000 and
    # 3 x 1 000 000 Float32 / Int64.  Latency-bound sizes; reported as time per call.  The one number
    # the reference's tree holds for this set: accumulate(+, 3x1e6 Float32; dims=1) 70.5 us on gfx1100.
    if want("ref"):
        def lat(name, fn, bytes_):
            ms = time_loop(pkg, st, fn, reps(200))
            out[name] = {"us": round(ms * 1e3, 2), "GB/s": round(bytes_ / ms / 1e6, 1)}
        for dt, tag in ((np.float32, "f32"), (np.int64, "i64")):
            isz = np.dtype(dt).itemsize
            def gen(shape):
                a = pkg.ROCArray(dt, shape)
                if dt == np.float32:
                    return R.fill_random_(a, R.UNIFORM01, seed=7)
                return R.fill_random_(a, R.INTEGERS, seed=7, lo=-10, hi=10)
            mat, lng = gen((512, 1000)), gen((3, 1_000_000))
            vec = mat.reshape(512_000)
            o_mat, o_lng, o_vec = pkg.ROCArray(dt, (512, 1000)), pkg.ROCArray(dt, (3, 1_000_000)), pkg.ROCArray(dt, 512_000)
            lat(f"ref_accumulate_1d_{tag}", pkg.accumulate_prepared("+", o_vec, vec), 2 * isz * 512_000)
            for d in (1, 2):
                lat(f"ref_accumulate_512x1000_dims{d}_{tag}", pkg.accumulate_prepared("+", o_mat, mat, dims=d), 2 * isz * 512_000)
                lat(f"ref_accumulate_3x1e6_dims{d}_{tag}", pkg.accumulate_prepared("+", o_lng, lng, dims=d), 2 * isz * 3_000_000)
            rdt = dt
            r0 = pkg.ROCArray(rdt, (1, 1))
            lat(f"ref_reduce_1d_{tag}", pkg.mapreduce_prepared("identity", "+", pkg.ROCArray(rdt, 1), vec, init=dt(0)), isz * 512_000)
            lat(f"ref_reduce_512x1000_dims1_{tag}", pkg.mapreduce_prepared("identity", "+", pkg.ROCArray(rdt, (1, 1000)), mat, init=dt(0)), isz * 512_000)
            lat(f"ref_reduce_512x1000_dims2_{tag}", pkg.mapreduce_prepared("identity", "+", pkg.ROCArray(rdt, (512, 1)), mat, init=dt(0)), isz * 512_000)
            lat(f"ref_reduce_3x1e6_dims1_{tag}", pkg.mapreduce_prepared("identity", "+", pkg.ROCArray(rdt, (1, 1_000_000)), lng, init=dt(0)), isz * 3_000_000)
            lat(f"ref_reduce_3x1e6_dims2_{tag}", pkg.mapreduce_prepared("identity", "+", pkg.ROCArray(rdt, (3, 1)), lng, init=dt(0)), isz * 3_000_000)
            lat(f"ref_mapreduce_x+1_1d_{tag}", pkg.mapreduce_prepared(None, "+", r0.reshape(1), vec.dot + dt(1), init=dt(0)), isz * 512_000)
            if dt == np.float32:
                lat("ref_broadcast_fill_512x1000_f32", pkg.broadcast.prepared(o_mat, np.float32(0)), isz * 512_000)
                keys = pkg.ROCArray(dt, 512_000)
                def sort_once(_k=keys, _v=vec):
                    pkg.copyto_(_k, _v); pkg.sort_(_k)
                lat("ref_sort_512000_f32(copy+sort)", sort_once, 2 * isz * 512_000)
            del mat, lng, vec, o_mat, o_lng, o_vec
    # config 3: 2^28 scans
    if want("c3") or want("c4_sort"):
        n = (1 << 28) >> shrink
        v = R.fill_random_(pkg.ROCArray(np.int32, n), R.INTEGERS, seed=2, lo=-100, hi=100)
        o = pkg.ROCArray(np.int32, n)
        if want("c3_scan_2p28_i32"):
            rec("c3_scan_2p28_i32", 8 * n, time_loop(pkg, st, pkg.accumulate_prepared("+", o, v), reps(10)))
        if want("c3_scan_2p28_f32"):
            vf, of = v.reinterpret(np.float32), o.reinterpret(np.float32)
            R.fill_random_(vf, R.UNIFORM01, seed=2, stream_id=1)
            rec("c3_scan_2p28_f32", 8 * n, time_loop(pkg, st, pkg.accumulate_prepared("+", of, vf), reps(10)))
        # config 4: radix sort (keys are copied back before every timed sort: it sorts in place)
        if want("c4_sort"):
            keys = R.fill_random_(v.reinterpret(np.uint32), R.RAWBITS, seed=3)
            work = o.reinterpret(np.uint32)
            ts = []
            for _ in range(reps(5) + 1):
                pkg.copyto_(work, keys)
                ts.append(time_loop(pkg, st, lambda: pkg.sort_(work), 1))
            ms = min(ts[1:]) if len(ts) > 1 else ts[0]
            out["c4_sort_2p28_u32"] = {"ms": round(ms, 3), "Gkeys/s": round(n / ms / 1e6, 2), "model_GB/s": round(36 * n / ms / 1e6, 1),
                                       "frac_of_8TBs_model36B": round(36 * n / ms / 1e6 / NOMINAL_HBM_GBS, 3)}
        del v, o
    # the consumers of the scan and of the sort (the "next" rows around the path): findall, logical
    # indexing, reverse, x[ix]; algorithmic bytes = inputs read once + outputs written once
    if want("next"):
        n = (1 << 26) >> shrink
        rng = np.random.default_rng(6)
        mask_h = rng.random(n) < 0.5
        nnz = int(mask_h.sum())
        mask = pkg.ROCArray.from_host(mask_h)
        xs = R.fill_random_(pkg.ROCArray(np.float32, n), R.UNIFORM01, seed=6)
        def timed_alloc(fn, k):
            def go():
                fn().unsafe_free_()
            return time_loop(pkg, st, go, reps(k))
        rec("next_findall_2p26_bool", n + 8 * nnz, timed_alloc(lambda: pkg.findall(mask), 10))
        rec("next_getindex_mask_2p26_f32", 5 * n + 4 * nnz, timed_alloc(lambda: pkg.getindex_mask(xs, mask), 10))
        rec("next_reverse_2p26_f32", 8 * n, timed_alloc(lambda: pkg.reverse(xs), 10))
        perm = pkg.sortperm(R.fill_random_(pkg.ROCArray(np.float32, n), R.UNIFORM01, seed=7))
        rec("next_getindex_perm_2p26_f32", 16 * n, timed_alloc(lambda: pkg.getindex(xs, perm), 10))
        del mask, xs, perm
        # wrapped operands: a transposed matrix as source of a copy and as operand of a fused expression
        m = 8192 >> (shrink // 2)
        A = R.fill_random_(pkg.ROCArray(np.float32, (m, m)), R.UNIFORM01, seed=8)
        Bm = R.fill_random_(pkg.ROCArray(np.float32, (m, m)), R.UNIFORM01, seed=9)
        Cm = pkg.ROCArray(np.float32, (m, m))
        rec("next_copy_transpose_8192_f32", 8 * m * m, time_loop(pkg, st, lambda: pkg.copyto_(Cm, A.transpose()), reps(5)))
        rec("next_add_transpose_8192_f32", 12 * m * m, time_loop(pkg, st, pkg.broadcast.prepared(Cm, A.dot + Bm.transpose().dot), reps(5)))
        del A, Bm, Cm
    # yardsticks only: the vendor library kernels torch ships (CUB scan / radix sort, its own
    # reductions) on the same sizes, timed the same way on torch's stream.  Not part of any path
    # of this library; they say what "good" is on this box.
    if want("yardstick"):
        try:
            import torch
            dev = torch.device("cuda", pkg.current_device())
            def ttime(fn, reps_):
                for _ in range(3):
                    fn()
                torch.cuda.synchronize(dev)
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(reps_):
                    fn()
                e1.record()
                e1.synchronize()
                return e0.elapsed_time(e1) / reps_
            with torch.cuda.device(dev):
                n28 = (1 << 28) >> shrink
                xi = torch.randint(-100, 101, (n28,), dtype=torch.int32, device=dev)
                ms = ttime(lambda: torch.cumsum(xi, 0, dtype=torch.int32), reps(10))
                out["yardstick_torch_cumsum_2p28_i32"] = {"ms": round(ms, 4), "GB/s": round(8 * n28 / ms / 1e6, 1)}
                xf = torch.rand(n28, dtype=torch.float32, device=dev)
                ms = ttime(lambda: torch.sum(xf), reps(10))
                out["yardstick_torch_sum_2p28_f32"] = {"ms": round(ms, 4), "GB/s": round(4 * n28 / ms / 1e6, 1)}
                ms = ttime(lambda: torch.cumsum(xf, 0), reps(10))
                out["yardstick_torch_cumsum_2p28_f32"] = {"ms": round(ms, 4), "GB/s": round(8 * n28 / ms / 1e6, 1)}
                del xf
                keys = xi.view(torch.int32)
                ms = ttime(lambda: torch.sort(keys), reps(3))
                out["yardstick_torch_sort_2p28_i32(keys+indices)"] = {"ms": round(ms, 3), "Gkeys/s": round(n28 / ms / 1e6, 2)}
                del xi, keys
                # the 2^24 cases, rotating over four buffer sets like the c1 cases above
                n24 = (1 << 24) >> shrink
                sets24 = [(torch.rand(n24, dtype=torch.float32, device=dev), torch.rand(n24, dtype=torch.float32, device=dev),
                           torch.empty(n24, dtype=torch.float32, device=dev)) for _ in range(4)]
                k = [0]
                def nxt():
                    k[0] += 1
                    return sets24[k[0] % 4]
                def t_axpy():
                    x_, y_, z_ = nxt()
                    torch.add(y_, x_, alpha=2.5, out=z_)
                def t_sum():
                    torch.sum(nxt()[0])
                def t_cumsum():
                    x_, _, z_ = nxt()
                    torch.cumsum(x_, 0, out=z_)
                for name, fn_, nb in (("axpy", t_axpy, 12), ("sum", t_sum, 4), ("cumsum", t_cumsum, 8)):
                    ms = ttime(fn_, reps(200))
                    out[f"yardstick_torch_{name}_2p24_f32"] = {"ms": round(ms, 4), "GB/s": round(nb * n24 / ms / 1e6, 1)}
                del sets24
                torch.cuda.empty_cache()
        except Exception as e:                      # no torch CUDA build on this box: no yardstick
            out["yardstick_torch"] = {"unavailable": str(e)[:200]}
    if want("c4_sortperm"):
        m2 = (1 << 26) >> shrink
        f = R.fill_random_(pkg.ROCArray(np.float32, m2), R.NORMAL_DUP1PCT, seed=3, hi=m2)
        ix = pkg.ROCArray(np.int64, m2)
        pkg.sortperm_(ix, f)
        ms = min(time_loop(pkg, st, lambda: pkg.sortperm_(ix, f), 1) for _ in range(reps(4)))
        out["c4_sortperm_2p26_f32"] = {"ms": round(ms, 3), "Gkeys/s": round(m2 / ms / 1e6, 2)}
    return out


METRIC = "achieved HBM GB/s (algorithmic bytes / time), fused broadcast + sum(abs2) with allreduce"
CPU_SAMPLE_LOG2 = 26


def host_threads() -> int:
    """Threads this process may run on.  (torchrun exports OMP_NUM_THREADS=1, so the OpenMP default
    is not the number to use; the count is passed to every parallel region explicitly.)"""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def cpu_reference_step(n_sample: int, steps: int, warmup: int, threads: int) -> float:
    """Seconds per step of the CPU arm: the same step (fused broadcast, then sum of squares) by the
    C restatement of Base's loops on `threads` host threads, over a bounded sample of the shard."""
    entry.load_oracle()
    from b200_oracle import c_oracle as co   # noqa: E402
    lib = co.load()
    rng = np.random.default_rng(4)
    x, y, z = (rng.random(n_sample, dtype=np.float32) * 2 - 1 for _ in range(3))
    r = np.empty_like(x)
    px, py, pz, pr = (co.ptr(v, C.c_float) for v in (x, y, z, r))

    def step():
        lib.ora_muladd_exp_f32(px, py, pz, pr, n_sample, threads)
        return lib.ora_sum_f32(pr, n_sample, 1, threads)
    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    return (time.perf_counter() - t0) / steps


def numpy_reference_step(n_sample: int, steps: int) -> float:
    """Second yardstick: the same step written with NumPy array expressions (temporaries and all)."""
    rng = np.random.default_rng(4)
    x, y, z = (rng.random(n_sample, dtype=np.float32) * 2 - 1 for _ in range(3))
    def step():
        r = x * y + np.exp(-np.abs(z))
        return float(np.sum(r * r, dtype=np.float32))
    step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    return (time.perf_counter() - t0) / steps


def cpu_baseline(steps: int, warmup: int) -> dict:
    """The CPU numbers that stand beside the GPU line: all host threads (the `value`), one thread,
    and NumPy; one protocol wherever it is reported."""
    n_sample = 1 << CPU_SAMPLE_LOG2
    threads = host_threads()
    gbs = lambda dt: round(BYTES_PER_ELEM * n_sample / dt / 1e9, 3)
    dt_all = cpu_reference_step(n_sample, steps, warmup, threads)
    dt_one = cpu_reference_step(n_sample, max(1, min(steps, 5)), 1, 1)
    dt_np = numpy_reference_step(n_sample, max(1, min(steps, 3)))
    return {"value": gbs(dt_all), "unit": "GB/s", "cores": threads, "kind": "port",
            "sample": f"2^{CPU_SAMPLE_LOG2}-element slice of the shard per step, {steps} steps after {warmup} warm-ups; "
                      "Julia Base cannot run on this box, this is its C restatement (oracle/base_oracle.c, OpenMP)",
            "all_threads": {"value": gbs(dt_all), "threads": threads, "ms_per_step": round(dt_all * 1e3, 3)},
            "single_thread": {"value": gbs(dt_one), "threads": 1, "ms_per_step": round(dt_one * 1e3, 3)},
            "numpy": {"value": gbs(dt_np), "threads": "numpy default", "ms_per_step": round(dt_np * 1e3, 3)},
            "julia_base": "unavailable on this box"}


def sharded_scan_record(pkg, dist, rank, world, local_rank, st, log2_elems: int = 27) -> dict:
    """Sharded inclusive scan of Int32 (the exclusive prefix of the per-shard totals seeds every
    rank's local scan): timed with events, checked exactly.  Every rank regenerates its own shard on
    the host, the shard totals travel over the host channel, so each rank knows the value its last
    element must have and can compare a stretch of its output bit for bit."""
    R = pkg.random
    n = 1 << log2_elems
    first = rank * n
    shard = R.fill_random_(pkg.ROCArray(np.int32, n), R.INTEGERS, seed=2, first_index=first, lo=-100, hi=100)
    out = pkg.ROCArray(np.int32, n)
    comm = None
    if world > 1:
        comm = pkg.sharded.init_comm(rank, world, local_rank, dist.exchange)
    ops = pkg.sharded.ShardedOps(pkg.sharded.DeviceBackend(comm, world, stream=st), rank, world)
    try:
        ops.accumulate("+", out, shard, timeout=60.0 if world > 1 else None)
        st.synchronize()
        dist.barrier()
        reps = 5
        a, b = pkg.Event(timing=True), pkg.Event(timing=True)
        a.record(st)
        for _ in range(reps):
            ops.accumulate("+", out, shard)
        b.record(st)
        b.synchronize()
        ms = dist.max(pkg.elapsed_ms(a, b) / reps)
        # the check: host totals of every shard -> the carry of this rank -> exact comparison
        host = np.empty(n, dtype=np.int32)
        blk = 1 << 22
        for s in range(0, n, blk):
            host[s:s + blk] = R.host_integers(2, 0, first + s, blk, -100, 100)
        totals = dist.allgather(int(host.sum(dtype=np.int64)))
        carry = sum(totals[:rank])
        wrap = lambda v: np.int64(v).astype(np.int32)
        last = int(out.view(n - 1, n).to_host()[0])
        head = out.view(0, 1 << 20).to_host()
        want_head = (np.cumsum(host[:1 << 20], dtype=np.int64) + carry).astype(np.int32)
        ok = last == int(wrap(carry + totals[rank])) and np.array_equal(head, want_head)
        exact = all(dist.allgather(bool(ok)))
    finally:
        pkg.device_synchronize()
        dist.barrier()
        if comm is not None:
            pkg.sharded.destroy_comm(comm)
    return {"elements_per_gpu": n, "dtype": "Int32", "ms": round(ms, 4), "GB/s": round(8 * n * world / ms / 1e6, 1),
            "exact": bool(exact), "method": "local totals -> all-gather of one element per rank -> carry folded on the device -> seeded local scan"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-suite", action="store_true", help="skip the per-configuration kernel numbers")
    ap.add_argument("--collective", default="fused", choices=["fused", "nccl", "none"],
                    help="fused: reduction and all-reduce in one kernel over exchange slots all ranks can write; nccl: reduction "
                         "kernel, then ncclAllReduce on the same stream; none: diagnostic, ranks run their shards without any exchange")
    ap.add_argument("--transport", default=None, choices=["host", "vmm", "ipc"],
                    help="where the fused exchange keeps its slots (default: B200_PEER_TRANSPORT or the library default)")
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"],
                    help="weak: 2^LOG2_ELEMS elements per GPU at every N; strong: 2^33 elements in total, split over the GPUs "
                         "(at N=1: 2^33 when at least 140 GiB are free, else 2^32)")
    ap.add_argument("--case", default=None, help="run only the suite cases whose name starts with this (e.g. c3_scan) and print them")
    ap.add_argument("--shrink", type=int, default=0, help="with --case: divide the sizes by 2^SHRINK (small cases for profiler captures)")
    ap.add_argument("--reps-scale", type=float, default=1.0, help="with --case: scale the repetition counts")
    ap.add_argument("--log2-elems", type=int, default=int(os.environ.get("B200_BENCH_LOG2_ELEMS", "30")),
                    help="log2 of the elements per GPU in weak mode (30 = the 2^33 / 8-GPU configuration)")
    args = ap.parse_args()
    rank, world, local_rank = (int(os.environ.get(k, d)) for k, d in (("RANK", "0"), ("WORLD_SIZE", "1"), ("LOCAL_RANK", "0")))
    warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    def workload_text(log2_per_gpu, total_log2):
        return (f"config5: r .= x.*y .+ exp.(-abs.(z)); sum(abs2, r) all-reduced over the ranks; Float32, U[-1,1), "
                f"2^{log2_per_gpu} elements per GPU, 2^{total_log2} in total ({args.scaling} scaling; the stated "
                f"configuration is 2^33 in total)")

    if args.impl == "reference":
        if rank != 0:
            return
        steps = max(1, args.steps)
        cpu = cpu_baseline(steps, args.warmup)
        val = cpu["value"]
        lg = args.log2_elems
        line = {"impl": "reference", "metric": METRIC,
                "value": val, "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": cpu["all_threads"]["ms_per_step"], "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None,
                "dtype": "f32", "data": "synthetic",
                "config": {"workload": workload_text(lg, lg + max(0, (world - 1).bit_length())),
                           "sample": f"2^{CPU_SAMPLE_LOG2} elements per step on the host ({cpu['cores']} threads)"},
                "cpu_baseline": cpu,
                "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line), flush=True)
        return

    pkg = entry.load_package()
    if not pkg.functional():
        raise SystemExit("bench.py needs a CUDA device and the built extension (there is no CPU fallback)")
    if args.case is not None:
        pkg.device_(local_rank)
        print(json.dumps({"case": args.case, "shrink": args.shrink,
                          "results": run_suite(pkg, measured_peak()[0], args.case, args.shrink, args.reps_scale)}), flush=True)
        return
    dist = Dist(rank, world)
    pkg.device_(local_rank)
    st = pkg.current_stream()
    if args.scaling == "strong":
        total_log2 = 33
        if world == 1 and pkg.mem_info()[0] < (140 << 30):
            total_log2 = 32
        n = (1 << total_log2) // world
    else:
        n = 1 << args.log2_elems
        total_log2 = args.log2_elems + (world - 1).bit_length()
    log2_per_gpu = n.bit_length() - 1
    workload = workload_text(log2_per_gpu, total_log2)
    comm = peer = None
    transport = None
    if args.collective == "fused":       # every N runs the same entry point, a group of one rank included
        peer = pkg.sharded.init_peer(rank, world, local_rank, dist.allgather, transport=args.transport)
        tr, sq = C.c_int32(), C.c_uint64()
        pkg._lib.check(pkg._lib.lib.b200_peer_info(peer, C.byref(tr), C.byref(sq)))
        transport = ("host", "vmm", "ipc")[tr.value]
    elif world > 1 and args.collective == "nccl":
        comm = pkg.sharded.init_comm(rank, world, local_rank, dist.exchange)
    R, bc = pkg.random, pkg.broadcast
    first = rank * n
    x, y, z = (R.fill_random_(pkg.ROCArray(np.float32, n), R.UNIFORM11, seed=4, stream_id=s, first_index=first) for s in range(3))
    r = pkg.ROCArray(np.float32, n)
    part = pkg.ROCArray(np.float32, 1)
    zero = np.float32(0)
    expr = x.dot * y.dot + bc.exp(-bc.abs_(z))
    launches = [0]
    fused_step = pkg.sharded.prepared_mapreduce_allreduce(peer, bc.abs2(r), "+", part, zero, st) if peer is not None else None
    bc_step = bc.prepared(r, expr, st)

    def step():
        bc_step()
        launches[0] += 2
        if fused_step is not None:
            fused_step()                       # sum(abs2, r) and the all-reduce, one kernel
            return
        pkg.mapreducedim_("abs2", "+", part, r, init=zero)
        if comm is not None:
            pkg._lib.check(pkg._lib.lib.b200_allreduce(comm, C.c_void_p(part.ptr), 1, pkg._lib.F32, pkg._lib.RED_ADD, st.handle))

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()            # nvidia-smi needs a moment before its first sample
    for _ in range(warmup):
        step()
    pkg.device_synchronize()
    dist.barrier()
    if rank == 0:
        sampler.lines.clear()      # keep only samples taken while the timed region runs
    launches[0] = 0
    a, b = pkg.Event(timing=True), pkg.Event(timing=True)
    a.record(st)
    for _ in range(args.steps):
        step()
    b.record(st)
    b.synchronize()
    pkg.device_synchronize()
    dist.barrier()
    ms_total = dist.max(pkg.elapsed_ms(a, b))
    timed_launches = launches[0]
    # nvidia-smi samples every 20 ms; a short timed region yields only a few samples.  The same
    # steps then keep running (untimed, on every rank alike - the count comes from the maximum
    # over the ranks) until 150 ms of load have been sampled.
    in_region = len(sampler.lines) if rank == 0 else 0
    if ms_total < 150.0:
        for _ in range(int((150.0 - ms_total) / max(ms_total / args.steps, 1e-3)) + 1):
            step()
        pkg.device_synchronize()
        dist.barrier()
    clocks = sampler.stop() if rank == 0 else None
    if clocks is not None:
        clocks["samples_in_timed_region"] = in_region
    total_sq = float(part.to_host()[0])
    ms_step = ms_total / args.steps
    value = BYTES_PER_ELEM * n * world / ms_step / 1e6

    # ---- kernel-level roofline: the broadcast kernel moves 16 of the 20 bytes per element
    peak, peak_kind = measured_peak()
    ms_bc = time_loop(pkg, st, bc_step, 10)
    ms_red = time_loop(pkg, st, lambda: pkg.mapreducedim_("abs2", "+", part, r, init=zero), 10)
    ach = 16 * n / ms_bc / 1e6
    ms_coll = None
    if fused_step is not None:
        dist.barrier()
        ms_coll = time_loop(pkg, st, fused_step, 10)     # reduction + all-reduce in one kernel
    per_rank = dist.allgather({"bc": ms_bc, "red": ms_red, "coll": ms_coll})
    spread = lambda k: None if per_rank[0][k] is None else {"min": round(min(p[k] for p in per_rank), 4), "max": round(max(p[k] for p in per_rank), 4)}

    # ---- checks that travel with the number.  (1) a stretch of rank 0's shard against a Float64
    # sum computed on the host from regenerated inputs; (2) the all-reduced value against the sum
    # of the ranks' own local reductions
    nc = min(n, 1 << 24)
    chk = pkg.ROCArray(np.float32, 1)
    pkg.mapreducedim_("abs2", "+", chk, r.view(0, nc), init=zero)
    gpu_sub = float(chk.to_host()[0])
    pkg.mapreducedim_("abs2", "+", chk, r, init=zero)
    locals_ = dist.allgather(float(chk.to_host()[0]))
    check = {"allreduce_vs_sum_of_local_reductions": abs(total_sq - sum(locals_)) <= 1e-5 * abs(sum(locals_))}
    if rank == 0:
        blk, host_sub = 1 << 22, 0.0
        for s in range(0, nc, blk):
            hx, hy, hz = (R.host_uniform11(4, k, first + s, min(blk, nc - s)).astype(np.float64) for k in range(3))
            hr = (hx.astype(np.float32) * hy.astype(np.float32)).astype(np.float64) + np.exp(-np.abs(hz))
            host_sub += float((hr * hr).sum())
        check.update({"sub_shard_elements": nc, "gpu_sum_abs2": gpu_sub, "host_float64_sum_abs2": host_sub,
                      "sub_shard_rel_err": abs(gpu_sub - host_sub) / host_sub, "sub_shard_ok": abs(gpu_sub - host_sub) <= 1e-5 * host_sub})

    # ---- end to end through the public API with host buffers
    ne = min(n, 1 << 28)
    hbuf = []
    for k in range(3):
        p = C.c_void_p()
        pkg._lib.check(pkg._lib.lib.b200_host_alloc(C.byref(p), 4 * ne))
        hv = np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_float)), shape=(ne,))
        blen = min(ne, 1 << 22)
        hv.reshape(-1, blen)[:] = R.host_uniform11(4, k, first, blen)
        hbuf.append((p, hv))
    hres = C.c_void_p()
    pkg._lib.check(pkg._lib.lib.b200_host_alloc(C.byref(hres), 4))
    xe, ye, ze, re_ = (v.view(0, ne) for v in (x, y, z, r))
    expr_e = xe.dot * ye.dot + bc.exp(-bc.abs_(ze))
    fused_e = pkg.sharded.prepared_mapreduce_allreduce(peer, bc.abs2(re_), "+", part, zero, st) if peer is not None else None
    L = pkg._lib.lib

    def e2e_step():
        for (p, _), d in zip(hbuf, (xe, ye, ze)):
            pkg._lib.check(L.b200_memcpy_async(C.c_void_p(d.ptr), p, 4 * ne, st.handle))
        pkg.materialize_(re_, expr_e)
        if fused_e is not None:
            fused_e()
        else:
            pkg.mapreducedim_("abs2", "+", part, re_, init=zero)
            if comm is not None:
                pkg._lib.check(L.b200_allreduce(comm, C.c_void_p(part.ptr), 1, pkg._lib.F32, pkg._lib.RED_ADD, st.handle))
        pkg._lib.check(L.b200_memcpy_async(hres, C.c_void_p(part.ptr), 4, st.handle))
        st.synchronize()          # the caller reads the scalar
    for _ in range(2):
        e2e_step()
    dist.barrier()
    ke = max(3, min(args.steps, 10))
    t0 = time.perf_counter()
    for _ in range(ke):
        e2e_step()
    e2e_ms = dist.max((time.perf_counter() - t0) * 1e3 / ke)
    e2e_val = BYTES_PER_ELEM * ne * world / e2e_ms / 1e6
    for p, _ in hbuf:
        L.b200_host_free(p)
    L.b200_host_free(hres)

    dist.barrier()
    if comm is not None:
        pkg.sharded.destroy_comm(comm)
    if peer is not None:
        pkg.device_synchronize()
        dist.barrier()
        pkg.sharded.destroy_peer(peer)
    del x, y, z, r, xe, ye, ze, re_, expr, expr_e, bc_step, fused_step, fused_e
    # ---- the sharded scan (after every timed region: it brings up an NCCL communicator)
    scan = sharded_scan_record(pkg, dist, rank, world, local_rank, st)

    suite = None
    cpu = None
    if rank == 0 and world == 1:
        cpu = cpu_baseline(max(1, min(args.steps, 20)), max(1, min(args.warmup, 5)))
        if not args.no_suite and args.scaling == "weak":
            suite = run_suite(pkg, peak)
    dist.barrier()
    dist.close()
    if rank != 0:
        return
    line = {
        "metric": METRIC,
        "value": round(value, 1), "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": warmup,
        "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload, "elements_per_gpu": n, "l2": f"inputs ({12 * n >> 30} GiB per GPU) are far larger than L2",
                   "frac_of_8TBs_per_gpu": round(value / world / NOMINAL_HBM_GBS, 3), "check_sum_abs2": total_sq, "check": check,
                   "collective": args.collective, "transport": transport, "sharded_scan": scan},
        "roofline": {"bound": "hbm", "kernel": "ew_stream_kernel<float, MulAddExpNegAbsF> (r .= x.*y .+ exp.(-abs.(z)))",
                     "achieved": round(ach, 1), "peak": peak, "unit": "GB/s", "frac": round(ach / peak, 3),
                     "peak_source": f"{peak_kind} copy bandwidth", "traffic": round(EW_TRAFFIC_BYTES_PER_ELEM * n),
                     "traffic_source": "ncu capture of a 2^28-element launch (profiles/ew_stream_kernel_c5_2p28_traffic.md) scaled by the "
                                       "element count; the reads are exactly the inputs, 2.7 % of the output was still dirty in L2 at the end",
                     "ms_per_launch": round(ms_bc, 4), "ms_per_launch_over_ranks": spread("bc"), "algorithmic_bytes_per_launch": 16 * n,
                     "reduce_kernel": {"ms_per_launch": round(ms_red, 4), "achieved": round(4 * n / ms_red / 1e6, 1),
                                       "frac": round(4 * n / ms_red / 1e6 / peak, 3), "ms_per_launch_over_ranks": spread("red")},
                     "fused_reduce_allreduce_ms": None if ms_coll is None else round(ms_coll, 4),
                     "fused_reduce_allreduce_ms_over_ranks": spread("coll")},
        "e2e": {"value": round(e2e_val, 2), "unit": "GB/s", "h2d_bytes_per_step": 12 * ne, "d2h_bytes_per_step": 4,
                "elements_per_gpu": ne, "ms_per_step": round(e2e_ms, 3),
                "note": "PCIe-bound: 12 B per element cross the link for 20 B of metric"},
        "gpu_launches": timed_launches,
        "clocks": clocks,
    }
    if cpu is not None:
        line["cpu_baseline"] = cpu
    if suite is not None:
        line["suite"] = suite
    print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
