"""World-size-2 runs of the sharded reduction / scan logic on CPU ranks (gloo).

The step sequence under test is the product's (`ShardedOps` in amdgpu.jl_b200/sharded.py); what
executes a step here is a NumPy stand-in for the device kernels plus gloo collectives, so the
shard arithmetic, the all-reduce / all-gather wiring and the carry fold are exercised without a
GPU.  The expected values come from the unsharded oracle.
"""
import os
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent


class NumpyGlooBackend:
    """Stand-in for DeviceBackend: one-element holders are NumPy arrays, collectives are gloo.
    `fused_supported` answers from the mapped function, operator and element type alone, as the
    device backend does; the stand-in for the fused kernel is a local fold followed by an
    all-gather, and it records which collective each call entered."""

    def __init__(self, dist, world, orc, fused=False):
        self.dist, self.world_size, self.orc, self.fused = dist, world, orc, fused
        self.entered: list[str] = []

    def fused_supported(self, f, op, dtype):
        return self.fused and f in (None, "identity", "abs", "abs2") and not (f == "abs2" and op != "+")

    def fused_mapreduce(self, f, op, shard):
        import torch
        self.entered.append("fused")
        part = self.local_mapreduce(f, op, shard, _record=False).astype(np.float64)
        outs = [torch.empty(1, dtype=torch.float64) for _ in range(self.world_size)]
        self.dist.all_gather(outs, torch.from_numpy(part))
        fold = {"+": np.add, "*": np.multiply, "max": np.maximum, "min": np.minimum}[op]
        total = outs[0].numpy().copy()
        for o in outs[1:]:
            total = fold(total, o.numpy())
        return total

    def wait(self, timeout):
        pass

    def local_mapreduce(self, f, op, shard, _record=True):
        import torch  # noqa: F401
        if _record:
            self.entered.append("local")
        if len(shard) == 0:
            ident = {"+": 0, "*": 1, "max": -np.inf, "min": np.inf}[op]
            return np.array([ident], dtype=np.float64 if shard.dtype.kind == "f" else np.int64)
        return np.array([self.orc.mapreduce(f, op, shard)])

    def allreduce(self, holder, op):
        import torch
        t = torch.from_numpy(holder)
        ops = {"+": self.dist.ReduceOp.SUM, "*": self.dist.ReduceOp.PRODUCT, "max": self.dist.ReduceOp.MAX, "min": self.dist.ReduceOp.MIN}
        self.dist.all_reduce(t, op=ops[op])
        return holder

    def allgather(self, holder):
        import torch
        outs = [torch.empty_like(torch.from_numpy(holder)) for _ in range(self.world_size)]
        self.dist.all_gather(outs, torch.from_numpy(holder))
        return np.concatenate([o.numpy() for o in outs])

    def fold_prefix(self, op, totals, rank):
        return np.array([self.orc.mapreduce(None, op, totals[:rank])])

    def combine_scalar(self, op, init, holder):
        f = {"+": np.add, "*": np.multiply, "max": np.maximum, "min": np.minimum}[op]
        return f(np.asarray(init, dtype=holder.dtype), holder)

    def local_accumulate(self, op, out_shard, shard, carry):
        init = None if carry is None else carry[0].astype(shard.dtype)
        out_shard[...] = self.orc.accumulate(op, shard, init=init).astype(shard.dtype)
        return out_shard


def _worker(rank, world, port, tmp):
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import torch.distributed as dist
    import __graft_entry__ as entry
    pkg, orc = entry.load_package(), entry.load_oracle()
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        ops = pkg.sharded.ShardedOps(NumpyGlooBackend(dist, world, orc), rank, world)
        rng = np.random.default_rng(7)                     # same stream on every rank
        for n in (1_000_003, 5, 1):
            x = rng.integers(-100, 101, n).astype(np.int64)
            lo, hi = pkg.sharded.shard_range(n, rank, world, 8)
            shard = x[lo:hi]
            total = ops.mapreduce(None, "+", shard)
            assert total[0] == x.sum(), (n, rank)
            assert ops.mapreduce("abs2", "+", shard)[0] == (x * x).sum()
            assert ops.mapreduce(None, "max", shard.astype(np.float64))[0] == x.max()
            assert ops.mapreduce(None, "+", shard, init=5)[0] == x.sum() + 5
            out = np.empty_like(shard)
            ops.accumulate("+", out, shard)
            assert np.array_equal(out, np.cumsum(x)[lo:hi]), (n, rank)
        f = rng.random(100_000)
        lo, hi = pkg.sharded.shard_range(len(f), rank, world, 8)
        out = np.empty(hi - lo)
        ops.accumulate("+", out, f[lo:hi])
        assert np.allclose(out, np.cumsum(f)[lo:hi], rtol=1e-12)
        # every rank must take the same branch whatever its shard holds: with fewer elements than
        # 4 x world some shards are empty (shard starts are rounded to 16 bytes) or hold one element
        for fused_on in (True, False):
            ops = pkg.sharded.ShardedOps(NumpyGlooBackend(dist, world, orc, fused=fused_on), rank, world)
            for n in range(0, 4 * world + 1):
                x = rng.integers(-100, 101, n).astype(np.int32)
                lo, hi = pkg.sharded.shard_range(n, rank, world, 4)
                shard = x[lo:hi]
                assert ops.mapreduce(None, "+", shard)[0] == x.sum(), (n, rank, fused_on)
                assert ops.mapreduce("abs2", "+", shard)[0] == (x.astype(np.int64) ** 2).sum()
                if n:
                    assert ops.mapreduce("abs", "max", shard.astype(np.float64))[0] == np.abs(x).max()
                assert ops.mapreduce("abs2", "max", shard.astype(np.float64), init=-1.0)[0] == max(-1.0, (x.astype(np.float64) ** 2).max(initial=-np.inf))
            traces = [None] * world
            dist.all_gather_object(traces, ops.trace)
            assert all(tr == traces[0] for tr in traces), "ranks disagreed on the collective to run"
            assert ("fused" in ops.trace) == fused_on and "collective" in ops.trace
        (Path(tmp) / f"ok{rank}").write_text("ok")
    finally:
        dist.destroy_process_group()


def test_sharded_ops_world_size_2(tmp_path):
    import torch.multiprocessing as mp
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "ok0").exists() and (tmp_path / "ok1").exists()


class TimedGlooBackend(NumpyGlooBackend):
    """Collectives are started asynchronously; `wait` gives them `timeout` seconds, as the device
    backend gives the stream (b200_comm_check)."""

    def __init__(self, dist, world, orc, pkg):
        super().__init__(dist, world, orc)
        self.pkg, self.pending = pkg, []

    def allreduce(self, holder, op):
        import torch
        self.pending.append(self.dist.all_reduce(torch.from_numpy(holder), op=self.dist.ReduceOp.SUM, async_op=True))
        return holder

    def wait(self, timeout):
        import datetime
        for work in self.pending:
            try:
                work.wait(timeout=datetime.timedelta(seconds=timeout))
            except RuntimeError as e:
                raise self.pkg.sharded.CollectiveTimeout(str(e)) from e
        self.pending.clear()


def _missing_rank_worker(rank, world, port, tmp):
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import torch.distributed as dist
    import __graft_entry__ as entry
    pkg, orc = entry.load_package(), entry.load_oracle()
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ops = pkg.sharded.ShardedOps(TimedGlooBackend(dist, world, orc, pkg), rank, world)
    x = np.arange(10, dtype=np.int64)
    # step 1: both ranks take part
    assert ops.mapreduce(None, "+", x, timeout=30.0)[0] == 2 * x.sum()
    # step 2: rank 1 leaves between steps and never joins the collective; rank 0 finds out on the
    # host, by its time limit, and gets an exception instead of a hang
    if rank == 1:
        (Path(tmp) / "left1").write_text("left")
        os._exit(0)
    try:
        ops.mapreduce(None, "+", x, timeout=2.0)
    except pkg.sharded.CollectiveTimeout:
        (Path(tmp) / "timeout0").write_text("ok")
    os._exit(0)          # the process group is broken by design: no orderly shutdown


def test_missing_rank_is_detected_on_the_host(tmp_path):
    import torch.multiprocessing as mp
    port = 31500 + (os.getpid() % 2000)
    ctx = mp.spawn(_missing_rank_worker, args=(2, port, str(tmp_path)), nprocs=2, join=False)
    for p in ctx.processes:
        p.join(120)
    assert (tmp_path / "left1").exists() and (tmp_path / "timeout0").exists()
