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
    """Stand-in for DeviceBackend: one-element holders are NumPy arrays, collectives are gloo."""

    def __init__(self, dist, world, orc):
        self.dist, self.world_size, self.orc = dist, world, orc

    def local_mapreduce(self, f, op, shard):
        import torch  # noqa: F401
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
        (Path(tmp) / f"ok{rank}").write_text("ok")
    finally:
        dist.destroy_process_group()


def test_sharded_ops_world_size_2(tmp_path):
    import torch.multiprocessing as mp
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "ok0").exists() and (tmp_path / "ok1").exists()
