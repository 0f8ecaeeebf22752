"""Sharded reduction and scan on two real GPUs (one process per GPU, NCCL through the C ABI).
Skipped on a single-GPU box; the same step logic runs on CPU ranks in test_sharded_gloo.py."""
import os
import sys
from pathlib import Path

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def _worker(rank, world, port, tmp):
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import torch.distributed as dist
    import __graft_entry__ as entry
    pkg, orc = entry.load_package(), entry.load_oracle()
    dist.init_process_group("gloo", rank=rank, world_size=world)
    pkg.device_(rank)

    def exchange(payload):
        box = [payload]
        dist.broadcast_object_list(box, src=0)
        return box[0]
    def allgather(payload):
        out = [None] * world
        dist.all_gather_object(out, payload)
        return out
    comm = pkg.sharded.init_comm(rank, world, rank, exchange)
    peer = pkg.sharded.init_peer(rank, world, rank, allgather)
    try:
        ops = pkg.sharded.ShardedOps(pkg.sharded.DeviceBackend(comm, world), rank, world)
        fused = pkg.sharded.ShardedOps(pkg.sharded.DeviceBackend(comm, world, peer=peer), rank, world)
        rng = np.random.default_rng(11)                    # same stream on every rank
        n = 3_000_004
        xi = rng.integers(-100, 101, n).astype(np.int32)
        xf = (rng.random(n) * 2 - 1).astype(np.float32)
        lo, hi = pkg.sharded.shard_range(n, rank, world, 4)
        si, sf = pkg.ROCArray.from_host(xi[lo:hi]), pkg.ROCArray.from_host(xf[lo:hi])
        # reductions: every rank ends up with the global value
        tot = ops.mapreduce(None, "+", si).to_host()[0]
        assert tot == xi.astype(np.int64).sum()
        sq = ops.mapreduce("abs2", "+", sf).to_host()[0]
        ref = (xf.astype(np.float64) ** 2).sum()
        assert abs(sq - ref) <= 1e-5 * ref
        assert ops.mapreduce(None, "max", sf).to_host()[0] == xf.max()
        # the same reductions through the one-kernel reduce + all-reduce over peer memory, several
        # in a row (alternating slot banks), every rank must hold the same bits
        for k in range(5):
            v = (rng.random(n) * 2 - 1).astype(np.float32)
            sv = pkg.ROCArray.from_host(v[lo:hi])
            got = fused.mapreduce("abs2", "+", sv).to_host()[0]
            ref = (v.astype(np.float64) ** 2).sum()
            assert abs(got - ref) <= 1e-5 * ref, (k, got, ref)
            assert len({g.tobytes() for g in allgather(got)}) == 1
            assert fused.mapreduce(None, "max", sv).to_host()[0] == v.max()
        assert fused.mapreduce(None, "+", si).to_host()[0] == xi.astype(np.int64).sum()
        # a case the fused kernel does not cover falls back to reduce + NCCL all-reduce
        two = fused.mapreduce(lambda t: t * t + 1, "+", sf).to_host()[0]
        ref2 = (xf.astype(np.float64) ** 2 + 1).sum()
        assert abs(two - ref2) <= 1e-5 * ref2
        # scans: carry stays on the device
        out = pkg.ROCArray(np.int32, hi - lo)
        ops.accumulate("+", out, si)
        assert np.array_equal(out.to_host(), np.cumsum(xi, dtype=np.int32)[lo:hi])
        outf = pkg.ROCArray(np.float32, hi - lo)
        ops.accumulate("+", outf, sf)
        reff = np.cumsum(xf.astype(np.float64))[lo:hi]
        assert np.all(np.abs(outf.to_host() - reff) <= 1e-4 * np.maximum(np.abs(reff), 1.0))
        pkg.synchronize()
        (Path(tmp) / f"ok{rank}").write_text("ok")
    finally:
        pkg.synchronize()
        dist.barrier()
        pkg.sharded.destroy_peer(peer)
        pkg.sharded.destroy_comm(comm)
        dist.destroy_process_group()


def test_two_gpu_sharded_ops(gpu, tmp_path):
    if gpu.ndevices() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    port = 29600 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "ok0").exists() and (tmp_path / "ok1").exists()
