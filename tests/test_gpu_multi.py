"""Sharded reduction and scan on two real GPUs (one process per GPU, the fused exchange over each
transport, NCCL through the C ABI).  Skipped on a single-GPU box; the same step logic runs on CPU
ranks in test_sharded_gloo.py."""
import os
import sys
from pathlib import Path

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def _setup(rank, world, port):
    import faulthandler
    faulthandler.enable()                     # a crash in native code names the Python line it came from
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
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
    return pkg, orc, dist, exchange, allgather


def _worker(rank, world, port, tmp):
    pkg, orc, dist, exchange, allgather = _setup(rank, world, port)
    comm = pkg.sharded.init_comm(rank, world, rank, exchange)
    peers = {}
    try:
        ops = pkg.sharded.ShardedOps(pkg.sharded.DeviceBackend(comm, world), rank, world)
        rng = np.random.default_rng(11)                    # same stream on every rank
        n = 3_000_004
        xi = rng.integers(-100, 101, n).astype(np.int32)
        xf = (rng.random(n) * 2 - 1).astype(np.float32)
        lo, hi = pkg.sharded.shard_range(n, rank, world, 4)
        si, sf = pkg.ROCArray.from_host(xi[lo:hi]), pkg.ROCArray.from_host(xf[lo:hi])
        # reductions through reduce + NCCL all-reduce: every rank ends up with the global value
        tot = ops.mapreduce(None, "+", si).to_host()[0]
        assert tot == xi.astype(np.int64).sum()
        sq = ops.mapreduce("abs2", "+", sf, timeout=60.0).to_host()[0]
        ref = (xf.astype(np.float64) ** 2).sum()
        assert abs(sq - ref) <= 1e-5 * ref
        assert ops.mapreduce(None, "max", sf).to_host()[0] == xf.max()
        assert ops.trace == ["collective"] * 3
        # the same reductions through the one-kernel reduce + all-reduce, over every transport,
        # several in a row (alternating slot banks); every rank must hold the same bits
        for transport in ("host", "vmm", "ipc"):
            peer = peers[transport] = pkg.sharded.init_peer(rank, world, rank, allgather, transport=transport)
            fused = pkg.sharded.ShardedOps(pkg.sharded.DeviceBackend(comm, world, peer=peer), rank, world)
            for k in range(5):
                v = (rng.random(n) * 2 - 1).astype(np.float32)
                sv = pkg.ROCArray.from_host(v[lo:hi])
                got = fused.mapreduce("abs2", "+", sv).to_host()[0]
                ref = (v.astype(np.float64) ** 2).sum()
                assert abs(got - ref) <= 1e-5 * ref, (transport, k, got, ref)
                assert len({g.tobytes() for g in allgather(got)}) == 1
                assert fused.mapreduce(None, "max", sv).to_host()[0] == v.max()
            assert fused.mapreduce(None, "+", si).to_host()[0] == xi.astype(np.int64).sum()
            # fewer elements than 4 x world: some shards are empty or hold one element, and every
            # rank still goes through the fused kernel
            for m in range(0, 4 * world + 1):
                y = rng.integers(-100, 101, m).astype(np.int32)
                a, b = pkg.sharded.shard_range(m, rank, world, 4)
                sy = pkg.ROCArray.from_host(y[a:b])
                assert fused.mapreduce(None, "+", sy).to_host()[0] == y.astype(np.int64).sum(), (transport, m)
                assert fused.mapreduce("abs", "max", sy, init=np.int32(-5)).to_host()[0] == max(-5, np.abs(y).max(initial=-5))
            # an expression the fused kernel does not cover goes to reduce + NCCL all-reduce on ALL ranks
            two = fused.mapreduce(lambda t: t * t + 1, "+", sf).to_host()[0]
            ref2 = (xf.astype(np.float64) ** 2 + 1).sum()
            assert abs(two - ref2) <= 1e-5 * ref2
            traces = allgather(fused.trace)
            assert all(tr == traces[0] for tr in traces) and fused.trace[-1] == "collective" and fused.trace[0] == "fused"
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
        for peer in peers.values():
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


def _skipped_step_worker(rank, world, port, tmp):
    """Rank 1 leaves out ONE fused call between steps.  Rank 0's kernel polls for rank 1's partial
    with a budget of a few thousand polls, gives up, and the error comes back as a status from the
    next synchronisation; nothing traps, both contexts stay usable, and after both ranks have
    created a new peer group the reductions agree again.  Plain peer stores only (host transport)."""
    pkg, orc, dist, exchange, allgather = _setup(rank, world, port)
    L = pkg._lib
    x = pkg.ROCArray.from_host(np.full(100_000, rank + 1, dtype=np.int32))
    peer = pkg.sharded.init_peer(rank, world, rank, allgather, transport="host")
    pkg.sharded.peer_set_poll_budget(peer, 4000)
    fused = pkg.sharded.ShardedOps(pkg.sharded.DeviceBackend(None, world, peer=peer), rank, world)
    try:
        assert fused.mapreduce(None, "+", x).to_host()[0] == 300_000
        dist.barrier()
        if rank == 0:
            part = fused.mapreduce(None, "+", x)             # rank 1 never joins this one
            with pytest.raises(pkg.B200Error) as ei:
                pkg.synchronize()
            assert ei.value.code == L.LOOKBACK_TIMEOUT
            pkg.synchronize()                                # reported once, the context is fine
            del part
        dist.barrier()
        # the group's sequence numbers now differ between the ranks: make a new group
        pkg.sharded.destroy_peer(peer)
        peer = pkg.sharded.init_peer(rank, world, rank, allgather, transport="host")
        fused = pkg.sharded.ShardedOps(pkg.sharded.DeviceBackend(None, world, peer=peer), rank, world)
        for _ in range(3):
            assert fused.mapreduce(None, "+", x).to_host()[0] == 300_000
        assert float(pkg.sum(x)) == 100_000 * (rank + 1)
        (Path(tmp) / f"ok{rank}").write_text("ok")
    finally:
        pkg.synchronize()
        dist.barrier()
        pkg.sharded.destroy_peer(peer)
        dist.destroy_process_group()


def test_missing_rank_times_out_and_group_recovers(gpu, tmp_path):
    if gpu.ndevices() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    port = 33600 + (os.getpid() % 2000)
    mp.spawn(_skipped_step_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "ok0").exists() and (tmp_path / "ok1").exists()


def test_arrays_on_two_devices_of_one_process(gpu):
    """One process, two devices, switched with ``device!`` (test/hip_rocarray/multi_gpu.jl:30-93):
    arrays stay on the device they were made on, reductions and broadcasts run on the current
    device, data moves between the devices through the host."""
    if gpu.ndevices() < 2:
        pytest.skip("needs two GPUs")
    try:
        gpu.device_(0)
        x1 = gpu.ones(np.int64, 16)
        assert x1.device == 0
        gpu.device_(1)
        x2 = gpu.ones(np.int64, 16)
        assert x2.device == 1 and gpu.current_device() == 1
        assert gpu.sum(x2) == 16
        gpu.device_(0)
        assert gpu.sum(x1) == 16
        # copyto! through a host array (multi_gpu.jl:52-68)
        h = np.arange(16, dtype=np.int32) * 3 - 7
        a = gpu.ROCArray.from_host(h)
        host = a.to_host()
        gpu.device_(1)
        b = gpu.zeros(np.int32, 16)
        b.copy_from_host(host)
        assert np.array_equal(b.to_host(), h)
        # the same operator on each device in turn (multi_gpu.jl:70-93, x .+= 1 in place of the kernel)
        gpu.device_(0)
        y1 = gpu.zeros(np.int32, 1 << 20)
        gpu.materialize_(y1, y1.dot + np.int32(1))
        gpu.device_(1)
        y2 = gpu.zeros(np.int32, 1 << 20)
        gpu.materialize_(y2, y2.dot + np.int32(1))
        assert gpu.sum(y2) == 1 << 20
        assert int(gpu.cumsum(y2).to_host()[-1]) == 1 << 20
        gpu.device_(0)
        assert gpu.sum(y1) == 1 << 20
        gpu.synchronize()
    finally:
        gpu.device_(0)
