"""Contiguously sharded vectors over the GPUs of one NVSwitch box, one process per GPU.

The reference has no sharded array type and no collective layer (one task per device with
copies through the host, docs/src/usage/multitasking.md:37-53, test/hip_rocarray/multi_gpu.jl);
this module adds exactly what the sharded workloads need:

* broadcast: purely local, every rank runs the fused kernel on its shard;
* reductions: local ``mapreducedim!`` into a one-element device array, then an in-place NCCL
  all-reduce of that element on the same stream (no host round trip in between);
* scans: local total -> all-gather of one element per rank -> carry = fold of the totals of the
  lower ranks (a tiny reduction over this rank's own copy) -> local look-back scan seeded by
  the carry, which stays in device memory.

The sequence of steps lives in :class:`ShardedOps`; what runs a step is a backend object, so
the same logic is exercised on CPU ranks (gloo + NumPy stand-ins) in the tests and on GPUs
(library kernels + NCCL) in production.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np


def shard_range(n: int, rank: int, world: int, itemsize: int = 4) -> tuple[int, int]:
    """Half-open element range of `rank`: blocks of ceil(n/world) elements whose starts are
    rounded up to 16 bytes so every shard can use 128-bit accesses."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError("rank outside [0, world)")
    grain = max(1, 16 // itemsize)
    per = -(-n // world)
    per = -(-per // grain) * grain
    lo = min(n, rank * per)
    hi = min(n, lo + per)
    return lo, hi


class ShardedOps:
    """Rank-local view of sharded reductions and scans."""

    def __init__(self, backend, rank: int, world: int):
        self.b, self.rank, self.world = backend, rank, world

    def mapreduce(self, f, op, shard, init=None):
        """All ranks receive op-fold over the whole (virtual) array of f(shard elements)."""
        fused = getattr(self.b, "fused_mapreduce", None)
        part = fused(f, op, shard) if (fused is not None and self.world > 1) else None
        if part is None:
            part = self.b.local_mapreduce(f, op, shard)      # one-element holder, op-neutral seeded
            if self.world > 1:
                self.b.allreduce(part, op)
        if init is not None:
            part = self.b.combine_scalar(op, init, part)
        return part

    def accumulate(self, op, out_shard, shard):
        """Inclusive scan of the whole (virtual) array; this rank writes its shard's part."""
        if self.world == 1:
            return self.b.local_accumulate(op, out_shard, shard, None)
        total = self.b.local_mapreduce(None, op, shard)
        totals = self.b.allgather(total)                       # holder with `world` elements
        carry = self.b.fold_prefix(op, totals, self.rank) if self.rank > 0 else None
        return self.b.local_accumulate(op, out_shard, shard, carry)


class DeviceBackend:
    """Library kernels + NCCL through the C ABI."""

    def __init__(self, comm, world_size: int, stream=None, peer=None):
        from .runtime import current_stream
        self.comm = comm
        self.peer = peer
        self.world_size = world_size
        self.stream = stream or current_stream()

    def fused_mapreduce(self, f, op, shard):
        """Reduction and all-reduce in ONE kernel over NVLink peer memory; None when the case is
        outside what that kernel handles (the caller then reduces locally and all-reduces)."""
        if self.peer is None or len(shard) == 0:
            return None
        from . import _lib
        from .array import ROCArray
        from .mapreduce import _apply_f, _neutral, _op_code, _result_dtype
        expr = _apply_f(f, shard)
        opc = _op_code(op)
        dt = _result_dtype(expr.dtype, opc)
        R = ROCArray(dt, (1,) * max(1, len(expr.shape())), stream=self.stream)
        try:
            launch = prepared_mapreduce_allreduce(self.peer, expr, op, R, _neutral(opc, dt), self.stream)
            launch()
        except _lib.B200Error as e:
            if e.code == _lib.UNSUPPORTED:
                return None
            raise
        return R

    def local_mapreduce(self, f, op, shard):
        from .array import ROCArray
        from .mapreduce import _apply_f, _neutral, _op_code, _result_dtype, mapreducedim_
        expr = _apply_f(f, shard)
        opc = _op_code(op)
        dt = _result_dtype(expr.dtype, opc)
        R = ROCArray(dt, (1,) * max(1, len(expr.shape())), stream=self.stream)
        seed = _neutral(opc, dt)
        if len(shard) == 0:
            return R.fill_(seed, self.stream)
        return mapreducedim_(lambda _: expr, op, R, shard, init=seed, stream=self.stream)

    def allreduce(self, holder, op):
        from . import _lib
        from ._lib import check, lib
        from .mapreduce import _op_code
        check(lib.b200_allreduce(self.comm, C.c_void_p(holder.ptr), holder.size, _lib.dtype_code(holder.dtype),
                                 _op_code(op), self.stream.handle))
        return holder

    def allgather(self, holder):
        from . import _lib
        from ._lib import check, lib
        from .array import ROCArray
        world = self.world_size
        out = ROCArray(holder.dtype, (world * holder.size,), stream=self.stream)
        check(lib.b200_allgather(self.comm, C.c_void_p(holder.ptr), C.c_void_p(out.ptr), holder.size,
                                 _lib.dtype_code(holder.dtype), self.stream.handle))
        return out

    def fold_prefix(self, op, totals, rank):
        return self.local_mapreduce(None, op, totals.view(0, rank))

    def combine_scalar(self, op, init, holder):
        from .broadcast import Broadcasted, materialize_
        name = {"+": "add", "*": "mul", "max": "max", "min": "min"}[op]
        return materialize_(holder, Broadcasted.call(name, holder.dtype.type(init), holder), self.stream)

    def local_accumulate(self, op, out_shard, shard, carry):
        from ._lib import check, lib
        from .accumulate import accumulate_
        from .mapreduce import _op_code
        if carry is None:
            return accumulate_(op, out_shard, shard, init=None, stream=self.stream)
        if carry.dtype != shard.dtype:
            from .broadcast import Broadcasted, materialize_
            from .array import ROCArray
            carry = materialize_(ROCArray(shard.dtype, (1,), stream=self.stream), Broadcasted.leaf(carry.reshape(1)), self.stream)
        tb, ta = out_shard.tensor(), shard.tensor()
        check(lib.b200_accumulate_carry(self.stream.handle, C.byref(tb), C.byref(ta), _op_code(op),
                                        C.c_void_p(carry.ptr), 0, 1))
        return out_shard


def prepared_mapreduce_allreduce(peer, expr, op, R, init, stream):
    """Zero-argument callable issuing one fused reduce + all-reduce of `expr` into the one-element
    array `R` (descriptors built once)."""
    from ._lib import check, lib
    from .broadcast import Broadcasted
    from .mapreduce import _op_code
    expr = Broadcasted.leaf(expr)
    shape = expr.shape()
    code, leaves, nleaves, keep = expr.flatten()
    shp = (C.c_int64 * max(1, len(shape)))(*shape)
    t = R.tensor()
    init_buf = None if init is None else np.asarray(init, dtype=R.dtype).tobytes()
    fn, ninstr, opc, nd = lib.b200_mapreduce_allreduce, len(code) // 2, _op_code(op), len(shape)

    def launch(_keep=(keep, R, stream)):
        check(fn(peer, stream.handle, C.byref(t), shp, nd, leaves, nleaves, code, ninstr, opc, init_buf))
    return launch


def init_peer(rank: int, world: int, device: int, allgather) -> C.c_void_p:
    """Creates this rank's peer-exchange group.  `allgather(bytes) -> list[bytes]` must return
    every rank's argument in rank order on every rank (any host channel)."""
    from ._lib import check, lib
    peer = C.c_void_p()
    buf = C.create_string_buffer(64)
    check(lib.b200_peer_create(device, rank, world, C.byref(peer), buf))
    handles = allgather(buf.raw)
    check(lib.b200_peer_connect(peer, b"".join(handles)))
    return peer


def destroy_peer(peer) -> None:
    from ._lib import check, lib
    check(lib.b200_peer_destroy(peer))


def init_comm(rank: int, world: int, device: int, exchange) -> C.c_void_p:
    """Creates the NCCL communicator of this rank.  `exchange(bytes_or_None) -> bytes` must
    return rank 0's argument on every rank (a store or a host-side broadcast)."""
    from ._lib import check, lib
    ident = None
    if rank == 0:
        buf = C.create_string_buffer(128)
        check(lib.b200_comm_unique_id(buf))
        ident = buf.raw
    ident = exchange(ident)
    comm = C.c_void_p()
    check(lib.b200_comm_init_rank(C.byref(comm), world, rank, ident, device))
    return comm


def destroy_comm(comm) -> None:
    from ._lib import check, lib
    check(lib.b200_comm_destroy(comm))


def env_rank_world() -> tuple[int, int, int]:
    """(rank, world, local_rank) as set by torchrun; a plain launch is rank 0 of 1."""
    return (int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")),
            int(os.environ.get("LOCAL_RANK", "0")))
