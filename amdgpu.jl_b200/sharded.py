"""Contiguously sharded vectors over the GPUs of one NVSwitch box, one process per GPU.

The reference has no sharded array type and no collective layer (one task per device with
copies through the host, docs/src/usage/multitasking.md:37-53, test/hip_rocarray/multi_gpu.jl);
this module adds exactly what the sharded workloads need:

* broadcast: purely local, every rank runs the fused kernel on its shard;
* reductions: one kernel that reduces the shard and exchanges + folds the partials of all ranks
  through slots every rank can write (``b200_mapreduce_allreduce``); expressions outside that
  kernel's set reduce into a one-element device array followed by an in-place NCCL all-reduce on
  the same stream (no host round trip in between).  Which of the two runs is decided from the
  expression, operator and element type alone, so all ranks always agree;
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


class CollectiveTimeout(RuntimeError):
    """A collective did not finish in time: a rank is missing or stuck."""


class ShardedOps:
    """Rank-local view of sharded reductions and scans.

    Every decision that selects which collective runs is taken from inputs that are the same on
    all ranks (the mapped function, the operator, the element type, the world size) - never from
    the length of the local shard, which differs between ranks and may be zero.  `trace` records
    the branch of each call ("fused" or "collective") so that tests can compare the ranks."""

    def __init__(self, backend, rank: int, world: int):
        self.b, self.rank, self.world = backend, rank, world
        self.trace: list[str] = []

    def mapreduce(self, f, op, shard, init=None, timeout: float | None = None):
        """All ranks receive op-fold over the whole (virtual) array of f(shard elements).  With
        `timeout` (seconds) the call waits for the result and raises :class:`CollectiveTimeout`
        when the collective does not finish in time."""
        supported = getattr(self.b, "fused_supported", None)
        if self.world > 1 and supported is not None and supported(f, op, shard.dtype):
            self.trace.append("fused")
            part = self.b.fused_mapreduce(f, op, shard)        # takes shards of any length, empty ones too
        else:
            self.trace.append("collective" if self.world > 1 else "local")
            part = self.b.local_mapreduce(f, op, shard)      # one-element holder, op-neutral seeded
            if self.world > 1:
                self.b.allreduce(part, op)
        if timeout is not None:
            self.b.wait(timeout)
        if init is not None:
            part = self.b.combine_scalar(op, init, part)
        return part

    def accumulate(self, op, out_shard, shard, timeout: float | None = None):
        """Inclusive scan of the whole (virtual) array; this rank writes its shard's part."""
        if self.world == 1:
            return self.b.local_accumulate(op, out_shard, shard, None)
        total = self.b.local_mapreduce(None, op, shard)
        totals = self.b.allgather(total)                       # holder with `world` elements
        if timeout is not None:
            self.b.wait(timeout)
        carry = self.b.fold_prefix(op, totals, self.rank) if self.rank > 0 else None
        return self.b.local_accumulate(op, out_shard, shard, carry)


_FUSED_MAPS = {None: "identity", "identity": "identity", "abs": "abs", abs: "abs", "abs2": "abs2"}


class DeviceBackend:
    """Library kernels + NCCL through the C ABI."""

    def __init__(self, comm, world_size: int, stream=None, peer=None):
        from .runtime import current_stream
        self.comm = comm
        self.peer = peer
        self.world_size = world_size
        self.stream = stream or current_stream()

    def fused_supported(self, f, op, dtype) -> bool:
        """Whether ``mapreduce(f, op, shard)`` goes through the one-kernel reduce + all-reduce.
        Depends on the mapped function, the operator and the element type only (what
        b200_mapreduce_allreduce accepts: f in {identity, abs, abs2}; ``*`` only with identity,
        abs2 only with ``+``; Float16/BFloat16/Float32/Float64/Int32/Int64 elements)."""
        if self.peer is None:
            return False
        from . import _lib
        from .mapreduce import _op_code
        try:
            name = _FUSED_MAPS.get(f)
        except TypeError:              # unhashable callable
            name = None
        if name is None:
            return False
        opc = _op_code(op)
        if name == "abs" and opc == _lib.RED_MUL:
            return False
        if name == "abs2" and opc != _lib.RED_ADD:
            return False
        return _lib.dtype_code(dtype) in (_lib.F16, _lib.BF16, _lib.F32, _lib.F64, _lib.I32, _lib.I64)

    def fused_mapreduce(self, f, op, shard):
        """Reduction and all-reduce in ONE kernel over the peer group's exchange slots.  The shard
        may be empty (this rank then contributes the operator's neutral element) or a single
        element.  Errors are raised, never turned into another collective: the other ranks are
        already inside this one."""
        from .array import ROCArray
        from .mapreduce import _apply_f, _neutral, _op_code, _result_dtype
        if not shard.is_contiguous:
            shard = shard.copy(self.stream)
        expr = _apply_f(f, shard)
        opc = _op_code(op)
        dt = _result_dtype(expr.dtype, opc)
        R = ROCArray(dt, (1,) * max(1, len(expr.shape())), stream=self.stream)
        prepared_mapreduce_allreduce(self.peer, expr, op, R, _neutral(opc, dt), self.stream)()
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
        from .array import with_managed
        from .mapreduce import _op_code
        with_managed(self.stream, holder)
        check(lib.b200_allreduce(self.comm, C.c_void_p(holder.ptr), holder.size, _lib.dtype_code(holder.dtype),
                                 _op_code(op), self.stream.handle))
        return holder

    def allgather(self, holder):
        from . import _lib
        from ._lib import check, lib
        from .array import ROCArray, with_managed
        world = self.world_size
        out = ROCArray(holder.dtype, (world * holder.size,), stream=self.stream)
        with_managed(self.stream, holder, out)
        check(lib.b200_allgather(self.comm, C.c_void_p(holder.ptr), C.c_void_p(out.ptr), holder.size,
                                 _lib.dtype_code(holder.dtype), self.stream.handle))
        return out

    def wait(self, timeout: float) -> None:
        """Waits for this rank's stream; a collective that does not finish within `timeout`
        seconds (a rank that never arrived) aborts the communicator and raises."""
        from . import _lib
        from ._lib import lib
        if self.comm is None:
            self.stream.synchronize()
            return
        status = lib.b200_comm_check(self.comm, self.stream.handle, int(timeout * 1000))
        if status == _lib.NCCL_ERROR:
            raise CollectiveTimeout(_lib.last_error())
        _lib.check(status)

    def fold_prefix(self, op, totals, rank):
        return self.local_mapreduce(None, op, totals.view(0, rank))

    def combine_scalar(self, op, init, holder):
        from .broadcast import Broadcasted, materialize_
        name = {"+": "add", "*": "mul", "max": "max", "min": "min"}[op]
        return materialize_(holder, Broadcasted.call(name, holder.dtype.type(init), holder), self.stream)

    def local_accumulate(self, op, out_shard, shard, carry):
        from ._lib import check, lib
        from .accumulate import accumulate_
        from .array import with_managed
        from .mapreduce import _op_code
        if carry is None:
            return accumulate_(op, out_shard, shard, init=None, stream=self.stream)
        if len(shard) == 0:
            return out_shard
        if carry.dtype != shard.dtype:
            from .broadcast import Broadcasted, materialize_
            from .array import ROCArray
            carry = materialize_(ROCArray(shard.dtype, (1,), stream=self.stream), Broadcasted.leaf(carry.reshape(1)), self.stream)
        tb, ta = out_shard.tensor(), shard.tensor()
        with_managed(self.stream, out_shard, shard, carry)
        check(lib.b200_accumulate_carry(self.stream.handle, C.byref(tb), C.byref(ta), _op_code(op),
                                        C.c_void_p(carry.ptr), 0, 1))
        return out_shard


def prepared_mapreduce_allreduce(peer, expr, op, R, init, stream):
    """Zero-argument callable issuing one fused reduce + all-reduce of `expr` into the one-element
    array `R` (descriptors built once)."""
    from ._lib import check, lib
    from .array import with_managed
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
        with_managed(stream, R, *keep)
        check(fn(peer, stream.handle, C.byref(t), shp, nd, leaves, nleaves, code, ninstr, opc, init_buf))
    return launch


_TRANSPORTS = {"host": 0, "vmm": 1, "ipc": 2}
DEFAULT_TRANSPORT = "vmm"


def _pass_descriptors(rank: int, world: int, handle: bytes, allgather) -> bytes:
    """VMM transport: a file descriptor means nothing outside its process, so every rank serves
    its descriptor on a Unix socket (SCM_RIGHTS) and fetches the descriptors of its peers; the
    handle that comes back names descriptors that are open in THIS process."""
    import array
    import socket
    import struct
    import tempfile
    import threading
    magic, pid, fd, _res, nbytes = struct.unpack_from("<IiiiQ", handle)
    path = os.path.join(tempfile.gettempdir(), f"b200peer-{os.getpid()}-{rank}.sock")
    try:
        os.unlink(path)
    except OSError:
        pass
    srv = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
    srv.bind(path)
    srv.listen(world)

    def serve():
        for _ in range(world - 1):
            conn, _ = srv.accept()
            with conn:
                conn.sendmsg([b"f"], [(socket.SOL_SOCKET, socket.SCM_RIGHTS, array.array("i", [fd]))])
    th = threading.Thread(target=serve, daemon=True)
    th.start()
    infos = allgather((path, handle))                  # also the rendezvous: every server listens by now
    out = bytearray()
    for r, (peer_path, peer_handle) in enumerate(infos):
        if r == rank:
            out += handle.ljust(64, b"\0")[:64]
            continue
        pm, _pp, _pf, _pr, pbytes = struct.unpack_from("<IiiiQ", peer_handle)
        with socket.socket(socket.AF_UNIX, socket.SOCK_STREAM) as c:
            c.connect(peer_path)
            fds = array.array("i")
            _msg, anc, _flags, _addr = c.recvmsg(1, socket.CMSG_LEN(fds.itemsize))
            for level, kind, data in anc:
                if level == socket.SOL_SOCKET and kind == socket.SCM_RIGHTS:
                    fds.frombytes(data[:fds.itemsize])
            if not len(fds):
                raise RuntimeError(f"rank {r} sent no descriptor")
        out += struct.pack("<IiiiQ", pm, os.getpid(), fds[0], 0, pbytes).ljust(64, b"\0")
    th.join(timeout=30)
    srv.close()
    try:
        os.unlink(path)
    except OSError:
        pass
    return bytes(out)


def init_peer(rank: int, world: int, device: int, allgather, transport: str | None = None) -> C.c_void_p:
    """Creates this rank's peer-exchange group.  `allgather(obj) -> list` must return every
    rank's argument in rank order on every rank (any host channel).  `transport` is "vmm" (one
    exported device allocation per rank, mapped by the peers over NVLink; peer access for that
    allocation only), "host" (slots in shared host memory, no GPU maps another GPU) or "ipc" (CUDA
    IPC, enables peer access device wide).  Default: environment B200_PEER_TRANSPORT, else "vmm"
    with "host" as the fallback when any rank cannot export or map device memory - the ranks
    agree on that over `allgather`, so they always end up on the same transport."""
    from . import _lib
    from ._lib import check, lib
    name = (transport or os.environ.get("B200_PEER_TRANSPORT") or "").lower()
    fallback = name == ""
    name = name or DEFAULT_TRANSPORT
    if name not in _TRANSPORTS:
        raise ValueError(f"unknown peer transport {name!r}: use one of {sorted(_TRANSPORTS)}")

    def agree(ok: bool) -> bool:
        """True when the step worked on every rank (one exchange over the host channel)."""
        return all(allgather(bool(ok))) if world > 1 else bool(ok)

    def attempt(kind: str):
        """Create, then connect; after each step the ranks agree on whether all of them got through,
        so that either every rank holds a connected group or none does."""
        peer = C.c_void_p()
        buf = C.create_string_buffer(64)
        status = lib.b200_peer_create(device, rank, world, _TRANSPORTS[kind], C.byref(peer), buf)
        msg = "" if status == _lib.OK else _lib.last_error()
        if not agree(status == _lib.OK):
            if status == _lib.OK:
                lib.b200_peer_destroy(peer)
                status, msg = _lib.UNSUPPORTED, f"another rank could not create a {kind} exchange buffer"
            return None, status, msg
        if world == 1:
            return peer, _lib.OK, ""
        try:
            if kind == "vmm":
                handles = _pass_descriptors(rank, world, buf.raw, allgather)
                try:
                    status = lib.b200_peer_connect(peer, handles)
                finally:
                    import struct
                    for r in range(world):          # the library duplicated what it needed
                        if r != rank:
                            os.close(struct.unpack_from("<IiiiQ", handles, 64 * r)[2])
            else:
                status = lib.b200_peer_connect(peer, b"".join(allgather(buf.raw)))
            msg = "" if status == _lib.OK else _lib.last_error()
        except OSError as e:                          # descriptor passing failed on this rank
            status, msg = _lib.UNSUPPORTED, str(e)
        if not agree(status == _lib.OK):
            lib.b200_peer_destroy(peer)
            if status == _lib.OK:
                status, msg = _lib.UNSUPPORTED, f"another rank could not map the {kind} exchange buffers"
            return None, status, msg
        lib.b200_peer_seal(peer)        # everyone holds its mappings: drop the names they were found by
        return peer, _lib.OK, ""

    peer, status, msg = attempt(name)
    if peer is None and fallback and name != "host":
        peer, status, msg = attempt("host")
    if peer is None:
        raise _lib.B200Error(status, msg)
    return peer


def peer_set_poll_budget(peer, polls: int) -> None:
    from ._lib import check, lib
    check(lib.b200_peer_set_poll_budget(peer, polls))


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
