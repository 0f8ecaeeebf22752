"""ctypes binding of libb200arrays.so (declarations follow include/b200arrays.h).

There is no CPU fallback: if the shared library is missing or was built without the CUDA
kernels, importing this module raises.  Every call goes through :func:`check`, which turns a
non-zero status into :class:`B200Error` the way the reference's ``@check`` macro turns a
``hipError_t`` into ``HIPError`` (src/hip/error.jl:143-161).
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import numpy as np

try:  # bfloat16 host representation
    import ml_dtypes
    bfloat16 = np.dtype(ml_dtypes.bfloat16)
except Exception:  # pragma: no cover - ml_dtypes ships with the image
    bfloat16 = None

import os

LIB_PATH = Path(os.environ.get("B200ARRAYS_LIB") or Path(__file__).resolve().parent / "lib" / "libb200arrays.so")

# status codes
OK, NOT_READY, INVALID_ARG, UNSUPPORTED, OOM, CUDA_ERROR, NCCL_ERROR, LOOKBACK_TIMEOUT, NOT_INITIALISED, TOO_LARGE = range(10)

# element types
F16, BF16, F32, F64, I8, I16, I32, I64, U8, U16, U32, U64, BOOL = range(13)
_NP2DT = {
    np.dtype(np.float16): F16, np.dtype(np.float32): F32, np.dtype(np.float64): F64,
    np.dtype(np.int8): I8, np.dtype(np.int16): I16, np.dtype(np.int32): I32, np.dtype(np.int64): I64,
    np.dtype(np.uint8): U8, np.dtype(np.uint16): U16, np.dtype(np.uint32): U32, np.dtype(np.uint64): U64,
    np.dtype(np.bool_): BOOL,
}
if bfloat16 is not None:
    _NP2DT[bfloat16] = BF16
_DT2NP = {v: k for k, v in _NP2DT.items()}

# opcodes
OP_LEAF, OP_CONVERT, OP_ADD, OP_SUB, OP_MUL, OP_DIV, OP_MULADD, OP_ABS, OP_ABS2, OP_EXP, OP_MAX, OP_MIN, OP_NEG = range(13)
RED_ADD, RED_MUL, RED_MAX, RED_MIN = range(4)
PEER_HOST, PEER_VMM, PEER_IPC = range(3)

MAX_DIMS, MAX_LEAVES, MAX_PROGRAM = 8, 8, 64


def dtype_code(dt) -> int:
    dt = np.dtype(dt)
    try:
        return _NP2DT[dt]
    except KeyError:
        raise TypeError(f"element type {dt} is not supported by the B200 array backend") from None


def dtype_numpy(code: int) -> np.dtype:
    return _DT2NP[code]


class Tensor(C.Structure):
    _fields_ = [("ptr", C.c_void_p), ("dtype", C.c_int32), ("ndim", C.c_int32),
                ("shape", C.c_int64 * MAX_DIMS), ("stride", C.c_int64 * MAX_DIMS)]


class Leaf(C.Structure):
    _fields_ = [("t", Tensor), ("is_scalar", C.c_int32), ("_pad", C.c_int32), ("scalar", C.c_uint64)]


class PoolStats(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in (
        "alloc_count", "free_count", "alloc_bytes", "free_bytes", "live_bytes", "peak_live_bytes",
        "pool_reserved", "pool_used", "hard_limit", "soft_limit")]


class Props(C.Structure):
    _fields_ = [("name", C.c_char * 128), ("cc_major", C.c_int32), ("cc_minor", C.c_int32),
                ("sm_count", C.c_int32), ("l2_bytes_mb", C.c_int32), ("total_mem", C.c_uint64),
                ("max_smem_per_block", C.c_int32), ("clock_khz", C.c_int32)]


class B200Error(RuntimeError):
    """Raised for every non-zero status (mirrors HIPError, src/hip/error.jl:1-10)."""

    def __init__(self, code: int, msg: str):
        super().__init__(f"B200Error(code {code} {status_name(code)}, {msg})")
        self.code = code
        self.msg = msg


class OutOfMemoryError(B200Error):
    pass


if not LIB_PATH.exists():
    raise ImportError(
        f"{LIB_PATH} is missing: build it with `python -c 'import __graft_entry__ as g; g.build()'`. "
        "This backend has no CPU fallback.")

lib = C.CDLL(str(LIB_PATH))

_vp, _i32, _i64, _u64, _sz = C.c_void_p, C.c_int32, C.c_int64, C.c_uint64, C.c_size_t
_P = C.POINTER
SIGNATURES = {
    "b200_init": [],
    "b200_device_count": [_P(_i32)],
    "b200_device_props": [_i32, _P(Props)],
    "b200_can_access_peer": [_i32, _i32, _P(_i32)],
    "b200_last_error": [C.c_char_p, _sz],
    "b200_version": [_P(_i32), _P(_i32), _P(_i32)],
    "b200_device_sync": [_i32],
    "b200_stream_create": [_i32, _i32, _P(_vp)],
    "b200_stream_wrap": [_i32, _vp, _P(_vp)],
    "b200_stream_destroy": [_vp],
    "b200_stream_sync": [_vp],
    "b200_stream_release_scratch": [_vp],
    "b200_stream_query": [_vp],
    "b200_stream_device": [_vp, _P(_i32)],
    "b200_stream_raw": [_vp, _P(_vp)],
    "b200_event_create": [_i32, _i32, _P(_vp)],
    "b200_event_destroy": [_vp],
    "b200_event_record": [_vp, _vp],
    "b200_event_sync": [_vp],
    "b200_event_query": [_vp],
    "b200_event_elapsed_ms": [_vp, _vp, _P(C.c_float)],
    "b200_stream_wait_event": [_vp, _vp],
    "b200_pool_configure": [_i32, _u64, _u64],
    "b200_malloc_async": [_P(_vp), _sz, _vp],
    "b200_free_async": [_vp, _vp],
    "b200_pool_trim": [_i32, _sz],
    "b200_pool_stats": [_i32, _P(PoolStats)],
    "b200_mem_info": [_i32, _P(_sz), _P(_sz)],
    "b200_memcpy_async": [_vp, _vp, _sz, _vp],
    "b200_memset_async": [_vp, _u64, _i32, _sz, _vp],
    "b200_host_alloc": [_P(_vp), _sz],
    "b200_host_free": [_vp],
    "b200_host_register": [_vp, _sz, _P(_vp)],
    "b200_host_unregister": [_vp],
    "b200_broadcast": [_vp, _P(Tensor), _P(Leaf), _i32, C.c_char_p, _i32],
    "b200_broadcast_prepare": [_P(Tensor), _P(Leaf), _i32, C.c_char_p, _i32],
    "b200_jit_configure": [_i32],
    "b200_jit_stats": [_P(C.c_uint64)],
    "b200_mapreduce": [_vp, _P(Tensor), _P(_i64), _i32, _P(Leaf), _i32, C.c_char_p, _i32, _i32, _vp],
    "b200_mapreduce_prepare": [_P(Tensor), _P(_i64), _i32, _P(Leaf), _i32, C.c_char_p, _i32, _i32],
    "b200_accumulate": [_vp, _P(Tensor), _P(Tensor), _i32, _vp, _i32, _i32],
    "b200_accumulate_carry": [_vp, _P(Tensor), _P(Tensor), _i32, _vp, _i32, _i32],
    "b200_accumulate_noalloc": [_vp, _P(Tensor), _P(Tensor), _i32, _vp, _i32, _i32],
    "b200_sort": [_vp, _P(Tensor), _i32],
    "b200_sortperm": [_vp, _P(Tensor), _P(Tensor), _i32],
    "b200_compact": [_vp, _P(Tensor), _P(Tensor), _P(Tensor), _P(Tensor)],
    "b200_reverse": [_vp, _P(Tensor), _P(Tensor), C.c_uint32],
    "b200_gather": [_vp, _P(Tensor), _P(Tensor), _P(Tensor)],
    "b200_graph_capture_begin": [_vp, C.c_int32],
    "b200_graph_capture_end": [_vp, _P(_vp)],
    "b200_stream_is_capturing": [_vp, _P(C.c_int32)],
    "b200_graph_destroy": [_vp],
    "b200_graph_instantiate": [_vp, _P(_vp)],
    "b200_graph_exec_destroy": [_vp],
    "b200_graph_launch": [_vp, _vp],
    "b200_graph_exec_update": [_vp, _vp, _P(C.c_int32)],
    "b200_fill_random": [_vp, _P(Tensor), _i32, _u64, _u64, _u64, _i64, _i64],
    "b200_selftest_wait_timeout": [_vp, C.c_uint32],
    "b200_peer_create": [_i32, _i32, _i32, _i32, _P(_vp), C.c_char_p],
    "b200_peer_connect": [_vp, C.c_char_p],
    "b200_peer_seal": [_vp],
    "b200_peer_set_poll_budget": [_vp, C.c_uint32],
    "b200_peer_info": [_vp, _P(_i32), _P(_u64)],
    "b200_peer_destroy": [_vp],
    "b200_mapreduce_allreduce": [_vp, _vp, _P(Tensor), _P(_i64), _i32, _P(Leaf), _i32, C.c_char_p, _i32, _i32, _vp],
    "b200_comm_unique_id": [C.c_char_p],
    "b200_comm_init_rank": [_P(_vp), _i32, _i32, C.c_char_p, _i32],
    "b200_comm_destroy": [_vp],
    "b200_comm_check": [_vp, _vp, _i32],
    "b200_allreduce": [_vp, _vp, _sz, _i32, _i32, _vp],
    "b200_allgather": [_vp, _vp, _vp, _sz, _i32, _vp],
}
for _name, _args in SIGNATURES.items():
    _fn = getattr(lib, _name)   # AttributeError here means header and library disagree
    _fn.argtypes = _args
    _fn.restype = _i32
lib.b200_status_name.argtypes = [_i32]
lib.b200_status_name.restype = C.c_char_p


def status_name(code: int) -> str:
    return lib.b200_status_name(code).decode()


def last_error() -> str:
    buf = C.create_string_buffer(512)
    lib.b200_last_error(buf, 512)
    return buf.value.decode(errors="replace")


def check(status: int) -> int:
    if status == OK or status == NOT_READY:
        return status
    msg = last_error()
    if status == OOM:
        raise OutOfMemoryError(status, msg)
    raise B200Error(status, msg)
