"""Counter-based synthetic data on the device (the role of ``AMDGPU.rand!`` / ``randn!``,
src/random.jl:30-70 of the reference, for the benchmark workloads).

Element ``i`` of stream ``stream_id`` is ``draw(key(seed, stream_id), first_index + i)``; the
NumPy restatement :func:`host_draw` gives the same raw 64-bit draws, so uniform, integer and
raw-bit arrays are bit-identical on host and device (normal deviates only statistically:
device libm).
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from ._lib import check, lib
from .array import ROCArray, with_managed
from .runtime import Stream, current_stream

UNIFORM01, UNIFORM11, NORMAL, INTEGERS, RAWBITS, NORMAL_DUP1PCT = range(6)
_M64 = np.uint64(0xFFFFFFFFFFFFFFFF)


def fill_random_(out: ROCArray, dist: int, seed: int, stream_id: int = 0, first_index: int = 0,
                 lo: int = 0, hi: int = 0, stream: Stream | None = None) -> ROCArray:
    t = out.tensor()
    st = with_managed(stream or current_stream(), out)
    check(lib.b200_fill_random(st.handle, C.byref(t), dist, seed, stream_id, first_index, lo, hi))
    return out


def _mix64(z: np.ndarray) -> np.ndarray:
    z = z.astype(np.uint64)
    with np.errstate(over="ignore"):
        z ^= z >> np.uint64(30); z *= np.uint64(0xBF58476D1CE4E5B9)
        z ^= z >> np.uint64(27); z *= np.uint64(0x94D049BB133111EB)
        z ^= z >> np.uint64(31)
    return z


def host_draw(seed: int, stream_id: int, first_index: int, n: int) -> np.ndarray:
    """Raw 64-bit draws, identical to the device generator."""
    with np.errstate(over="ignore"):
        key = _mix64(np.array([np.uint64(seed) + np.uint64(0x9E3779B97F4A7C15) * np.uint64(stream_id + 1)], dtype=np.uint64))[0]
        idx = np.arange(first_index + 1, first_index + n + 1, dtype=np.uint64)
        return _mix64(key + idx * np.uint64(0x9E3779B97F4A7C15))


def host_uniform01(seed, stream_id, first_index, n) -> np.ndarray:
    r = host_draw(seed, stream_id, first_index, n)
    return ((r >> np.uint64(40)).astype(np.float32) * np.float32(2.0 ** -24)).astype(np.float32)


def host_uniform11(seed, stream_id, first_index, n) -> np.ndarray:
    return (np.float32(2.0) * host_uniform01(seed, stream_id, first_index, n) - np.float32(1.0)).astype(np.float32)


def host_integers(seed, stream_id, first_index, n, lo, hi, dtype=np.int32) -> np.ndarray:
    r = host_draw(seed, stream_id, first_index, n)
    return (np.int64(lo) + (r % np.uint64(hi - lo + 1)).astype(np.int64)).astype(dtype)


def host_rawbits(seed, stream_id, first_index, n, dtype=np.uint32) -> np.ndarray:
    return host_draw(seed, stream_id, first_index, n).astype(dtype)
