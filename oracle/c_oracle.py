"""ctypes access to the C restatement (checker and CPU-baseline timing only)."""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
SO = HERE / "build" / "libbase_oracle.so"


def load():
    if not SO.exists():
        subprocess.run(["make", "-s", "-C", str(HERE)], check=True)
    lib = C.CDLL(str(SO))
    f32p, i32p, u32p, i64p = (C.POINTER(C.c_float), C.POINTER(C.c_int32), C.POINTER(C.c_uint32), C.POINTER(C.c_int64))
    lib.ora_max_threads.restype = C.c_int
    lib.ora_axpy_f32.argtypes = [C.c_float, f32p, f32p, f32p, C.c_int64, C.c_int]
    lib.ora_muladd_exp_f32.argtypes = [f32p, f32p, f32p, f32p, C.c_int64, C.c_int]
    lib.ora_sum_f32.argtypes = [f32p, C.c_int64, C.c_int, C.c_int]
    lib.ora_sum_f32.restype = C.c_float
    lib.ora_sum_f64acc.argtypes = [f32p, C.c_int64, C.c_int, C.c_int]
    lib.ora_sum_f64acc.restype = C.c_double
    lib.ora_cumsum_f32.argtypes = [f32p, f32p, C.c_int64]
    lib.ora_cumsum_i32.argtypes = [i32p, i32p, C.c_int64]
    lib.ora_cumsum_i32_mt.argtypes = [i32p, i32p, C.c_int64, C.c_int]
    lib.ora_sort_u32.argtypes = [u32p, C.c_int64]
    lib.ora_sortperm_f32.argtypes = [f32p, i64p, C.c_int64]
    return lib


def ptr(a: np.ndarray, ctype):
    return a.ctypes.data_as(C.POINTER(ctype))
