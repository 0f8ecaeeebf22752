"""The C-ABI library loads and exports every symbol the header declares (no GPU needed)."""
import ctypes as C
import re

import numpy as np
import pytest
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols():
    text = (ROOT / "include" / "b200arrays.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported(pkg):
    names = declared_symbols()
    assert len(names) >= 40
    lib = C.CDLL(str(ROOT / "amdgpu.jl_b200" / "lib" / "libb200arrays.so"))
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, f"declared in include/b200arrays.h but not exported: {missing}"


def test_python_binding_covers_header(pkg):
    bound = set(pkg._lib.SIGNATURES) | {"b200_status_name"}
    assert set(declared_symbols()) <= bound


def test_status_names_and_error_text(pkg):
    lib = pkg._lib
    assert lib.status_name(0) == "B200_OK" and lib.status_name(7) == "B200_LOOKBACK_TIMEOUT"
    # argument validation happens before any device work
    st = lib.lib.b200_stream_sync(None)
    assert st == lib.INVALID_ARG and "null stream" in lib.last_error()


def test_struct_layout_matches_header(pkg):
    lib = pkg._lib
    assert C.sizeof(lib.Tensor) == 8 + 4 + 4 + 8 * 8 * 2
    assert C.sizeof(lib.Leaf) == C.sizeof(lib.Tensor) + 16
    assert C.sizeof(lib.PoolStats) == 80


def test_runtime_compiler_builds_a_kernel_without_a_device(pkg):
    """b200_broadcast_prepare needs NVRTC but no GPU: compile one expression here."""
    import ctypes as C

    class FakeBuffer:
        ptr, freed, stream = 1 << 20, False, None

    x = pkg.ROCArray(np.float32, 4096, _buf=FakeBuffer())
    o = pkg.ROCArray(np.float64, 4096, _buf=FakeBuffer())
    B = pkg.broadcast
    before = B.jit_stats()
    ok = B.precompile(o, B.exp(x.dot) * 2.0 - B.abs_(x.dot))
    after = B.jit_stats()
    if not ok:
        buf = C.create_string_buffer(1024)
        pkg._lib.lib.b200_last_error(buf, 1024)
        assert b"libnvrtc could not be loaded" in buf.value, buf.value      # a compile ERROR is a bug
        pytest.skip("libnvrtc is not installed here")
    assert after["compiled"] == before["compiled"] + 1
    assert B.precompile(o, B.exp(x.dot) * 3.0 - B.abs_(x.dot))               # other scalar: same kernel
    assert B.jit_stats()["compiled"] == after["compiled"]


def test_runtime_compiler_builds_a_reduction_kernel_without_a_device(pkg):
    """The same for mapreduce over an expression: b200_mapreduce_prepare compiles the specialised
    reduction kernel (full reduction and reduction along one dimension)."""
    class FakeBuffer:
        ptr, freed, stream = 1 << 20, False, None

    x = pkg.ROCArray(np.float32, (64, 64), _buf=FakeBuffer())
    y = pkg.ROCArray(np.float32, (64, 64), _buf=FakeBuffer())
    B = pkg.broadcast
    if not B.precompile(pkg.ROCArray(np.float32, (64, 64), _buf=FakeBuffer()), x.dot - y.dot):
        pytest.skip("libnvrtc is not installed here")
    before = B.jit_stats()
    assert pkg.mapreduce_precompile(None, "+", pkg.ROCArray(np.float32, 1, _buf=FakeBuffer()), x.dot * y.dot)
    assert pkg.mapreduce_precompile(None, "max", pkg.ROCArray(np.float32, (1, 64), _buf=FakeBuffer()), B.abs_(x.dot - y.dot))
    after = B.jit_stats()
    assert after["compiled"] == before["compiled"] + 2 and after["failures"] == before["failures"]
    # a plain sum of one dense array needs no compilation
    assert pkg.mapreduce_precompile("identity", "+", pkg.ROCArray(np.float32, 1, _buf=FakeBuffer()), x)
    assert B.jit_stats()["compiled"] == after["compiled"]
