"""The C-ABI library loads and exports every symbol the header declares (no GPU needed)."""
import ctypes as C
import re
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
