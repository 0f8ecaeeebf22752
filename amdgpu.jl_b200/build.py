"""Builds libb200arrays.so (sm_100a only) from csrc/*.cu with nvcc, in tree.

The shared object lands in ``lib/`` next to this file so that it travels with the source
tree; nothing is installed into site-packages and nothing is cached outside the tree.
"""
from __future__ import annotations

import hashlib
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
OBJ = HERE / "build"
LIB = HERE / "lib" / "libb200arrays.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-std=c++17", "-O3", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
    "-fmad=false",            # separate multiply/add stay separately rounded (Base semantics)
    "-Xptxas", "-v" if os.environ.get("B200_PTXAS_V") else "-O3",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    raise RuntimeError("nvcc not found")


def _stamp(src: Path) -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    h.update(src.read_bytes())
    for hdr in sorted(CSRC.glob("*.cuh")) + [HERE.parent / "include" / "b200arrays.h"]:
        h.update(hdr.read_bytes())
    return h.hexdigest()


def _write_rtc_sources() -> None:
    """The run-time compiler (csrc/jit.cu) builds its kernels from the evaluator's own sources:
    they are embedded in the library as string literals through this generated include file."""
    def lit(name: str, path: Path) -> str:
        text = path.read_text()
        # one literal per ~8 KB: compilers limit the length of a single string literal
        chunks = [text[i:i + 8000] for i in range(0, len(text), 8000)] or [""]
        body = "\n".join(f'R"b200src({c})b200src"' for c in chunks)
        return f"static const char {name}[] =\n{body};\n"
    out = OBJ / "rtc_sources.inc"
    # of the public header only the types and constants: host prototypes mean nothing to NVRTC
    header = (HERE.parent / "include" / "b200arrays.h").read_text()
    marker = "/* ---- library / device"
    assert marker in header, "b200arrays.h lost the marker that separates types from entry points"
    types_only = OBJ / "b200arrays_types.h"
    types_only.write_text(header[:header.index(marker)] + "#ifdef __cplusplus\n}\n#endif\n#endif\n")
    text = (lit("kRtcCommon", CSRC / "common.cuh") + lit("kRtcProgram", CSRC / "program.cuh")
            + lit("kRtcReduce", CSRC / "reduce_program.cuh") + lit("kRtcHeader", types_only))
    if not out.exists() or out.read_text() != text:
        out.write_text(text)


def _compile_one(src: Path, verbose: bool) -> Path:
    obj = OBJ / (src.stem + ".o")
    stamp = OBJ / (src.stem + ".stamp")
    want = _stamp(src)
    if obj.exists() and stamp.exists() and stamp.read_text() == want:
        return obj
    cmd = [_nvcc(), *NVCC_FLAGS, "-I", str(OBJ), "-c", str(src), "-o", str(obj)]
    if verbose:
        print(" ".join(cmd), flush=True)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stdout}\n{res.stderr}")
    if verbose and res.stderr.strip():
        print(res.stderr, file=sys.stderr)
    stamp.write_text(want)
    return obj


def build_library(verbose: bool = False, force: bool = False) -> Path:
    OBJ.mkdir(parents=True, exist_ok=True)
    LIB.parent.mkdir(exist_ok=True)
    if force:
        for f in OBJ.glob("*.stamp"):
            f.unlink()
    _write_rtc_sources()
    srcs = sorted(CSRC.glob("*.cu"))
    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        objs = list(ex.map(lambda s: _compile_one(s, verbose), srcs))
    newest = max(o.stat().st_mtime for o in objs)
    if LIB.exists() and LIB.stat().st_mtime >= newest and not force:
        return LIB
    cmd = [_nvcc(), "-shared", "-o", str(LIB), *map(str, objs),
           "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC", "-ldl", "-lpthread"]
    if verbose:
        print(" ".join(cmd), flush=True)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return LIB


if __name__ == "__main__":
    print(build_library(verbose=True, force="--force" in sys.argv))
