"""Host-side failure detection of the collective layer (b200_comm_check) against a stand-in for
libnccl (tests/stubs/nccl_stub.c) whose health state the test scripts.  No GPU and no peer is
involved: an asynchronous error or a collective that never finishes is reported as a status and
the communicator is aborted, nothing hangs."""
import ctypes as C
import subprocess
import sys
import textwrap
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent

CHILD = textwrap.dedent("""
    import ctypes as C, sys
    sys.path.insert(0, {root!r})
    import __graft_entry__ as entry
    pkg = entry.load_package()
    L = pkg._lib
    stub = C.CDLL({stub!r}, mode=C.RTLD_GLOBAL)
    ident = C.create_string_buffer(128)
    L.check(L.lib.b200_comm_unique_id(ident))
    assert ident.raw == bytes([7]) * 128                      # the stand-in answered, not a real NCCL
    comm = C.c_void_p()
    L.check(L.lib.b200_comm_init_rank(C.byref(comm), 2, 0, ident.raw, -1))   # not bound to a device
    # healthy communicator
    assert L.lib.b200_comm_check(comm, None, 50) == L.OK
    # NCCL still working on something when the time is up: not an error while no stream is watched
    stub.stub_script(7)
    assert L.lib.b200_comm_check(comm, None, 30) == L.NOT_READY
    assert stub.stub_aborts() == 0
    # a peer died: the asynchronous error surfaces, the communicator is aborted
    stub.stub_script(6)
    assert L.lib.b200_comm_check(comm, None, 1000) == L.NCCL_ERROR
    assert "aborted" in L.last_error() and stub.stub_aborts() == 1
    # afterwards only destroy is accepted
    assert L.lib.b200_comm_check(comm, None, 10) == L.NCCL_ERROR
    assert L.lib.b200_allreduce(comm, None, 1, L.F32, L.RED_ADD, None) == L.NCCL_ERROR
    L.check(L.lib.b200_comm_destroy(comm))
    assert stub.stub_destroys() == 0 and stub.stub_aborts() == 1   # an aborted communicator is not destroyed twice
    print("comm-check-ok")
""")


def test_comm_check_against_stub_nccl(pkg, tmp_path):
    stub = tmp_path / "libnccl_stub.so"
    subprocess.run(["gcc", "-shared", "-fPIC", "-O1", "-o", str(stub), str(ROOT / "tests" / "stubs" / "nccl_stub.c")], check=True)
    env = dict(__import__("os").environ, B200_NCCL_LIB=str(stub))
    res = subprocess.run([sys.executable, "-c", CHILD.format(root=str(ROOT), stub=str(stub))],
                         capture_output=True, text=True, env=env, timeout=300)
    assert res.returncode == 0 and "comm-check-ok" in res.stdout, res.stdout + res.stderr
