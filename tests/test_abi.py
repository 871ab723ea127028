"""CPU test: the C-ABI library loads and exports every symbol the public header declares."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = []
    inc = os.path.join(ROOT, "include")
    for f in sorted(os.listdir(inc)):
        if f.endswith(".h"):
            txt = open(os.path.join(inc, f)).read()
            txt = re.sub(r"/\*.*?\*/", "", txt, flags=re.S)
            names += re.findall(r"\b(tpx_[a-z0-9_]+)\s*\(", txt)
    return sorted(set(names))


def test_library_exports_header_symbols():
    from tpp_pytorch_extension_b200 import _build
    so = _build.build()
    L = ctypes.CDLL(so)
    names = declared_symbols()
    assert len(names) >= 10
    missing = [n for n in names if not hasattr(L, n)]
    assert not missing, missing
    L.tpx_version.restype = ctypes.c_int
    assert L.tpx_version() >= 100


def test_argument_errors_are_reported_not_fatal():
    """Bad arguments come back as status codes with a message (the reference exits the process)."""
    from tpp_pytorch_extension_b200 import _lib
    L = _lib.lib()
    rc = L.tpx_packed_bytes(1, 30, 128, 32, None, None)
    assert rc == 1 and b"multiple of 16" in L.tpx_last_error()
    rc = L.tpx_qlinear(7, None, None, None, None, 32, None, 1, 16, 64, None, 0, None, None, 1.0, None, None, 0, None)
    assert rc == 1 and b"unknown weight kind" in L.tpx_last_error()
    rc = L.tpx_qlinear(1, None, None, None, None, 32, None, 0, 16, 64, None, 0, None, None, 1.0, None, None, 0, None)
    assert rc == 0, L.tpx_last_error()  # an empty batch is a no-op
