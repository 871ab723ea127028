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


def header_prototypes():
    """name -> list of parameter declarations, parsed from the public header."""
    protos = {}
    inc = os.path.join(ROOT, "include")
    for f in sorted(os.listdir(inc)):
        if not f.endswith(".h"):
            continue
        txt = open(os.path.join(inc, f)).read()
        txt = re.sub(r"/\*.*?\*/", "", txt, flags=re.S)
        for m in re.finditer(r"\b(tpx_[a-z0-9_]+)\s*\(([^)]*)\)\s*;", txt, flags=re.S):
            params = [p.strip() for p in m.group(2).split(",")]
            if params == ["void"] or params == [""]:
                params = []
            protos[m.group(1)] = params
    return protos


def test_ctypes_signatures_match_the_header():
    """Every ctypes signature of the Python binding has the header's parameter count, pointers where the header has
    pointers and floats where it has floats: a changed prototype cannot drift away from its binding silently."""
    from tpp_pytorch_extension_b200 import _lib
    protos = header_prototypes()
    checked = 0
    for name, (_, argtypes) in _lib._SIGS.items():
        if name not in protos:
            continue  # debug hooks outside the public header
        params = protos[name]
        assert len(params) == len(argtypes), (name, len(params), len(argtypes))
        for decl, ct in zip(params, argtypes):
            if "*" in decl:
                assert ct is ctypes.c_void_p or ct is ctypes.c_char_p or hasattr(ct, "contents"), (name, decl, ct)
            elif decl.startswith("float"):
                assert ct is ctypes.c_float, (name, decl, ct)
            else:
                assert ct not in (ctypes.c_void_p, ctypes.c_float), (name, decl, ct)
        checked += 1
    assert checked >= 20
    unbound = [n for n in protos if n not in _lib._SIGS]
    assert not unbound, f"header entry points without a Python binding: {unbound}"
