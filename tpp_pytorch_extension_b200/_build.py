"""Builds the CUDA library in-tree with nvcc for sm_100a (cross-compiles without a GPU).

Every csrc/*.cu is compiled to an object under build/ (in parallel, only where the source or a header is newer than the
object) and the objects are linked into libtpx_b200.so beside this file. `TPX_DEBUG=1` in the environment adds
-DTPX_DEBUG, which compiles in the timing-experiment knobs and debug exports; the default build has none of them."""
import concurrent.futures
import glob
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
SO = os.path.join(HERE, "libtpx_b200.so")
OBJ_DIR = os.path.join(HERE, "build")
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
]


def sources():
    return sorted(glob.glob(os.path.join(HERE, "csrc", "*.cu")))


def _headers():
    return glob.glob(os.path.join(HERE, "csrc", "*.cuh")) + glob.glob(os.path.join(HERE, "..", "include", "*.h"))


def _flags():
    return NVCC_FLAGS + (["-DTPX_DEBUG"] if os.environ.get("TPX_DEBUG", "0") == "1" else [])


def _obj(src):
    tag = "dbg" if os.environ.get("TPX_DEBUG", "0") == "1" else "rel"
    return os.path.join(OBJ_DIR, os.path.basename(src)[:-3] + "." + tag + ".o")


def stale():
    if not os.path.exists(SO):
        return True
    t = os.path.getmtime(SO)
    return any(os.path.getmtime(d) > t for d in sources() + _headers())


def build(force=False, verbose=False):
    if not force and not stale():
        return SO
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    os.makedirs(OBJ_DIR, exist_ok=True)
    hdr_t = max(os.path.getmtime(h) for h in _headers())
    todo = []
    for s in sources():
        o = _obj(s)
        if force or not os.path.exists(o) or os.path.getmtime(o) < max(os.path.getmtime(s), hdr_t):
            todo.append((s, o))

    def compile_one(so):
        s, o = so
        cmd = [nvcc] + _flags() + (["-Xptxas", "-v"] if verbose else []) + ["-c", "-o", o, s]
        subprocess.check_call(cmd)

    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        list(ex.map(compile_one, todo))
    subprocess.check_call([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-o", SO] + [_obj(s) for s in sources()])
    return SO


if __name__ == "__main__":
    print(build(force=True, verbose=True))
