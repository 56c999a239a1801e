"""In-tree build of the native library ``fastfold_b200/lib/libffb200.so``.

Every ``csrc/*.cu`` is compiled for sm_100a only (``-gencode
arch=compute_100a,code=sm_100a``) with relocatable device code and linked into
one shared object that the Python side loads through ``ctypes``.  The sources
do not include PyTorch headers, so a full rebuild takes well under a minute
and the result has no ABI tie to a particular PyTorch build.

Replaces the reference's ``setup.py`` CUDAExtension build (setup.py:89-125),
which targets sm_70/sm_80.
"""
import hashlib
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIBDIR = os.path.join(HERE, "lib")
LIBNAME = "libffb200.so"
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-rdc=true", "-Xcompiler", "-fPIC", "-Xptxas", "-v",
]


def _nvcc():
    cand = os.environ.get("NVCC") or os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    return cand if os.path.exists(cand) else "nvcc"


def sources():
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _digest():
    h = hashlib.sha256()
    for f in sorted(os.listdir(CSRC)):
        if f.endswith((".cu", ".cuh", ".h")):
            with open(os.path.join(CSRC, f), "rb") as fh:
                h.update(f.encode())
                h.update(fh.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def lib_path():
    return os.path.join(LIBDIR, LIBNAME)


def is_current():
    stamp = os.path.join(LIBDIR, "build.stamp")
    if not (os.path.exists(lib_path()) and os.path.exists(stamp)):
        return False
    with open(stamp) as fh:
        return fh.read().strip() == _digest()


def build(force=False, verbose=True):
    """Compile and link; returns the path of the shared object."""
    if not force and is_current():
        return lib_path()
    os.makedirs(LIBDIR, exist_ok=True)
    objdir = os.path.join(LIBDIR, "obj")
    os.makedirs(objdir, exist_ok=True)
    nvcc = _nvcc()
    srcs = sources()
    logs = {}

    def compile_one(src):
        obj = os.path.join(objdir, os.path.basename(src)[:-3] + ".o")
        cmd = [nvcc] + NVCC_FLAGS + ["-I", CSRC, "-c", src, "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        logs[src] = r.stdout + r.stderr
        if r.returncode != 0:
            raise RuntimeError("nvcc failed for %s:\n%s" % (src, logs[src]))
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        objs = list(ex.map(compile_one, srcs))
    link = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "--shared", "-Xcompiler", "-fPIC",
            "-o", lib_path()] + objs + ["-lcudart"]
    r = subprocess.run(link, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("link failed:\n" + r.stdout + r.stderr)
    with open(os.path.join(LIBDIR, "ptxas.log"), "w") as fh:
        for s in srcs:
            fh.write("==== %s\n%s\n" % (os.path.basename(s), logs[s]))
    with open(os.path.join(LIBDIR, "build.stamp"), "w") as fh:
        fh.write(_digest())
    if verbose:
        print("built", lib_path())
    return lib_path()


if __name__ == "__main__":
    build(force="--force" in sys.argv)
