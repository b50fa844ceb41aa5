"""Builds the library's CUDA sources into ``pippy_b200/lib/libpippy_b200.so`` with plain nvcc.

The kernels are exported with C linkage and called through ctypes, so the build needs neither the
PyTorch headers nor a GPU: nvcc cross-compiles for sm_100a in a few seconds per file.
"""
from __future__ import annotations

import hashlib
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

CSRC = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(CSRC)
LIB_DIR = os.path.join(PKG, "lib")
LIB_PATH = os.path.join(LIB_DIR, "libpippy_b200.so")
OBJ_DIR = os.path.join(LIB_DIR, "obj")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]
# Debug build (``build_all(debug=True)`` or PIPPY_BOUNDS_CHECK=1): kernels validate indices they read from tensors and
# report violations through the device error word instead of reading out of bounds (csrc/dbgcheck.cuh).  It is a
# second library, libpippy_b200_dbg.so, with its own object directory; ops._lib loads it when PIPPY_BOUNDS_CHECK=1.
DEBUG_FLAGS = ["-DPB_BOUNDS_CHECK"]
DEBUG_LIB_PATH = os.path.join(LIB_DIR, "libpippy_b200_dbg.so")
DEBUG_OBJ_DIR = os.path.join(LIB_DIR, "obj_dbg")


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def sources() -> list[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _digest(path: str, flags=None) -> str:
    h = hashlib.sha1()
    for dep in [path] + sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))):
        with open(dep, "rb") as f:
            h.update(f.read())
    h.update(" ".join(flags if flags is not None else NVCC_FLAGS).encode())
    return h.hexdigest()


def _compile_one(src: str, verbose: bool, ptxas_v: bool, obj_dir: str = OBJ_DIR, flags=None) -> str:
    flags = list(NVCC_FLAGS) if flags is None else flags
    os.makedirs(obj_dir, exist_ok=True)
    obj = os.path.join(obj_dir, os.path.basename(src)[:-3] + ".o")
    stamp = obj + ".sha1"
    dig = _digest(src, flags)
    if os.path.exists(obj) and os.path.exists(stamp) and open(stamp).read() == dig:
        return obj
    cmd = [_nvcc(), *flags, "-c", src, "-o", obj]
    if ptxas_v:
        cmd[1:1] = ["-Xptxas", "-v"]
    if verbose:
        print(" ".join(cmd), flush=True)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{res.stdout}\n{res.stderr}")
    if ptxas_v:
        print(res.stderr, flush=True)
    with open(stamp, "w") as f:
        f.write(dig)
    return obj


def build_all(verbose: bool = False, ptxas_v: bool = False, force: bool = False, debug: bool = False) -> str:
    """Compile every ``.cu`` under csrc/ for sm_100a and link the shared library (with ``debug`` the bounds-checking
    one). Returns its path."""
    lib_path, obj_dir = (DEBUG_LIB_PATH, DEBUG_OBJ_DIR) if debug else (LIB_PATH, OBJ_DIR)
    flags = NVCC_FLAGS + DEBUG_FLAGS if debug else list(NVCC_FLAGS)
    os.makedirs(LIB_DIR, exist_ok=True)
    if force and os.path.isdir(obj_dir):
        for f in os.listdir(obj_dir):
            os.remove(os.path.join(obj_dir, f))
    srcs = sources()
    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        objs = list(ex.map(lambda s: _compile_one(s, verbose, ptxas_v, obj_dir, flags), srcs))
    newest = max(os.path.getmtime(o) for o in objs)
    if not os.path.exists(lib_path) or os.path.getmtime(lib_path) < newest or force:
        cmd = [_nvcc(), "-shared", "-o", lib_path, *objs, "-gencode", "arch=compute_100a,code=sm_100a"]
        if verbose:
            print(" ".join(cmd), flush=True)
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return lib_path


if __name__ == "__main__":
    want_debug = "--debug" in sys.argv or os.environ.get("PIPPY_BOUNDS_CHECK", "0") == "1"
    path = build_all(verbose=True, ptxas_v="-v" in sys.argv, force="--force" in sys.argv, debug=want_debug)
    print("built", path)
