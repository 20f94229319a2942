"""Build the CUDA kernel library (``shadow_b200/lib/libsb200.so``) and the C++ host library
(``shadow_b200/lib/libshadow_b200.so``) in-tree with nvcc / g++ for sm_100a, and the NCCL combine library
(``shadow_b200/lib/libsb200_nccl.so``).

    python -m shadow_b200.build [--force]
"""
from __future__ import annotations

import concurrent.futures as cf
import glob
import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
HOST = os.path.join(PKG, "host")
LIB_DIR = os.path.join(PKG, "lib")
OBJ_DIR = os.path.join(PKG, "build")
KERNEL_LIB = os.path.join(LIB_DIR, "libsb200.so")
HOST_LIB = os.path.join(LIB_DIR, "libshadow_b200.so")
COMM_LIB = os.path.join(LIB_DIR, "libsb200_nccl.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    # IEEE arithmetic: no fast-math; FMA contraction is irrelevant for the parity-critical code
    # (it uses explicit __f*_rn intrinsics) but is disabled anyway so that nothing depends on it.
    "-fmad=false", "-prec-div=true", "-prec-sqrt=true", "-ftz=false",
    "-Xcompiler", "-fPIC", "-I" + os.path.join(REPO, "include"),
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found")
    return exe


def _run(cmd):
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("command failed: %s\n%s\n%s" % (" ".join(cmd), proc.stdout, proc.stderr))
    return proc.stdout + proc.stderr


def _stale(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def build_kernels(force: bool = False, verbose: bool = False) -> str:
    srcs = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    deps = srcs + glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(REPO, "include", "*.h"))
    if not force and not _stale(KERNEL_LIB, deps + [os.path.abspath(__file__)]):
        return KERNEL_LIB
    os.makedirs(LIB_DIR, exist_ok=True)
    os.makedirs(OBJ_DIR, exist_ok=True)
    nvcc = _nvcc()

    def one(src):
        obj = os.path.join(OBJ_DIR, os.path.basename(src)[:-3] + ".o")
        out = _run([nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", src, "-o", obj])
        if verbose:
            print(out)
        return obj

    with cf.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 4)) as pool:
        objs = list(pool.map(one, srcs))
    _run([nvcc, "-shared", "-o", KERNEL_LIB] + objs + ["-gencode", "arch=compute_100a,code=sm_100a"])
    return KERNEL_LIB


def build_host(force: bool = False) -> str | None:
    srcs = sorted(glob.glob(os.path.join(HOST, "*.cpp")) + glob.glob(os.path.join(HOST, "src", "*.cpp")))
    if not os.path.isdir(os.path.join(HOST, "shadow")):
        return None
    deps = srcs + glob.glob(os.path.join(HOST, "shadow", "**", "*.hpp"), recursive=True) + \
        glob.glob(os.path.join(REPO, "include", "*.h"))
    if not force and not _stale(HOST_LIB, deps + [os.path.abspath(__file__), KERNEL_LIB]):
        return HOST_LIB
    os.makedirs(LIB_DIR, exist_ok=True)
    os.makedirs(OBJ_DIR, exist_ok=True)
    cuda_home = os.path.dirname(os.path.dirname(_nvcc()))
    # SHADOW_CAPI_PRODUCT_EXTENSIONS: adapter entry points that exist only on this library's side
    # (binary model parsing, NetParam dump); the reference-side build of the adapter omits them
    flags = ["-O2", "-std=c++17", "-fPIC", "-Wall", "-DSHADOW_CAPI_PRODUCT_EXTENSIONS", "-I" + os.path.join(HOST, "shadow"),
             "-I" + os.path.join(REPO, "include"), "-I" + os.path.join(cuda_home, "include")]

    def one(src):
        obj = os.path.join(OBJ_DIR, "host_" + os.path.basename(src)[:-4] + ".o")
        _run(["g++"] + flags + ["-c", src, "-o", obj])
        return obj

    with cf.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 4)) as pool:
        objs = list(pool.map(one, srcs))
    _run(["g++", "-shared", "-o", HOST_LIB] + objs +
         ["-L" + LIB_DIR, "-lsb200", "-Wl,-rpath,$ORIGIN", "-L" + os.path.join(cuda_home, "lib64"),
          "-lcudart_static", "-ldl", "-lrt", "-lpthread"])
    return HOST_LIB


def _nccl_paths():
    """(include dir, library file) of an NCCL to build against: the system one, else the copy that
    ships inside the Python environment (the soname is libnccl.so.2 either way, so at run time the
    process's already loaded NCCL - torch's, in a Python job - is the one that is used)."""
    candidates = [("/usr/include", "/usr/lib/x86_64-linux-gnu/libnccl.so.2")]
    for base in sys.path:
        candidates.append((os.path.join(base, "nvidia", "nccl", "include"), os.path.join(base, "nvidia", "nccl", "lib", "libnccl.so.2")))
    for inc, lib in candidates:
        if os.path.exists(os.path.join(inc, "nccl.h")) and os.path.exists(lib):
            return inc, lib
    return None


def build_comm(force: bool = False) -> str | None:
    """libsb200_nccl.so: the cross-GPU combine entry points (include/sb200_nccl.h).  None when no
    NCCL header/library is installed."""
    src = os.path.join(PKG, "comm", "sb200_nccl.cpp")
    nccl = _nccl_paths()
    if nccl is None or not os.path.exists(src):
        return None
    deps = [src, KERNEL_LIB, os.path.abspath(__file__)] + glob.glob(os.path.join(REPO, "include", "*.h"))
    if not force and not _stale(COMM_LIB, deps):
        return COMM_LIB
    cuda_home = os.path.dirname(os.path.dirname(_nvcc()))
    _run(["g++", "-O2", "-std=c++17", "-fPIC", "-Wall", "-shared", "-o", COMM_LIB, src,
          "-I" + os.path.join(REPO, "include"), "-I" + os.path.join(cuda_home, "include"), "-I" + nccl[0],
          "-L" + LIB_DIR, "-lsb200", "-Wl,-rpath,$ORIGIN", nccl[1], "-L" + os.path.join(cuda_home, "lib64"), "-lcudart"])
    return COMM_LIB


def build_all(force: bool = False, verbose: bool = False):
    return {"kernels": build_kernels(force, verbose), "host": build_host(force), "comm": build_comm(force)}


if __name__ == "__main__":
    print(build_all(force="--force" in sys.argv, verbose="-v" in sys.argv))
