"""Build recipe for the parity oracle.  TEST INFRASTRUCTURE ONLY: nothing the product ships
imports, links or executes anything under oracle/.

Two artefacts:

* ``oracle/liboracle_port.so``  - the plain-C restatement of the reference's CPU algorithms
  (``oracle/oracle_port.c``), always buildable (gcc only).
* ``oracle/_ref/libshadow_ref.so`` - the reference's own CPU ``Default`` kernels, compiled from
  the sources where they lie (the checkout named by ``$SHADOW_REFERENCE_ROOT``, by default the directory
  ``reference`` beside this repository) with no
  ``USE_*`` define (plain-loop kernels, glibc libm, no Eigen/DNNL/NNPACK, CPUContext only),
  plus the C adapter ``shadow_b200/host/net_capi.cpp`` compiled against the reference's headers
  with the symbol prefix ``sref_``.  Built only when the reference tree is present; a machine
  without it uses the prebuilt file.  No reference source is copied: the one generated file the
  reference's CMake would write into its tree (``core/config.hpp`` from ``config.hpp.in``,
  version 0.1.0, no ``USE_Protobuf``) is written to ``oracle/_gen/`` and found through ``-I``.

Flags mirror the reference's Release build (``CMakeLists.txt:32-38``: ``-std=c++11 -fPIC``, -O3,
NDEBUG; no ``-march``, no ``-ffast-math``, no OpenMP).  ``-include cstdint`` is needed because
``shadow/core/blob.hpp`` uses ``std::int64_t`` without including ``<cstdint>``.
"""
from __future__ import annotations

import concurrent.futures as cf
import glob
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(HERE)
REF_ROOT = os.environ.get("SHADOW_REFERENCE_ROOT", os.path.join(os.path.dirname(REPO), "reference"))
REF_DIR = os.path.join(HERE, "_ref")
GEN_DIR = os.path.join(HERE, "_gen")
REF_LIB = os.path.join(REF_DIR, "libshadow_ref.so")
REF_GPU_LIB = os.path.join(REF_DIR, "libshadow_ref_b200.so")
PORT_LIB = os.path.join(HERE, "liboracle_port.so")

CONFIG_HPP = """#ifndef SHADOW_CORE_CONFIG_HPP_
#define SHADOW_CORE_CONFIG_HPP_
#define SHADOW_VERSION_MAJOR 0
#define SHADOW_VERSION_MINOR 1
#define SHADOW_VERSION_PATCH 0
#define SHADOW_VERSION_STRING "0.1.0"
#endif
"""


def _run(cmd: list[str]) -> None:
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("command failed: %s\n%s\n%s" % (" ".join(cmd), proc.stdout, proc.stderr))


def _newer(target: str, sources: list[str]) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources if os.path.exists(s))


def build_port(force: bool = False) -> str:
    """Compile the C restatement.  -O2 without -ffast-math / -march so the arithmetic is plain
    IEEE single/double with no FMA contraction (-ffp-contract=off), like the reference build."""
    src = os.path.join(HERE, "oracle_port.c")
    if not force and _newer(PORT_LIB, [src]):
        return PORT_LIB
    _run(["gcc", "-O2", "-std=c11", "-fPIC", "-shared", "-ffp-contract=off", "-fno-fast-math",
          "-o", PORT_LIB, src, "-lm"])
    return PORT_LIB


def reference_available() -> bool:
    return os.path.isdir(os.path.join(REF_ROOT, "shadow", "core"))


def build_ref(force: bool = False) -> str | None:
    """Compile the reference CPU library + the sref_ adapter into oracle/_ref/.  Returns the
    path, or None when the reference tree is absent and no prebuilt library exists."""
    if not reference_available():
        return REF_LIB if os.path.exists(REF_LIB) else None
    shadow = os.path.join(REF_ROOT, "shadow")
    shim = os.path.join(REPO, "shadow_b200", "host", "net_capi.cpp")
    sources = []
    for pat in ("core/*.cpp", "operators/*.cpp", "operators/kernels/*.cpp"):
        sources += sorted(glob.glob(os.path.join(shadow, pat)))
    sources += [os.path.join(shadow, p) for p in
                ("backends/native/native.cpp", "util/io.cpp", "util/json.cpp", "util/boxes.cpp")]
    if not force and _newer(REF_LIB, sources + [shim, os.path.abspath(__file__)]):
        return REF_LIB
    os.makedirs(REF_DIR, exist_ok=True)
    os.makedirs(GEN_DIR, exist_ok=True)
    with open(os.path.join(GEN_DIR, "config.hpp"), "w") as f:
        f.write(CONFIG_HPP)
    obj_dir = os.path.join(GEN_DIR, "obj")
    os.makedirs(obj_dir, exist_ok=True)
    flags = ["-O3", "-DNDEBUG", "-std=c++11", "-fPIC", "-include", "cstdint", "-w",
             "-I" + shadow, "-I" + GEN_DIR]

    def compile_one(item):
        idx, src = item
        obj = os.path.join(obj_dir, "%03d_%s.o" % (idx, os.path.basename(src)[:-4]))
        _run(["g++"] + flags + ["-c", src, "-o", obj])
        return obj

    with cf.ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as pool:
        objs = list(pool.map(compile_one, enumerate(sources)))
    shim_obj = os.path.join(obj_dir, "net_capi_sref.o")
    _run(["g++"] + flags + ["-DSHADOW_CAPI_PREFIX=sref_", "-I" + os.path.join(REPO, "include"),
                            "-c", shim, "-o", shim_obj])
    # -Bsymbolic + a version script: only the sref_ adapter is visible, so the library can sit in
    # one process with other code that also defines `namespace Shadow` symbols.
    vers = os.path.join(GEN_DIR, "sref.map")
    with open(vers, "w") as f:
        f.write("{ global: sref_*; local: *; };\n")
    _run(["g++", "-shared", "-o", REF_LIB] + objs + [shim_obj,
         "-Wl,-Bsymbolic", "-Wl,--version-script=" + vers, "-ldl"])
    return REF_LIB


def build_ref_gpu(force: bool = False) -> str | None:
    """The reference's own host stack - Network, NetworkImpl, the Native backend, the operator
    front-ends, Workspace, Blob, the GPU Context and allocator (``core/context.cu``,
    ``core/allocator.cu``) - compiled from the reference tree with ``-DUSE_CUDA`` (no cuDNN), WITHOUT
    any of its ``operators/kernels/*.cu``: the GPU kernel registry keys are taken by this
    repository's binding translation units (``shadow_b200/host/src/gpu_kernels*.cpp``, compiled here
    against the reference's headers) and resolve to ``libsb200.so``.  The result,
    ``oracle/_ref/libshadow_ref_b200.so`` with the adapter prefix ``srefgpu_``, is the drop-in proof:
    the reference's Network runs an operator graph unchanged on this library's kernels.  Needs the
    reference tree, nvcc and the built ``libsb200.so``; returns the prebuilt file (or None) otherwise."""
    kernel_lib = os.path.join(REPO, "shadow_b200", "lib", "libsb200.so")
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not reference_available() or not os.path.exists(nvcc) or not os.path.exists(kernel_lib):
        return REF_GPU_LIB if os.path.exists(REF_GPU_LIB) else None
    shadow = os.path.join(REF_ROOT, "shadow")
    host_src = os.path.join(REPO, "shadow_b200", "host", "src")
    shim = os.path.join(REPO, "shadow_b200", "host", "net_capi.cpp")
    binding = sorted(glob.glob(os.path.join(host_src, "gpu_kernels*.cpp")))
    sources = []
    for pat in ("core/*.cpp", "operators/*.cpp", "operators/kernels/*.cpp"):
        sources += sorted(glob.glob(os.path.join(shadow, pat)))
    sources += [os.path.join(shadow, p) for p in
                ("backends/native/native.cpp", "util/io.cpp", "util/json.cpp", "util/boxes.cpp")]
    cuda_sources = [os.path.join(shadow, "core", "context.cu"), os.path.join(shadow, "core", "allocator.cu")]
    deps = sources + cuda_sources + binding + [shim, kernel_lib, os.path.abspath(__file__),
                                               os.path.join(host_src, "gpu_kernels_common.hpp")]
    if not force and _newer(REF_GPU_LIB, deps):
        return REF_GPU_LIB
    os.makedirs(REF_DIR, exist_ok=True)
    os.makedirs(GEN_DIR, exist_ok=True)
    with open(os.path.join(GEN_DIR, "config.hpp"), "w") as f:
        f.write(CONFIG_HPP)
    obj_dir = os.path.join(GEN_DIR, "obj_gpu")
    os.makedirs(obj_dir, exist_ok=True)
    cuda_inc = os.path.join(os.path.dirname(os.path.dirname(nvcc)), "include")
    cuda_lib = os.path.join(os.path.dirname(os.path.dirname(nvcc)), "lib64")
    flags = ["-O2", "-DNDEBUG", "-DUSE_CUDA", "-std=c++11", "-fPIC", "-include", "cstdint", "-w",
             "-I" + shadow, "-I" + GEN_DIR, "-I" + cuda_inc, "-I" + os.path.join(REPO, "include"), "-I" + host_src]

    def compile_one(item):
        idx, src = item
        obj = os.path.join(obj_dir, "%03d_%s.o" % (idx, os.path.splitext(os.path.basename(src))[0]))
        if src.endswith(".cu"):
            _run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O2", "-DNDEBUG", "-DUSE_CUDA", "-std=c++11",
                  "-Xcompiler", "-fPIC,-w", "-include", "cstdint", "-I" + shadow, "-I" + GEN_DIR, "-c", src, "-o", obj])
        else:
            _run(["g++"] + flags + ["-c", src, "-o", obj])
        return obj

    with cf.ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as pool:
        objs = list(pool.map(compile_one, enumerate(sources + cuda_sources + binding)))
    shim_obj = os.path.join(obj_dir, "net_capi_srefgpu.o")
    _run(["g++"] + flags + ["-DSHADOW_CAPI_PREFIX=srefgpu_", "-c", shim, "-o", shim_obj])
    vers = os.path.join(GEN_DIR, "srefgpu.map")
    with open(vers, "w") as f:
        f.write("{ global: srefgpu_*; local: *; };\n")
    # $ORIGIN-relative path to libsb200.so: the library is found wherever the repository is copied
    _run(["g++", "-shared", "-o", REF_GPU_LIB] + objs + [shim_obj,
         "-Wl,-Bsymbolic", "-Wl,--version-script=" + vers,
         "-L" + os.path.dirname(kernel_lib), "-lsb200", "-Wl,-rpath,$ORIGIN/../../shadow_b200/lib",
         "-L" + cuda_lib, "-lcudart", "-lcublas", "-ldl"])
    return REF_GPU_LIB


def build_all(force: bool = False) -> dict:
    out = {"port": None, "ref": None, "ref_gpu": None}
    if os.path.exists(os.path.join(HERE, "oracle_port.c")):
        out["port"] = build_port(force)
    out["ref"] = build_ref(force)
    out["ref_gpu"] = build_ref_gpu(force)
    return out


if __name__ == "__main__":
    print(build_all(force="--force" in sys.argv))
