"""The drop-in boundary seen from the reference's side.

CPU part: the kernel-binding translation units of the host library (shadow_b200/host/src/gpu_kernels*.cpp)
compile against the REFERENCE's own headers (shadow/core/kernel.hpp:13-41, shadow/core/registry.hpp:15-58,
shadow/operators/kernels/<op>.hpp) - they use no member that only this repository's re-creation of the
host API has.

GPU part: the reference's own Network / Native backend / operator front-ends / Workspace / GPU context,
compiled from the reference tree with USE_CUDA and WITHOUT its operators/kernels/*.cu, with those
translation units taking the "<Op>GPU(Default)" registry keys (oracle/build.py: build_ref_gpu), run
every parity case and a multi-operator graph.  The results must equal, bit for bit, what this
repository's host library produces for the same graph (the kernels are the same; only the host stack
differs), which in turn is compared with the reference's CPU results by tests/test_host_api.py."""
import os
import shutil
import subprocess

import numpy as np
import pytest

import cases
import shadow_b200
from oracle import build as obuild
from oracle import oracle as orc
from shadow_b200.netapi import Net, NetLibrary

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HOST_SRC = os.path.join(ROOT, "shadow_b200", "host", "src")
UNITS = ["gpu_kernels.cpp", "gpu_kernels_reduce.cpp", "gpu_kernels_eltwise.cpp"]
SMALL = cases.small_cases()


@pytest.mark.parametrize("unit", UNITS)
def test_binding_compiles_against_the_reference_headers(unit, tmp_path):
    if not obuild.reference_available():
        pytest.skip("reference tree not present on this machine")
    gen = tmp_path / "gen"
    gen.mkdir()
    (gen / "config.hpp").write_text(obuild.CONFIG_HPP)   # the one header the reference's CMake generates
    cmd = ["g++", "-std=c++11", "-fsyntax-only", "-Wall", "-include", "cstdint",
           "-I" + os.path.join(obuild.REF_ROOT, "shadow"), "-I" + str(gen), "-I" + os.path.join(ROOT, "include"),
           "-I" + HOST_SRC, os.path.join(HOST_SRC, unit)]
    out = subprocess.run(cmd, capture_output=True, text=True)
    assert out.returncode == 0, out.stderr


def test_binding_names_no_private_header():
    """The units include the per-operator headers by the reference's paths, never this repository's
    umbrella headers."""
    for unit in UNITS + ["gpu_kernels_common.hpp"]:
        text = open(os.path.join(HOST_SRC, unit)).read()
        assert "op_kernels.hpp" not in text and "shadow_api.hpp" not in text, unit


def test_reference_hosted_library_exports_the_adapter():
    if not os.path.exists(obuild.REF_GPU_LIB):
        pytest.skip("oracle/_ref/libshadow_ref_b200.so not built (needs the reference tree and nvcc)")
    nm = shutil.which("nm")
    if nm is None:
        pytest.skip("nm not available")
    syms = subprocess.run([nm, "-D", "--defined-only", obuild.REF_GPU_LIB], capture_output=True, text=True).stdout
    for name in ("net_create", "net_add_op", "net_load", "net_forward", "net_blob_data"):
        assert "srefgpu_" + name in syms
    # nothing of the reference's namespace leaks: the adapter is the only interface
    assert "Shadow" not in syms


@pytest.fixture(scope="module")
def hosted():
    if not os.path.exists(obuild.REF_GPU_LIB):
        pytest.skip("oracle/_ref/libshadow_ref_b200.so not built (needs the reference tree and nvcc)")
    return NetLibrary(obuild.REF_GPU_LIB, "srefgpu_")


@pytest.fixture(scope="module")
def own():
    return shadow_b200.host_library()


@pytest.mark.gpu
@pytest.mark.parametrize("case", SMALL, ids=[c["name"] for c in SMALL])
def test_reference_network_on_these_kernels(case, hosted, own):
    got = cases.run_net(hosted, case)
    want = cases.run_net(own, case)
    assert got.shape == want.shape
    assert orc.bit_equal(got, want), case["name"]


@pytest.mark.gpu
def test_reference_network_runs_a_graph_unchanged(hosted, own):
    def graph(library):
        a = cases.uniform(1, (4, 6, 10, 12))
        b = cases.normal(2, (1, 6, 1, 1))
        g, bt = cases.normal(3, (6,), 1, 0.1), cases.normal(4, (6,), 0, 0.1)
        net = Net(library, "graph").input({"a": a.shape, "b": b.shape})
        net.weight("gamma", g).weight("beta", bt)
        net.op("Binary", ["a", "b"], ["m"], operation=2)
        net.op("Scale", ["m", "gamma", "beta"], ["s"], axis=1, has_scale=True, has_bias=True)
        net.op("Activate", ["s"], ["s"], type=2, slope=float(np.float32(0.1)))
        net.op("Unary", ["s"], ["e"], operation=4)
        net.op("Reduce", ["e"], ["r"], operation=1, axes=[2, 3], keep_dims=False)
        net.op("Softmax", ["r"], ["p"], axis=-1)
        net.load("Native", out_blobs=["p", "r", "e"])
        net.forward({"a": a, "b": b})
        return [net.blob(n) for n in ("s", "e", "r", "p")]
    for x, y in zip(graph(hosted), graph(own)):
        assert orc.bit_equal(x, y)
