"""The C++ host library (Shadow Operator/Kernel/Blob/Workspace/Network API).  CPU part: it loads,
exports the adapter, and reports errors the reference's way.  GPU part: every parity case and a
multi-operator graph through Network::Forward with host buffers."""
import hashlib
import os

import numpy as np
import pytest

import cases
import shadow_b200
from shadow_b200 import build as sbuild
from shadow_b200.netapi import Net, ShadowError

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "small_cases.npz")
SMALL = cases.small_cases()


@pytest.fixture(scope="module")
def lib():
    sbuild.build_all()
    return shadow_b200.host_library()


@pytest.fixture(scope="module")
def golden():
    return np.load(GOLDEN)


def test_adapter_symbols(lib):
    for name in ("net_create", "net_destroy", "net_add_op", "net_add_blob", "net_load", "net_forward",
                 "net_blob_shape", "net_blob_data", "last_error"):
        assert hasattr(lib.lib, "sb200net_" + name)


def test_front_end_checks_fire_at_load(lib):
    """Argument checks of the operator constructors (no device needed to reach them? they run after
    the Workspace is created, so without a GPU the CUDA error comes first) - either way an error."""
    with pytest.raises(ShadowError):
        Net(lib).input({"a": [2]}).op("Binary", ["a"], ["y"]).load("Native", out_blobs=["y"])
    with pytest.raises(ShadowError):
        Net(lib).input({"a": [2]}).op("NoSuchOp", ["a"], ["y"]).load("Native", out_blobs=["y"])
    with pytest.raises(ShadowError):
        Net(lib).input({"a": [2]}).op("Unary", ["a"], ["y"], operation=0).load("NoSuchBackend", out_blobs=["y"])


@pytest.mark.gpu
def test_error_messages_follow_the_reference(lib):
    with pytest.raises(ShadowError, match=r"Check Failed: operation_ >= 0 \(-1 vs 0\)"):
        Net(lib).input({"a": [2]}).op("Binary", ["a"], ["y"]).load("Native", out_blobs=["y"])
    with pytest.raises(ShadowError, match="Op type: NoSuchOp is not registered"):
        Net(lib).input({"a": [2]}).op("NoSuchOp", ["a"], ["y"]).load("Native", out_blobs=["y"])
    net = Net(lib).input({"a": [2, 3], "b": [2, 4]}).op("Binary", ["a", "b"], ["y"], operation=0)
    net.load("Native", out_blobs=["y"])
    with pytest.raises(ShadowError, match="Check Failed"):
        net.forward({"a": np.zeros((2, 3), np.float32), "b": np.zeros((2, 4), np.float32)})
    net = Net(lib).input({"a": [2, 3]}).op("Reduce", ["a"], ["a"], operation=1)
    net.load("Native", out_blobs=["a"])
    with pytest.raises(ShadowError, match="Check Failed"):       # in-place reduce is refused
        net.forward({"a": np.zeros((2, 3), np.float32)})


@pytest.mark.gpu
@pytest.mark.parametrize("case", SMALL, ids=[c["name"] for c in SMALL])
def test_network_api_matches_reference_golden(case, lib, golden):
    want, digest, shape = cases.golden_lookup(golden, case["name"])
    if want is None:
        want = cases.run_port(case)
        assert hashlib.sha256(np.ascontiguousarray(want).tobytes()).digest() == digest
    got = cases.run_net(lib, case)
    assert list(got.shape) == shape
    cases.assert_parity(case, got.reshape(want.shape), want)


def _graph(library):
    """Input -> Binary(bcast Mul) -> Scale -> Activate(LeakyReLU) -> Reduce(Sum {2,3}) and Softmax."""
    a = cases.uniform(1, (4, 6, 10, 12))
    b = cases.normal(2, (1, 6, 1, 1))
    g, bt = cases.normal(3, (6,), 1, 0.1), cases.normal(4, (6,), 0, 0.1)
    net = Net(library, "graph").input({"a": a.shape, "b": b.shape})
    net.weight("gamma", g).weight("beta", bt)
    net.op("Binary", ["a", "b"], ["m"], operation=2)
    net.op("Scale", ["m", "gamma", "beta"], ["s"], axis=1, has_scale=True, has_bias=True)
    net.op("Activate", ["s"], ["s"], type=2, slope=float(np.float32(0.1)))      # in place
    net.op("Reduce", ["s"], ["r"], operation=1, axes=[2, 3], keep_dims=False)
    net.op("Softmax", ["r"], ["p"], axis=-1)
    net.load("Native", out_blobs=["p", "r"])
    net.forward({"a": a, "b": b})
    return net.blob("s"), net.blob("r"), net.blob("p"), net.shape("r")


@pytest.mark.gpu
def test_multi_operator_graph(lib):
    from oracle import oracle as orc
    s, r, p, r_shape = _graph(lib)
    ref = orc.ref_library()
    if ref is not None:
        s0, r0, p0, r0_shape = _graph(ref)
    else:
        a, b = cases.uniform(1, (4, 6, 10, 12)), cases.normal(2, (1, 6, 1, 1))
        g, bt = cases.normal(3, (6,), 1, 0.1), cases.normal(4, (6,), 0, 0.1)
        s0 = orc.activate(orc.scale(orc.binary(a, b, 2), 1, g, bt), 2, np.float32(0.1))
        r0 = orc.reduce(s0, 1, [2, 3], keep_dims=False)
        p0 = orc.softmax(r0, -1)
        r0_shape = list(r0.shape)
    assert r_shape == r0_shape == [4, 6]
    assert orc.bit_equal(s, s0)                       # Mul, unfused Scale, LeakyReLU: exact
    assert np.allclose(r, r0, rtol=1e-5 * np.log2(120), atol=0)
    assert np.allclose(p, p0, rtol=1e-5 * np.log2(6) + 1e-5, atol=1e-7)
