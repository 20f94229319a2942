"""Pins the C restatement (oracle/oracle_port.c) to the reference: bit-for-bit against the golden
outputs the compiled reference produced (tests/golden/small_cases.npz), and, where the compiled
reference library is present, live against it on medium-size seeded tensors."""
import hashlib
import os

import numpy as np
import pytest

import cases
from oracle import oracle as orc

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "small_cases.npz")
SMALL = cases.small_cases()


@pytest.fixture(scope="module")
def golden():
    return np.load(GOLDEN)


@pytest.mark.parametrize("case", SMALL, ids=[c["name"] for c in SMALL])
def test_port_matches_reference_golden(case, golden):
    want, digest, want_shape = cases.golden_lookup(golden, case["name"])
    got = cases.run_port(case)
    assert list(got.shape) == want_shape
    if want is None:
        assert hashlib.sha256(np.ascontiguousarray(got).tobytes()).digest() == digest
    else:
        assert orc.bit_equal(got.reshape(want.shape), want), (
            "max ulp %d" % int(orc.ulp_distance(got, want).max()))


def test_golden_covers_every_case(golden):
    names = {k[:-len("/shape")] for k in golden.files if k.endswith("/shape")}
    assert names == {c["name"] for c in SMALL}


def test_known_answers(golden):
    """Edge semantics measured on the compiled reference."""
    f = np.float32
    mx = lambda a, b: orc.binary(np.array([a], f), np.array([b], f), 5)[0]
    assert np.signbit(mx(0.0, -0.0)) == False and np.signbit(mx(-0.0, 0.0)) == True  # noqa: E712
    assert np.isnan(mx(np.nan, 1.0)) and mx(1.0, np.nan) == 1.0
    relu = orc.activate(np.array([np.nan, -0.0, 2.0], f), 1)
    assert relu[0] == 0.0 and not np.signbit(relu[1]) and relu[2] == 2.0
    kat = golden["scale_unfused_kat"]
    assert np.all(kat.view(np.uint32) == 0)  # unfused multiply-add gives +0, a fused one 0x30088888
    r = orc.reduce(np.array([[1.0, np.nan, 3.0]], f), 2, [1])
    assert r.ravel()[0] == 3.0  # Reduce-Max skips NaN
    assert orc.reduce(np.ones((2, 3), f), 1, [], keep_dims=False).shape == ()


REF = orc.ref_library()


def _medium_cases():
    c = cases._case
    return [
        c("m_bcast_mul", "Binary", {"operation": 2}, [cases.uniform(1, (8, 16, 28, 28)), cases.normal(2, (1, 16, 1, 1))]),
        c("m_bcast_both", "Binary", {"operation": 2}, [cases.uniform(3, (4, 1, 64, 96)), cases.normal(4, (1, 6, 1, 96))]),
        c("m_tanh", "Activate", {"type": 5}, [cases.normal(5, (16, 64, 14, 14), 0, 2)]),
        c("m_sigmoid", "Activate", {"type": 3}, [cases.normal(6, (16, 64, 14, 14), 0, 2)]),
        c("m_exp", "Unary", {"operation": 4}, [cases.uniform(7, (200000,), -10, 10)]),
        c("m_log", "Unary", {"operation": 3}, [cases.uniform(8, (200000,), 0.01, 10)]),
        c("m_scale", "Scale", {"axis": 1, "has_scale": True, "has_bias": True},
          [cases.normal(9, (8, 256, 14, 14)), cases.normal(10, (256,), 1, 0.1), cases.normal(11, (256,), 0, 0.1)]),
        c("m_reduce_023", "Reduce", {"operation": 1, "axes": [0, 2, 3]}, [cases.normal(12, (16, 64, 14, 14))]),
        c("m_reduce_1", "Reduce", {"operation": 4, "axes": [1]}, [cases.normal(13, (16, 64, 14, 14))]),
        c("m_reduce_all", "Reduce", {"operation": 6, "axes": [], "keep_dims": False}, [cases.normal(14, (16, 64, 14, 14))]),
        c("m_softmax_rows", "Softmax", {"axis": -1}, [cases.normal(15, (256, 4096), 0, 3)]),
        c("m_softmax_strided", "Softmax", {"axis": 1}, [cases.normal(16, (8, 1000, 7, 7))]),
    ]


@pytest.mark.skipif(REF is None, reason="compiled reference (oracle/_ref) not built on this machine")
@pytest.mark.parametrize("case", _medium_cases(), ids=lambda c: c["name"])
def test_port_matches_live_reference(case):
    want = cases.run_net(REF, case)
    got = cases.run_port(case)
    assert got.shape == want.shape
    assert orc.bit_equal(got, want), "max ulp %d" % int(orc.ulp_distance(got, want).max())
