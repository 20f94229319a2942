"""GPU parity tests proper: every small case through the kernel C ABI against (a) the golden
outputs of the compiled reference and (b) the C oracle run on the spot."""
import os

import numpy as np
import pytest

import cases

pytestmark = pytest.mark.gpu

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "small_cases.npz")
SMALL = cases.small_cases()


@pytest.fixture(scope="module")
def golden():
    return np.load(GOLDEN)


@pytest.mark.parametrize("case", SMALL, ids=[c["name"] for c in SMALL])
def test_cabi_matches_reference_golden(case, golden):
    want = golden[case["name"]]
    got = cases.run_cuda(case)
    cases.assert_parity(case, got.reshape(want.shape), want)
    assert list(got.shape) == list(golden[case["name"] + "/shape"])
