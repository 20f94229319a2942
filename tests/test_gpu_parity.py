"""GPU parity tests proper: every small case through the kernel C ABI against (a) the golden
outputs of the compiled reference and (b) the C oracle run on the spot."""
import hashlib
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
    want, digest, shape = cases.golden_lookup(golden, case["name"])
    if want is None:
        # digest-only fixture: the C oracle (itself pinned to that digest) supplies the values
        want = cases.run_port(case)
        assert hashlib.sha256(np.ascontiguousarray(want).tobytes()).digest() == digest
    got = cases.run_cuda(case)
    assert list(got.shape) == shape
    cases.assert_parity(case, got.reshape(want.shape), want)


@pytest.mark.parametrize("operation", range(7), ids=["prod", "sum", "max", "min", "avg", "l1", "l2"])
@pytest.mark.parametrize("axes", [[], [0, 2], [0]], ids=["all", "ax02", "ax0"])
def test_sharded_partials_combine_to_the_full_reduction(operation, axes):
    """The multi-GPU path on one GPU: dim-0 slabs of a tensor are reduced to double partials
    (sb200_reduce_partial), the per-slab records are laid out as an all-gather would leave them, and
    sb200_reduce_combine must give the oracle's reduction of the whole tensor."""
    import torch
    from oracle import oracle as orc
    from shadow_b200 import functional as F
    shape = (7, 33, 20)
    full = cases.uniform(77, shape, 0.9, 1.1) if operation == 0 else cases.normal(78, shape)
    want = orc.reduce(full, operation, axes, keep_dims=True)
    ax = axes or list(range(len(shape)))
    count = int(np.prod([1 if n in ax else d for n, d in enumerate(shape)]))
    slabs = [(0, 3), (3, 4), (4, 7)]
    record_len = count + 5                      # records may carry other reductions' partials too
    gathered = torch.zeros(len(slabs) * record_len, dtype=torch.float64, device="cuda")
    for r, (lo, hi) in enumerate(slabs):
        x = torch.from_numpy(np.ascontiguousarray(full[lo:hi])).cuda()
        F.reduce_partial(x, operation, axes, out=gathered[r * record_len:r * record_len + count])
    total = int(np.prod([shape[a] for a in ax]))
    got = F.reduce_combine(gathered, len(slabs), record_len, count, operation, total)
    torch.cuda.synchronize()
    case = {"name": "combine", "op": "Reduce", "args": {"operation": operation, "axes": axes}, "inputs": [full]}
    cases.assert_parity(case, got.cpu().numpy().reshape(want.shape), want)
