"""The five baseline configurations at their FULL sizes.  C1-C4 are compared element for element
with the C oracle (it finishes each in about a second); C5 (2 GiB output) is checked through
size-independent properties plus an oracle comparison of one dim-0 slice."""
import numpy as np
import pytest

import cases
from oracle import oracle as orc

pytestmark = pytest.mark.gpu

SEED = 20240600


def _dev(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _host(t):
    import torch
    torch.cuda.synchronize()
    return t.cpu().numpy()


def _check(name, op, args, inputs, got):
    case = {"name": name, "op": op, "args": args, "inputs": inputs}
    want = cases.run_port(case)
    cases.assert_parity(case, got.reshape(want.shape), want)


def test_c1_binary_broadcast_and_same_shape():
    from shadow_b200 import functional as F
    a = cases.uniform(SEED + 10, (32, 64, 56, 56))
    b = cases.normal(SEED + 11, (1, 64, 1, 1))
    c = cases.uniform(SEED + 12, (32, 64, 56, 56))
    da, db, dc = _dev(a), _dev(b), _dev(c)
    for code in (0, 2, 5):   # Add, Mul, Max
        _check("c1_bcast_%d" % code, "Binary", {"operation": code}, [a, b], _host(F.binary(da, db, code)))
    _check("c1_same_add", "Binary", {"operation": 0}, [a, c], _host(F.binary(da, dc, 0)))


def test_c2_unary_activation_scale():
    from shadow_b200 import functional as F
    shape = (64, 256, 28, 28)
    x = cases.normal(SEED + 20, shape, 0.0, 2.0)
    dx = _dev(x)
    for t in (1, 2, 3, 5):   # ReLU, LeakyReLU(0.1), Sigmoid, Tanh
        slope = float(np.float32(0.1))
        _check("c2_act_%d" % t, "Activate", {"type": t, "slope": slope}, [x], _host(F.activate(dx, t, slope)))
    xe = cases.uniform(SEED + 21, shape, -10.0, 10.0)
    _check("c2_exp", "Unary", {"operation": 4}, [xe], _host(F.unary(_dev(xe), 4)))
    xl = cases.uniform(SEED + 22, shape, 0.01, 10.0)
    dl = _dev(xl)
    _check("c2_log", "Unary", {"operation": 3}, [xl], _host(F.unary(dl, 3)))
    _check("c2_sqrt", "Unary", {"operation": 2}, [xl], _host(F.unary(dl, 2)))
    g, bt = cases.normal(SEED + 23, (256,), 1.0, 0.1), cases.normal(SEED + 24, (256,), 0.0, 0.1)
    _check("c2_scale", "Scale", {"axis": 1, "has_scale": True, "has_bias": True}, [x, g, bt],
           _host(F.scale(dx, 1, _dev(g), _dev(bt))))


def test_c3_axis_reductions():
    from shadow_b200 import functional as F
    shape = (128, 512, 14, 14)
    x = cases.normal(SEED + 30, shape)
    dx = _dev(x)
    for axes in ([2, 3], [1], [0, 2, 3]):
        for code in (1, 4, 2, 3):   # Sum, Avg, Max, Min
            for keep in (True, False):
                got = _host(F.reduce(dx, code, axes, keep))
                _check("c3_%d_%s_%d" % (code, axes, keep), "Reduce", {"operation": code, "axes": axes, "keep_dims": keep},
                       [x], got)
    xp = cases.uniform(SEED + 31, shape, 0.99, 1.01)
    _check("c3_prod", "Reduce", {"operation": 0, "axes": [2, 3], "keep_dims": True}, [xp],
           _host(F.reduce(_dev(xp), 0, [2, 3], True)))


def test_c4_softmax_rows_and_strided():
    from shadow_b200 import functional as F
    logits = cases.normal(SEED + 40, (16384, 4096), 0.0, 3.0)
    _check("c4a", "Softmax", {"axis": -1}, [logits], _host(F.softmax(_dev(logits), -1)))
    x = cases.normal(SEED + 41, (64, 1000, 7, 7))
    _check("c4b", "Softmax", {"axis": 1}, [x], _host(F.softmax(_dev(x), 1)))


def test_c5_large_chain_properties():
    import torch
    from shadow_b200 import functional as F
    a = cases.uniform(SEED + 50, (8, 1, 2048, 2048))
    b = cases.normal(SEED + 51, (1, 16, 1, 2048))
    da, db = _dev(a), _dev(b)
    o = F.binary(da, db, 2)                                      # [8,16,2048,2048], 2 GiB
    assert tuple(o.shape) == (8, 16, 2048, 2048)
    # (1) one dim-0 slice against the oracle, bit for bit
    want = orc.binary(a[3:4], b, 2)
    assert orc.bit_equal(_host(o[3:4]), want)
    # (2) random positions of the whole tensor: each output is the float product of its operands
    rng = np.random.Generator(np.random.PCG64(7))
    idx = rng.integers(0, [8, 16, 2048, 2048], size=(200000, 4))
    flat = ((idx[:, 0] * 16 + idx[:, 1]) * 2048 + idx[:, 2]) * 2048 + idx[:, 3]
    picked = _host(o.view(-1)[torch.from_numpy(flat).cuda()])
    assert np.array_equal(picked, a[idx[:, 0], 0, idx[:, 2], idx[:, 3]] * b[0, idx[:, 1], 0, idx[:, 3]])
    # (3) full sum: linearity.  sum(O) = sum_w colsum_A[w] * colsum_B[w] up to the rounding of the
    #     individual products (each <= 2^-24 relative), far inside the reduction tolerance
    s = float(F.reduce(o, 1, [], False).item())
    exact = float((a.astype(np.float64).sum(axis=(0, 1, 2)) * b.astype(np.float64).sum(axis=(0, 1, 2))).sum())
    scale = float((np.abs(a).astype(np.float64).sum(axis=(0, 1, 2)) * np.abs(b).astype(np.float64).sum(axis=(0, 1, 2))).sum())
    assert abs(s - exact) <= 1e-5 * np.log2(o.numel()) * abs(exact) + 2.0 ** -23 * scale
    # (4) the full sum agrees with the sum of the per-slice sums (a different kernel path), and the
    #     full max is the max of the per-slice maxima and is attained
    per_n_sum = _host(F.reduce(o, 1, [1, 2, 3], False)).astype(np.float64)
    assert abs(per_n_sum.sum() - s) <= 1e-6 * abs(s) + 1e-3
    m = float(F.reduce(o, 2, [], False).item())
    per_n_max = _host(F.reduce(o, 2, [1, 2, 3], False))
    assert m == per_n_max.max()
    assert bool((o == m).any().item())
    assert m >= picked.max()
    # (5) one slice of each reduction against the oracle
    o1 = _host(o[5:6])
    case = {"name": "c5_slice_sum", "op": "Reduce", "args": {"operation": 1, "axes": []}, "inputs": [o1]}
    cases.assert_parity(case, _host(F.reduce(o[5:6].contiguous(), 1, [], True)), orc.reduce(o1, 1, [], True))
    assert _host(F.reduce(o[5:6].contiguous(), 2, [], True)).ravel()[0] == o1.max()
