"""Edge conditions of the kernel entry points: in-place calls, sub-buffers that are not 16-byte
aligned (head/tail peeling and the scalar fallbacks), ragged sizes, guard bands around outputs."""
import numpy as np
import pytest

import cases
from oracle import oracle as orc

pytestmark = pytest.mark.gpu

GUARD = 64   # floats of sentinel before and after every output


def _torch():
    import torch
    return torch


def _view(arr, offset, pad=GUARD):
    """Device copy of `arr` placed `offset` floats after a 256-byte aligned address, with sentinel
    guard bands; returns (view, whole_buffer)."""
    torch = _torch()
    n = arr.size
    buf = torch.full((pad + offset + n + pad + 8,), 12345.0, dtype=torch.float32, device="cuda")
    v = buf[pad + offset:pad + offset + n]
    v.copy_(torch.from_numpy(np.ascontiguousarray(arr).ravel()))
    return v.view(arr.shape), buf


def _guards_intact(buf, offset, n, pad=GUARD):
    b = buf.cpu().numpy()
    return bool(np.all(b[:pad + offset] == 12345.0) and np.all(b[pad + offset + n:] == 12345.0))


@pytest.mark.parametrize("off_in,off_out", [(0, 0), (1, 1), (3, 3), (2, 2), (1, 2), (0, 3), (3, 0)])
@pytest.mark.parametrize("n", [1, 5, 1023, 4100])
def test_unaligned_elementwise(off_in, off_out, n):
    from shadow_b200 import functional as F
    torch = _torch()
    x = cases.uniform(n + off_in, (n,), -3, 3)
    b = cases.uniform(n + 99, (n,), -3, 3)
    dx, _ = _view(x, off_in)
    db, _ = _view(b, off_in)
    for name, fn, want in (
        ("neg", lambda o: F.unary(dx, 13, out=o), orc.unary(x, 13)),
        ("exp", lambda o: F.unary(dx, 4, out=o), orc.unary(x, 4)),
        ("relu", lambda o: F.activate(dx, 1, 0.1, out=o), orc.activate(x, 1)),
        ("add", lambda o: F.binary(dx, db, 0, out=o), orc.binary(x, b, 0)),
        ("mul_scalar", lambda o: F.binary_scalar(dx, 0.7, 2, out=o), orc.binary_scalar(x, 0.7, 2)),
        ("eltwise_max", lambda o: F.eltwise([dx, db], 2, out=o), orc.eltwise([x, b], 2)),
    ):
        out, buf = _view(np.zeros(n, np.float32), off_out)
        fn(out)
        torch.cuda.synchronize()
        got = out.cpu().numpy()
        tol = 1 if name == "exp" else 0
        assert int(orc.ulp_distance(got, want).max()) <= tol, name
        assert _guards_intact(buf, off_out, n), name
    fill, buf = _view(np.zeros(n, np.float32), off_out)
    F.fill(fill, 2.5)
    torch.cuda.synchronize()
    assert bool((fill == 2.5).all().item()) and _guards_intact(buf, off_out, n)


@pytest.mark.parametrize("offset", [0, 1, 2, 3])
def test_unaligned_channel_broadcast_reduce_softmax(offset):
    from shadow_b200 import functional as F
    torch = _torch()
    x = cases.normal(50 + offset, (3, 6, 5, 7))
    dx, _ = _view(x, offset)
    g, bt = cases.normal(60, (6,)), cases.normal(61, (6,))
    dg, dbt = torch.from_numpy(g).cuda(), torch.from_numpy(bt).cuda()
    out, buf = _view(np.zeros_like(x), offset)
    F.scale(dx, 1, dg, dbt, out=out)
    assert orc.bit_equal(out.cpu().numpy(), orc.scale(x, 1, g, bt)) and _guards_intact(buf, offset, x.size)
    out, buf = _view(np.zeros_like(x), (offset + 1) % 4)            # input and output misaligned differently
    F.scale(dx, 1, dg, dbt, out=out)
    assert orc.bit_equal(out.cpu().numpy(), orc.scale(x, 1, g, bt)) and _guards_intact(buf, (offset + 1) % 4, x.size)
    out, buf = _view(np.zeros_like(x), offset)
    F.activate(dx, 0, 0.1, dg, out=out)                             # PReLU
    assert orc.bit_equal(out.cpu().numpy(), orc.activate(x, 0, 0.1, g))
    b = cases.normal(62, (1, 6, 1, 7))
    db, _ = _view(b, offset)
    out, buf = _view(np.zeros_like(x), offset)
    F.binary(dx, db, 1, out=out)                                    # broadcast Sub
    assert orc.bit_equal(out.cpu().numpy(), orc.binary(x, b, 1)) and _guards_intact(buf, offset, x.size)
    for axes in ([2, 3], [1], [0, 2, 3], []):
        for op in (1, 2):
            want = orc.reduce(x, op, axes, True)
            out, buf = _view(np.zeros_like(want), offset)
            F.reduce(dx, op, axes, True, out=out)
            torch.cuda.synchronize()
            case = {"name": "r", "op": "Reduce", "args": {"operation": op, "axes": axes}, "inputs": [x]}
            cases.assert_parity(case, out.cpu().numpy().reshape(want.shape), want)
            assert _guards_intact(buf, offset, want.size)
    for axis in (1, 3):
        want = orc.softmax(x, axis)
        out, buf = _view(np.zeros_like(x), offset)
        F.softmax(dx, axis, out=out)
        torch.cuda.synchronize()
        case = {"name": "s", "op": "Softmax", "args": {"axis": axis}, "inputs": [x]}
        cases.assert_parity(case, out.cpu().numpy(), want)
        assert _guards_intact(buf, offset, x.size)
    alpha = cases.normal(63, (3, 6))
    y = cases.normal(64, x.shape)
    dy, _ = _view(y, offset)
    out, buf = _view(np.zeros_like(x), offset)
    F.axpy(torch.from_numpy(alpha).cuda(), dx, dy, out=out)
    assert orc.bit_equal(out.cpu().numpy(), orc.axpy(alpha, x, y)) and _guards_intact(buf, offset, x.size)


def test_in_place_calls():
    from shadow_b200 import functional as F
    torch = _torch()
    x = cases.normal(70, (4, 8, 9, 11), 0, 2)
    b = cases.normal(71, x.shape)
    bc = cases.normal(72, (1, 8, 1, 1))
    g, bt = cases.normal(73, (8,)), cases.normal(74, (8,))
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()   # noqa: E731
    t = dev(x); F.unary(t, 13, out=t); assert orc.bit_equal(t.cpu().numpy(), orc.unary(x, 13))
    t = dev(x); F.activate(t, 2, 0.1, out=t); assert orc.bit_equal(t.cpu().numpy(), orc.activate(x, 2, np.float32(0.1)))
    t = dev(x); F.activate(t, 5, 0.1, out=t); assert int(orc.ulp_distance(t.cpu().numpy(), orc.activate(x, 5)).max()) <= 2
    t = dev(x); F.binary_scalar(t, 1.5, 0, out=t); assert orc.bit_equal(t.cpu().numpy(), orc.binary_scalar(x, 1.5, 0))
    t = dev(x); F.binary(t, dev(b), 2, out=t); assert orc.bit_equal(t.cpu().numpy(), orc.binary(x, b, 2))
    t = dev(b); F.binary(dev(x), t, 1, out=t); assert orc.bit_equal(t.cpu().numpy(), orc.binary(x, b, 1))   # out aliases the 2nd input
    t = dev(x); F.binary(t, dev(bc), 0, out=t); assert orc.bit_equal(t.cpu().numpy(), orc.binary(x, bc, 0))  # broadcast, full input in place
    t = dev(x); F.scale(t, 1, dev(g), dev(bt), out=t); assert orc.bit_equal(t.cpu().numpy(), orc.scale(x, 1, g, bt))
    t = dev(x); F.activate(t, 0, 0.1, dev(g), out=t); assert orc.bit_equal(t.cpu().numpy(), orc.activate(x, 0, 0.1, g))
    t = dev(x); F.eltwise([t, dev(b)], 0, out=t); assert orc.bit_equal(t.cpu().numpy(), orc.eltwise([x, b], 0))
    t = dev(x); F.softmax(t, 1, out=t)
    cases.assert_parity({"name": "s", "op": "Softmax", "args": {"axis": 1}, "inputs": [x]}, t.cpu().numpy(), orc.softmax(x, 1))
    t = dev(x); F.softmax(t, 3, out=t)
    cases.assert_parity({"name": "s", "op": "Softmax", "args": {"axis": 3}, "inputs": [x]}, t.cpu().numpy(), orc.softmax(x, 3))


@pytest.mark.parametrize("offset", [0, 1, 2, 3])
def test_unaligned_normalisation_family(offset):
    """BatchNorm / Normalize / SSDNormalize / LayerNorm / GroupNorm / InstanceNorm on sub-buffers that
    start 0-3 floats past a 16-byte boundary: scalar fall-backs, guard bands intact."""
    from shadow_b200 import functional as F
    torch = _torch()
    x = cases.normal(80 + offset, (3, 8, 4, 6), 0.3, 1.5)
    dx, _ = _view(x, offset)
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()   # noqa: E731
    g, bt = cases.normal(81, (8,), 1.0, 0.2), cases.normal(82, (8,))
    var = cases.uniform(83, (8,), 0.2, 2.0)

    def check(name, op, args, inputs, fn):
        want = cases.run_port({"name": name, "op": op, "args": args, "inputs": inputs})
        out, buf = _view(np.zeros_like(x), (offset + 1) % 4)
        fn(out)
        torch.cuda.synchronize()
        cases.assert_parity({"name": name, "op": op, "args": args, "inputs": inputs}, out.cpu().numpy(), want)
        assert _guards_intact(buf, (offset + 1) % 4, x.size), name

    check("bn", "BatchNorm", {}, [x, bt, var], lambda o: F.batch_norm(dx, dev(bt), dev(var), 1.0, 1e-5, out=o))
    for p in (1.0, 2.0):
        for axis in (1, 3):
            check("norm", "Normalize", {"p": p, "axis": axis}, [x], lambda o: F.normalize(dx, axis, p, 1e-12, out=o))
    check("ssd_pos", "SSDNormalize", {"across_spatial": False, "channel_shared": False}, [x, g],
          lambda o: F.ssd_normalize(dx, dev(g), False, False, 1e-5, out=o))
    check("ssd_all", "SSDNormalize", {"across_spatial": True, "channel_shared": True}, [x, g[:1]],
          lambda o: F.ssd_normalize(dx, dev(g[:1]), True, True, 1e-5, out=o))
    check("gn", "GroupNorm", {"group": 2}, [x, g, bt], lambda o: F.group_norm(dx, 2, dev(g), dev(bt), 1e-5, out=o))
    check("in", "InstanceNorm", {}, [x], lambda o: F.instance_norm(dx, None, None, 1e-5, out=o))
    ls, lb = cases.normal(84, (4, 6)), cases.normal(85, (4, 6))
    check("ln", "LayerNorm", {"normalized_shape": [4, 6]}, [x, ls, lb],
          lambda o: F.layer_norm(dx, [4, 6], dev(ls), dev(lb), 1e-5, out=o))


@pytest.mark.parametrize("offset", [0, 1, 2])
def test_unaligned_data_movement(offset):
    from shadow_b200 import functional as F
    torch = _torch()
    a, b = cases.normal(90, (3, 5, 8, 12)), cases.normal(91, (3, 2, 8, 12))
    da, _ = _view(a, offset)
    db, _ = _view(b, (offset + 2) % 4)
    want = np.concatenate([a, b], 1)
    out, buf = _view(np.zeros_like(want), offset)
    F.concat([da, db], 1, out=out)
    assert orc.bit_equal(out.cpu().numpy(), want) and _guards_intact(buf, offset, want.size)
    wide_a, wide_b = cases.normal(92, (2, 1000)), cases.normal(93, (2, 600))
    dwa, _ = _view(wide_a, offset)
    dwb, _ = _view(wide_b, 0)
    want = np.concatenate([wide_a, wide_b], 1)
    out, buf = _view(np.zeros_like(want), offset)
    F.concat([dwa, dwb], 1, out=out)                                  # tile kernel, scalar units when offset != 0
    assert orc.bit_equal(out.cpu().numpy(), want) and _guards_intact(buf, offset, want.size)
    pieces = F.slice_(out, 1, [1000, 600])
    assert orc.bit_equal(pieces[0].cpu().numpy(), wide_a) and orc.bit_equal(pieces[1].cpu().numpy(), wide_b)
    want = a.transpose(0, 2, 3, 1)
    out, buf = _view(np.zeros(want.shape, np.float32), offset)
    F.permute(da, [0, 2, 3, 1], out=out)
    assert orc.bit_equal(out.cpu().numpy(), np.ascontiguousarray(want)) and _guards_intact(buf, offset, want.size)
    want = a.transpose(3, 1, 0, 2)
    out, buf = _view(np.zeros(want.shape, np.float32), offset)
    F.permute(da, [3, 1, 0, 2], out=out)
    assert orc.bit_equal(out.cpu().numpy(), np.ascontiguousarray(want)) and _guards_intact(buf, offset, want.size)
    want = np.pad(a, ((0, 0), (0, 0), (2, 1), (0, 3)), constant_values=-7.0)
    out, buf = _view(np.zeros(want.shape, np.float32), offset)
    F.pad(da, [2, 1, 0, 3], -7.0, out=out)
    assert orc.bit_equal(out.cpu().numpy(), want) and _guards_intact(buf, offset, want.size)
    idx = torch.tensor([4, 0, 4, 1], dtype=torch.int32, device="cuda")
    want = a[:, [4, 0, 4, 1]]
    out, buf = _view(np.zeros(want.shape, np.float32), offset)
    F.gather(da, idx, 1, out=out)
    assert orc.bit_equal(out.cpu().numpy(), np.ascontiguousarray(want)) and _guards_intact(buf, offset, want.size)
    bad = torch.tensor([9, -1, 2], dtype=torch.int32, device="cuda")   # out-of-range indexes give zeros, no fault
    got = F.gather(da, bad, 1).cpu().numpy()
    assert np.all(got[:, 0] == 0) and np.all(got[:, 1] == 0) and orc.bit_equal(got[:, 2], a[:, 2])


def test_every_permutation_of_small_tensors():
    """All 24 + 120 axis orders of a 4-d and a 5-d tensor (tile transposes, gathers and plain copies)."""
    import itertools
    from shadow_b200 import functional as F
    torch = _torch()
    for shape in ((3, 33, 5, 70), (2, 3, 35, 2, 40), (1, 9, 1, 64)):
        x = cases.normal(95 + len(shape), shape)
        dx = torch.from_numpy(x).cuda()
        for order in itertools.permutations(range(len(shape))):
            got = F.permute(dx, list(order)).cpu().numpy()
            assert got.shape == tuple(shape[a] for a in order)
            assert orc.bit_equal(got, np.ascontiguousarray(x.transpose(order))), (shape, order)


@pytest.mark.parametrize("rows,inner,group_affine", [
    (400, 8448, True),      # 33 KB rows, more rows than blocks: the double-buffered loop runs several rounds
    (300, 8196, False),     # the same kernel just above the row-in-registers limit
    (5, 30000, True),       # 120 KB rows: one buffer
    (3, 57344, False),      # the longest row that fits shared memory
    (2, 60000, True),       # longer: block-per-row kernel re-reading from L2
    (150, 8450, False),     # not a multiple of 4 floats: scalar long-row kernel
])
def test_long_row_normalisation(rows, inner, group_affine):
    """GroupNorm / LayerNorm on rows that do not fit the registers of a block."""
    from shadow_b200 import functional as F
    torch = _torch()
    spatial = inner // 2 if inner % 2 == 0 else inner
    channels = inner // spatial
    x = cases.normal(7000 + rows, (rows, channels, spatial), 0.5, 2.0)
    if group_affine:
        sc, bs = cases.normal(7001, (channels,), 1.0, 0.3), cases.normal(7002, (channels,))
        got = F.group_norm(torch.from_numpy(x).cuda(), 1, torch.from_numpy(sc).cuda(), torch.from_numpy(bs).cuda(), 1e-5)
        case = {"name": "long_rows", "op": "GroupNorm", "args": {"group": 1, "eps": 1e-5}, "inputs": [x, sc, bs]}
    else:
        flat = x.reshape(rows, inner)
        got = F.layer_norm(torch.from_numpy(flat).cuda(), [inner], None, None, 1e-5)
        case = {"name": "long_rows", "op": "LayerNorm", "args": {"normalized_shape": [inner], "eps": 1e-5}, "inputs": [flat]}
    torch.cuda.synchronize()
    want = cases.run_port(case)
    cases.assert_parity(case, got.cpu().numpy().reshape(want.shape), want)


def test_permute_vector_tiles_with_ragged_edges():
    """The 128-bit tile transpose on extents that are multiples of 4 but not of the 64-wide tile, and
    the scalar tile kernel right beside it (extents not multiples of 4)."""
    from shadow_b200 import functional as F
    torch = _torch()
    for shape, order in (((3, 68, 100), (0, 2, 1)), ((2, 4, 260), (2, 0, 1)), ((5, 132, 12, 8), (0, 2, 3, 1)),
                         ((3, 66, 100), (0, 2, 1)), ((2, 8, 6, 36), (1, 3, 0, 2)), ((7, 64, 64), (0, 2, 1))):
        x = cases.normal(7100 + len(shape) + shape[1], shape)
        got = F.permute(torch.from_numpy(x).cuda(), list(order))
        torch.cuda.synchronize()
        assert orc.bit_equal(got.cpu().numpy(), np.ascontiguousarray(np.transpose(x, order))), (shape, order)


def test_pad_vector_stores_cross_row_boundaries():
    """Output rows of 58, 7 and 3 floats: most float4 of the flat output straddle two rows (or three)."""
    from shadow_b200 import functional as F
    torch = _torch()
    for shape, pads, value in (((3, 5, 56, 56), (1, 1, 1, 1), 0.0), ((2, 3, 4, 5), (2, 0, 1, 1), -7.5),
                               ((4, 1, 6, 1), (0, 3, 1, 1), 2.0), ((2, 2, 9, 9), (-2, -1, -3, 0), 0.0), ((1, 1, 1, 1), (0, 0, 0, 0), 1.0),
                               # input widths that are multiples of 4: bands of output rows assembled in shared memory
                               ((2, 3, 8, 12), (0, 2, 3, 1), -1.0), ((1, 1, 4, 4), (0, 0, 0, 1), 9.0), ((300, 1, 1, 4), (1, 0, 0, 0), 0.5),
                               ((1, 2, 3, 6000), (1, 1, 2, 2), 0.0), ((7, 9, 20, 16), (3, 0, 0, 5), 1.5), ((2, 1, 1, 4), (0, 0, 0, 0), 0.0),
                               ((40, 16, 28, 28), (1, 2, 2, 1), 0.0)):
        x = cases.normal(7200 + shape[2], shape)
        got = F.pad(torch.from_numpy(x).cuda(), list(pads), value)
        torch.cuda.synchronize()
        want = orc.pad(x, list(pads), value)
        assert orc.bit_equal(got.cpu().numpy(), want), (shape, pads)


@pytest.mark.parametrize("shape", [(300, 1000, 7, 7), (310, 600, 9, 9), (300, 2500, 10), (297, 500, 14, 7), (600, 1002, 6, 4)],
                         ids=lambda s: "x".join(str(d) for d in s))
def test_softmax_with_the_plane_resident_in_shared_memory(shape):
    """Planes of 96..200 KB with enough of them to pipeline: the persistent kernel that keeps a plane in
    shared memory and streams the next one in by bulk asynchronous copies.  Ragged inner (49, 81, 10,
    98, 24), a partial last chunk, several planes per block; none of its bounded waits may run out."""
    from shadow_b200 import capi
    from shadow_b200 import functional as F
    torch = _torch()
    x = cases.normal(7300 + shape[1], shape, 0.0, 3.0)
    x[1, 5, 2] = -np.inf
    x[2, :, 1] = 80.0          # a column of equal large values
    got = F.softmax(torch.from_numpy(x).cuda(), 1)
    torch.cuda.synchronize()
    assert capi.lib().sb200_softmax_ring_timeouts() == 0
    case = {"name": "softmax_resident", "op": "Softmax", "args": {"axis": 1}, "inputs": [x]}
    want = cases.run_port(case)
    cases.assert_parity(case, got.cpu().numpy(), want)


POOL_GEOMETRIES = [
    # shape, pool, kernel, stride, pad, global, full
    ((3, 5, 70, 66), 0, [3], [2], [1], False, False),      # bands of rows of one plane, halo rows shared by two bands
    ((3, 5, 70, 66), 1, [3], [2], [1], False, True),       # ceil sizing: the last windows hang over the padded edge
    ((2, 3, 61, 63), 1, [2], [2], [0], False, True),       # odd extents: clipped windows at the bottom and the right
    ((2, 3, 61, 63), 0, [2, 3], [2, 1], [0, 1], False, False),
    ((41, 50, 7, 7), 1, [], [1], [0], True, True),         # many small planes per block, input count not a multiple of 4
    ((7, 33, 6, 10), 1, [3], [1], [1], False, True),       # planes per block does not divide the plane count
    ((7, 33, 6, 10), 0, [3], [1], [1], False, True),
    ((1, 2, 3, 1500), 0, [2], [1], [0], False, True),      # rows wider than a block's thread count
    ((1, 1, 2, 4000), 1, [2, 4], [1, 3], [0, 2], False, True),   # one output row per band at the larger shared-memory size
    ((2, 2, 40, 40), 0, [2], [3], [0], False, True),       # stride above the kernel: rows that no window reads
    ((1, 1, 1, 1), 1, [1], [1], [0], False, True),
    # planes above 12 KB whose width is a multiple of 4, with padding or overhang: the copy is laid out with its padding
    ((2, 3, 72, 64), 0, [3], [2], [1], False, False),
    ((2, 3, 72, 64), 1, [3], [2], [1], False, True),
    ((1, 2, 100, 68), 1, [2], [2], [1], False, True),
    ((1, 2, 200, 64), 1, [3], [2], [1], False, True),      # three bands
    ((1, 2, 200, 64), 0, [3], [2], [1], False, True),
    ((1, 1, 150, 64), 0, [3], [1], [1], False, True),
    ((1, 2, 80, 48), 1, [2, 5], [2, 3], [1, 2], False, True),   # run-time window loops over the padded copy
    ((1, 2, 80, 48), 0, [2], [3], [0], False, True),       # no padding, but the last window hangs over the edge
    ((2, 2, 64, 64), 1, [2], [2], [0], False, True),       # every window inside the tensor
    ((1, 1, 3, 6000), 0, [3], [1], [1], False, True),      # one band needs 72 KB of shared memory (opted into per device)
    ((1, 1, 3, 9000), 1, [3], [1], [1], False, True),      # and this one more than a block may have: windows through the caches
    ((300, 2, 7, 7), 1, [], [1], [0], True, True),         # whole passes of 256 one-output planes, then a short last block
]


@pytest.mark.parametrize("geometry", POOL_GEOMETRIES, ids=lambda g: "x".join(str(d) for d in g[0]) + ("_avg" if g[1] else "_max"))
@pytest.mark.parametrize("offset", [0, 1])
def test_pooling_from_shared_memory_rows(geometry, offset):
    """2-D pooling with the block's input range staged in shared memory (offset 0), and the same
    geometries from a base that is not 16-byte aligned (offset 1: windows read through the caches).
    Small windows add floats in the reference's order, so every result is bit-exact."""
    from shadow_b200 import functional as F
    shape, pool, kernel, stride, pad, global_pooling, full = geometry
    x = cases.normal(7400 + shape[2] + shape[3], shape)
    if pool == 0 and x.size > 64:
        # windows whose maximum is a zero, of either sign and in either order: std::max keeps the one it meets first
        flat = x.reshape(-1)
        flat[: flat.size // 2] = -np.abs(flat[: flat.size // 2])
        flat[3: flat.size // 2: 7] = -0.0
        flat[5: flat.size // 2: 11] = 0.0
    xv, _ = _view(x, offset)
    want = orc.pooling(x, pool, kernel, stride, pad, global_pooling, full)
    yv, ybuf = _view(np.zeros(want.shape, np.float32), 0)
    got = F.pooling(xv, pool, kernel, stride, pad, global_pooling, full, out=yv)
    _torch().cuda.synchronize()
    assert orc.bit_equal(got.cpu().numpy(), want)
    assert _guards_intact(ybuf, 0, want.size)


@pytest.mark.parametrize("offset", [0, 2])
def test_gather_with_vector_rows(offset):
    """Gather whose inner extent is a multiple of 4: 128-bit moves from an aligned base, the 4-byte kernel
    from a base that is not; repeated and out-of-order indexes, more float4 than one block moves."""
    from shadow_b200 import functional as F
    torch = _torch()
    for shape, axis, idx in (((3, 10, 4, 8), 1, [9, 0, 0, 5, 3]), ((6, 40, 36), 0, [5, 5, 1]), ((2, 7, 1028), 1, [6, 0, 3, 3, 1, 2]),
                             ((5, 12), 0, [4, 0])):
        x = cases.normal(7500 + shape[1], shape)
        xv, _ = _view(x, offset)
        want = np.take(x, idx, axis=axis)
        yv, ybuf = _view(np.zeros(want.shape, np.float32), offset)
        got = F.gather(xv, torch.tensor(idx, dtype=torch.int32, device="cuda"), axis, out=yv)
        torch.cuda.synchronize()
        assert orc.bit_equal(got.cpu().numpy(), want), (shape, axis)
        assert _guards_intact(ybuf, offset, want.size)
