"""sb200_reduce_static: the reduction for callers that cannot hand over (or allocate) a scratch
buffer - a serving loop whose device memory was all assigned at start-up, or code that holds only
the input and output pointers.  Its cross-block partials live in a 1 MiB array built into the
library.  Checked here through the C ABI against sb200_reduce (caller scratch) on the same input,
bit for bit, twice in a row with different data, so that partials left behind by the first call
cannot leak into the second.  Collected last on purpose (file name)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

STATIC_BYTES = 1 << 20

# (shape, axes): all of them split the reduction over blocks, i.e. really use the scratch
GEOMETRIES = [
    ((8, 1024, 1024), [0, 1, 2]),      # full tensor: 256 splits x 1 output
    ((64, 96, 56, 56), [0, 2, 3]),     # R K R: several splits x 96 outputs
    ((3000, 196), [0]),                # column reduce split along the reduced dim
    ((4, 50000, 12), [1]),             # K R K
]


def _ptr(t):
    return t.data_ptr()


@pytest.mark.parametrize("shape,axes", GEOMETRIES, ids=lambda v: str(v).replace(" ", ""))
@pytest.mark.parametrize("operation", [1, 2, 4, 6], ids=["sum", "max", "avg", "l2"])
def test_static_scratch_matches_caller_scratch_twice(shape, axes, operation):
    import torch
    from shadow_b200 import capi
    lib = capi.lib()
    stream = torch.cuda.current_stream().cuda_stream
    shape_c, axes_c = capi.ints(shape), capi.ints(axes)
    need = lib.sb200_reduce_scratch_bytes(shape_c, len(shape), axes_c, len(axes), operation)
    assert 0 < need <= STATIC_BYTES, need
    out_shape = [1 if n in axes else d for n, d in enumerate(shape)]
    scratch = torch.empty(need, dtype=torch.uint8, device="cuda")
    gen = torch.Generator(device="cuda").manual_seed(1234)
    for call in range(2):
        x = torch.randn(shape, device="cuda", generator=gen) * (1.0 + call)
        want = torch.full(out_shape, float("nan"), device="cuda")
        got = torch.full(out_shape, float("nan"), device="cuda")
        capi.check(lib.sb200_reduce(_ptr(x), shape_c, len(shape), axes_c, len(axes), operation, _ptr(want),
                                    _ptr(scratch), need, stream), "sb200_reduce")
        before = capi.launch_count()
        capi.check(lib.sb200_reduce_static(_ptr(x), shape_c, len(shape), axes_c, len(axes), operation, _ptr(got),
                                           stream), "sb200_reduce_static")
        assert capi.launch_count() - before == 2        # first-stage kernel + finishing kernel
        torch.cuda.synchronize()
        # the property the entry point exists for: the call takes no device memory.  Free memory as
        # the driver reports it (not torch's caching allocator) is the same before and after a call.
        free_before = torch.cuda.mem_get_info()[0]
        capi.check(lib.sb200_reduce_static(_ptr(x), shape_c, len(shape), axes_c, len(axes), operation, _ptr(got),
                                           stream), "sb200_reduce_static")
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free_before
        w, g = want.cpu().numpy(), got.cpu().numpy()
        # same plan, same kernels, same combination order: identical bits (the tests' bar for
        # reductions is 1e-5*log2(n) relative; this is far inside it)
        assert np.array_equal(w.view(np.uint32), g.view(np.uint32))
        assert not np.isnan(g).any()
        if call == 1:
            # and against the CPU oracle, at the reductions' bar
            from oracle import oracle as orc
            ref = orc.reduce(x.cpu().numpy(), operation, axes, keep_dims=True)
            n = int(np.prod([shape[a] for a in axes]))
            if operation == 2:
                assert np.array_equal(ref, g)
            else:
                assert np.allclose(g, ref, rtol=1e-5 * np.log2(n), atol=0)


def test_static_scratch_without_split_needs_no_buffer():
    import torch
    from shadow_b200 import capi
    lib = capi.lib()
    x = torch.randn(37, 5, 8, 7, device="cuda")
    shape_c, axes_c = capi.ints(x.shape), capi.ints([2, 3])
    assert lib.sb200_reduce_scratch_bytes(shape_c, 4, axes_c, 2, 1) == 0
    y = torch.empty(37, 5, 1, 1, device="cuda")
    capi.check(lib.sb200_reduce_static(_ptr(x), shape_c, 4, axes_c, 2, 1, _ptr(y), torch.cuda.current_stream().cuda_stream),
               "sb200_reduce_static")
    torch.cuda.synchronize()
    assert torch.allclose(y, x.double().sum(dim=(2, 3), keepdim=True).float(), rtol=1e-6)


def test_oversized_reduction_is_refused_before_launch():
    import torch
    from shadow_b200 import capi
    lib = capi.lib()
    shape, axes = (4096, 65536), [0]        # 16 splits x 65536 outputs x 8 B = 8 MiB of partials
    shape_c, axes_c = capi.ints(shape), capi.ints(axes)
    need = lib.sb200_reduce_scratch_bytes(shape_c, 2, axes_c, 1, 1)
    assert need > STATIC_BYTES
    dummy = torch.zeros(16, device="cuda")   # never dereferenced: the call is refused first
    before = capi.launch_count()
    rc = lib.sb200_reduce_static(_ptr(dummy), shape_c, 2, axes_c, 1, 1, _ptr(dummy), None)
    assert rc == 4
    assert capi.launch_count() == before
    # a geometry that the planner refuses keeps its own status (more than 8 axes after collapsing)
    many_axes = [2, 3] * 9
    odd_axes = list(range(0, 18, 2))
    rc2 = lib.sb200_reduce_static(_ptr(dummy), capi.ints(many_axes), 18, capi.ints(odd_axes), 9, 1, _ptr(dummy), None)
    assert rc2 == lib.sb200_reduce(_ptr(dummy), capi.ints(many_axes), 18, capi.ints(odd_axes), 9, 1, _ptr(dummy), None, 0, None)
    assert rc2 in (1, 2)
    rc3 = lib.sb200_reduce_static(_ptr(dummy), shape_c, 2, capi.ints([5]), 1, 1, _ptr(dummy), None)   # axis out of range
    assert rc3 == 1
    assert capi.launch_count() == before
    text = lib.sb200_last_cuda_error().decode()
    assert str(need) in text and str(STATIC_BYTES) in text
    with pytest.raises(capi.Sb200Error, match="built-in buffer"):
        capi.check(rc, "sb200_reduce_static")
