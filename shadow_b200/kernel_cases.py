"""One small workload per CUDA kernel of the library, for profiling a kernel in isolation:

    python -m shadow_b200.kernel_cases <case> [launches]          # runs the case (default 2 launches)
    python -m shadow_b200.kernel_cases --list

Every case moves more than the 126 MB L2 (so DRAM counters mean something) and holds well under a
GB on the device, so that a profiler capture of one launch ends within seconds.  The first column
of the table is the case name, the second the kernel it launches (what to give `ncu -k regex:`),
the third the algorithmic bytes of one launch.
"""
from __future__ import annotations

import sys


def _cases(torch, F):
    dev = torch.device("cuda", 0)

    def normal(shape, sd=1.0):
        return torch.empty(shape, device=dev).normal_(0, sd)

    def uniform(shape, lo, hi):
        return torch.empty(shape, device=dev).uniform_(lo, hi)

    table = {}

    def case(name, kernel, make):
        table[name] = (kernel, make)

    n_ew = (128, 256, 28, 28)   # 25.7 M floats, 103 MB per tensor

    def unary(code, lo, hi):
        def make():
            x = uniform(n_ew, lo, hi)
            y = torch.empty_like(x)
            return (lambda: F.unary(x, code, out=y)), 8 * x.numel()
        return make

    def activate(code):
        def make():
            x = normal(n_ew, 2.0)
            y = torch.empty_like(x)
            return (lambda: F.activate(x, code, 0.1, out=y)), 8 * x.numel()
        return make

    case("unary_neg", "ew_vec_kernel", unary(13, -1, 1))
    case("unary_exp", "ew_vec_kernel", unary(4, -10, 10))
    case("unary_log", "ew_vec_kernel", unary(3, 0.01, 10))
    case("activate_relu", "ew_vec_kernel", activate(1))
    case("activate_sigmoid", "ew_vec_kernel", activate(3))
    case("activate_tanh", "ew_vec_kernel", activate(5))

    case("unary_sin", "ew_vec_kernel", unary(5, -10, 10))
    case("unary_tan", "ew_vec_kernel", unary(7, -10, 10))
    case("activate_softplus", "ew_vec_kernel", activate(4))
    case("activate_gelu", "ew_vec_kernel", activate(8))

    def binary_pow():
        a, c = uniform(n_ew, 0.5, 2.0), uniform(n_ew, 0.5, 2.0)
        y = torch.empty_like(a)
        return (lambda: F.binary(a, c, 4, out=y)), 12 * a.numel()
    case("binary_same_pow", "ew_vec_kernel", binary_pow)

    def binary_same():
        a, c = uniform(n_ew, -1, 1), uniform(n_ew, -1, 1)
        y = torch.empty_like(a)
        return (lambda: F.binary(a, c, 0, out=y)), 12 * a.numel()
    case("binary_same_add", "ew_vec_kernel", binary_same)

    def binary_scalar():
        a = uniform(n_ew, -1, 1)
        y = torch.empty_like(a)
        return (lambda: F.binary_scalar(a, 1.5, 2, out=y)), 8 * a.numel()
    case("binary_scalar_mul", "ew_vec_kernel", binary_scalar)

    def binary_channel():
        a, b = uniform((128, 64, 56, 56), -1, 1), normal((1, 64, 1, 1))
        y = torch.empty_like(a)
        return (lambda: F.binary(a, b, 2, out=y)), 8 * a.numel() + 256
    case("binary_broadcast_channel", "chan_vec_kernel", binary_channel)

    def binary_rowvec():
        a, b = uniform((2, 1, 2048, 2048), -1, 1), normal((1, 1, 1, 2048))
        y = torch.empty((2, 1, 2048, 2048), device=dev)
        return (lambda: F.binary(a, b, 2, out=y)), 8 * a.numel() + 4 * 2048
    case("binary_broadcast_rowvec", "bcast_rowvec_kernel", binary_rowvec)

    def binary_reuse():
        a, b = uniform((2, 1, 2048, 2048), -1, 1), normal((1, 16, 1, 2048))
        y = torch.empty((2, 16, 2048, 2048), device=dev)
        return (lambda: F.binary(a, b, 2, out=y)), 4 * (a.numel() + b.numel() + y.numel())
    case("binary_broadcast_reuse", "bcast_reuse_kernel", binary_reuse)

    def scale():
        x = normal(n_ew, 2.0)
        g, bt = normal((256,), 0.1) + 1, normal((256,), 0.1)
        y = torch.empty_like(x)
        return (lambda: F.scale(x, 1, g, bt, out=y)), 8 * x.numel() + 8 * 256
    case("scale_channel", "chan_vec_kernel", scale)

    red_shape = (256, 512, 14, 14)   # 25.7 M floats

    def reduce(code, axes, outs, lo=None):
        def make():
            x = normal(red_shape) if lo is None else uniform(red_shape, lo, 2 - lo)
            r = torch.empty(outs, device=dev)
            return (lambda: F.reduce(x, code, axes, out=r)), 4 * (x.numel() + outs)
        return make

    case("reduce_sum_spatial", "redA_rows_kernel", reduce(1, (2, 3), 256 * 512))
    case("reduce_max_spatial", "redA_rows_kernel", reduce(2, (2, 3), 256 * 512))
    case("reduce_prod_spatial", "redA_rows_kernel", reduce(0, (2, 3), 256 * 512, 0.99))
    def reduce_channel(code):
        def make():
            x = normal((512, 512, 14, 14))          # enough planes for the fixed-column walk
            r = torch.empty(512 * 196, device=dev)
            return (lambda: F.reduce(x, code, (1,), out=r)), 4 * (x.numel() + 512 * 196)
        return make

    case("reduce_sum_channel", "redC_kernel", reduce_channel(1))
    case("reduce_max_channel", "redC_kernel", reduce_channel(2))
    case("reduce_sum_batch_spatial", "redB_kernel", reduce(1, (0, 2, 3), 512))
    case("reduce_sum_all", "redA_block_kernel", reduce(1, (), 1))

    def softmax(shape, sd, axis):
        def make():
            x = normal(shape, sd)
            y = torch.empty_like(x)
            return (lambda: F.softmax(x, axis, out=y)), 8 * x.numel()
        return make

    case("softmax_rows", "softmax_rows_kernel", softmax((6144, 4096), 3.0, -1))
    case("softmax_strided_c4b", "softmax_ring_kernel", softmax((512, 1000, 7, 7), 1.0, 1))
    case("softmax_strided_c4b_few_planes", "softmax_colvec_kernel", softmax((280, 1000, 7, 7), 1.0, 1))
    case("softmax_strided_wide", "softmax_colreg_kernel", softmax((5, 21, 512, 512), 1.0, 1))

    def normalize():
        x = normal((32, 512, 38, 38))
        y = torch.empty_like(x)
        return (lambda: F.normalize(x, 1, 2.0, 1e-12, out=y)), 8 * x.numel()
    case("normalize_l2_channel", "normalize_colvec_kernel", normalize)

    def layer_norm():
        x = normal((32768, 768))
        g, bt = normal((768,)), normal((768,))
        y = torch.empty_like(x)
        return (lambda: F.layer_norm(x, [768], g, bt, 1e-5, out=y)), 8 * x.numel()
    case("layer_norm_rows", "rownorm_rows_kernel", layer_norm)

    def group_norm():
        x = normal((128, 64, 56, 56))
        g, bt = normal((64,)), normal((64,))
        y = torch.empty_like(x)
        return (lambda: F.group_norm(x, 8, g, bt, 1e-5, out=y)), 8 * x.numel()
    case("group_norm_100kb_rows", "rownorm_smem_rows_kernel", group_norm)

    def permute():
        x = normal((32, 256, 56, 56))
        y = torch.empty((32, 56, 56, 256), device=dev)
        return (lambda: F.permute(x, [0, 2, 3, 1], out=y)), 8 * x.numel()
    case("permute_nchw_nhwc", "permute_tile4_kernel", permute)

    def pad():
        x = normal((64, 160, 56, 56))
        y = torch.empty((64, 160, 58, 58), device=dev)
        return (lambda: F.pad(x, [1, 1, 1, 1], 0.0, out=y)), 4 * (x.numel() + y.numel())
    case("pad_border_1", "pad_vec_kernel", pad)

    def gather():
        x = normal((64, 160, 56, 56))
        idx = torch.arange(0, 160, 2, device=dev, dtype=torch.int32)
        y = torch.empty((64, 80, 56, 56), device=dev)
        return (lambda: F.gather(x, idx, 1, out=y)), 8 * y.numel()
    case("gather_every_2nd_channel", "gather_vec_kernel", gather)

    def pooling(pool, kernel, stride, pad, full):
        def make():
            x = normal((64, 64, 112, 112))
            y = torch.empty((64, 64, 56, 56), device=dev)
            return (lambda: F.pooling(x, pool, [kernel], [stride], [pad], full_pooling=full, out=y)), 4 * (x.numel() + y.numel())
        return make
    case("pooling_max_k2_s2", "pool_smem_kernel", pooling(0, 2, 2, 0, True))
    case("pooling_max_k3_s2_p1", "pool_smem_kernel", pooling(0, 3, 2, 1, False))

    def pooling_global():
        x = normal((512, 2048, 7, 7))
        y = torch.empty((512, 2048, 1, 1), device=dev)
        return (lambda: F.pooling(x, 1, global_pooling=True, out=y)), 4 * (x.numel() + y.numel())
    case("pooling_avg_global_7x7", "pool_smem_kernel", pooling_global)
    return table


def main(argv) -> int:
    import torch
    from . import functional as F
    table = _cases(torch, F)
    if len(argv) < 2 or argv[1] == "--list":
        for name, (kernel, _) in table.items():
            print("%-28s %s" % (name, kernel))
        return 0
    name = argv[1]
    launches = int(argv[2]) if len(argv) > 2 else 2
    if name not in table:
        print("unknown case %s (try --list)" % name, file=sys.stderr)
        return 2
    kernel, make = table[name]
    fn, nbytes = make()
    for _ in range(launches):
        fn()
    torch.cuda.synchronize()
    print("ok %s kernel=%s algorithmic_bytes=%d" % (name, kernel, nbytes))
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv))
