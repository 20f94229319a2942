"""Operator-level calls on CUDA tensors that are already resident in HBM.

Each function applies the shape rule of the reference operator front-end
(shadow/operators/{binary,unary,activate,scale,reduce,softmax}_op.cpp) and then makes exactly the
C-ABI call(s) of ``include/sb200.h`` on the tensor's device pointers and the current torch stream.
torch is used only for device memory and streams; all arithmetic happens in ``libsb200.so``.
Inputs must be contiguous float32 CUDA tensors; there is no CPU path.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Sequence

import torch

from . import capi


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _chk(t: torch.Tensor, name: str) -> torch.Tensor:
    if not (t.is_cuda and t.dtype == torch.float32 and t.is_contiguous()):
        raise ValueError("%s must be a contiguous float32 CUDA tensor" % name)
    return t


def fill(y: torch.Tensor, val: float) -> torch.Tensor:
    _chk(y, "y")
    capi.check(capi.lib().sb200_fill(y.data_ptr(), y.numel(), val, _stream()), "sb200_fill")
    return y


def unary(x: torch.Tensor, operation: int, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _chk(x, "x")
    y = torch.empty_like(x) if out is None else _chk(out, "out")
    capi.check(capi.lib().sb200_unary(x.data_ptr(), y.data_ptr(), x.numel(), operation, _stream()), "sb200_unary")
    return y


def activate(x: torch.Tensor, type: int = 1, slope: float = 0.1, slope_blob: Optional[torch.Tensor] = None,
             out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _chk(x, "x")
    y = torch.empty_like(x) if out is None else _chk(out, "out")
    if type == 0:
        s = _chk(slope_blob, "slope_blob")
        if x.dim() < 2:
            raise ValueError("PRelu needs >= 2 axes")
        shared = s.numel() == 1
        if not shared and s.numel() != x.shape[1]:
            raise ValueError("PRelu slope count must be 1 or channels")
        dim = 1
        for d in x.shape[2:]:
            dim *= d
        capi.check(capi.lib().sb200_prelu(x.data_ptr(), y.data_ptr(), x.shape[0], x.shape[1], dim,
                                          s.data_ptr(), int(shared), _stream()), "sb200_prelu")
    else:
        capi.check(capi.lib().sb200_activate(x.data_ptr(), y.data_ptr(), x.numel(), type, slope, _stream()),
                   "sb200_activate")
    return y


def binary_scalar(a: torch.Tensor, scalar: float, operation: int, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _chk(a, "a")
    y = torch.empty_like(a) if out is None else _chk(out, "out")
    capi.check(capi.lib().sb200_binary_scalar(a.data_ptr(), scalar, y.data_ptr(), a.numel(), operation, _stream()),
               "sb200_binary_scalar")
    return y


def broadcast_shapes(sa: Sequence[int], sb: Sequence[int]):
    sa, sb = list(sa), list(sb)
    nd = max(len(sa), len(sb))
    pa, pb = [1] * (nd - len(sa)) + sa, [1] * (nd - len(sb)) + sb
    out = []
    for da, db in zip(pa, pb):
        if not (da == db or da == 1 or db == 1):
            raise ValueError("shapes %s and %s do not broadcast" % (sa, sb))
        out.append(max(da, db))
    return pa, pb, out


def binary(a: torch.Tensor, b: torch.Tensor, operation: int, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _chk(a, "a"), _chk(b, "b")
    if tuple(a.shape) == tuple(b.shape):
        y = torch.empty_like(a) if out is None else _chk(out, "out")
        capi.check(capi.lib().sb200_binary(a.data_ptr(), b.data_ptr(), y.data_ptr(), a.numel(), operation,
                                           _stream()), "sb200_binary")
        return y
    pa, pb, po = broadcast_shapes(a.shape, b.shape)
    y = torch.empty(po, dtype=torch.float32, device=a.device) if out is None else _chk(out, "out")
    capi.check(capi.lib().sb200_binary_broadcast(a.data_ptr(), capi.ints(pa), b.data_ptr(), capi.ints(pb),
                                                 capi.ints(po), len(po), y.data_ptr(), operation, _stream()),
               "sb200_binary_broadcast")
    return y


def scale(x: torch.Tensor, axis: int = 1, scale: Optional[torch.Tensor] = None,
          bias: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _chk(x, "x")
    ref = scale if scale is not None else bias
    if ref is None:
        raise ValueError("scale or bias required")
    if scale is not None and bias is not None and tuple(scale.shape) != tuple(bias.shape):
        raise ValueError("scale and bias shapes differ")
    inner = 1
    for d in x.shape[axis + ref.dim():]:
        inner *= d
    y = torch.empty_like(x) if out is None else _chk(out, "out")
    capi.check(capi.lib().sb200_scale_bias(
        x.data_ptr(), y.data_ptr(), x.numel(), scale.data_ptr() if scale is not None else None,
        bias.data_ptr() if bias is not None else None, ref.numel(), inner, _stream()), "sb200_scale_bias")
    return y


class ReduceScratch:
    """Grow-only device scratch, the analogue of Workspace::GrowTempBuffer for Python callers: one
    buffer per (device, stream), because kernels of two streams may run at the same time and a
    reduction's partials must not be shared between them.  A buffer that is outgrown is handed back
    to torch's allocator only after the stream that used it has been told so (record_stream), so its
    memory cannot be reused while a kernel of that stream may still write it.  A CUDA graph captures the
    buffer's address: do not outgrow the buffer of a stream between capture and replay."""

    def __init__(self):
        self.bufs = {}

    def get(self, nbytes: int, device) -> int:
        if nbytes <= 0:
            return 0
        stream = torch.cuda.current_stream(device)
        key = (torch.device(device).index, stream.cuda_stream)
        buf = self.bufs.get(key)
        if buf is None or buf.numel() < nbytes:
            if buf is not None:
                buf.record_stream(stream)
            buf = torch.empty(nbytes, dtype=torch.uint8, device=device)
            self.bufs[key] = buf
        return buf.data_ptr()


_scratch = ReduceScratch()


def reduce(x: torch.Tensor, operation: int = 0, axes: Sequence[int] = (), keep_dims: bool = True,
           out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _chk(x, "x")
    axes = list(axes) if len(axes) else list(range(x.dim()))
    out_shape = list(x.shape)
    for ax in axes:
        out_shape[ax] = 1
    y = torch.empty(out_shape, dtype=torch.float32, device=x.device) if out is None else _chk(out, "out")
    shape_c, axes_c = capi.ints(x.shape), capi.ints(axes)
    nbytes = capi.lib().sb200_reduce_scratch_bytes(shape_c, x.dim(), axes_c, len(axes), operation)
    if nbytes < 0:
        raise capi.Sb200Error(1, "sb200_reduce_scratch_bytes")
    capi.check(capi.lib().sb200_reduce(x.data_ptr(), shape_c, x.dim(), axes_c, len(axes), operation, y.data_ptr(),
                                       _scratch.get(nbytes, x.device), nbytes, _stream()), "sb200_reduce")
    if not keep_dims:
        y = y.reshape([d for n, d in enumerate(out_shape) if n not in axes])
    return y


def reduce_partial(x: torch.Tensor, operation: int, axes: Sequence[int],
                   out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Double partial per kept position (see sb200_reduce_partial); shape = x.shape with reduced dims 1.
    ``out``: a contiguous float64 CUDA tensor with that many elements to write into."""
    _chk(x, "x")
    axes = list(axes) if len(axes) else list(range(x.dim()))
    out_shape = list(x.shape)
    for ax in axes:
        out_shape[ax] = 1
    if out is None:
        part = torch.empty(out_shape, dtype=torch.float64, device=x.device)
    else:
        n = 1
        for d in out_shape:
            n *= d
        if not (out.is_cuda and out.dtype == torch.float64 and out.is_contiguous() and out.numel() == n):
            raise ValueError("out must be a contiguous float64 CUDA tensor of %d elements" % n)
        part = out
    shape_c, axes_c = capi.ints(x.shape), capi.ints(axes)
    nbytes = capi.lib().sb200_reduce_scratch_bytes(shape_c, x.dim(), axes_c, len(axes), operation)
    capi.check(capi.lib().sb200_reduce_partial(x.data_ptr(), shape_c, x.dim(), axes_c, len(axes), operation,
                                               part.data_ptr(), _scratch.get(nbytes, x.device), nbytes, _stream()),
               "sb200_reduce_partial")
    return part


def reduce_finalize(part: torch.Tensor, operation: int, total_reduced_count: int) -> torch.Tensor:
    y = torch.empty(part.shape, dtype=torch.float32, device=part.device)
    capi.check(capi.lib().sb200_reduce_finalize(part.data_ptr(), y.data_ptr(), part.numel(), operation,
                                                total_reduced_count, _stream()), "sb200_reduce_finalize")
    return y


def reduce_combine(parts: torch.Tensor, n_parts: int, part_stride: int, count: int, operation: int,
                   total_reduced_count: int, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Merge ``n_parts`` double records (``parts[p*part_stride + o]``) and finish to float
    (see sb200_reduce_combine)."""
    y = torch.empty(count, dtype=torch.float32, device=parts.device) if out is None else _chk(out, "out")
    capi.check(capi.lib().sb200_reduce_combine(parts.data_ptr(), n_parts, part_stride, y.data_ptr(), count, operation,
                                               total_reduced_count, _stream()), "sb200_reduce_combine")
    return y


def softmax(x: torch.Tensor, axis: int = 1, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _chk(x, "x")
    if not -x.dim() <= axis < x.dim():
        raise ValueError("axis out of range")
    axis %= x.dim()
    outer = 1
    for d in x.shape[:axis]:
        outer *= d
    inner = 1
    for d in x.shape[axis + 1:]:
        inner *= d
    y = torch.empty_like(x) if out is None else _chk(out, "out")
    capi.check(capi.lib().sb200_softmax(x.data_ptr(), y.data_ptr(), outer, x.shape[axis], inner, _stream()),
               "sb200_softmax")
    return y


def eltwise(inputs: Sequence[torch.Tensor], operation: int, coeff: Sequence[float] = (),
            out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Eltwise operator (shadow/operators/eltwise_op.cpp:7-56): >= 2 inputs of one shape."""
    import ctypes as C
    xs = [_chk(x, "input") for x in inputs]
    if len(xs) < 2 or any(tuple(x.shape) != tuple(xs[0].shape) for x in xs):
        raise ValueError("eltwise needs >= 2 inputs of one shape")
    if len(coeff) and (operation != 1 or len(coeff) != len(xs)):
        raise ValueError("coefficients only for Sum, one per input")
    y = torch.empty_like(xs[0]) if out is None else _chk(out, "out")
    ptrs = (C.c_void_p * len(xs))(*[x.data_ptr() for x in xs])
    cf = (C.c_float * len(coeff))(*[float(c) for c in coeff]) if len(coeff) else None
    capi.check(capi.lib().sb200_eltwise(ptrs, len(xs), cf, y.data_ptr(), y.numel(), operation, _stream()),
               "sb200_eltwise")
    return y


def axpy(alpha: torch.Tensor, x: torch.Tensor, y: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Axpy operator (shadow/operators/axpy_op.cpp:16-51): out = alpha[n,c] * x + y."""
    _chk(alpha, "alpha"), _chk(x, "x"), _chk(y, "y")
    if tuple(x.shape) != tuple(y.shape) or alpha.shape[0] != x.shape[0] or alpha.shape[1] != x.shape[1]:
        raise ValueError("axpy shapes")
    inner = 1
    for d in x.shape[2:]:
        inner *= d
    o = torch.empty_like(x) if out is None else _chk(out, "out")
    capi.check(capi.lib().sb200_axpy(alpha.data_ptr(), x.data_ptr(), y.data_ptr(), o.data_ptr(), alpha.numel(), inner,
                                     _stream()), "sb200_axpy")
    return o


def batch_norm(x: torch.Tensor, mean: torch.Tensor, variance: torch.Tensor, scale_factor: float = 1.0,
               eps: float = 1e-5, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Inference BatchNorm (shadow/operators/batch_norm_op.cpp:9-43); `scale_factor` is what the
    operator front-end derives from its optional 4th input."""
    _chk(x, "x"), _chk(mean, "mean"), _chk(variance, "variance")
    if mean.numel() != x.shape[1] or variance.numel() != x.shape[1]:
        raise ValueError("mean/variance must have one value per channel")
    inner = 1
    for d in x.shape[2:]:
        inner *= d
    y = torch.empty_like(x) if out is None else _chk(out, "out")
    capi.check(capi.lib().sb200_batch_norm(x.data_ptr(), y.data_ptr(), x.numel(), mean.data_ptr(), variance.data_ptr(),
                                           x.shape[1], inner, scale_factor, eps, _stream()), "sb200_batch_norm")
    return y


def normalize(x: torch.Tensor, axis: int = 1, p: float = 2.0, eps: float = 1e-12,
              out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Normalize (shadow/operators/normalize_op.cpp:9-37): x / max(||x||_p over `axis`, eps)."""
    _chk(x, "x")
    axis = axis + x.dim() if axis < 0 else axis
    if not 0 <= axis < x.dim():
        raise ValueError("axis out of range")
    outer = 1
    for d in x.shape[:axis]:
        outer *= d
    inner = 1
    for d in x.shape[axis + 1:]:
        inner *= d
    y = torch.empty_like(x) if out is None else _chk(out, "out")
    capi.check(capi.lib().sb200_normalize(x.data_ptr(), y.data_ptr(), outer, x.shape[axis], inner, p, eps, _stream()),
               "sb200_normalize")
    return y


def _row_norm(x, rows, inner, eps, scale, bias, mode, groups, cpg, spatial, out):
    y = torch.empty_like(x) if out is None else _chk(out, "out")
    sp = _chk(scale, "scale").data_ptr() if scale is not None else None
    bp = _chk(bias, "bias").data_ptr() if bias is not None else None
    capi.check(capi.lib().sb200_row_norm(x.data_ptr(), y.data_ptr(), rows, inner, eps, sp, bp, mode, groups, cpg, spatial,
                                         _stream()), "sb200_row_norm")
    return y


def layer_norm(x: torch.Tensor, normalized_shape, scale: Optional[torch.Tensor] = None,
               bias: Optional[torch.Tensor] = None, eps: float = 1e-5, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """LayerNorm (shadow/operators/layer_norm_op.cpp:9-50): statistics over the trailing
    `normalized_shape` dims; scale and bias (both or neither) have that shape."""
    _chk(x, "x")
    k = len(normalized_shape)
    if k < 1 or tuple(x.shape[x.dim() - k:]) != tuple(normalized_shape):
        raise ValueError("normalized_shape must equal the trailing dims of x")
    inner = 1
    for d in normalized_shape:
        inner *= d
    if (scale is None) != (bias is None):
        raise ValueError("scale and bias come together")
    if scale is not None and (scale.numel() != inner or bias.numel() != inner):
        raise ValueError("scale/bias must have normalized_shape")
    return _row_norm(x, x.numel() // inner, inner, eps, scale, bias, 1 if scale is not None else 0, 1, 1, 1, out)


def group_norm(x: torch.Tensor, group: int, scale: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None,
               eps: float = 1e-5, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """GroupNorm (shadow/operators/group_norm_op.cpp:9-45): statistics per (sample, group of
    channels); scale and bias (both or neither) per channel.  InstanceNorm is group == channels."""
    _chk(x, "x")
    channel = x.shape[1]
    if group < 1 or channel % group:
        raise ValueError("channels must be divisible by group")
    spatial = 1
    for d in x.shape[2:]:
        spatial *= d
    cpg = channel // group
    if (scale is None) != (bias is None):
        raise ValueError("scale and bias come together")
    if scale is not None and (scale.numel() != channel or bias.numel() != channel):
        raise ValueError("scale/bias must have one value per channel")
    return _row_norm(x, x.shape[0] * group, cpg * spatial, eps, scale, bias, 2 if scale is not None else 0, group, cpg,
                     spatial, out)


def instance_norm(x: torch.Tensor, scale: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None,
                  eps: float = 1e-5, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """InstanceNorm (shadow/operators/instance_norm_op.cpp:9-40): GroupNorm with one channel per group."""
    return group_norm(x, x.shape[1], scale, bias, eps, out)


def ssd_normalize(x: torch.Tensor, scale: Optional[torch.Tensor] = None, across_spatial: bool = True,
                  channel_shared: bool = True, eps: float = 1e-5, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """SSDNormalize (shadow/operators/ssd_normalize_op.cpp:9-45)."""
    _chk(x, "x")
    if x.dim() < 2:
        raise ValueError("x needs a channel axis")
    spatial = 1
    for d in x.shape[2:]:
        spatial *= d
    if scale is not None:
        _chk(scale, "scale")
        if scale.numel() != (1 if channel_shared else x.shape[1]):
            raise ValueError("scale must hold one value (channel_shared) or one per channel")
    y = torch.empty_like(x) if out is None else _chk(out, "out")
    capi.check(capi.lib().sb200_ssd_normalize(x.data_ptr(), y.data_ptr(), x.shape[0], x.shape[1], spatial,
                                              1 if across_spatial else 0, eps,
                                              scale.data_ptr() if scale is not None else None,
                                              1 if channel_shared else 0, _stream()), "sb200_ssd_normalize")
    return y


def _prod(dims) -> int:
    n = 1
    for d in dims:
        n *= int(d)
    return n


def concat(inputs, axis: int = 1, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Concat (shadow/operators/concat_op.cpp:9-45)."""
    first = _chk(inputs[0], "inputs[0]")
    axis = axis + first.dim() if axis < 0 else axis
    shape = list(first.shape)
    for t in inputs[1:]:
        _chk(t, "input")
        if t.dim() != first.dim() or any(t.shape[d] != shape[d] for d in range(first.dim()) if d != axis):
            raise ValueError("inputs must agree except on the concat axis")
        shape[axis] += t.shape[axis]
    y = torch.empty(shape, dtype=torch.float32, device=first.device) if out is None else _chk(out, "out")
    inner = _prod(first.shape[axis + 1:])
    ptrs = (ctypes.c_void_p * len(inputs))(*[t.data_ptr() for t in inputs])
    widths = (ctypes.c_int64 * len(inputs))(*[t.shape[axis] * inner for t in inputs])
    capi.check(capi.lib().sb200_concat(ptrs, widths, len(inputs), y.data_ptr(), _prod(first.shape[:axis]), _stream()),
               "sb200_concat")
    return y


def stack(inputs, axis: int = 0, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Stack (shadow/operators/stack_op.cpp:9-40)."""
    first = _chk(inputs[0], "inputs[0]")
    axis = axis + first.dim() + 1 if axis < 0 else axis
    for t in inputs[1:]:
        if _chk(t, "input").shape != first.shape:
            raise ValueError("inputs must share one shape")
    shape = list(first.shape)
    shape.insert(axis, len(inputs))
    y = torch.empty(shape, dtype=torch.float32, device=first.device) if out is None else _chk(out, "out")
    width = _prod(first.shape[axis:])
    ptrs = (ctypes.c_void_p * len(inputs))(*[t.data_ptr() for t in inputs])
    widths = (ctypes.c_int64 * len(inputs))(*[width] * len(inputs))
    capi.check(capi.lib().sb200_concat(ptrs, widths, len(inputs), y.data_ptr(), _prod(first.shape[:axis]), _stream()),
               "sb200_concat")
    return y


def slice_(x: torch.Tensor, axis: int, sizes) -> list:
    """Slice (shadow/operators/slice_op.cpp:9-60): split `axis` into pieces of the given sizes."""
    _chk(x, "x")
    axis = axis + x.dim() if axis < 0 else axis
    if sum(sizes) != x.shape[axis] or min(sizes) < 1:
        raise ValueError("sizes must be positive and add up to the axis extent")
    inner = _prod(x.shape[axis + 1:])
    outs = []
    for sz in sizes:
        shape = list(x.shape)
        shape[axis] = sz
        outs.append(torch.empty(shape, dtype=torch.float32, device=x.device))
    ptrs = (ctypes.c_void_p * len(outs))(*[t.data_ptr() for t in outs])
    widths = (ctypes.c_int64 * len(outs))(*[sz * inner for sz in sizes])
    capi.check(capi.lib().sb200_slice(x.data_ptr(), ptrs, widths, len(outs), _prod(x.shape[:axis]), _stream()), "sb200_slice")
    return outs


def permute(x: torch.Tensor, order, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Permute (shadow/operators/permute_op.cpp:9-35)."""
    _chk(x, "x")
    if sorted(order) != list(range(x.dim())):
        raise ValueError("order must be a permutation of the axes")
    shape = [x.shape[a] for a in order]
    y = torch.empty(shape, dtype=torch.float32, device=x.device) if out is None else _chk(out, "out")
    ishape = (ctypes.c_int * x.dim())(*x.shape)
    iorder = (ctypes.c_int * x.dim())(*order)
    capi.check(capi.lib().sb200_permute(x.data_ptr(), y.data_ptr(), ishape, iorder, x.dim(), _stream()), "sb200_permute")
    return y


def gather(x: torch.Tensor, indexes: torch.Tensor, axis: int = 0, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Gather (shadow/operators/gather_op.cpp:9-50); `indexes` is a 1-d int32 device tensor."""
    _chk(x, "x")
    if indexes.dtype != torch.int32 or indexes.dim() != 1 or not indexes.is_cuda or not indexes.is_contiguous():
        raise TypeError("indexes must be a contiguous 1-d int32 CUDA tensor")
    axis = axis + x.dim() if axis < 0 else axis
    shape = list(x.shape)
    shape[axis] = indexes.numel()
    y = torch.empty(shape, dtype=torch.float32, device=x.device) if out is None else _chk(out, "out")
    capi.check(capi.lib().sb200_gather(x.data_ptr(), indexes.data_ptr(), indexes.numel(), _prod(x.shape[:axis]), x.shape[axis],
                                       _prod(x.shape[axis + 1:]), y.data_ptr(), _stream()), "sb200_gather")
    return y


def pad(x: torch.Tensor, paddings, value: float = 0.0, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Pad (shadow/operators/pad_op.cpp:9-40): paddings = [top, bottom, left, right] on axes 2 and 3."""
    _chk(x, "x")
    if x.dim() != 4 or len(paddings) != 4:
        raise ValueError("x must be 4-d and paddings hold four values")
    shape = [x.shape[0], x.shape[1], x.shape[2] + paddings[0] + paddings[1], x.shape[3] + paddings[2] + paddings[3]]
    y = torch.empty(shape, dtype=torch.float32, device=x.device) if out is None else _chk(out, "out")
    pads = (ctypes.c_int * 4)(*paddings)
    capi.check(capi.lib().sb200_pad(x.data_ptr(), y.data_ptr(), x.shape[0] * x.shape[1], x.shape[2], x.shape[3], pads, value,
                                    _stream()), "sb200_pad")
    return y


def pooling_out_size(dim: int, kernel: int, stride: int, pad: int, full_pooling: bool) -> int:
    """shadow/operators/pooling_op.cpp:7-16: ceil (full_pooling) or floor of (dim + 2*pad - kernel)/stride, plus 1,
    evaluated in float as the reference does."""
    import numpy as np
    q = np.float32(np.float32(dim) + np.float32(2.0) * np.float32(pad) - np.float32(kernel)) / np.float32(stride)
    return int(np.ceil(q) if full_pooling else np.floor(q)) + 1


def pooling(x: torch.Tensor, pool: int = 0, kernel_size=(), stride=(1,), pad=(0,), global_pooling: bool = False,
            full_pooling: bool = True, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Pooling (shadow/operators/pooling_op.cpp:27-100): pool 0 = max, 1 = average, over the 2 or 3
    axes after (batch, channel); one-element kernel_size / stride / pad apply to every axis."""
    _chk(x, "x")
    ns = x.dim() - 2
    if ns not in (2, 3):
        raise ValueError("Only support 2D or 3D Pooling")
    if global_pooling:
        kernel_size, stride, pad = list(x.shape[2:]), [1], [0]
    expand = lambda v: [int(v[0])] * ns if len(v) == 1 else [int(t) for t in v]   # noqa: E731
    k, s, p = expand(list(kernel_size)), expand(list(stride)), expand(list(pad))
    if not (len(k) == len(s) == len(p) == ns):
        raise ValueError("kernel_size / stride / pad need one value or one per spatial axis")
    out_sp = [pooling_out_size(x.shape[2 + n], k[n], s[n], p[n], full_pooling) for n in range(ns)]
    y = torch.empty(list(x.shape[:2]) + out_sp, dtype=torch.float32, device=x.device) if out is None else _chk(out, "out")
    lead = 3 - ns
    arr = lambda v, fill: (ctypes.c_int * 3)(*([fill] * lead + list(v)))   # noqa: E731
    capi.check(capi.lib().sb200_pooling(x.data_ptr(), y.data_ptr(), x.shape[0] * x.shape[1], arr(x.shape[2:], 1), arr(out_sp, 1),
                                        arr(k, 1), arr(s, 1), arr(p, 0), pool, _stream()), "sb200_pooling")
    return y
