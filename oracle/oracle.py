"""numpy front-end of the CPU oracle.  TEST INFRASTRUCTURE ONLY (see oracle_port.c): imported by
tests/, the smoke check and the benchmark's CPU-baseline leg; never by the product package.

``port`` functions run the C restatement (``liboracle_port.so``) and apply the operator
front-ends' shape rules in Python; ``ref_library()`` gives the compiled reference itself
(``oracle/_ref/libshadow_ref.so``) through the same Network adapter the product uses, or None.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Sequence

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
PORT_LIB = os.path.join(HERE, "liboracle_port.so")
REF_LIB = os.path.join(HERE, "_ref", "libshadow_ref.so")

# operation codes (shadow/operators/kernels/{binary,unary,activate,reduce}.hpp)
BINARY = {"Add": 0, "Sub": 1, "Mul": 2, "Div": 3, "Pow": 4, "Max": 5, "Min": 6}
UNARY = {"Abs": 0, "Square": 1, "Sqrt": 2, "Log": 3, "Exp": 4, "Sin": 5, "Cos": 6, "Tan": 7,
         "Asin": 8, "Acos": 9, "Atan": 10, "Floor": 11, "Ceil": 12, "Neg": 13, "Reciprocal": 14}
ACTIVATE = {"PRelu": 0, "Relu": 1, "Leaky": 2, "Sigmoid": 3, "SoftPlus": 4, "Tanh": 5,
            "Relu6": 6, "HardSwish": 7, "Gelu": 8}
REDUCE = {"Prod": 0, "Sum": 1, "Max": 2, "Min": 3, "Avg": 4, "LpNorm1": 5, "LpNorm2": 6}

_lib = None
_FP = C.POINTER(C.c_float)
_IP = C.POINTER(C.c_int)


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _fp(a: np.ndarray):
    return a.ctypes.data_as(_FP)


def _ip(seq: Sequence[int]):
    return (C.c_int * max(len(seq), 1))(*[int(v) for v in seq])


def port():
    """Load (building on demand) the C restatement."""
    global _lib
    if _lib is None:
        if not os.path.exists(PORT_LIB) or os.path.getmtime(PORT_LIB) < os.path.getmtime(
                os.path.join(HERE, "oracle_port.c")):
            import importlib.util
            spec = importlib.util.spec_from_file_location("_oracle_build", os.path.join(HERE, "build.py"))
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
            mod.build_port(force=True)
        L = C.CDLL(PORT_LIB)
        i64 = C.c_int64
        L.orc_binary.argtypes = [i64, _FP, _FP, _FP, C.c_int]
        L.orc_binary_scalar.argtypes = [i64, _FP, C.c_float, _FP, C.c_int]
        L.orc_broadcast_binary.argtypes = [_FP, _IP, _FP, _IP, C.c_int, C.c_int, i64, _IP, _FP]
        L.orc_unary.argtypes = [i64, _FP, _FP, C.c_int]
        L.orc_activate.argtypes = [_FP, _FP, i64, C.c_int, C.c_float]
        L.orc_prelu.argtypes = [_FP, _FP, _IP, C.c_int, C.c_int, _FP]
        L.orc_scale_bias.argtypes = [_FP, i64, _FP, _FP, i64, i64, _FP]
        L.orc_reduce.argtypes = [_FP, _IP, C.c_int, _IP, C.c_int, C.c_int, _FP]
        L.orc_softmax.argtypes = [_FP, i64, i64, i64, _FP, _FP]
        L.orc_fill.argtypes = [i64, C.c_float, _FP]
        L.orc_eltwise.argtypes = [C.POINTER(_FP), C.c_int, _FP, i64, C.c_int, _FP]
        L.orc_axpy.argtypes = [_FP, _FP, _FP, i64, i64, _FP]
        IP = C.POINTER(C.c_int)
        L.orc_pooling.argtypes = [_FP, i64, IP, IP, IP, IP, IP, C.c_int, _FP]
        L.orc_copy_part.argtypes = [_FP, _FP, i64, i64, i64, i64, C.c_int]
        L.orc_permute.argtypes = [_FP, IP, IP, C.c_int, _FP]
        L.orc_gather.argtypes = [_FP, IP, i64, i64, i64, i64, _FP]
        L.orc_pad.argtypes = [_FP, i64, i64, i64, i64, IP, C.c_float, _FP]
        L.orc_ssd_normalize.argtypes = [_FP, i64, i64, i64, C.c_int, C.c_float, _FP, C.c_int, _FP, _FP]
        L.orc_row_norm.argtypes = [_FP, i64, i64, C.c_float, _FP, _FP, i64, i64, _FP]
        L.orc_normalize.argtypes = [_FP, i64, i64, i64, _FP, C.c_float, C.c_float, _FP]
        L.orc_batch_norm.argtypes = [_FP, i64, _FP, _FP, i64, i64, C.c_float, C.c_float, _FP]
        _lib = L
    return _lib


def ref_library():
    """NetLibrary over the compiled reference, or None if it was never built."""
    if not os.path.exists(REF_LIB):
        return None
    from shadow_b200.netapi import NetLibrary  # the adapter binding is shared with the product
    return NetLibrary(REF_LIB, "sref_")


def _ok(rc: int, what: str):
    if rc != 0:
        raise ValueError("oracle %s: bad argument" % what)


# ---- operator-level functions (front-end shape rules + C loops) -------------------------------

def binary_scalar(a, scalar: float, operation: int) -> np.ndarray:
    """BinaryOp scalar form (shadow/operators/binary_op.cpp:31-33)."""
    a = _f32(a)
    y = np.empty_like(a)
    _ok(port().orc_binary_scalar(a.size, _fp(a), np.float32(scalar), _fp(y), operation), "binary_scalar")
    return y


def broadcast_shapes(sa: Sequence[int], sb: Sequence[int]):
    """Left-pad the lower rank with 1s; each dim equal or 1; out = max
    (shadow/operators/binary_op.cpp:36-57)."""
    sa, sb = list(sa), list(sb)
    nd = max(len(sa), len(sb))
    pa, pb = [1] * (nd - len(sa)) + sa, [1] * (nd - len(sb)) + sb
    out = []
    for da, db in zip(pa, pb):
        if not (da == db or da == 1 or db == 1):
            raise ValueError("shapes %s and %s do not broadcast" % (sa, sb))
        out.append(max(da, db))
    return pa, pb, out


def binary(a, b, operation: int) -> np.ndarray:
    """BinaryOp tensor form (shadow/operators/binary_op.cpp:34-63)."""
    a, b = _f32(a), _f32(b)
    if a.shape == b.shape:
        y = np.empty_like(a)
        _ok(port().orc_binary(a.size, _fp(a), _fp(b), _fp(y), operation), "binary")
        return y
    pa, pb, out = broadcast_shapes(a.shape, b.shape)
    y = np.empty(out, dtype=np.float32)
    _ok(port().orc_broadcast_binary(_fp(a), _ip(pa), _fp(b), _ip(pb), operation, len(out), y.size,
                                    _ip(out), _fp(y)), "broadcast_binary")
    return y


def unary(x, operation: int) -> np.ndarray:
    x = _f32(x)
    y = np.empty_like(x)
    _ok(port().orc_unary(x.size, _fp(x), _fp(y), operation), "unary")
    return y


def activate(x, type: int = 1, slope: float = 0.1, slope_blob=None) -> np.ndarray:
    """ActivateOp (shadow/operators/activate_op.cpp:9-34; kernels/activate.hpp:45-73)."""
    x = _f32(x)
    y = np.empty_like(x)
    if type == 0:
        s = _f32(slope_blob)
        if x.ndim < 2:
            raise ValueError("PRelu needs >= 2 axes")
        shared = s.size == 1
        if not shared and s.size != x.shape[1]:
            raise ValueError("PRelu slope count must be 1 or channels")
        _ok(port().orc_prelu(_fp(x), _fp(y), _ip(x.shape), x.ndim, int(shared), _fp(s)), "prelu")
    else:
        _ok(port().orc_activate(_fp(x), _fp(y), x.size, type, np.float32(slope)), "activate")
    return y


def scale(x, axis: int = 1, scale=None, bias=None) -> np.ndarray:
    """ScaleOp blob / value forms (shadow/operators/kernels/scale.hpp:44-110):
    inner = count(axis + scale.ndim), scale_num = scale.size."""
    x = _f32(x)
    s = None if scale is None else _f32(scale)
    b = None if bias is None else _f32(bias)
    ref = s if s is not None else b
    if ref is None:
        raise ValueError("scale or bias required")
    if s is not None and b is not None and s.shape != b.shape:
        raise ValueError("scale and bias shapes differ")
    start = axis + ref.ndim
    inner = int(np.prod(x.shape[start:], dtype=np.int64)) if start <= x.ndim else 1
    y = np.empty_like(x)
    _ok(port().orc_scale_bias(_fp(x), x.size, _fp(s) if s is not None else None,
                              _fp(b) if b is not None else None, ref.size, inner, _fp(y)), "scale")
    return y


def reduce(x, operation: int = 0, axes: Sequence[int] = (), keep_dims: bool = True) -> np.ndarray:
    """ReduceOp (shadow/operators/reduce_op.cpp:22-65)."""
    x = _f32(x)
    axes = list(axes) if len(axes) else list(range(x.ndim))
    out_shape = list(x.shape)
    for ax in axes:
        out_shape[ax] = 1
    y = np.empty(out_shape, dtype=np.float32)
    _ok(port().orc_reduce(_fp(x), _ip(x.shape), x.ndim, _ip(axes), len(axes), operation, _fp(y)), "reduce")
    if not keep_dims:
        y = y.reshape([d for n, d in enumerate(out_shape) if n not in axes])
    return y


def softmax(x, axis: int = 1) -> np.ndarray:
    """SoftmaxOp (shadow/operators/softmax_op.cpp:18-28; kernels/softmax.hpp:29-41)."""
    x = _f32(x)
    if not -x.ndim <= axis < x.ndim:
        raise ValueError("axis out of range")
    axis = axis % x.ndim
    outer = int(np.prod(x.shape[:axis], dtype=np.int64))
    dim = x.shape[axis]
    inner = int(np.prod(x.shape[axis + 1:], dtype=np.int64))
    val = np.empty(outer * inner, dtype=np.float32)
    y = np.empty_like(x)
    _ok(port().orc_softmax(_fp(x), outer, dim, inner, _fp(val), _fp(y)), "softmax")
    return y


def eltwise(inputs, operation: int, coeff=None) -> np.ndarray:
    """EltwiseOp (shadow/operators/eltwise_op.cpp:7-56): >= 2 same-shape inputs; Prod 0, Sum 1 (optional
    one coefficient per input), Max 2, Min 3."""
    xs = [_f32(x) for x in inputs]
    if len(xs) < 2 or any(x.shape != xs[0].shape for x in xs):
        raise ValueError("eltwise needs >= 2 inputs of one shape")
    if coeff is not None and len(coeff) and (operation != 1 or len(coeff) != len(xs)):
        raise ValueError("coefficients only for Sum, one per input")
    ptrs = (_FP * len(xs))(*[_fp(x) for x in xs])
    cf = _f32(coeff) if coeff is not None and len(coeff) else None
    y = np.empty_like(xs[0])
    _ok(port().orc_eltwise(ptrs, len(xs), _fp(cf) if cf is not None else None, xs[0].size, operation, _fp(y)), "eltwise")
    return y


def axpy(alpha, x, y) -> np.ndarray:
    """AxpyOp (shadow/operators/axpy_op.cpp:16-51): alpha [N,C] or [N,C,1,1], x and y [N,C,...]."""
    alpha, x, y = _f32(alpha), _f32(x), _f32(y)
    if x.shape != y.shape or alpha.shape[0] != x.shape[0] or alpha.shape[1] != x.shape[1]:
        raise ValueError("axpy shapes")
    inner = int(np.prod(x.shape[2:], dtype=np.int64))
    out = np.empty_like(x)
    _ok(port().orc_axpy(_fp(alpha), _fp(x), _fp(y), alpha.size, inner, _fp(out)), "axpy")
    return out


def _ints(v):
    a = np.ascontiguousarray(np.asarray(v, dtype=np.int32))
    return a, a.ctypes.data_as(C.POINTER(C.c_int))


def concat(inputs, axis: int = 1) -> np.ndarray:
    """ConcatOp + ConcatKernelDefault (shadow/operators/concat_op.cpp:9-45, kernels/concat.hpp:30-47)."""
    xs = [_f32(t) for t in inputs]
    axis = axis + xs[0].ndim if axis < 0 else axis
    shape = list(xs[0].shape)
    shape[axis] = sum(t.shape[axis] for t in xs)
    y = np.empty(shape, np.float32)
    num = int(np.prod(shape[:axis], dtype=np.int64))
    inner = int(np.prod(shape[axis + 1:], dtype=np.int64))
    off = 0
    for t in xs:
        _ok(port().orc_copy_part(_fp(t), _fp(y), num, t.shape[axis] * inner, shape[axis] * inner, off * inner, 1), "concat")
        off += t.shape[axis]
    return y


def stack(inputs, axis: int = 0) -> np.ndarray:
    """StackOp + StackKernelDefault (shadow/operators/stack_op.cpp:9-40, kernels/stack.hpp:29-42)."""
    xs = [_f32(t) for t in inputs]
    axis = axis + xs[0].ndim + 1 if axis < 0 else axis
    shape = list(xs[0].shape)
    shape.insert(axis, len(xs))
    y = np.empty(shape, np.float32)
    num = int(np.prod(shape[:axis], dtype=np.int64))
    size = int(np.prod(shape[axis + 1:], dtype=np.int64))
    for n, t in enumerate(xs):
        _ok(port().orc_copy_part(_fp(t), _fp(y), num, size, len(xs) * size, n * size, 1), "stack")
    return y


def slice_(x, axis: int, sizes) -> list:
    """SliceOp + SliceKernelDefault (shadow/operators/slice_op.cpp:9-60, kernels/slice.hpp:30-48)."""
    x = _f32(x)
    axis = axis + x.ndim if axis < 0 else axis
    num = int(np.prod(x.shape[:axis], dtype=np.int64))
    inner = int(np.prod(x.shape[axis + 1:], dtype=np.int64))
    outs, off = [], 0
    for sz in sizes:
        shape = list(x.shape)
        shape[axis] = sz
        y = np.empty(shape, np.float32)
        _ok(port().orc_copy_part(_fp(y), _fp(x), num, sz * inner, x.shape[axis] * inner, off * inner, 0), "slice")
        outs.append(y)
        off += sz
    return outs


def permute(x, order) -> np.ndarray:
    """PermuteOp (shadow/operators/permute_op.cpp:9-35)."""
    x = _f32(x)
    y = np.empty([x.shape[a] for a in order], np.float32)
    sh, shp = _ints(x.shape)
    od, odp = _ints(order)
    _ok(port().orc_permute(_fp(x), shp, odp, x.ndim, _fp(y)), "permute")
    return y


def gather(x, indexes, axis: int = 0) -> np.ndarray:
    """GatherOp (shadow/operators/gather_op.cpp:9-50)."""
    x = _f32(x)
    axis = axis + x.ndim if axis < 0 else axis
    idx, idxp = _ints(indexes)
    shape = list(x.shape)
    shape[axis] = idx.size
    y = np.empty(shape, np.float32)
    _ok(port().orc_gather(_fp(x), idxp, idx.size, x.shape[axis], int(np.prod(x.shape[axis + 1:], dtype=np.int64)), y.size,
                          _fp(y)), "gather")
    return y


def pad(x, paddings, value: float = 0.0) -> np.ndarray:
    """PadOp (shadow/operators/pad_op.cpp:9-40)."""
    x = _f32(x)
    pd, pdp = _ints(paddings)
    y = np.empty([x.shape[0], x.shape[1], x.shape[2] + pd[0] + pd[1], x.shape[3] + pd[2] + pd[3]], np.float32)
    _ok(port().orc_pad(_fp(x), x.shape[0], x.shape[1], x.shape[2], x.shape[3], pdp, np.float32(value), _fp(y)), "pad")
    return y


def pooling(x, pool: int = 0, kernel_size=(), stride=(1,), pad=(0,), global_pooling: bool = False,
            full_pooling: bool = True) -> np.ndarray:
    """PoolingOp (shadow/operators/pooling_op.cpp:7-100): output size ceil/floor((dim + 2*pad - kernel)/stride) + 1
    in float arithmetic."""
    x = _f32(x)
    ns = x.ndim - 2
    if global_pooling:
        kernel_size, stride, pad = list(x.shape[2:]), [1], [0]
    expand = lambda v: [int(v[0])] * ns if len(v) == 1 else [int(t) for t in v]   # noqa: E731
    k, s, p = expand(list(kernel_size)), expand(list(stride)), expand(list(pad))
    out_sp = []
    for n in range(ns):
        q = np.float32(np.float32(x.shape[2 + n]) + np.float32(2.0) * np.float32(p[n]) - np.float32(k[n])) / np.float32(s[n])
        out_sp.append(int(np.ceil(q) if full_pooling else np.floor(q)) + 1)
    lead = 3 - ns
    y = np.empty(list(x.shape[:2]) + out_sp, np.float32)
    a_in, p_in = _ints([1] * lead + list(x.shape[2:]))
    a_out, p_out = _ints([1] * lead + out_sp)
    a_k, p_k = _ints([1] * lead + k)
    a_s, p_s = _ints([1] * lead + s)
    a_p, p_p = _ints([0] * lead + p)
    _ok(port().orc_pooling(_fp(x), x.shape[0] * x.shape[1], p_in, p_out, p_k, p_s, p_p, pool, _fp(y)), "pooling")
    return y


def ssd_normalize(x, scale=None, across_spatial: bool = True, channel_shared: bool = True, eps: float = 1e-5) -> np.ndarray:
    """SSDNormalizeOp (shadow/operators/ssd_normalize_op.cpp:9-45)."""
    x = _f32(x)
    spatial = int(np.prod(x.shape[2:], dtype=np.int64))
    val = np.empty(max(x.shape[0] * spatial, 1), np.float32)
    y = np.empty_like(x)
    sc = _f32(scale) if scale is not None else None
    _ok(port().orc_ssd_normalize(_fp(x), x.shape[0], x.shape[1], spatial, int(across_spatial), np.float32(eps),
                                 _fp(sc) if sc is not None else None, int(channel_shared), _fp(val), _fp(y)), "ssd_normalize")
    return y


def _row_norm(x, rows, inner, eps, scale, bias, scale_num, scale_inner):
    y = np.empty_like(x)
    sc = _f32(scale) if scale is not None else None     # kept alive across the call
    bs = _f32(bias) if bias is not None else None
    sp = _fp(sc) if sc is not None else None
    bp = _fp(bs) if bs is not None else None
    _ok(port().orc_row_norm(_fp(x), rows, inner, np.float32(eps), sp, bp, scale_num, scale_inner, _fp(y)), "row_norm")
    return y


def layer_norm(x, normalized_shape, scale=None, bias=None, eps: float = 1e-5) -> np.ndarray:
    """LayerNormOp (shadow/operators/layer_norm_op.cpp:9-50)."""
    x = _f32(x)
    inner = int(np.prod(normalized_shape, dtype=np.int64))
    return _row_norm(x, x.size // inner, inner, eps, scale, bias, inner, 1)


def group_norm(x, group: int, scale=None, bias=None, eps: float = 1e-5) -> np.ndarray:
    """GroupNormOp (shadow/operators/group_norm_op.cpp:9-45); InstanceNormOp is group == channels."""
    x = _f32(x)
    rows = x.shape[0] * group
    spatial = int(np.prod(x.shape[2:], dtype=np.int64))
    return _row_norm(x, rows, x.size // rows, eps, scale, bias, x.shape[1], spatial)


def normalize(x, axis: int = 1, p: float = 2.0, eps: float = 1e-12) -> np.ndarray:
    """NormalizeOp (shadow/operators/normalize_op.cpp:9-37)."""
    x = _f32(x)
    axis = axis + x.ndim if axis < 0 else axis
    outer = int(np.prod(x.shape[:axis], dtype=np.int64))
    inner = int(np.prod(x.shape[axis + 1:], dtype=np.int64))
    val = np.empty(max(outer * inner, 1), np.float32)
    y = np.empty_like(x)
    _ok(port().orc_normalize(_fp(x), outer, x.shape[axis], inner, _fp(val), np.float32(p), np.float32(eps), _fp(y)),
        "normalize")
    return y


def batch_norm(x, mean, variance, scale=None, eps: float = 1e-5) -> np.ndarray:
    """BatchNormOp, inference (shadow/operators/batch_norm_op.cpp:9-43): optional 4th input `scale`
    (one element) gives scale_factor = scale == 0 ? 0 : 1/scale."""
    x, mean, variance = _f32(x), _f32(mean), _f32(variance)
    if mean.size != x.shape[1] or variance.size != x.shape[1]:
        raise ValueError("mean/variance must have one value per channel")
    sf = np.float32(1)
    if scale is not None:
        sc = np.float32(_f32(scale).ravel()[0])
        sf = np.float32(0) if sc == 0 else np.float32(1) / sc
    inner = int(np.prod(x.shape[2:], dtype=np.int64))
    y = np.empty_like(x)
    _ok(port().orc_batch_norm(_fp(x), x.size, _fp(mean), _fp(variance), x.shape[1], inner, sf, np.float32(eps), _fp(y)),
        "batch_norm")
    return y


def fill(n: int, val: float) -> np.ndarray:
    y = np.empty(n, dtype=np.float32)
    port().orc_fill(n, np.float32(val), _fp(y))
    return y


# ---- comparison helpers ----------------------------------------------------------------------

def ulp_distance(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """Distance in float32 units-in-the-last-place, on the monotone integer line (so +0 and -0
    are 0 apart, and adjacent floats are 1 apart).  NaN vs NaN is 0; NaN vs number is 2**31."""
    a = np.ascontiguousarray(a, dtype=np.float32).ravel()
    b = np.ascontiguousarray(b, dtype=np.float32).ravel()
    ia = a.view(np.int32).astype(np.int64)
    ib = b.view(np.int32).astype(np.int64)
    ia = np.where(ia < 0, -(ia & 0x7FFFFFFF), ia)
    ib = np.where(ib < 0, -(ib & 0x7FFFFFFF), ib)
    d = np.abs(ia - ib)
    na, nb = np.isnan(a), np.isnan(b)
    d = np.where(na & nb, 0, d)
    d = np.where(na ^ nb, 2 ** 31, d)
    return d


def bit_equal(a: np.ndarray, b: np.ndarray) -> bool:
    a = np.ascontiguousarray(a, dtype=np.float32)
    b = np.ascontiguousarray(b, dtype=np.float32)
    return a.shape == b.shape and bool(np.array_equal(a.view(np.uint32), b.view(np.uint32)))
