"""ctypes binding of the Network C adapter declared in ``include/shadow_net_capi.h``.

``NetLibrary(path, prefix)`` wraps one shared library exporting ``<prefix>net_create`` ... ;
``Net`` builds a ``shadow::NetParam`` op by op, loads it into a ``Shadow::Network``
(shadow/core/network.hpp:15-43) and runs ``Forward``.  The product library exports the prefix
``sb200net_``; a library built from the reference's own sources with the same adapter exports
``sref_`` and is driven by exactly the same Python code (the parity tests do that).
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Iterable, Mapping, Sequence

import numpy as np

ARG_S_I, ARG_S_F, ARG_V_I, ARG_V_F, ARG_S_S, ARG_V_S = range(6)


class ShadowError(RuntimeError):
    """A CHECK / LOG(FATAL) failure inside the C++ library (shadow/util/log.hpp:111-117)."""


def _cstr_array(items: Sequence[str]):
    arr = (C.c_char_p * max(len(items), 1))()
    for i, s in enumerate(items):
        arr[i] = s.encode()
    return arr


class NetLibrary:
    def __init__(self, path: str, prefix: str = "sb200net_"):
        if not os.path.exists(path):
            raise FileNotFoundError(path)
        self.path, self.prefix = path, prefix
        self.lib = C.CDLL(path, mode=C.RTLD_LOCAL)
        f = self._fn
        f("net_create", C.c_void_p, [C.c_char_p])
        f("net_destroy", None, [C.c_void_p])
        f("net_add_op", C.c_int, [C.c_void_p, C.c_char_p, C.c_char_p, C.c_int,
                                  C.POINTER(C.c_char_p), C.c_int, C.POINTER(C.c_char_p), C.c_int,
                                  C.POINTER(C.c_char_p), C.POINTER(C.c_int), C.POINTER(C.c_int),
                                  C.POINTER(C.c_double), C.POINTER(C.c_char_p)])
        f("net_add_blob", C.c_int, [C.c_void_p, C.c_char_p, C.c_int, C.POINTER(C.c_int), C.c_void_p])
        f("net_parse_text", C.c_int, [C.c_void_p, C.c_char_p])
        if prefix == "sb200net_":     # extensions of this repository's build of the adapter
            f("net_parse_binary", C.c_int, [C.c_void_p, C.c_char_p, C.c_int, C.c_int])
            f("net_dump", C.c_int, [C.c_void_p, C.c_char_p, C.c_int])
        f("net_load", C.c_int, [C.c_void_p, C.c_char_p, C.c_int, C.c_int, C.POINTER(C.c_char_p)])
        f("net_forward", C.c_int, [C.c_void_p, C.c_int, C.POINTER(C.c_char_p), C.POINTER(C.c_void_p)])
        f("net_blob_shape", C.c_int, [C.c_void_p, C.c_char_p, C.POINTER(C.c_int), C.c_int])
        f("net_blob_data", C.c_void_p, [C.c_void_p, C.c_char_p, C.c_int])
        f("last_error", C.c_char_p, [])

    def _fn(self, name, restype, argtypes):
        fn = getattr(self.lib, self.prefix + name)
        fn.restype, fn.argtypes = restype, argtypes
        setattr(self, name, fn)

    def error(self) -> str:
        return (self.last_error() or b"").decode(errors="replace")

    def check(self, rc: int, what: str) -> None:
        if rc != 0:
            raise ShadowError("%s: %s" % (what, self.error()))


def encode_args(args: Mapping[str, object]):
    """Map a Python dict onto shadow::Argument fields: int/bool -> s_i, float -> s_f,
    str -> s_s, list of int -> v_i, list of float -> v_f, list of str -> v_s.  An empty list
    is sent as an empty v_i.  Use ``np.float32`` / ``float`` explicitly for s_f."""
    names, kinds, counts, values, strings = [], [], [], [], []
    for key, val in args.items():
        names.append(key)
        if isinstance(val, (bool, np.bool_)):
            kinds.append(ARG_S_I), counts.append(1), values.append(float(int(val)))
        elif isinstance(val, (int, np.integer)):
            kinds.append(ARG_S_I), counts.append(1), values.append(float(val))
        elif isinstance(val, (float, np.floating)):
            kinds.append(ARG_S_F), counts.append(1), values.append(float(val))
        elif isinstance(val, str):
            kinds.append(ARG_S_S), counts.append(1), strings.append(val)
        else:
            seq = list(val)
            counts.append(len(seq))
            if seq and all(isinstance(v, str) for v in seq):
                kinds.append(ARG_V_S), strings.extend(seq)
            elif seq and any(isinstance(v, (float, np.floating)) for v in seq):
                kinds.append(ARG_V_F), values.extend(float(v) for v in seq)
            else:
                kinds.append(ARG_V_I), values.extend(float(int(v)) for v in seq)
    return names, kinds, counts, values, strings


def _text_value(val) -> str:
    """`type, [values]` of one argument in the model text format."""
    if isinstance(val, (bool, np.bool_, int, np.integer)):
        return "s_i, [%d]" % int(val)
    if isinstance(val, (float, np.floating)):
        return "s_f, [%s]" % repr(float(np.float32(val)))
    if isinstance(val, str):
        return "s_s, [%s]" % val
    seq = list(val)
    if seq and all(isinstance(v, str) for v in seq):
        return "v_s, [%s]" % " # ".join(seq)
    if seq and any(isinstance(v, (float, np.floating)) for v in seq):
        return "v_f, [%s]" % " # ".join(repr(float(np.float32(v))) for v in seq)
    return "v_i, [%s]" % " # ".join(str(int(v)) for v in seq)


def model_text(net_name: str, ops, net_args: Mapping[str, object] | None = None, blobs=()) -> str:
    """Serialise a graph in the reference's protobuf-free model text format
    (shadow/core/parser.cpp:1844-1917; written on the reference side by
    python/converter/shadow/transformer.py).  `ops` holds (type, name, bottoms, tops, args) tuples,
    `blobs` (name, type, shape) tuples.  Floats are written with enough digits to round-trip float32."""
    def arg_list(args):
        return "; ".join("{%s, %s}" % (k, _text_value(v)) for k, v in args.items())
    lines = ["[%s]" % net_name, "[%s]" % arg_list(net_args or {}),
             "[%s]" % "; ".join("{%s, %s, [%s]}" % (n, t, " # ".join(str(int(d)) for d in shp)) for n, t, shp in blobs)]
    for op_type, name, bottoms, tops, args in ops:
        lines.append("[%s] | [%s] | [%d %d %d] | [%s] | [%s] | [%s]" % (
            op_type, name, len(bottoms), len(tops), len(args), "; ".join(bottoms), "; ".join(tops), arg_list(args)))
    return "\n".join(lines)


class Net:
    """One NetParam + Network.  Typical use::

        net = Net(lib).input({"a": [2, 3]}).op("Unary", ["a"], ["y"], operation=4)
        net.load("Native", out_blobs=["y"])
        net.forward({"a": a_host})
        y = net.blob("y")
    """

    def __init__(self, library: NetLibrary, name: str = "net"):
        self.L = library
        self.h = library.net_create(name.encode())
        self._n_ops = 0
        self._keep = []

    def __del__(self):
        try:
            if getattr(self, "h", None):
                self.L.net_destroy(self.h)
                self.h = None
        except Exception:
            pass

    def op(self, op_type: str, bottoms: Iterable[str], tops: Iterable[str], /, op_name: str | None = None,
           **args) -> "Net":
        bottoms, tops = list(bottoms), list(tops)
        names, kinds, counts, values, strings = encode_args(args)
        n = len(names)
        rc = self.L.net_add_op(
            self.h, op_type.encode(), (op_name or "%s_%d" % (op_type.lower(), self._n_ops)).encode(),
            len(bottoms), _cstr_array(bottoms), len(tops), _cstr_array(tops), n, _cstr_array(names),
            (C.c_int * max(n, 1))(*kinds), (C.c_int * max(n, 1))(*counts),
            (C.c_double * max(len(values), 1))(*values), _cstr_array(strings))
        self.L.check(rc, "net_add_op(%s)" % op_type)
        self._n_ops += 1
        return self

    def input(self, shapes: Mapping[str, Sequence[int]]) -> "Net":
        """The ``Input`` operator: one top per input blob, its shape in a v_i argument named
        after the blob (shadow/backends/native/native.cpp:174-180)."""
        return self.op("Input", [], list(shapes), op_name="input",
                       **{k: [int(d) for d in v] for k, v in shapes.items()})

    def weight(self, name: str, array: np.ndarray) -> "Net":
        arr = np.ascontiguousarray(array, dtype=np.float32)
        shape = (C.c_int * max(arr.ndim, 1))(*arr.shape)
        rc = self.L.net_add_blob(self.h, name.encode(), arr.ndim, shape, arr.ctypes.data_as(C.c_void_p))
        self.L.check(rc, "net_add_blob(%s)" % name)
        return self

    def parse_text(self, text: str) -> "Net":
        """Replace the net under construction by the one parsed from the model text format
        (IO::ReadProtoFromText, shadow/util/io.hpp:47-52)."""
        self.L.check(self.L.net_parse_text(self.h, text.encode()), "net_parse_text")
        return self

    def parse_binary(self, data: bytes, network: int = -1) -> "Net":
        """Replace the net under construction by the one decoded from a protobuf binary model
        (IO::ReadProtoFromArray); `network` >= 0 picks that network of a MetaNetParam."""
        self.L.check(self.L.net_parse_binary(self.h, data, len(data), network), "net_parse_binary")
        return self

    def dump(self) -> str:
        """Line-based description of the net under construction (floats as C99 hex literals)."""
        need = self.L.net_dump(self.h, None, 0)
        buf = C.create_string_buffer(need)
        self.L.net_dump(self.h, buf, need)
        return buf.value.decode()

    def load(self, backend_type: str = "Native", device_id: int = 0, out_blobs: Sequence[str] = ()) -> "Net":
        outs = list(out_blobs)
        rc = self.L.net_load(self.h, backend_type.encode(), device_id, len(outs), _cstr_array(outs))
        self.L.check(rc, "net_load")
        return self

    def forward(self, inputs: Mapping[str, np.ndarray] | None = None) -> "Net":
        """``inputs`` values are C-contiguous numpy arrays or raw integer host addresses."""
        inputs = inputs or {}
        names = list(inputs)
        ptrs = (C.c_void_p * max(len(names), 1))()
        for i, k in enumerate(names):
            v = inputs[k]
            if isinstance(v, np.ndarray):
                if not v.flags["C_CONTIGUOUS"]:
                    raise ValueError("input %s must be C-contiguous" % k)
                self._keep.append(v)
                ptrs[i] = v.ctypes.data
            else:
                ptrs[i] = int(v)
        rc = self.L.net_forward(self.h, len(names), _cstr_array(names), ptrs)
        self._keep.clear()
        self.L.check(rc, "net_forward")
        return self

    def shape(self, name: str) -> list[int]:
        buf = (C.c_int * 16)()
        nd = self.L.net_blob_shape(self.h, name.encode(), buf, 16)
        if nd < 0:
            raise ShadowError("net_blob_shape(%s): %s" % (name, self.L.error()))
        return [buf[i] for i in range(nd)]

    def device_ptr(self, name: str) -> int:
        p = self.L.net_blob_data(self.h, name.encode(), 0)
        if not p:
            raise ShadowError("net_blob_data(%s): %s" % (name, self.L.error()))
        return int(p)

    def blob(self, name: str) -> np.ndarray:
        """Host copy of a blob (Network::GetBlobDataByName<float>(name, "host"))."""
        shape = self.shape(name)
        p = self.L.net_blob_data(self.h, name.encode(), 1)
        if not p:
            raise ShadowError("net_blob_data(%s): %s" % (name, self.L.error()))
        count = int(np.prod(shape, dtype=np.int64)) if shape else 1
        arr = np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_float)), shape=(count,)).copy()
        return arr.reshape(shape)
