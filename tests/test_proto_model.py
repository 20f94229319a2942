"""Protobuf binary models: the reader in the host library (no protobuf runtime linked) against bytes
produced by the official Python protobuf runtime for the reference's schema
(shadow/proto/shadow.proto:5-47, rebuilt here as a descriptor - field numbers, types, labels and the
packed options are the schema's).  Also checks that the reader and the text-format reader agree on
the NetParam they produce (dump of one == dump of the other)."""
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.dirname(__file__))
import cases  # noqa: E402
from oracle import oracle as orc  # noqa: E402
from shadow_b200.netapi import Net, ShadowError, model_text  # noqa: E402

pb = pytest.importorskip("google.protobuf")
from google.protobuf import descriptor_pb2, descriptor_pool, message_factory  # noqa: E402

F = descriptor_pb2.FieldDescriptorProto


def _schema():
    fd = descriptor_pb2.FileDescriptorProto(name="shadow_test.proto", package="shadow", syntax="proto2")

    def message(name, fields):
        m = fd.message_type.add(name=name)
        for fname, number, ftype, label, extra in fields:
            f = m.field.add(name=fname, number=number, type=ftype, label=label)
            if extra.get("packed"):
                f.options.packed = True
            if "msg" in extra:
                f.type_name = ".shadow." + extra["msg"]
    O, R = F.LABEL_OPTIONAL, F.LABEL_REPEATED
    message("Blob", [("name", 1, F.TYPE_STRING, O, {}), ("type", 2, F.TYPE_STRING, O, {}), ("shape", 3, F.TYPE_INT32, R, {}),
                     ("data_f", 4, F.TYPE_FLOAT, R, {"packed": True}), ("data_i", 5, F.TYPE_INT32, R, {"packed": True}),
                     ("data_b", 6, F.TYPE_BYTES, R, {})])
    message("Argument", [("name", 1, F.TYPE_STRING, O, {}), ("s_f", 2, F.TYPE_FLOAT, O, {}), ("s_i", 3, F.TYPE_INT32, O, {}),
                         ("s_s", 4, F.TYPE_STRING, O, {}), ("v_f", 5, F.TYPE_FLOAT, R, {}), ("v_i", 6, F.TYPE_INT32, R, {}),
                         ("v_s", 7, F.TYPE_STRING, R, {})])
    message("OpParam", [("name", 1, F.TYPE_STRING, O, {}), ("type", 2, F.TYPE_STRING, O, {}), ("bottom", 3, F.TYPE_STRING, R, {}),
                        ("top", 4, F.TYPE_STRING, R, {}), ("arg", 11, F.TYPE_MESSAGE, R, {"msg": "Argument"})])
    message("NetParam", [("name", 1, F.TYPE_STRING, O, {}), ("blob", 5, F.TYPE_MESSAGE, R, {"msg": "Blob"}),
                         ("op", 11, F.TYPE_MESSAGE, R, {"msg": "OpParam"}), ("arg", 12, F.TYPE_MESSAGE, R, {"msg": "Argument"})])
    message("MetaNetParam", [("name", 1, F.TYPE_STRING, O, {}), ("network", 11, F.TYPE_MESSAGE, R, {"msg": "NetParam"}),
                             ("arg", 12, F.TYPE_MESSAGE, R, {"msg": "Argument"})])
    pool = descriptor_pool.DescriptorPool()
    pool.Add(fd)
    get = lambda n: message_factory.GetMessageClass(pool.FindMessageTypeByName("shadow." + n))   # noqa: E731
    return get("NetParam"), get("MetaNetParam")


NetParam, MetaNetParam = _schema()


def _set_arg(arg, name, val):
    arg.name = name
    if isinstance(val, (bool, np.bool_, int, np.integer)):
        arg.s_i = int(val)
    elif isinstance(val, (float, np.floating)):
        arg.s_f = float(np.float32(val))
    elif isinstance(val, str):
        arg.s_s = val
    else:
        seq = list(val)
        if seq and all(isinstance(v, str) for v in seq):
            arg.v_s.extend(seq)
        elif seq and any(isinstance(v, (float, np.floating)) for v in seq):
            arg.v_f.extend(float(np.float32(v)) for v in seq)
        else:
            arg.v_i.extend(int(v) for v in seq)


def _message(name, ops, net_args=None, blobs=()):
    net = NetParam(name=name)
    for k, v in (net_args or {}).items():
        _set_arg(net.arg.add(), k, v)
    for bname, btype, shape, data in blobs:
        b = net.blob.add(name=bname, type=btype)
        b.shape.extend(shape)
        if data is not None and btype == "float":
            b.data_f.extend(float(v) for v in np.asarray(data, np.float32).ravel())
        elif data is not None:   # every other type travels as raw bytes
            b.data_b.append(np.ascontiguousarray(data).tobytes())
    for op_type, op_name, bottoms, tops, args in ops:
        op = net.op.add(name=op_name, type=op_type)
        op.bottom.extend(bottoms)
        op.top.extend(tops)
        for k, v in args.items():
            _set_arg(op.arg.add(), k, v)
    return net


def _lib():
    import shadow_b200
    return shadow_b200.host_library()


GRAPH = [("Input", "input", [], ["x", "g"], {"x": [2, 3, 4], "g": [3]}),
         ("Scale", "s", ["x", "g"], ["y"], {"axis": 1, "has_scale": True, "has_bias": False}),
         ("Activate", "a", ["y"], ["z"], {"type": 2, "slope": 0.125}),
         ("Reduce", "r", ["z"], ["out"], {"operation": 2, "axes": [0, 2], "keep_dims": False}),
         ("Eltwise", "e", ["z", "z"], ["w"], {"operation": 1, "coeff": [0.5, -1.5]})]
WEIGHT = ("w0", "float", [2, 2], np.array([[1.5, -2.25], [3e-7, 1e9]], np.float32))


def test_reader_reproduces_every_field():
    graph = list(GRAPH)
    graph[3] = ("Reduce", "r", ["z"], ["out"], {"operation": 2, "axes": [0, -1], "keep_dims": False})   # parsed, never run
    msg = _message("net-a", graph, {"out_blob": ["out", "w"], "note": "hello world", "version": 3, "ratio": 0.1},
                   [WEIGHT, ("empty", "float", [4, 0], None)])
    dump = Net(_lib(), "x").parse_binary(msg.SerializeToString()).dump().splitlines()
    assert dump[0] == "net net-a"
    assert "netarg out_blob v_s out w" in dump and "netarg note s_s hello world" in dump and "netarg version s_i 3" in dump
    assert "netarg ratio s_f " + float(np.float32(0.1)).hex() in [" ".join(line.split()[:3] + [float.fromhex(line.split()[3]).hex()])
                                                                   for line in dump if line.startswith("netarg ratio")]
    blob = [line.split() for line in dump if line.startswith("blob w0")][0]
    assert blob[2:6] == ["float", "2", "2", "2"] and blob[6] == "4"
    assert [np.float32(float.fromhex(v)) for v in blob[7:]] == list(WEIGHT[3].ravel())
    assert "blob empty float 2 4 0 0" in dump
    ops = [line for line in dump if line.startswith("op ")]
    assert ops == ["op Input input 0 2 x g 2", "op Scale s 2 x g 1 y 3", "op Activate a 1 y 1 z 2",
                   "op Reduce r 1 z 1 out 3", "op Eltwise e 2 z z 1 w 2"]
    assert "arg axes v_i 0 -1" in dump and "arg keep_dims s_i 0" in dump           # negative int32: 10-byte varint
    slope = [line.split() for line in dump if line.startswith("arg slope")][0]
    assert float.fromhex(slope[3]) == 0.125


def test_packed_and_unpacked_repeated_scalars_are_both_accepted():
    """A parser must take either encoding whatever the schema says: hand-encoded v_i (declared
    unpacked) as a packed payload and data_f (declared packed) as single values."""
    def varint(v):
        v &= (1 << 64) - 1
        out = b""
        while True:
            b = v & 0x7f
            v >>= 7
            out += bytes([b | (0x80 if v else 0)])
            if not v:
                return out
    def ld(field, payload):
        return varint(field << 3 | 2) + varint(len(payload)) + payload
    arg = ld(1, b"axes") + ld(6, varint(5) + varint(-2) + varint(300))
    op = ld(1, b"r") + ld(2, b"Reduce") + ld(3, b"x") + ld(4, b"y") + ld(11, arg)
    blob = ld(1, b"w") + varint(3 << 3 | 0) + varint(2) + b"".join(varint(4 << 3 | 5) + np.float32(v).tobytes() for v in (1.5, -3.0))
    unknown = varint(99 << 3 | 0) + varint(7) + ld(98, b"ignored")
    net = ld(1, b"n") + unknown + ld(5, blob) + ld(11, op)
    dump = Net(_lib(), "x").parse_binary(net).dump()
    assert "arg axes v_i 5 -2 300" in dump
    blob_line = [line.split() for line in dump.splitlines() if line.startswith("blob w ")][0]
    assert blob_line[2:6] == ["float", "1", "2", "2"] and [float.fromhex(v) for v in blob_line[6:]] == [1.5, -3.0]


def test_meta_net_and_errors():
    meta = MetaNetParam(name="pack")
    meta.network.add().CopyFrom(_message("first", GRAPH[:2]))
    meta.network.add().CopyFrom(_message("second", GRAPH[:3]))
    data = meta.SerializeToString()
    assert Net(_lib(), "x").parse_binary(data, network=1).dump().startswith("net second\n")
    with pytest.raises(ShadowError, match="fewer networks"):
        Net(_lib(), "x").parse_binary(data, network=2)
    good = _message("n", GRAPH).SerializeToString()
    for cut in (1, len(good) // 2, len(good) - 1):
        with pytest.raises(ShadowError):
            Net(_lib(), "x").parse_binary(good[:cut])            # truncated payloads are refused, not read past


def test_binary_and_text_readers_agree():
    """The same graph through both readers (all arguments given, so the text format's own defaults
    add nothing): identical NetParam apart from the text format's argument order."""
    ops = [GRAPH[0], ("Reduce", "r", ["x"], ["out"], {"operation": 1, "axes": [2], "keep_dims": True}),
           ("Softmax", "s", ["out"], ["p"], {"axis": 1})]
    fill = {"net_args": {"from_text": 1}, "blobs": [("unused_blob", "float", [1])]}
    a = Net(_lib(), "x").parse_text(model_text("n", ops, **fill)).dump()
    b = Net(_lib(), "x").parse_binary(_message("n", ops, fill["net_args"], [("unused_blob", "float", [1], None)]).SerializeToString()).dump()
    assert sorted(a.splitlines()) == sorted(b.splitlines())


def test_protobuf_text_format_reader_agrees_with_the_binary_reader():
    """`.shadowtxt`: every way the official runtime prints the message (multi-line, one line, short
    repeated form, floats at full precision) parses to the NetParam the binary reader gives."""
    from google.protobuf import text_format
    graph = list(GRAPH)
    graph[3] = ("Reduce", "r", ["z"], ["out"], {"operation": 2, "axes": [0, -1], "keep_dims": False})
    msg = _message("net \"quoted\" \\ name\n2nd line", graph, {"out_blob": ["out", "w"], "note": "tab\there 'single' \x01", "ratio": 0.1},
                   [WEIGHT, ("empty", "float", [4, 0], None)])
    want = Net(_lib(), "x").parse_binary(msg.SerializeToString()).dump()
    variants = [text_format.MessageToString(msg), text_format.MessageToString(msg, as_one_line=True),
                text_format.MessageToString(msg, use_short_repeated_primitives=True),
                text_format.MessageToString(msg, pointy_brackets=True), text_format.MessageToString(msg, as_utf8=True)]
    for text in variants:
        assert Net(_lib(), "x").parse_text(text).dump() == want, text[:200]
    hand = """
      # hand-written, with the looser forms the grammar allows
      name: "n"   op: { type: 'Unary' name: "u" bottom: "a", top: "b"; arg < name: "operation" s_i: 0x4 > }
      op { name: "s" type: "Scale" bottom: ["b"] top: "c"
           arg { name: "scale_value" v_f: [1.5f, -2e-3, inf] } arg { name: "axis" s_i: -1 } }
      blob { name: "w" "0" shape: [2, 1] data_f: 1 data_f: 2.5 }
    """
    dump = Net(_lib(), "x").parse_text(hand).dump().splitlines()
    assert "op Unary u 1 a 1 b 1" in dump and "arg operation s_i 4" in dump and "arg axis s_i -1" in dump
    sv = [line.split() for line in dump if line.startswith("arg scale_value")][0]
    assert [float.fromhex(v) for v in sv[3:]] == [1.5, float(np.float32(-2e-3)), float("inf")]
    assert [line for line in dump if line.startswith("blob w0 float 2 2 1 2")]
    for bad in ('name: "n" bogus: 1', 'op { name: "x" ', 'op { name: x }', 'arg { s_i: 99999999999 }'):
        with pytest.raises(ShadowError):
            Net(_lib(), "x").parse_text(bad)


@pytest.mark.gpu
def test_binary_model_runs_like_the_programmatic_net():
    lib = _lib()
    x, g = cases.normal(11, (2, 3, 4)), cases.normal(12, (3,))
    msg = _message("n", GRAPH, blobs=[WEIGHT])
    net = Net(lib, "n").parse_binary(msg.SerializeToString())
    net.load("Native", out_blobs=["out", "w", "w0"])
    net.forward({"x": x, "g": g})
    z = orc.activate(orc.scale(x, 1, g, None), 2, np.float32(0.125))
    assert orc.bit_equal(net.blob("out"), orc.reduce(z, 2, [0, 2], False))
    assert orc.bit_equal(net.blob("w"), orc.eltwise([z, z], 1, [0.5, -1.5]))
    assert orc.bit_equal(net.blob("w0"), WEIGHT[3])


@pytest.mark.gpu
def test_int32_weight_blob_reaches_the_device():
    """A non-float weight blob (data_b, shadow/backends/native/native.cpp:158-167): the int32 index
    list of a Gather stored in the model, not passed as an argument."""
    lib = _lib()
    x = cases.normal(21, (5, 7))
    idx = np.array([3, 0, 0, 2, 4], np.int32)
    graph = [("Input", "input", [], ["x"], {"x": [5, 7]}),
             ("Gather", "g", ["x", "idx"], ["out"], {"axis": 0})]
    msg = _message("n", graph, blobs=[("idx", "int32", [5], idx)])
    net = Net(lib, "n").parse_binary(msg.SerializeToString())
    net.load("Native", out_blobs=["out"])
    net.forward({"x": x})
    assert orc.bit_equal(net.blob("out"), x[idx])
    # a byte count that does not match the blob's shape is refused at load time
    bad = _message("n", graph, blobs=[("idx", "int32", [5], idx[:3])])
    with pytest.raises(ShadowError):
        Net(lib, "n").parse_binary(bad.SerializeToString()).load("Native", out_blobs=["out"])


def _expected_dump(msg):
    """What Net.dump() must print for `msg`, computed from the message itself."""
    def arg(word, a):
        if a.HasField("s_f"):
            return [word, a.name, "s_f", float(a.s_f).hex()]
        if a.HasField("s_i"):
            return [word, a.name, "s_i", str(a.s_i)]
        if a.HasField("s_s"):
            return [word, a.name, "s_s", a.s_s]
        if len(a.v_f):
            return [word, a.name, "v_f"] + [float(v).hex() for v in a.v_f]
        if len(a.v_s):
            return [word, a.name, "v_s"] + list(a.v_s)
        return [word, a.name, "v_i"] + [str(v) for v in a.v_i]
    lines = [["net", msg.name]]
    lines += [arg("netarg", a) for a in msg.arg]
    for b in msg.blob:
        lines.append(["blob", b.name, b.type if b.HasField("type") else "float", str(len(b.shape))] + [str(d) for d in b.shape] +
                     [str(len(b.data_f))] + [float(v).hex() for v in b.data_f])
    for op in msg.op:
        lines.append(["op", op.type, op.name, str(len(op.bottom))] + list(op.bottom) + [str(len(op.top))] + list(op.top) +
                     [str(len(op.arg))])
        lines += [arg("arg", a) for a in op.arg]
    return lines


def _normalise(dump):
    out = []
    for line in dump.splitlines():
        tok = line.split(" ")
        if tok[0] in ("arg", "netarg") and tok[2] in ("s_f", "v_f"):
            tok = tok[:3] + [float.fromhex(t).hex() for t in tok[3:]]
        if tok[0] == "blob":
            nd = int(tok[3])
            tok = tok[:5 + nd] + [float.fromhex(t).hex() for t in tok[5 + nd:]]
        out.append(tok)
    return out


def test_random_messages_through_both_protobuf_readers():
    """Seeded random NetParams (names without spaces, so that the dump tokenises): the official
    encoder's bytes and the official text printer's output both decode to exactly the message."""
    from google.protobuf import text_format
    rng = np.random.Generator(np.random.PCG64(2024))
    word = lambda: "".join(rng.choice(list("abcXYZ_019/.-"), size=int(rng.integers(1, 9))))   # noqa: E731
    f32 = lambda: float(np.float32(rng.choice([0.0, -0.0, 1.0, 1e-38, 3.4e38, -2.5, 1 / 3, 1e-45, 123456.789])))   # noqa: E731
    i32 = lambda: int(rng.choice([0, 1, -1, 127, 128, -129, 2 ** 31 - 1, -2 ** 31, 300, 65536]))   # noqa: E731

    def fill(a):
        a.name = word()
        kind = int(rng.integers(0, 6))
        if kind == 0:
            a.s_f = f32()
        elif kind == 1:
            a.s_i = i32()
        elif kind == 2:
            a.s_s = word()
        elif kind == 3:
            a.v_f.extend(f32() for _ in range(int(rng.integers(1, 5))))
        elif kind == 4:
            a.v_i.extend(i32() for _ in range(int(rng.integers(1, 5))))
        else:
            a.v_s.extend(word() for _ in range(int(rng.integers(1, 4))))
    for _ in range(40):
        msg = NetParam(name=word())
        for _ in range(int(rng.integers(0, 4))):
            fill(msg.arg.add())
        for _ in range(int(rng.integers(0, 3))):
            b = msg.blob.add(name=word())
            if rng.integers(0, 2):
                b.type = word()
            b.shape.extend(int(rng.integers(0, 5)) for _ in range(int(rng.integers(0, 4))))
            b.data_f.extend(f32() for _ in range(int(rng.integers(0, 6))))
        for _ in range(int(rng.integers(0, 5))):
            op = msg.op.add(name=word(), type=word())
            op.bottom.extend(word() for _ in range(int(rng.integers(0, 3))))
            op.top.extend(word() for _ in range(int(rng.integers(0, 3))))
            for _ in range(int(rng.integers(0, 4))):
                fill(op.arg.add())
        want = _expected_dump(msg)
        assert _normalise(Net(_lib(), "x").parse_binary(msg.SerializeToString()).dump()) == want
        if len(msg.arg) or len(msg.blob) or len(msg.op):   # an otherwise empty message prints as one name line, also fine
            assert _normalise(Net(_lib(), "x").parse_text(text_format.MessageToString(msg)).dump()) == want
