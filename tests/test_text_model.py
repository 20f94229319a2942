"""The protobuf-free model text format: the same text is parsed by the reference (compiled from its own
sources, CPU) and by this library's IO::ReadProtoFromText; both must produce the net the golden
fixtures were made from - including the PARSER's defaults, which differ from the operators' own
(Scale: has_scale / has_bias default to 1 in the text format)."""
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.dirname(__file__))
import cases  # noqa: E402
from oracle import oracle as orc  # noqa: E402
from shadow_b200.netapi import Net, ShadowError, model_text  # noqa: E402

TEXT_OPS = ("Activate", "BatchNorm", "Binary", "Concat", "Eltwise", "Flatten", "Gather", "InstanceNorm", "Pad", "Permute",
            "Pooling", "Reduce", "Reshape", "Scale", "Slice", "Softmax", "Squeeze", "SSDNormalize", "Stack", "Unary", "Unsqueeze")


def _text_cases():
    out = []
    for c in cases.small_cases():
        if c["op"] not in TEXT_OPS or c["inputs"][0].size > 4096:
            continue
        a = c["args"]
        if c["op"] == "Scale" and not ("has_scale" in a and "has_bias" in a):
            continue          # the text format defaults has_scale/has_bias to 1: such a case would mean another net
        if c["op"] == "Pooling" and not a.get("global_pooling", False) and not ("stride" in a and "pad" in a):
            continue          # the text format emits empty stride / pad lists when they are absent, which the operator refuses
        if c["op"] == "SSDNormalize" and "eps" in a:
            continue          # the text format does not carry eps for SSDNormalize
        if sum(1 for o in out if o["op"] == c["op"]) < 4:   # a few per operator type keep the suite short
            out.append(c)
    return out


CASES = _text_cases()
# The reference's tokenizer turns an empty list into one empty token and then fails on it, so a text it
# can read has at least one net argument and one blob; this library's reader also accepts "[]".
FILLERS = {"net_args": {"from_text": 1}, "blobs": [("unused_blob", "float", [1])]}


def _as_text(case):
    names = ["in%d" % i for i in range(len(case["inputs"]))]
    tops = ["out"] if case.get("n_tops", 1) == 1 else ["out%d" % k for k in range(case["n_tops"])]
    ops = [("Input", "input", [], names, {n: [int(d) for d in (x.shape if x.ndim else (1,))] for n, x in zip(names, case["inputs"])}),
           (case["op"], "op0", names, tops, case["args"])]
    return model_text(case["name"], ops, **FILLERS), names, tops


def _run_text(library, case):
    text, names, tops = _as_text(case)
    net = Net(library, "t").parse_text(text)
    net.load("Native", out_blobs=tops)
    net.forward(dict(zip(names, case["inputs"])))
    return net.blob(tops[0]) if len(tops) == 1 else np.concatenate([net.blob(t).ravel() for t in tops])


def test_every_text_operator_type_is_covered():
    assert {c["op"] for c in CASES} == set(TEXT_OPS)


@pytest.mark.parametrize("case", CASES, ids=[c["name"] for c in CASES])
def test_reference_parses_the_writer_output(case):
    ref = orc.ref_library()
    if ref is None:
        pytest.skip("compiled reference not available")
    got = _run_text(ref, case)
    want = cases.run_net(ref, case)
    assert got.shape == want.shape and orc.bit_equal(got, want)


@pytest.mark.gpu
@pytest.mark.parametrize("case", CASES, ids=[c["name"] for c in CASES])
def test_product_parser_matches_programmatic_net(case):
    import shadow_b200
    lib = shadow_b200.host_library()
    got = _run_text(lib, case)
    want = cases.run_net(lib, case)
    assert got.shape == want.shape and orc.bit_equal(got, want)


@pytest.mark.gpu
def test_parser_defaults_are_the_text_formats():
    """A Scale line without has_scale / has_bias means scale AND bias inputs (parser default 1);
    a Reduce line without keep_dims keeps the dims."""
    import shadow_b200
    lib = shadow_b200.host_library()
    ref = orc.ref_library()
    x, g, b = cases.normal(5, (2, 3, 4)), cases.normal(6, (3,)), cases.normal(7, (3,))
    text = model_text("n", [("Input", "input", [], ["x", "g", "b"], {"x": [2, 3, 4], "g": [3], "b": [3]}),
                            ("Scale", "s", ["x", "g", "b"], ["y"], {}),
                            ("Reduce", "r", ["y"], ["z"], {"operation": 1, "axes": [2]})], **FILLERS)
    outs = []
    for library in (lib, ref):
        if library is None:
            continue
        net = Net(library, "n").parse_text(text)
        net.load("Native", out_blobs=["y", "z"])
        net.forward({"x": x, "g": g, "b": b})
        assert net.shape("z") == [2, 3, 1]
        outs.append((net.blob("y"), net.blob("z")))
    assert orc.bit_equal(outs[0][0], orc.scale(x, 1, g, b))
    if len(outs) == 2:
        assert orc.bit_equal(outs[0][0], outs[1][0])
        cases.assert_parity({"name": "z", "op": "Reduce", "args": {"operation": 1, "axes": [2]}, "inputs": [outs[0][0]]},
                            outs[0][1], outs[1][1])


def test_malformed_text_and_unknown_operator_are_refused():
    import shadow_b200
    lib = shadow_b200.host_library()
    with pytest.raises(ShadowError):
        Net(lib, "n").parse_text("[n]")
    with pytest.raises(ShadowError, match="is not recognized"):
        Net(lib, "n").parse_text("[n]\n[]\n[]\n[Conv] | [c] | [1 1 0] | [x] | [y] | []")
