"""The model-file reader (mace_b200/host/netdef.cc) against a NetDef serialized by the real protobuf
runtime from the reference's mace/proto/mace.proto (tests/golden/netdef_fixture.*, written by
tests/golden/make_netdef_fixture.py), against malformed input, and against the test-side encoder
the GPU model-file tests build their networks with.  No GPU needed: only the parser is called."""
import json
import os
import struct

import numpy as np
import pytest

from mace_b200.harness import netdef_wire as W
from mace_b200 import capi, hostapi

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _same(expected, got, path=""):
    if isinstance(expected, dict):
        assert set(expected) == set(got), (path, set(expected) ^ set(got))
        for k in expected:
            _same(expected[k], got[k], path + "/" + k)
    elif isinstance(expected, list):
        assert len(expected) == len(got), (path, expected, got)
        for i, (x, y) in enumerate(zip(expected, got)):
            _same(x, y, "%s/%d" % (path, i))
    elif isinstance(expected, float) or isinstance(got, float):
        assert np.float32(expected) == np.float32(got), (path, expected, got)  # floats print with 9 digits
    else:
        assert expected == got, (path, expected, got)


def _fixture():
    raw = open(os.path.join(GOLDEN, "netdef_fixture.bin"), "rb").read()
    meta = json.load(open(os.path.join(GOLDEN, "netdef_fixture.json")))
    assert len(raw) == meta["bytes"]
    return raw, meta["expected"]


def test_reader_matches_protobuf_serialization():
    raw, expected = _fixture()
    got = json.loads(hostapi.describe_netdef(raw))
    _same(expected, got)
    # spot checks of the awkward values, independent of the comparison helper
    assert got["arg"][1]["i"] == -(1 << 40) and got["arg"][1]["ints"] == [0, -1, 1 << 35, 127, 128]
    assert got["tensors"][0]["int32_data"] == [-2147483648, 2147483647, 0, -1]
    assert got["tensors"][0]["offset"] == 1 << 33 and got["tensors"][0]["node_id"] == 4000000000
    assert got["infer_order"] == -1 and got["op"][0]["mem_id"] == [0, -1, 5]
    # defaults of unset fields (mace.proto: data_type DT_FLOAT, data_format NHWC, quantized false)
    assert got["tensors"][1]["data_type"] == 1 and got["tensors"][1]["quantized"] is False
    assert got["input_info"][1]["data_format"] == 1 and got["input_info"][1]["data_type"] == 1


def test_every_truncation_is_rejected_or_a_valid_prefix():
    raw, _ = _fixture()
    ok = 0
    for n in range(len(raw)):
        try:
            hostapi.describe_netdef(raw[:n])
            ok += 1  # cut at a field boundary of the top-level message: a shorter valid NetDef
        except capi.MaceB200Error as e:
            assert e.code == 1, e  # MACE_INVALID_ARGS
    assert 0 < ok < len(raw) // 4


@pytest.mark.parametrize("bad, why", [
    (b"\x0a\x05ab", "runs past the end"),                      # length 5, 2 bytes left
    (b"\x20" + b"\xff" * 10 + b"\x01", "varint"),              # 11-byte varint
    (b"\x20" + b"\xff" * 9 + b"\x02", "64 bits"),              # 10th byte carries more than bit 63
    (b"\xbb\x3e", "group"),                                     # unknown field 999, wire type 3
    (b"\x0b", "does not fit"),                                  # op (field 1) as a group
    (b"\x00", "tag"),                                           # field number 0
    (b"\x25\x00\x00\x00\x00", "does not fit"),                  # data_type as fixed32
    (b"\x0a\x02\x1a\x05", "runs past the end"),                 # op { name: <length 5, nothing left> }
    (b"\x1a\x03\x45\x00\x00", "truncated"),                     # tensors { scale: 2 of 4 bytes }
])
def test_malformed_messages(bad, why):
    with pytest.raises(capi.MaceB200Error) as e:
        hostapi.describe_netdef(bad)
    assert e.value.code == 1 and why in str(e.value), str(e.value)


def test_unknown_fields_are_skipped_and_both_repeated_encodings_read():
    raw, expected = _fixture()
    extra = (W.varint((999 << 3) | 0) + W.varint(12345)            # unknown varint
             + W.varint((998 << 3) | 2) + W.varint(3) + b"xyz"    # unknown bytes
             + W.varint((997 << 3) | 5) + b"\x00\x00\x80\x3f"     # unknown fixed32
             + W.varint((996 << 3) | 1) + b"\x00" * 8)            # unknown fixed64
    got = json.loads(hostapi.describe_netdef(extra + raw + extra))
    _same(expected, got)
    # ConstTensor.float_data is packed in the .proto; a writer may still send it one by one, and
    # Argument.ints (unpacked in the .proto) may arrive packed: parsers must take both
    tensor = (W.varint((3 << 3) | 5) + struct.pack("<f", 1.5) + W.varint((3 << 3) | 5) + struct.pack("<f", -2.0))
    arg = W.varint((6 << 3) | 2) + W.varint(3) + W.varint(7) + W.varint(300)  # ints packed: 7, 300
    net = (W.varint((3 << 3) | 2) + W.varint(len(tensor)) + tensor + W.varint((2 << 3) | 2) + W.varint(len(arg)) + arg)
    got = json.loads(hostapi.describe_netdef(net))
    assert got["tensors"][0]["float_data"] == [1.5, -2.0]
    assert got["arg"][0]["ints"] == [7, 300]


def test_empty_message_is_an_empty_net():
    got = json.loads(hostapi.describe_netdef(b""))
    assert got["op"] == [] and got["tensors"] == [] and got["data_type"] == 1 and got["name"] == ""


def test_encoder_used_by_the_gpu_tests_round_trips_through_the_reader():
    w = W.NetDefWriter(quantized=True, name="roundtrip")
    w.add_tensor("input", shape=(2, 8, 8, 3), dtype=W.DT_UINT8, scale=1.0 / 255, zero_point=0)
    filt = np.arange(4 * 3 * 3 * 3, dtype=np.uint8).reshape(4, 3, 3, 3)
    bias = np.array([-5, 0, 7, 1 << 20], dtype=np.int32)
    w.add_tensor("f", filt, scale=0.02, zero_point=120, is_weight=True)
    w.add_tensor("b", bias, scale=0.02 / 255, zero_point=0, is_weight=True)
    w.op("Conv2D", "conv", ["input", "f", "b"], ["conv"], T=W.DT_UINT8, out_quant=[(0.05, 3)],
         ints={"strides": [2, 2], "dilations": [1, 1]}, i={"padding": 1}, s={"activation": "RELU"},
         f={"max_limit": 6.0}, floats={"coeff": [1.0, -1.0]})
    w.add_output("conv", (2, 4, 4, 4), data_type=W.DT_UINT8)
    got = json.loads(hostapi.describe_netdef(w.netdef()))
    assert got["name"] == "roundtrip" and got["arg"] == [{"name": "quantize_flag", "i": 1}]
    t0, t1 = got["tensors"]
    assert (t0["name"], t0["dims"], t0["data_type"], t0["offset"], t0["data_size"]) == ("f", [4, 3, 3, 3], 2, 0, 108)
    assert (t1["name"], t1["dims"], t1["data_type"], t1["offset"], t1["data_size"]) == ("b", [4], 4, 108, 4)
    assert np.float32(t0["scale"]) == np.float32(0.02) and t0["zero_point"] == 120
    blob = w.weights()
    assert np.array_equal(np.frombuffer(blob, np.uint8, 108, 0).reshape(filt.shape), filt)
    assert np.array_equal(np.frombuffer(blob, np.int32, 4, 108), bias)
    op = got["op"][0]
    assert op["type"] == "Conv2D" and op["input"] == ["input", "f", "b"] and op["output"] == ["conv"]
    args = {a["name"]: a for a in op["arg"]}
    assert args["T"]["i"] == 2 and args["strides"]["ints"] == [2, 2] and args["padding"]["i"] == 1
    assert args["activation"]["s"] == "RELU" and args["max_limit"]["f"] == 6.0
    assert args["coeff"]["floats"] == [1.0, -1.0]
    assert np.float32(op["quantize_info"][0]["scale"]) == np.float32(0.05) and op["quantize_info"][0]["zero_point"] == 3
    info = got["input_info"][0]
    assert info["name"] == "input" and info["dims"] == [2, 8, 8, 3] and info["data_type"] == 2
    assert got["output_info"][0]["name"] == "conv" and got["output_info"][0]["data_type"] == 2


def test_half_weights_widen_exactly_for_every_bit_pattern():
    bits = np.arange(65536, dtype=np.uint16)
    got = hostapi.half_to_float(bits).view(np.uint32)
    want = bits.view(np.float16).astype(np.float32).view(np.uint32)
    assert np.array_equal(got, want)  # normals, subnormals, zeros, infinities, NaN payloads
