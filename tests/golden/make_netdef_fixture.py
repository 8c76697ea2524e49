"""Writes tests/golden/netdef_fixture.bin / .json: a NetDef that uses every field of every message
of the reference's mace/proto/mace.proto, serialized by the REAL protobuf runtime, plus what a
correct reader must find in it.  The message classes are built from the .proto text itself (there
is no protoc in the image): the simple proto2 subset the file uses is parsed into a
FileDescriptorProto and handed to protobuf's message factory.

Run where the reference tree is present:   python tests/golden/make_netdef_fixture.py <mace.proto>
The tests read only the two written files.
"""
import json
import os
import re
import sys

from google.protobuf import descriptor_pb2, descriptor_pool, message_factory

HERE = os.path.dirname(os.path.abspath(__file__))

SCALARS = {"float": 2, "int64": 3, "int32": 5, "bool": 8, "string": 9, "bytes": 12, "uint32": 13}
LABELS = {"optional": 1, "repeated": 3}


def parse_proto(text):
    text = re.sub(r"//[^\n]*", "", text)
    fd = descriptor_pb2.FileDescriptorProto(name="mace.proto", package="mace", syntax="proto2")
    enums = set()
    for m in re.finditer(r"enum\s+(\w+)\s*\{([^}]*)\}", text):
        e = fd.enum_type.add(name=m.group(1))
        enums.add(m.group(1))
        for v in re.finditer(r"(\w+)\s*=\s*(\d+)\s*;", m.group(2)):
            e.value.add(name=v.group(1), number=int(v.group(2)))
    for m in re.finditer(r"message\s+(\w+)\s*\{([^}]*)\}", text):
        msg = fd.message_type.add(name=m.group(1))
        for f in re.finditer(r"(optional|repeated)\s+(\w+)\s+(\w+)\s*=\s*(\d+)\s*(\[[^\]]*\])?\s*;", m.group(2)):
            label, typ, name, number, opts = f.groups()
            fld = msg.field.add(name=name, number=int(number), label=LABELS[label])
            if typ in SCALARS:
                fld.type = SCALARS[typ]
            elif typ in enums:
                fld.type = 14
                fld.type_name = ".mace." + typ
            else:
                fld.type = 11
                fld.type_name = ".mace." + typ
            if opts:
                if re.search(r"packed\s*=\s*true", opts):
                    fld.options.packed = True
                d = re.search(r"default\s*=\s*(\w+)", opts)
                if d:
                    fld.default_value = d.group(1)
    return fd


def build(classes):
    net = classes["NetDef"]()
    net.name = "fixture-net"
    net.data_type = 2
    net.data_offset = 7
    net.data_size = 1234567
    net.infer_order = -1
    a = net.arg.add(name="quantize_flag")
    a.i = 1
    a = net.arg.add(name="everything")
    a.f = -2.5
    a.i = -(1 << 40)
    a.s = b"bytes \x00\x01 with a quote \" and a backslash \\"
    a.floats.extend([0.1, -3.25, 1e-30])
    a.ints.extend([0, -1, 1 << 35, 127, 128])

    t = net.tensors.add(name="weights:0")
    t.dims.extend([3, 1, 300, 4])
    t.data_type = 2
    t.float_data.extend([1.5, -0.0, 3.4028234663852886e38])
    t.int32_data.extend([-2147483648, 2147483647, 0, -1])
    t.offset = 1 << 33
    t.data_size = 3600
    t.scale = 0.0123
    t.zero_point = -128
    t.minval = -6.0
    t.maxval = 6.0
    t.quantized = True
    t.node_id = 4000000000
    t = net.tensors.add(name="defaults")  # every optional field left unset

    op = net.op.add(name="conv1", type="Conv2D")
    op.input.extend(["input", "weights:0", "bias"])
    op.output.extend(["conv1:0", "conv1:1"])
    op.device_type = 0
    a = op.arg.add(name="strides")
    a.ints.extend([2, 2])
    a = op.arg.add(name="padding")
    a.i = 1
    a = op.arg.add(name="activation")
    a.s = b"RELUX"
    a = op.arg.add(name="max_limit")
    a.f = 6.0
    a = op.arg.add(name="T")
    a.i = 2
    op.output_shape.add().dims.extend([1, 112, 112, 32])
    op.output_shape.add().dims.extend([])
    op.output_type.extend([2, 4])
    q = op.quantize_info.add()
    q.scale = 0.0235
    q.zero_point = 3
    q.minval = -0.07
    q.maxval = 5.9
    op.quantize_info.add()
    op.mem_id.extend([0, -1, 5])
    op.node_id = 17
    op.op_id = 23
    op.padding = 1
    n = op.node_input.add()
    n.node_id = 5
    n.output_port = 1
    op.out_max_byte_size.extend([1605632, 4])
    op = net.op.add(name="empty", type="Identity")

    i = net.input_info.add(name="input")
    i.node_id = 1
    i.dims.extend([1, 224, 224, 3])
    i.max_byte_size = 602112
    i.data_type = 1
    i.data_format = 2
    i.scale = 0.5
    i.zero_point = 7
    i.alias = "image"
    net.input_info.add(name="second")
    o = net.output_info.add(name="conv1:0")
    o.dims.extend([1, 112, 112, 32])
    o.data_type = 2
    return net


def describe(net):
    """The structure mbh_netdef_describe prints, computed from the protobuf message."""

    def arg(a):
        d = {"name": a.name}
        if a.HasField("f"):
            d["f"] = a.f
        if a.HasField("i"):
            d["i"] = a.i
        if a.HasField("s"):
            d["s"] = a.s.decode("latin-1")
        if len(a.floats):
            d["floats"] = list(a.floats)
        if len(a.ints):
            d["ints"] = list(a.ints)
        return d

    def info(m):
        return {"name": m.name, "node_id": m.node_id, "dims": list(m.dims), "max_byte_size": m.max_byte_size,
                "data_type": int(m.data_type), "data_format": m.data_format, "scale": m.scale,
                "zero_point": m.zero_point, "alias": m.alias}

    return {
        "name": net.name, "data_type": int(net.data_type), "data_offset": net.data_offset,
        "data_size": net.data_size, "infer_order": net.infer_order,
        "arg": [arg(a) for a in net.arg],
        "tensors": [{"name": t.name, "dims": list(t.dims), "data_type": int(t.data_type),
                     "float_data": list(t.float_data), "int32_data": list(t.int32_data), "offset": t.offset,
                     "data_size": t.data_size, "scale": t.scale, "zero_point": t.zero_point, "minval": t.minval,
                     "maxval": t.maxval, "quantized": t.quantized, "node_id": t.node_id} for t in net.tensors],
        "op": [{"name": o.name, "type": o.type, "input": list(o.input), "output": list(o.output),
                "device_type": o.device_type, "arg": [arg(a) for a in o.arg],
                "output_shape": [list(s.dims) for s in o.output_shape],
                "output_type": [int(x) for x in o.output_type],
                "quantize_info": [{"scale": q.scale, "zero_point": q.zero_point, "minval": q.minval,
                                   "maxval": q.maxval} for q in o.quantize_info],
                "mem_id": list(o.mem_id), "node_id": o.node_id, "op_id": o.op_id, "padding": o.padding,
                "node_input": [[n.node_id, n.output_port] for n in o.node_input],
                "out_max_byte_size": list(o.out_max_byte_size)} for o in net.op],
        "input_info": [info(m) for m in net.input_info],
        "output_info": [info(m) for m in net.output_info],
    }


def main(proto_path):
    fd = parse_proto(open(proto_path).read())
    pool = descriptor_pool.DescriptorPool()
    pool.Add(fd)
    classes = {m.name: message_factory.GetMessageClass(pool.FindMessageTypeByName("mace." + m.name))
               for m in fd.message_type}
    net = build(classes)
    raw = net.SerializeToString(deterministic=True)
    again = classes["NetDef"]()
    again.ParseFromString(raw)
    assert again == net
    with open(os.path.join(HERE, "netdef_fixture.bin"), "wb") as f:
        f.write(raw)
    with open(os.path.join(HERE, "netdef_fixture.json"), "w") as f:
        json.dump({"source": "mace/proto/mace.proto, serialized by protobuf " +
                             __import__("google.protobuf").protobuf.__version__,
                   "bytes": len(raw), "expected": describe(net)}, f, indent=1)
    print("wrote", len(raw), "bytes")


if __name__ == "__main__":
    main(sys.argv[1])
