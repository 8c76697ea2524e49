"""Test-side writer of MACE model files: a minimal proto2 wire ENCODER for the messages of
mace/proto/mace.proto:25-117 (field numbers and types below), and a recorder with the
add_tensor() / op() interface of mace_b200.hostapi.HostEngine that turns the test networks into a
serialized NetDef plus a weights blob, the pair of files MACE's converter writes.

The encoder writes fields in field-number order, repeated scalars unpacked unless the .proto
says [packed = true], exactly as protobuf's own serializer does; tests/golden/netdef_fixture.*
(written by the real protobuf runtime from the reference's mace.proto) pins both this encoder and
the C++ decoder under test to the real field numbers.
"""
import struct

import numpy as np

DT_FLOAT, DT_UINT8, DT_HALF, DT_INT32 = 1, 2, 3, 4
DF_NONE, DF_NHWC, DF_NCHW = 0, 1, 2

# field name -> (number, kind[, message schema]); kinds: int (varint, two's complement 64-bit),
# float (fixed32), str, bytes, bool, msg; "r" prefix = repeated, "p" prefix = packed repeated
ARGUMENT = {"name": (1, "str"), "f": (2, "float"), "i": (3, "int"), "s": (4, "bytes"),
            "floats": (5, "rfloat"), "ints": (6, "rint")}
CONST_TENSOR = {"dims": (1, "rint"), "data_type": (2, "int"), "float_data": (3, "pfloat"),
                "int32_data": (4, "pint"), "name": (5, "str"), "offset": (6, "int"),
                "data_size": (7, "int"), "scale": (8, "float"), "zero_point": (9, "int"),
                "minval": (10, "float"), "maxval": (11, "float"), "quantized": (12, "bool"),
                "node_id": (100, "int")}
NODE_INPUT = {"node_id": (1, "int"), "output_port": (2, "int")}
OUTPUT_SHAPE = {"dims": (1, "rint")}
QUANTIZE_INFO = {"scale": (1, "float"), "zero_point": (2, "int"), "minval": (3, "float"),
                 "maxval": (4, "float")}
OPERATOR_DEF = {"input": (1, "rstr"), "output": (2, "rstr"), "name": (3, "str"), "type": (4, "str"),
                "device_type": (5, "int"), "arg": (6, "rmsg", ARGUMENT),
                "output_shape": (7, "rmsg", OUTPUT_SHAPE), "output_type": (8, "rint"),
                "quantize_info": (9, "rmsg", QUANTIZE_INFO), "mem_id": (10, "rint"),
                "node_id": (100, "int"), "op_id": (101, "int"), "padding": (102, "int"),
                "node_input": (103, "rmsg", NODE_INPUT), "out_max_byte_size": (104, "rint")}
IO_INFO = {"name": (1, "str"), "node_id": (2, "int"), "dims": (3, "rint"), "max_byte_size": (4, "int"),
           "data_type": (5, "int"), "data_format": (6, "int"), "scale": (7, "float"),
           "zero_point": (8, "int"), "alias": (100, "str")}
NET_DEF = {"op": (1, "rmsg", OPERATOR_DEF), "arg": (2, "rmsg", ARGUMENT),
           "tensors": (3, "rmsg", CONST_TENSOR), "data_type": (4, "int"), "name": (5, "str"),
           "data_offset": (6, "int"), "data_size": (7, "int"), "infer_order": (8, "int"),
           "input_info": (100, "rmsg", IO_INFO), "output_info": (101, "rmsg", IO_INFO)}


def varint(v):
    v &= (1 << 64) - 1  # negative int32 / int64 values travel as 10-byte varints
    out = bytearray()
    while True:
        b = v & 0x7F
        v >>= 7
        if v:
            out.append(b | 0x80)
        else:
            out.append(b)
            return bytes(out)


def _tag(number, wire_type):
    return varint((number << 3) | wire_type)


def _scalar(number, kind, value, schema=None):
    if kind in ("int", "bool"):
        return _tag(number, 0) + varint(int(value))
    if kind == "float":
        return _tag(number, 5) + struct.pack("<f", value)
    if kind in ("str", "bytes"):
        raw = value.encode() if isinstance(value, str) else bytes(value)
        return _tag(number, 2) + varint(len(raw)) + raw
    if kind == "msg":
        raw = encode(value, schema)
        return _tag(number, 2) + varint(len(raw)) + raw
    raise ValueError(kind)


def encode(message, schema):
    """message: dict field name -> value (lists for repeated fields); absent = not set."""
    out = bytearray()
    for name, spec in sorted(schema.items(), key=lambda kv: kv[1][0]):
        if name not in message:
            continue
        number, kind = spec[0], spec[1]
        sub = spec[2] if len(spec) > 2 else None
        value = message[name]
        if kind[0] == "r":
            for v in value:
                out += _scalar(number, kind[1:], v, sub)
        elif kind[0] == "p":
            if len(value):
                if kind == "pfloat":
                    raw = b"".join(struct.pack("<f", v) for v in value)
                else:
                    raw = b"".join(varint(int(v)) for v in value)
                out += _tag(number, 2) + varint(len(raw)) + raw
        else:
            out += _scalar(number, kind, value, sub)
    return bytes(out)


_NP_TO_DT = {np.dtype(np.float32): DT_FLOAT, np.dtype(np.uint8): DT_UINT8, np.dtype(np.int32): DT_INT32,
             np.dtype(np.float16): DT_HALF}


class NetDefWriter:
    """Records add_tensor() / op() calls (the HostEngine interface the test networks are built
    through) and serializes them: netdef() -> bytes, weights() -> bytes."""

    def __init__(self, device=0, quantized=False, name="net"):
        self.quantized = quantized
        self.net = {"op": [], "arg": [], "tensors": [], "name": name, "input_info": [], "output_info": []}
        if quantized:
            self.net["arg"].append({"name": "quantize_flag", "i": 1})
        self.blob = bytearray()

    # -- HostEngine interface --
    def add_tensor(self, name, array=None, shape=None, dtype=None, scale=0.0, zero_point=0, is_weight=False,
                   data_format=DF_NHWC):
        if array is None:  # a model input
            info = {"name": name, "dims": list(shape), "data_type": int(dtype), "data_format": data_format}
            if scale:
                info["scale"] = float(scale)
                info["zero_point"] = int(zero_point)
            self.net["input_info"].append(info)
            return
        a = np.ascontiguousarray(array)
        while len(self.blob) % 4:  # the converter keeps tensors 4-byte aligned
            self.blob.append(0)
        t = {"dims": list(a.shape), "data_type": _NP_TO_DT[a.dtype], "name": name, "offset": len(self.blob),
             "data_size": int(a.size)}
        if scale:
            t["scale"] = float(scale)
            t["zero_point"] = int(zero_point)
        self.net["tensors"].append(t)
        self.blob += a.tobytes()

    def op(self, type_, name, inputs, outputs, T=DT_UINT8, out_dtype=None, out_quant=None, ints=None, i=None,
           f=None, s=None, floats=None):
        args = [{"name": "T", "i": int(T)}]
        for k, v in (i or {}).items():
            args.append({"name": k, "i": int(v)})
        for k, v in (ints or {}).items():
            args.append({"name": k, "ints": [int(x) for x in v]})
        for k, v in (floats or {}).items():
            args.append({"name": k, "floats": [float(x) for x in v]})
        for k, v in (f or {}).items():
            args.append({"name": k, "f": float(v)})
        for k, v in (s or {}).items():
            args.append({"name": k, "s": v})
        od = {"input": list(inputs), "output": list(outputs), "name": name, "type": type_, "arg": args}
        if out_dtype is not None:
            od["output_type"] = [int(out_dtype)] * len(outputs)
        if out_quant:
            # (scale, zero_point) or (scale, zero_point, minval, maxval)
            od["quantize_info"] = [dict({"scale": float(q[0]), "zero_point": int(q[1])},
                                        **({"minval": float(q[2]), "maxval": float(q[3])} if len(q) == 4 else {}))
                                   for q in out_quant]
        self.net["op"].append(od)

    # -- model outputs --
    def add_output(self, name, dims, data_type=DT_FLOAT, data_format=DF_NHWC):
        self.net["output_info"].append({"name": name, "dims": list(dims), "data_type": int(data_type),
                                        "data_format": data_format})

    def netdef(self):
        return encode(self.net, NET_DEF)

    def weights(self):
        return bytes(self.blob)


class WriterModule:
    """Stands in for the hostapi module where a network builder expects one: HostEngine(device)
    returns the shared NetDefWriter; the constants are hostapi's."""

    def __init__(self, hostapi, writer):
        self._writer = writer
        for k in dir(hostapi):
            if k.isupper():
                setattr(self, k, getattr(hostapi, k))

    def HostEngine(self, device=0):
        return self._writer
