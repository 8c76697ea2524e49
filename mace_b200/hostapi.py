"""ctypes binding of ``libmace_b200_host.so``: the C entry points of the C++ host layer
(operators, delegators, sequential net).  Used by the tests and the benchmark to drive the
host layer the way the reference's OpsTestNet / OpDefBuilder drive MACE's operators
(test/ccutils/mace/ops/ops_test_util.h:122-316)."""
import ctypes as C
import os

import numpy as np

from . import capi

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = os.path.join(_HERE, "libmace_b200_host.so")

DT_FLOAT, DT_UINT8, DT_INT32 = 1, 2, 4
VALID, SAME, FULL = 0, 1, 2
AVG, MAX = 1, 2
_NP = {DT_FLOAT: np.float32, DT_UINT8: np.uint8, DT_INT32: np.int32}
_DT = {np.dtype(np.float32): DT_FLOAT, np.dtype(np.uint8): DT_UINT8, np.dtype(np.int32): DT_INT32}

_vp, _int, _i32, _f32, _sz, _cp = C.c_void_p, C.c_int, C.c_int32, C.c_float, C.c_size_t, C.c_char_p
_PROTOS = {
    "mbh_engine_create": [_int, C.POINTER(_vp)],
    "mbh_engine_destroy": [_vp],
    "mbh_engine_context": [_vp],
    "mbh_add_tensor": [_vp, _cp, _int, _int, C.POINTER(C.c_int64), _vp, _f32, _i32, _int],
    "mbh_set_tensor_quant": [_vp, _cp, _f32, _i32],
    "mbh_tensor_rank": [_vp, _cp, C.POINTER(_int)],
    "mbh_tensor_shape": [_vp, _cp, C.POINTER(C.c_int64), _int],
    "mbh_tensor_quant": [_vp, _cp, C.POINTER(_f32), C.POINTER(_i32)],
    "mbh_tensor_read": [_vp, _cp, _vp, _sz],
    "mbh_tensor_write": [_vp, _cp, _vp, _sz],
    "mbh_tensor_device_ptr": [_vp, _cp, C.POINTER(_vp), C.POINTER(_sz)],
    "mbh_op_begin": [_vp, _cp, _cp],
    "mbh_op_input": [_vp, _cp],
    "mbh_op_output": [_vp, _cp, _int, _f32, _i32],
    "mbh_op_arg_int": [_vp, _cp, _int],
    "mbh_op_arg_ints": [_vp, _cp, _int, C.POINTER(_int)],
    "mbh_op_arg_floats": [_vp, _cp, _int, C.POINTER(C.c_float)],
    "mbh_op_arg_float": [_vp, _cp, _f32],
    "mbh_op_arg_str": [_vp, _cp, _cp],
    "mbh_op_end": [_vp],
    "mbh_run": [_vp],
    "mbh_sync": [_vp],
    "mbh_capture": [_vp],
    "mbh_fuse_activations": [_vp, C.POINTER(_int)],
    "mbh_plan_memory": [_vp, C.POINTER(_sz), C.POINTER(_sz)],
    "mbh_fuse_residual_sums": [_vp, C.POINTER(_int)],
    "mbh_share_subsampled_inputs": [_vp, C.POINTER(_int)],
    "mbh_run_host": [_vp, _cp, _vp, _sz, _cp, _vp, _sz],
    "mbh_run_host_pipelined": [_vp, _cp, _vp, _sz, _cp, _vp, _sz, C.POINTER(_int)],
    "mbh_wait_slot": [_vp, _int],
    "mbh_run_profiled": [_vp, C.POINTER(_f32), _int, C.c_char_p, _sz, C.POINTER(_int)],
    "mbh_run_profiled_graph": [_vp, _int, C.POINTER(_f32), _int, C.c_char_p, _sz, C.POINTER(_int)],
    "mbh_netdef_describe": [_vp, _sz, C.c_char_p, _sz, C.POINTER(_sz)],
    "mbh_half_to_float": [_vp, _vp, _sz],
    "mbh_model_destroy": [_vp],
    "mbh_model_captured": [_vp],
    "mbh_model_run_metadata": [_vp, C.c_char_p, _sz, C.POINTER(_sz)],
    "mbh_shard_bounds": [C.c_int64, _int, _int, C.POINTER(C.c_int64), C.POINTER(C.c_int64)],
    "mbh_multi_destroy": [_vp],
    "mbh_multi_shards": [_vp],
    "mbh_set_vlog_level": [_int],
    "mbh_vlog_is_on": [_int],
    "mbh_log": [_int, _cp],
}
LOG_SINK = C.CFUNCTYPE(None, _int, _cp)
_lib = None


def lib():
    global _lib
    if _lib is None:
        capi.lib()  # the device library must load first (and must exist)
        if not os.path.exists(_LIB):
            raise ImportError("libmace_b200_host.so is missing: build with make -C mace_b200/host")
        _lib = C.CDLL(_LIB)
        for name, args in _PROTOS.items():
            fn = getattr(_lib, name)
            fn.argtypes = args
            fn.restype = _int
        _lib.mbh_last_error.restype = _cp
        _lib.mbh_last_error.argtypes = [_vp]
        _lib.mbh_engine_context.restype = _vp
        _lib.mbh_model_create.restype = _int
        _lib.mbh_model_create.argtypes = [_int, _vp, _sz, _vp, _sz, _int, _int, _int, C.POINTER(_vp), C.c_char_p, _sz]
        _lib.mbh_model_run.restype = _int
        _lib.mbh_model_run.argtypes = [_vp, _int, C.POINTER(IoTensor), _int, C.POINTER(IoTensor)]
        _lib.mbh_model_last_error.restype = _cp
        _lib.mbh_model_last_error.argtypes = [_vp]
        _lib.mbh_model_context.restype = _vp
        _lib.mbh_model_context.argtypes = [_vp]
        _lib.mbh_multi_create.restype = _int
        _lib.mbh_multi_create.argtypes = [_int, C.POINTER(_int), _vp, _sz, _vp, _sz, _int, _int, _int,
                                          C.POINTER(_vp), C.c_char_p, _sz]
        _lib.mbh_multi_run.restype = _int
        _lib.mbh_multi_run.argtypes = [_vp, _int, C.POINTER(IoTensor), _int, C.POINTER(IoTensor)]
        _lib.mbh_multi_last_error.restype = _cp
        _lib.mbh_multi_last_error.argtypes = [_vp]
        _lib.mbh_set_log_sink.restype = _int
        _lib.mbh_set_log_sink.argtypes = [LOG_SINK]
    return _lib


DF_NONE, DF_NHWC, DF_NCHW = 0, 1, 2


class IoTensor(C.Structure):
    """mbh_io_tensor: one input or output of a model in host memory."""
    _fields_ = [("name", _cp), ("data", _vp), ("shape", C.c_int64 * 8), ("rank", _int), ("data_format", _int),
                ("data_type", _int)]


def describe_netdef(graph):
    """Parses a serialized NetDef (bytes) and returns its JSON rendering; needs no GPU."""
    need = _sz()
    L = lib()
    L.mbh_netdef_describe(graph, len(graph), None, 0, C.byref(need))
    buf = C.create_string_buffer(need.value)
    st = L.mbh_netdef_describe(graph, len(graph), buf, need.value, None)
    if st != 0:
        raise capi.MaceB200Error(st, buf.value.decode())
    return buf.value.decode()


def half_to_float(h):
    """uint16 bit patterns of IEEE halves -> float32, by the loader's own routine; needs no GPU."""
    h = np.ascontiguousarray(h, np.uint16)
    out = np.empty(h.shape, np.float32)
    st = lib().mbh_half_to_float(h.ctypes.data, out.ctypes.data, h.size)
    if st != 0:
        raise capi.MaceB200Error(st, "mbh_half_to_float")
    return out


class Model:
    """A converted model (serialized NetDef + weights blob) on one GPU: the C++ MaceEngine of
    mace_b200/host/mace_engine.h, i.e. CreateMaceEngineFromProto + MaceEngine::Run."""

    def __init__(self, graph, weights, device=0, fuse=False, plan_memory=False, cuda_graph=False):
        self.h = _vp()
        err = C.create_string_buffer(1024)
        st = lib().mbh_model_create(int(device), graph, len(graph), weights, len(weights), int(fuse),
                                    int(plan_memory), int(cuda_graph), C.byref(self.h), err, len(err))
        if st != 0:
            self.h = None
            raise capi.MaceB200Error(st, err.value.decode())

    def close(self):
        if self.h:
            lib().mbh_model_destroy(self.h)
            self.h = None

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    @property
    def context(self):
        return lib().mbh_model_context(self.h)

    @property
    def captured(self):
        return bool(lib().mbh_model_captured(self.h))

    def run(self, inputs, outputs):
        """inputs: {name: (array, data_format)}; outputs: {name: (array sized for the largest result,
        data_format)}.  Returns {name: view of the output array with the actual shape}."""
        ins, outs, keep = _marshal_io(inputs, outputs)
        st = lib().mbh_model_run(self.h, len(inputs), ins, len(outputs), outs)
        if st != 0:
            raise capi.MaceB200Error(st, lib().mbh_model_last_error(self.h).decode())
        return _unmarshal_outputs(outputs, outs)

    def run_metadata(self):
        """Runs the net once more on the inputs of the last run() and returns RunMetadata's
        per-operator statistics as a list of dicts (times from device events)."""
        import json
        need = _sz()
        buf = C.create_string_buffer(1 << 20)
        st = lib().mbh_model_run_metadata(self.h, buf, len(buf), C.byref(need))
        if st != 0:
            raise capi.MaceB200Error(st, lib().mbh_model_last_error(self.h).decode())
        assert need.value <= len(buf)
        return json.loads(buf.value.decode())


def _marshal_io(inputs, outputs):
    ins = (IoTensor * max(1, len(inputs)))()
    keep = []
    for k, (name, (a, fmt)) in enumerate(inputs.items()):
        a = np.ascontiguousarray(a)
        keep.append(a)
        ins[k].name, ins[k].data, ins[k].rank = name.encode(), a.ctypes.data, a.ndim
        ins[k].data_format, ins[k].data_type = fmt, _DT[a.dtype]
        for d in range(a.ndim):
            ins[k].shape[d] = a.shape[d]
    outs = (IoTensor * max(1, len(outputs)))()
    for k, (name, (a, fmt)) in enumerate(outputs.items()):
        assert a.flags["C_CONTIGUOUS"]
        outs[k].name, outs[k].data, outs[k].rank = name.encode(), a.ctypes.data, a.ndim
        outs[k].data_format, outs[k].data_type = fmt, _DT[a.dtype]
        for d in range(a.ndim):
            outs[k].shape[d] = a.shape[d]
    return ins, outs, keep


def _unmarshal_outputs(outputs, outs):
    result = {}
    for k, (name, (a, fmt)) in enumerate(outputs.items()):
        shape = tuple(outs[k].shape[d] for d in range(outs[k].rank))
        n = int(np.prod(shape)) if shape else 1
        result[name] = a.reshape(-1)[:n].reshape(shape)
    return result


def shard_bounds(total, parts, index):
    """Rows [begin, end) of shard `index` of `parts` (the C++ runner's rule); needs no GPU."""
    b, e = C.c_int64(), C.c_int64()
    st = lib().mbh_shard_bounds(int(total), int(parts), int(index), C.byref(b), C.byref(e))
    if st != 0:
        raise capi.MaceB200Error(st, "mbh_shard_bounds: bad argument")
    return b.value, e.value


class MultiModel:
    """A converted model replicated over several shards (normally one per GPU): the C++
    MultiGpuRunner -- one MaceEngine, stream and host thread per shard, the batch split along the
    first dimension, every shard's output rows copied straight into the caller's buffer."""

    def __init__(self, graph, weights, devices, fuse=False, plan_memory=False, cuda_graph=False):
        self.h = _vp()
        err = C.create_string_buffer(1024)
        dev = (_int * len(devices))(*[int(d) for d in devices])
        st = lib().mbh_multi_create(len(devices), dev, graph, len(graph), weights, len(weights), int(fuse),
                                    int(plan_memory), int(cuda_graph), C.byref(self.h), err, len(err))
        if st != 0:
            self.h = None
            raise capi.MaceB200Error(st, err.value.decode())

    def close(self):
        if self.h:
            lib().mbh_multi_destroy(self.h)
            self.h = None

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    @property
    def shards(self):
        return lib().mbh_multi_shards(self.h)

    def run(self, inputs, outputs):
        """As Model.run, on the whole batch."""
        ins, outs, keep = _marshal_io(inputs, outputs)
        st = lib().mbh_multi_run(self.h, len(inputs), ins, len(outputs), outs)
        if st != 0:
            raise capi.MaceB200Error(st, lib().mbh_multi_last_error(self.h).decode())
        return _unmarshal_outputs(outputs, outs)


class LogCapture:
    """Collects the host layer's log lines (LOG / VLOG) while active, optionally with another
    VLOG level than the environment's."""

    def __init__(self, vlog_level=None):
        self.lines = []
        self.vlog_level = vlog_level
        self._cb = LOG_SINK(lambda sev, line: self.lines.append((sev, line.decode())))

    def __enter__(self):
        lib().mbh_set_log_sink(self._cb)
        if self.vlog_level is not None:
            lib().mbh_set_vlog_level(int(self.vlog_level))
        return self

    def __exit__(self, *a):
        lib().mbh_set_log_sink(C.cast(None, LOG_SINK))
        lib().mbh_set_vlog_level(-2 ** 31)


class HostEngine:
    """One engine: CudaRuntime + workspace + SerialNet on one GPU."""

    def __init__(self, device=0):
        self.h = _vp()
        st = lib().mbh_engine_create(int(device), C.byref(self.h))
        if st != 0:
            raise capi.MaceB200Error(st, "mbh_engine_create failed (no sm_100a CUDA device?)")

    def _check(self, st):
        if st != 0:
            raise capi.MaceB200Error(st, lib().mbh_last_error(self.h).decode())

    def close(self):
        if self.h:
            lib().mbh_engine_destroy(self.h)
            self.h = None

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    @property
    def context(self):
        """The raw mb_context pointer of the engine's runtime."""
        return lib().mbh_engine_context(self.h)

    # -- tensors ------------------------------------------------------------------
    def add_tensor(self, name, array=None, shape=None, dtype=None, scale=0.0, zero_point=0,
                   is_weight=False):
        if array is not None:
            array = np.ascontiguousarray(array)
            shape, dt = array.shape, _DT[array.dtype]
            ptr = array.ctypes.data
        else:
            dt, ptr = dtype, None
        dims = (C.c_int64 * len(shape))(*shape)
        self._check(lib().mbh_add_tensor(self.h, name.encode(), dt, len(shape), dims, ptr,
                                         float(scale), int(zero_point), int(is_weight)))

    def set_quant(self, name, scale, zero_point):
        self._check(lib().mbh_set_tensor_quant(self.h, name.encode(), float(scale), int(zero_point)))

    def shape(self, name):
        r = _int()
        self._check(lib().mbh_tensor_rank(self.h, name.encode(), C.byref(r)))
        dims = (C.c_int64 * max(r.value, 1))()
        self._check(lib().mbh_tensor_shape(self.h, name.encode(), dims, r.value))
        return tuple(dims[i] for i in range(r.value))

    def quant(self, name):
        s, z = _f32(), _i32()
        self._check(lib().mbh_tensor_quant(self.h, name.encode(), C.byref(s), C.byref(z)))
        return np.float32(s.value), int(z.value)

    def read(self, name, dtype):
        out = np.empty(self.shape(name), dtype)
        self._check(lib().mbh_tensor_read(self.h, name.encode(), out.ctypes.data, out.nbytes))
        return out

    def device_ptr(self, name):
        """(device address, bytes) of a tensor after the last run."""
        p, n = _vp(), _sz()
        self._check(lib().mbh_tensor_device_ptr(self.h, name.encode(), C.byref(p), C.byref(n)))
        return p.value, n.value

    def write(self, name, array):
        array = np.ascontiguousarray(array)
        self._check(lib().mbh_tensor_write(self.h, name.encode(), array.ctypes.data, array.nbytes))

    # -- operators ----------------------------------------------------------------
    def op(self, type_, name, inputs, outputs, T=DT_UINT8, out_dtype=None, out_quant=None,
           ints=None, i=None, f=None, s=None, floats=None):
        """Adds one operator; the keyword groups are the typed args of an OperatorDef."""
        L = lib()
        self._check(L.mbh_op_begin(self.h, type_.encode(), name.encode()))
        for t in inputs:
            self._check(L.mbh_op_input(self.h, t.encode()))
        for k, t in enumerate(outputs):
            q = out_quant[k] if out_quant else (0.0, 0)
            self._check(L.mbh_op_output(self.h, t.encode(), -1 if out_dtype is None else out_dtype,
                                        float(q[0]), int(q[1])))
        self._check(L.mbh_op_arg_int(self.h, b"T", int(T)))
        for k, v in (i or {}).items():
            self._check(L.mbh_op_arg_int(self.h, k.encode(), int(v)))
        for k, v in (ints or {}).items():
            arr = (C.c_int * len(v))(*v)
            self._check(L.mbh_op_arg_ints(self.h, k.encode(), len(v), arr))
        for k, v in (floats or {}).items():
            arr = (C.c_float * len(v))(*v)
            self._check(L.mbh_op_arg_floats(self.h, k.encode(), len(v), arr))
        for k, v in (f or {}).items():
            self._check(L.mbh_op_arg_float(self.h, k.encode(), float(v)))
        for k, v in (s or {}).items():
            self._check(L.mbh_op_arg_str(self.h, k.encode(), v.encode()))
        self._check(L.mbh_op_end(self.h))

    def run(self, sync=True):
        self._check(lib().mbh_run(self.h))
        if sync:
            self.sync()

    def sync(self):
        self._check(lib().mbh_sync(self.h))

    def fuse_activations(self):
        """Merge Activation operators into the Eltwise that feeds them; returns how many."""
        n = _int()
        self._check(lib().mbh_fuse_activations(self.h, C.byref(n)))
        return n.value

    def fuse_residual_sums(self):
        """After one run and fuse_activations(): merge residual sums into the 1x1 convolutions
        that feed them; returns how many."""
        n = _int()
        self._check(lib().mbh_fuse_residual_sums(self.h, C.byref(n)))
        return n.value

    def share_subsampled_inputs(self):
        """One gather for the strided 1x1 convolutions that read the same tensor; returns the
        number of shared gathers.  Call before the first run."""
        n = _int()
        self._check(lib().mbh_share_subsampled_inputs(self.h, C.byref(n)))
        return n.value

    def plan_memory(self):
        """Share activation memory between tensors with disjoint lifetimes (after one run);
        returns (bytes before, bytes after)."""
        a, b = _sz(), _sz()
        self._check(lib().mbh_plan_memory(self.h, C.byref(a), C.byref(b)))
        return a.value, b.value

    def capture(self):
        """Record the chain into a CUDA graph (after one plain run); later runs replay it."""
        self._check(lib().mbh_capture(self.h))

    def run_host(self, input_name, host_in, output_name, host_out):
        self._check(lib().mbh_run_host(self.h, input_name.encode(), host_in.ctypes.data,
                                       host_in.nbytes, output_name.encode(),
                                       host_out.ctypes.data, host_out.nbytes))

    def run_host_pipelined(self, input_name, host_in, output_name, host_out):
        """Enqueue upload + run + download without waiting (pinned host arrays); returns the slot
        to pass to wait_slot().  The upload overlaps the previous call's run."""
        slot = _int()
        self._check(lib().mbh_run_host_pipelined(self.h, input_name.encode(), host_in.ctypes.data,
                                                 host_in.nbytes, output_name.encode(),
                                                 host_out.ctypes.data, host_out.nbytes, C.byref(slot)))
        return slot.value

    def wait_slot(self, slot):
        self._check(lib().mbh_wait_slot(self.h, int(slot)))

    def run_profiled(self, max_ops=256):
        ms = (C.c_float * max_ops)()
        names = C.create_string_buffer(64 * max_ops)
        n = _int()
        self._check(lib().mbh_run_profiled(self.h, ms, max_ops, names, len(names), C.byref(n)))
        labels = names.value.decode().strip().split("\n")
        return [(labels[k], float(ms[k])) for k in range(min(n.value, max_ops))]

    def run_profiled_graph(self, replays=5, max_ops=256):
        """Per-operator device times inside a graph replay (event nodes between the operators of
        a recorded graph): [(type:name, ms)], adding up to the graph's duration."""
        ms = (C.c_float * max_ops)()
        names = C.create_string_buffer(64 * max_ops)
        n = _int()
        self._check(lib().mbh_run_profiled_graph(self.h, int(replays), ms, max_ops, names, len(names), C.byref(n)))
        labels = names.value.decode().strip().split("\n")
        return [(labels[k], float(ms[k])) for k in range(min(n.value, max_ops))]
