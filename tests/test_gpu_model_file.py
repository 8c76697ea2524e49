"""Converted-model files on the GPU: a serialized NetDef plus weights blob, loaded and run by the
C++ MaceEngine (CreateMaceEngineFromProto / MaceEngine::Run), against the CPU oracle.  The
networks are the quantized MobileNet-v1 and the float ResNet-50 the other tests drive operator
by operator; here they travel through the model-file format and the host-buffer API, with the
NHWC <-> NCHW handling of the CPU flow.  uint8 results bit-exact, fp32 within 1e-4 of the
largest magnitude (1e-3 where Winograd convolutions are involved)."""
import numpy as np
import pytest

from mace_b200.harness import mobilenet_v1 as mn
from mace_b200.harness import netdef_wire as W
from mace_b200.harness import resnet50 as rn

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    import mace_b200
    c = mace_b200.Context(0)
    yield c
    c.close()


# ---- layout conversion kernel -------------------------------------------------------------------

@pytest.mark.parametrize("batch, rows, cols", [(1, 1, 1), (3, 49, 1000), (2, 224 * 224, 3), (5, 33, 31),
                                                 (1, 3, 50176), (4, 64, 64), (7, 1, 129), (2, 130, 1)])
@pytest.mark.parametrize("dtype", [np.uint8, np.float32])
def test_transpose2d_batched_moves_every_element(ctx, batch, rows, cols, dtype):
    rng = np.random.Generator(np.random.PCG64(batch * 1000 + rows + cols))
    x = rng.integers(0, 255, size=(batch, rows, cols)).astype(dtype)
    dx, dout = ctx.upload(x), ctx.alloc(x.nbytes)
    ctx.transpose2d_batched(dx, dout, batch, rows, cols, x.dtype.itemsize)
    got = ctx.download(dout, (batch, cols, rows), dtype)
    assert np.array_equal(got, x.transpose(0, 2, 1))


def test_transpose2d_batched_round_trip_at_full_size(ctx):
    """The input of the benchmarked networks (64 x 224 x 224 x 3 uint8, 256 x 3 x 224 x 224 fp32):
    NHWC -> NCHW -> NHWC gives the bytes back, and the middle tensor is the numpy transpose of a
    sample of images."""
    rng = np.random.Generator(np.random.PCG64(99))
    for batch, dtype in ((64, np.uint8), (256, np.float32)):
        x = rng.integers(0, 256, size=(batch, 224 * 224, 3)).astype(dtype)
        dx, dm, db = ctx.upload(x), ctx.alloc(x.nbytes), ctx.alloc(x.nbytes)
        ctx.transpose2d_batched(dx, dm, batch, 224 * 224, 3, x.dtype.itemsize)
        ctx.transpose2d_batched(dm, db, batch, 3, 224 * 224, x.dtype.itemsize)
        assert np.array_equal(ctx.download(db, x.shape, dtype), x)
        mid = ctx.download(dm, (batch, 3, 224 * 224), dtype)
        for n in (0, batch // 2, batch - 1):
            assert np.array_equal(mid[n], x[n].T)
        for b in (dx, dm, db):
            b.free()


def test_transpose2d_batched_edge_cases(ctx):
    from mace_b200 import MaceB200Error
    d = ctx.alloc(64)
    ctx.transpose2d_batched(d, d, 0, 4, 4, 4)  # nothing to do: accepted even with aliased buffers
    with pytest.raises(MaceB200Error):
        ctx.transpose2d_batched(d, d, 1, 4, 4, 4)
    with pytest.raises(MaceB200Error):
        ctx.transpose2d_batched(d, ctx.alloc(64), 1, 4, 4, 2)


# ---- shape operators through the host engine ------------------------------------------------------

def test_transpose_squeeze_reshape_ops():
    from mace_b200 import hostapi as H
    from mace_b200 import MaceB200Error
    rng = np.random.Generator(np.random.PCG64(5))
    x = rng.standard_normal((2, 5, 7, 3)).astype(np.float32)
    q = rng.integers(0, 256, size=(2, 1, 1, 10), dtype=np.uint8)
    with H.HostEngine(0) as net:
        net.add_tensor("X", x)
        net.add_tensor("Q", q, scale=0.5, zero_point=3)
        net.add_tensor("Shape", np.array([2, -1, 3], np.int32), is_weight=True)
        net.op("Transpose", "t1", ["X"], ["ToNCHW"], T=H.DT_FLOAT, ints={"dims": [0, 3, 1, 2]})
        net.op("Transpose", "t2", ["ToNCHW"], ["Back"], T=H.DT_FLOAT, ints={"dims": [0, 2, 3, 1]})
        net.op("Transpose", "t3", ["X"], ["Swap"], T=H.DT_FLOAT, ints={"dims": [0, 1, 3, 2]})
        net.op("Transpose", "t4", ["X"], ["Same"], T=H.DT_FLOAT, ints={"dims": [0, 1, 2, 3]})
        net.op("Squeeze", "s1", ["Q"], ["Squeezed"], T=H.DT_UINT8, ints={"axis": [1, 2]})
        net.op("Squeeze", "s2", ["Q"], ["SqueezedAll"], T=H.DT_UINT8)
        net.op("Reshape", "r1", ["X"], ["Flat"], T=H.DT_FLOAT, ints={"dim": [0, -1]})
        net.op("Reshape", "r2", ["X", "Shape"], ["ByTensor"], T=H.DT_FLOAT)
        net.run()
        assert np.array_equal(net.read("ToNCHW", np.float32), x.transpose(0, 3, 1, 2))
        assert np.array_equal(net.read("Back", np.float32), x)
        assert np.array_equal(net.read("Swap", np.float32), x.transpose(0, 1, 3, 2))
        assert np.array_equal(net.read("Same", np.float32), x)
        assert net.shape("Squeezed") == (2, 10) and net.shape("SqueezedAll") == (2, 10)
        assert np.array_equal(net.read("Squeezed", np.uint8), q.reshape(2, 10))
        assert net.quant("Squeezed") == (0.5, 3)
        assert net.shape("Flat") == (2, 105) and net.shape("ByTensor") == (2, 35, 3)
        assert np.array_equal(net.read("ByTensor", np.float32), x.reshape(2, 35, 3))
    with H.HostEngine(0) as net:
        net.add_tensor("X", x)
        net.op("Transpose", "t", ["X"], ["Y"], T=H.DT_FLOAT, ints={"dims": [3, 2, 1, 0]})
        with pytest.raises(MaceB200Error) as e:
            net.run()
        assert "batched 2-D transpose" in str(e.value)


# ---- whole models ----------------------------------------------------------------------------------

def _mobilenet_model(orc, image):
    from mace_b200 import hostapi
    layers = mn.build(orc, seed=0, calib_images=1, image=image)
    w = W.NetDefWriter(quantized=True, name="mobilenet_v1_u8")
    mn.build_engine(W.WriterModule(hostapi, w), layers, 1, image=image)
    w.add_output("fc", (1, 1, 1, 1000), data_type=W.DT_UINT8)
    return layers, w.netdef(), w.weights()


def test_quantized_mobilenet_model_file_is_bit_exact(orc):
    from mace_b200 import hostapi as H
    image, batch = 64, 3
    layers, graph, weights = _mobilenet_model(orc, image)
    x = mn.random_images(batch, seed=21, image=image)
    want = mn.oracle_forward(orc, layers, x)
    out = np.zeros((batch, 1, 1, 1000), np.uint8)   # the quantized FullyConnected writes [N, 1, 1, O]
    for cfg in ({}, {"plan_memory": True, "cuda_graph": True}):
        with H.Model(graph, weights, **cfg) as m:
            # the model was written for batch 1: the engine follows the input's actual shape
            got = m.run({"input": (x, H.DF_NHWC)}, {"fc": (out, H.DF_NHWC)})["fc"]
            assert got.shape == (batch, 1, 1, 1000) and np.array_equal(got.reshape(want.shape), want)
            # a quantized model runs NHWC: an NCHW input is transposed on the way in
            got = m.run({"input": (x.transpose(0, 3, 1, 2), H.DF_NCHW)}, {"fc": (out, H.DF_NHWC)})["fc"]
            assert np.array_equal(got.reshape(want.shape), want)
            for _ in range(2):
                got = m.run({"input": (x, H.DF_NHWC)}, {"fc": (out, H.DF_NHWC)})["fc"]
                assert np.array_equal(got.reshape(want.shape), want)
            assert m.captured == bool(cfg.get("cuda_graph"))
            # another batch size drops the recording and still gives the oracle's bytes
            got = m.run({"input": (x[:2], H.DF_NHWC)}, {"fc": (out, H.DF_NHWC)})["fc"]
            assert got.shape == (2, 1, 1, 1000) and np.array_equal(got.reshape(2, 1000), want[:2])


def test_full_size_mobilenet_model_file_equals_the_operator_chain(orc):
    """224 x 224 at batch 8: the model-file path must give the bytes of the operator-by-operator
    engine (which test_gpu_mobilenet.py holds against the oracle at this size)."""
    from mace_b200 import hostapi as H
    batch = 8
    layers, graph, weights = _mobilenet_model(orc, 224)
    x = mn.random_images(batch, seed=5)
    eng = mn.build_engine(H, layers, batch)
    try:
        eng.write("input", x)
        eng.run()
        want = eng.read("fc", np.uint8).reshape(batch, 1000)
    finally:
        eng.close()
    out = np.zeros((batch, 1, 1, 1000), np.uint8)
    with H.Model(graph, weights, plan_memory=True, cuda_graph=True) as m:
        for _ in range(3):
            got = m.run({"input": (x, H.DF_NHWC)}, {"fc": (out, H.DF_NHWC)})["fc"]
            assert np.array_equal(got.reshape(batch, 1000), want)
        assert m.captured
    assert len(np.unique(want)) > 50


def _resnet_model(image, width_div, tail=True):
    from mace_b200 import hostapi
    nodes, weights = rn.build(seed=0, image=image, width_div=width_div)
    w = W.NetDefWriter(quantized=False, name="resnet50_f32")
    # the model file states the input the way a converter does: NHWC, to be run NCHW
    w.add_tensor("input", shape=(1, image, image, 3), dtype=W.DT_FLOAT, data_format=W.DF_NHWC)
    recorder = W.WriterModule(hostapi, w)
    real_add = w.add_tensor
    w.add_tensor = lambda name, *a, **k: None if name == "input" else real_add(name, *a, **k)
    rn.build_engine(recorder, nodes, weights, 1, image=image)
    w.add_tensor = real_add
    if tail:
        w.op("Squeeze", "squeeze", ["fc"], ["logits"], T=W.DT_FLOAT, ints={"axis": [1, 2]}, i={"has_data_format": 1})
        w.op("Softmax", "softmax", ["logits"], ["prob"], T=W.DT_FLOAT)
        w.add_output("prob", (1, 1000), data_format=W.DF_NONE)
    w.add_output("fc", (1, 1, 1, 1000), data_format=W.DF_NHWC)
    w.add_output("conv1", (1, image // 2, image // 2, 64 // width_div), data_format=W.DF_NHWC)
    return nodes, weights, w.netdef(), w.weights()


def _softmax(z):
    z = z.astype(np.float64)
    e = np.exp(z - z.max(1, keepdims=True))
    return e / e.sum(1, keepdims=True)


def test_float_resnet_model_file_nhwc_in_and_out(orc):
    from mace_b200 import hostapi as H
    image, width_div, batch = 64, 4, 2
    nodes, weights, graph, blob = _resnet_model(image, width_div)
    x = rn.random_images(batch, 3, image)                       # NCHW, what the oracle takes
    ref_logits, ref = rn.oracle_forward(orc, nodes, weights, x, keep=True)
    x_nhwc = np.ascontiguousarray(x.transpose(0, 2, 3, 1))     # what a MACE user hands over
    stem_c = 64 // width_div
    prob = np.zeros((batch, 1000), np.float32)
    fc = np.zeros((batch, 1, 1, 1000), np.float32)
    stem = np.zeros((batch, image // 2, image // 2, stem_c), np.float32)
    stem_nchw = np.zeros((batch, stem_c, image // 2, image // 2), np.float32)
    want_prob = _softmax(ref_logits.reshape(batch, 1000))
    with H.Model(graph, blob) as m:
        got = m.run({"input": (x_nhwc, H.DF_NHWC)},
                    {"prob": (prob, H.DF_NONE), "fc": (fc, H.DF_NHWC), "conv1": (stem, H.DF_NHWC)})
        scale = np.abs(ref_logits).max()
        assert got["fc"].shape == (batch, 1, 1, 1000)
        assert np.abs(got["fc"].reshape(batch, 1000) - ref_logits.reshape(batch, 1000)).max() <= 1e-3 * scale
        assert got["prob"].shape == (batch, 1000)
        assert np.abs(got["prob"] - want_prob).max() <= 1e-4
        # a 4-D output comes back in the layout the caller names: NHWC here, NCHW below
        want_stem = ref["conv1"]
        assert got["conv1"].shape == (batch, image // 2, image // 2, stem_c)
        assert np.abs(got["conv1"].transpose(0, 3, 1, 2) - want_stem).max() <= 1e-4 * np.abs(want_stem).max()
        plain_fc = got["fc"].copy()
        got = m.run({"input": (x, H.DF_NCHW)}, {"conv1": (stem_nchw, H.DF_NCHW)})
        assert got["conv1"].shape == want_stem.shape
        assert np.array_equal(got["conv1"], stem.transpose(0, 3, 1, 2))
    # merged residual sums, shared activation memory and graph replay: the same logits
    with H.Model(graph, blob, fuse=True, plan_memory=True, cuda_graph=True) as m:
        for k in range(4):
            got = m.run({"input": (x_nhwc, H.DF_NHWC)}, {"fc": (fc, H.DF_NHWC), "prob": (prob, H.DF_NONE)})
            assert np.abs(got["fc"] - plain_fc).max() <= 1e-4 * scale, k
            assert np.abs(got["prob"] - want_prob).max() <= 1e-4
        assert m.captured


def test_model_with_half_and_compressed_weights(orc):
    """DT_HALF weights are widened and uint8-compressed weights of a float model dequantized when
    the file is loaded (mace/core/workspace.cc:147-169): the convolution sees floats."""
    from mace_b200 import hostapi as H
    rng = np.random.Generator(np.random.PCG64(9))
    filt = (rng.standard_normal((8, 4, 3, 3)) * 0.2).astype(np.float16)           # OIHW
    q = rng.integers(0, 256, size=(8, 8, 1, 1), dtype=np.uint8)
    scale, zp = np.float32(0.004), 131
    bias = rng.standard_normal(8).astype(np.float32)
    x = rng.standard_normal((2, 4, 9, 11)).astype(np.float32)
    w = W.NetDefWriter(name="mixed")
    w.add_tensor("input", shape=(2, 4, 9, 11), dtype=W.DT_FLOAT, data_format=W.DF_NCHW)
    w.add_tensor("f1", filt)
    w.add_tensor("f2", q, scale=float(scale), zero_point=zp)
    w.net["tensors"][-1]["quantized"] = True
    w.add_tensor("b", bias)
    w.op("Conv2D", "c1", ["input", "f1", "b"], ["c1"], T=W.DT_FLOAT, ints={"strides": [1, 1], "dilations": [1, 1]},
         i={"padding": H.SAME}, s={"activation": "RELU"})
    w.op("Conv2D", "c2", ["c1", "f2"], ["c2"], T=W.DT_FLOAT, ints={"strides": [1, 1], "dilations": [1, 1]},
         i={"padding": H.VALID})
    w.add_output("c2", (2, 8, 9, 11), data_format=W.DF_NCHW)
    f1 = filt.astype(np.float32)
    f2 = (scale * (q.astype(np.int32) - zp).astype(np.float32)).astype(np.float32)
    ho, wo, ph, pw = orc.calc_padding_and_output_size(9, 11, 3, 3, (1, 1), (1, 1), 1)
    mid = orc.conv2d_f32(x, f1, bias, (1, 1), (1, 1), (ph >> 1, pw >> 1), (ho, wo), act=1)
    want = orc.conv2d_f32(mid, f2, np.zeros(8, np.float32), (1, 1), (1, 1), (0, 0), (9, 11))
    out = np.zeros((2, 8, 9, 11), np.float32)
    with H.Model(w.netdef(), w.weights()) as m:
        got = m.run({"input": (x, H.DF_NCHW)}, {"c2": (out, H.DF_NCHW)})["c2"]
    assert np.abs(got - want).max() <= 1e-4 * np.abs(want).max()


def test_float_in_float_out_quantized_model(orc):
    """Quantize -> uint8 Conv2D -> Dequantize: float host buffers on both sides of a quantized
    model; the NCHW output the caller asks for is produced from the NHWC tensor."""
    from mace_b200 import hostapi as H
    rng = np.random.Generator(np.random.PCG64(13))
    x = rng.uniform(-1, 1, size=(2, 10, 12, 8)).astype(np.float32)
    filt = rng.integers(0, 256, size=(16, 3, 3, 8), dtype=np.uint8)   # OHWI
    s_in, zp_in, s_f, zp_f, s_out, zp_out = 1 / 127.5, 128, 0.01, 127, 0.05, 120
    bias = rng.integers(-2000, 2000, size=16).astype(np.int32)
    w = W.NetDefWriter(quantized=True, name="qdq")
    w.add_tensor("input", shape=(2, 10, 12, 8), dtype=W.DT_FLOAT)
    w.add_tensor("f", filt, scale=s_f, zero_point=zp_f)
    w.add_tensor("b", bias, scale=s_in * s_f, zero_point=0)
    w.op("Quantize", "q", ["input"], ["xq"], T=W.DT_UINT8, out_dtype=W.DT_UINT8, out_quant=[(s_in, zp_in)])
    w.op("Conv2D", "conv", ["xq", "f", "b"], ["yq"], T=W.DT_UINT8, out_quant=[(s_out, zp_out)],
         ints={"strides": [1, 1], "dilations": [1, 1]}, i={"padding": H.SAME})
    w.op("Dequantize", "dq", ["yq"], ["y"], T=W.DT_UINT8, out_dtype=W.DT_FLOAT)
    w.add_output("y", (2, 10, 12, 16))
    xq = orc.quantize(x, s_in, zp_in)
    ho, wo, ph, pw = orc.calc_padding_and_output_size(10, 12, 3, 3, (1, 1), (1, 1), 1)
    mult, shift = orc.output_multiplier_and_shift(s_f, s_in, s_out)
    yq = orc.conv2d_u8(xq, filt, bias, (1, 1), (ph, pw), (ho, wo), zp_in, zp_f, mult, shift, zp_out)
    want = orc.dequantize(yq, s_out, zp_out)
    out = np.zeros((2, 16, 10, 12), np.float32)
    with H.Model(w.netdef(), w.weights()) as m:
        got = m.run({"input": (x, H.DF_NHWC)}, {"y": (out, H.DF_NCHW)})["y"]
    assert got.shape == (2, 16, 10, 12)
    assert np.array_equal(got, want.transpose(0, 3, 1, 2))


def test_two_inputs_in_different_layouts():
    """Each input is transposed (or not) by its own MaceTensor's layout; 2-D tensors never are."""
    from mace_b200 import hostapi as H
    rng = np.random.Generator(np.random.PCG64(17))
    a = rng.standard_normal((2, 5, 6, 3)).astype(np.float32)      # NHWC
    b = rng.standard_normal((2, 5, 6, 3)).astype(np.float32)
    v = rng.standard_normal((4, 9)).astype(np.float32)
    w = W.NetDefWriter(name="two_inputs")
    w.add_tensor("a", shape=a.shape, dtype=W.DT_FLOAT)
    w.add_tensor("b", shape=b.shape, dtype=W.DT_FLOAT)
    w.add_tensor("v", shape=v.shape, dtype=W.DT_FLOAT, data_format=W.DF_NONE)
    w.op("Eltwise", "sum", ["a", "b"], ["s"], T=W.DT_FLOAT, i={"type": 0})
    w.op("Eltwise", "prod", ["s", "a"], ["p"], T=W.DT_FLOAT, i={"type": 2})
    w.op("Activation", "relu", ["v"], ["r"], T=W.DT_FLOAT, s={"activation": "RELU"})
    w.add_output("p", a.shape)
    w.add_output("r", v.shape, data_format=W.DF_NONE)
    out = np.zeros(a.shape, np.float32)
    r = np.zeros(v.shape, np.float32)
    with H.Model(w.netdef(), b"") as m:
        got = m.run({"a": (a, H.DF_NHWC), "b": (b.transpose(0, 3, 1, 2), H.DF_NCHW), "v": (v, H.DF_NONE)},
                    {"p": (out, H.DF_NHWC), "r": (r, H.DF_NHWC)})
        assert np.array_equal(got["p"], (a + b) * a)
        assert np.array_equal(got["r"], np.maximum(v, 0))


def test_model_errors():
    from mace_b200 import hostapi as H
    from mace_b200 import MaceB200Error
    w = W.NetDefWriter(name="bad")
    w.add_tensor("input", shape=(1, 4, 4, 2), dtype=W.DT_FLOAT)
    w.op("NoSuchOp", "mystery", ["input"], ["out"], T=W.DT_FLOAT)
    with pytest.raises(MaceB200Error) as e:
        H.Model(w.netdef(), b"")
    assert "NoSuchOp" in str(e.value) and "mystery" in str(e.value)
    # a tensor that reaches past the end of the weights blob
    w = W.NetDefWriter(name="short")
    w.add_tensor("input", shape=(1, 4, 4, 2), dtype=W.DT_FLOAT)
    w.add_tensor("f", np.zeros((2, 2, 1, 1), np.float32))
    with pytest.raises(MaceB200Error) as e:
        H.Model(w.netdef(), w.weights()[:-4])
    assert "tensor_end" in str(e.value)
    with pytest.raises(MaceB200Error) as e:
        H.Model(b"\x0a\x05ab", b"")
    assert "malformed NetDef" in str(e.value)
    # run-time argument errors leave the engine usable
    w = W.NetDefWriter(name="relu")
    w.add_tensor("input", shape=(1, 2, 2, 3), dtype=W.DT_FLOAT)
    w.op("Activation", "relu", ["input"], ["out"], T=W.DT_FLOAT, s={"activation": "RELU"})
    w.add_output("out", (1, 2, 2, 3))
    x = np.arange(-6, 6, dtype=np.float32).reshape(1, 2, 2, 3)
    out = np.zeros((1, 2, 2, 3), np.float32)
    with H.Model(w.netdef(), b"") as m:
        with pytest.raises(MaceB200Error) as e:
            m.run({"nope": (x, H.DF_NHWC)}, {"out": (out, H.DF_NHWC)})
        assert "does not belong to model's inputs" in str(e.value)
        with pytest.raises(MaceB200Error) as e:
            m.run({"input": (x, H.DF_NHWC)}, {"input": (out, H.DF_NHWC)})
        assert "does not belong to model's outputs" in str(e.value)
        with pytest.raises(MaceB200Error) as e:
            m.run({"input": (x, H.DF_NHWC)}, {"out": (np.zeros(5, np.float32), H.DF_NONE)})
        assert "exceeds buffer size" in str(e.value)
        with pytest.raises(MaceB200Error) as e:
            m.run({"input": (x.astype(np.uint8), H.DF_NHWC)}, {"out": (out, H.DF_NHWC)})
        assert "data type" in str(e.value)
        got = m.run({"input": (x, H.DF_NHWC)}, {"out": (out, H.DF_NHWC)})["out"]
        assert np.array_equal(got, np.maximum(x, 0))
