"""Per-tensor range logging for post-training quantization (MACE_LOG_TENSOR_RANGE,
mace/core/net/serial_net.cc:185-224), per-operator RunMetadata and VLOG lines of a run, on a
small float network loaded from a model file."""
import os

import numpy as np
import pytest

from mace_b200.harness import netdef_wire as W
from mace_b200.harness import quantize_stat as qs

pytestmark = pytest.mark.gpu


def _small_float_model(rng, with_ranges):
    w = W.NetDefWriter(quantized=False, name="small_f32")
    w.add_tensor("input", shape=(1, 8, 12, 12), dtype=W.DT_FLOAT, data_format=W.DF_NCHW)
    w.add_tensor("w1", (rng.standard_normal((16, 8, 3, 3)) * 0.2).astype(np.float32), is_weight=True)
    w.add_tensor("b1", (rng.standard_normal(16) * 0.1).astype(np.float32), is_weight=True)
    w.add_tensor("w2", (rng.standard_normal((8, 16, 1, 1)) * 0.3).astype(np.float32), is_weight=True)
    q1 = [(0.1, 0, -3.0, 5.0)] if with_ranges else None
    w.op("Conv2D", "conv1", ["input", "w1", "b1"], ["c1"], T=W.DT_FLOAT, ints={"strides": [1, 1], "dilations": [1, 1]},
         i={"padding": 1}, s={"activation": "RELU"}, out_quant=q1)
    w.op("Conv2D", "conv2", ["c1", "w2"], ["c2"], T=W.DT_FLOAT, ints={"strides": [2, 2], "dilations": [1, 1]},
         i={"padding": 0})
    w.op("Pooling", "pool", ["c2"], ["p"], T=W.DT_FLOAT, ints={"kernels": [2, 2], "strides": [2, 2], "dilations": [1, 1]},
         i={"padding": 0, "pooling_type": 2})
    for name, dims in (("c1", (1, 16, 12, 12)), ("c2", (1, 8, 6, 6)), ("p", (1, 8, 3, 3))):
        w.add_output(name, dims, data_format=W.DF_NCHW)
    return w.netdef(), w.weights()


def _run(model, H, x):
    outs = {"c1": (np.zeros((x.shape[0], 16, 12, 12), np.float32), H.DF_NCHW),
            "c2": (np.zeros((x.shape[0], 8, 6, 6), np.float32), H.DF_NCHW),
            "p": (np.zeros((x.shape[0], 8, 3, 3), np.float32), H.DF_NCHW)}
    return {k: v.copy() for k, v in model.run({"input": (x, H.DF_NCHW)}, outs).items()}


def test_tensor_ranges_are_logged_and_feed_the_range_tool():
    from mace_b200 import hostapi as H
    rng = np.random.Generator(np.random.PCG64(2))
    graph, weights = _small_float_model(rng, with_ranges=False)
    xs = [rng.standard_normal((2, 8, 12, 12)).astype(np.float32) * (1 + i) for i in range(3)]
    os.environ["MACE_LOG_TENSOR_RANGE"] = "1"
    try:
        with H.Model(graph, weights, cuda_graph=True) as model, H.LogCapture() as cap:
            results = [_run(model, H, x) for x in xs]  # (a recorded graph is not replayed while logging)
    finally:
        os.environ.pop("MACE_LOG_TENSOR_RANGE")
    lines = [line for _, line in cap.lines if qs.MARK in line]
    assert len(lines) == 3 * 3
    ranges, order = qs.parse_ranges(lines)
    assert order == ["c1", "c2", "p"]
    for run, res in enumerate(results):
        for name in order:
            # the logged text is "%g"-like stream output of a float: six significant digits
            assert ranges[name][0][run] == pytest.approx(float(res[name].min()), rel=2e-5, abs=1e-6)
            assert ranges[name][1][run] == pytest.approx(float(res[name].max()), rel=2e-5, abs=1e-6)
    overall = dict(qs.overall_ranges(lines))
    assert overall["c1"][0] == 0.0 and overall["c1"][1] == pytest.approx(max(r["c1"].max() for r in results), rel=2e-5)
    scale, zp, _, _ = qs.adjust_range(overall["c2"][0], overall["c2"][1], non_zero=False)
    assert 0 < zp < 255 and scale > 0
    # switched off again: nothing is logged and the graph is used
    with H.Model(graph, weights, cuda_graph=True) as model, H.LogCapture() as cap:
        for x in xs:
            _run(model, H, x)
        assert model.captured
    assert not [line for _, line in cap.lines if qs.MARK in line]


def test_histogram_mode_with_a_quantize_info_range():
    from mace_b200 import hostapi as H
    rng = np.random.Generator(np.random.PCG64(4))
    graph, weights = _small_float_model(rng, with_ranges=True)
    x = rng.standard_normal((2, 8, 12, 12)).astype(np.float32) * 2
    os.environ["MACE_LOG_TENSOR_RANGE"] = "1"
    try:
        with H.Model(graph, weights) as model, H.LogCapture() as cap:
            res = _run(model, H, x)
    finally:
        os.environ.pop("MACE_LOG_TENSOR_RANGE")
    line = [line for _, line in cap.lines if "@@c1@@" in line][0]
    fields = line.split("@@")
    assert fields[2] == "-3,5"
    bins = np.array([int(v) for v in fields[3].strip().strip("[]").split(",")])
    assert bins.size == 2048 and bins.sum() == res["c1"].size
    bin_v = np.float32(np.float32(5.0 - (-3.0)) / np.float32(2048))
    idx = np.clip(((res["c1"].ravel() - np.float32(-3.0)) / bin_v).astype(np.int64), 0, 2047)
    assert np.array_equal(bins, np.bincount(idx, minlength=2048))


def test_histogram_entry_point_against_numpy():
    import ctypes as C
    import mace_b200
    L = mace_b200.lib()
    ctx = mace_b200.Context(0)
    try:
        rng = np.random.Generator(np.random.PCG64(8))
        for size, lo, hi, bins in ((1000003, -2.0, 3.0, 2048), (17, 0.0, 1.0, 5), (4096, -1.0, 1.0, 8192)):
            x = rng.standard_normal(size).astype(np.float32)
            x[::97] = np.float32(hi)          # the upper edge lands in the last bin
            counts = (C.c_int32 * bins)()
            dx = ctx.upload(x)
            assert L.mb_histogram_f32(ctx.h, dx.ptr, size, lo, hi, bins, counts) == 0
            bin_v = np.float32(np.float32(hi - lo) / np.float32(bins))
            idx = np.clip(((x - np.float32(lo)) / bin_v).astype(np.int64), 0, bins - 1)
            assert np.array_equal(np.array(counts[:]), np.bincount(idx, minlength=bins))
        assert L.mb_histogram_f32(ctx.h, dx.ptr, 10, 1.0, 1.0, 16, counts) == 1
    finally:
        ctx.close()


def test_run_metadata_and_vlog_lines():
    from mace_b200 import hostapi as H
    rng = np.random.Generator(np.random.PCG64(6))
    graph, weights = _small_float_model(rng, with_ranges=False)
    x = rng.standard_normal((2, 8, 12, 12)).astype(np.float32)
    with H.Model(graph, weights) as model:
        _run(model, H, x)
        with H.LogCapture(vlog_level=3) as cap:
            stats = model.run_metadata()
    assert [s["name"] for s in stats] == ["conv1", "conv2", "pool"]
    assert [s["type"] for s in stats] == ["Conv2D", "Conv2D", "Pooling"]
    assert stats[0]["output_shape"] == [[2, 16, 12, 12]] and stats[2]["output_shape"] == [[2, 8, 3, 3]]
    assert stats[0]["strides"] == [1, 1] and stats[0]["padding_type"] == 1 and stats[0]["kernels"] == [16, 8, 3, 3]
    assert stats[1]["strides"] == [2, 2] and stats[2]["kernels"] == [2, 2]
    assert all(s["device_ms"] > 0 for s in stats)
    assert stats[0]["start_micros"] == 0 and stats[2]["end_micros"] >= stats[1]["end_micros"] >= stats[0]["end_micros"]
    text = "\n".join(line for _, line in cap.lines)
    assert "Running net started" in text and "Running net latency:" in text
    assert "Running operator conv1<CUDA, Conv2D> started" in text
    assert "Operator pool has shape: [2, 8, 3, 3]" in text
    # at the default level none of this is printed
    with H.Model(graph, weights) as model, H.LogCapture() as cap:
        _run(model, H, x)
    assert not cap.lines
