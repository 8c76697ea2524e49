"""The C++ multi-GPU runner (one engine, stream and host thread per shard; no collective): the
quantized MobileNet model file over 1 and 2 shards -- on one GPU both shards share it, with two
or more GPUs visible each shard gets its own -- against the single-engine result and the CPU
oracle, with even, ragged and too-small batches."""
import numpy as np
import pytest

from mace_b200.harness import mobilenet_v1 as mn
from mace_b200.harness import netdef_wire as W

pytestmark = pytest.mark.gpu


def _devices(n):
    import ctypes
    count = ctypes.c_int(0)
    rt = ctypes.CDLL("libcudart.so")
    assert rt.cudaGetDeviceCount(ctypes.byref(count)) == 0
    return [i % max(1, count.value) for i in range(n)]


def test_batch_sharded_over_engines_gives_the_single_engine_bytes(orc):
    from mace_b200 import hostapi as H
    image = 64
    layers = mn.build(orc, seed=0, calib_images=1, image=image)
    w = W.NetDefWriter(quantized=True, name="mobilenet_v1_u8")
    mn.build_engine(W.WriterModule(H, w), layers, 1, image=image)
    w.add_output("fc", (1, 1, 1, 1000), data_type=W.DT_UINT8)
    graph, weights = w.netdef(), w.weights()
    x = mn.random_images(7, seed=12, image=image)
    want = mn.oracle_forward(orc, layers, x)
    for n_shards in (1, 2, 3):
        with H.MultiModel(graph, weights, _devices(n_shards), plan_memory=True, cuda_graph=True) as mm:
            assert mm.shards == n_shards
            for batch in (7, 6, 1, 7):  # ragged, even, fewer images than shards, and back
                out = np.full((batch, 1, 1, 1000), 0xA5, np.uint8)
                got = mm.run({"input": (x[:batch], H.DF_NHWC)}, {"fc": (out, H.DF_NHWC)})["fc"]
                assert got.shape == (batch, 1, 1, 1000)
                assert np.array_equal(got.reshape(batch, 1000), want[:batch]), (n_shards, batch)
            # an NCHW input is still split along the batch
            out = np.zeros((4, 1, 1, 1000), np.uint8)
            got = mm.run({"input": (np.ascontiguousarray(x[:4].transpose(0, 3, 1, 2)), H.DF_NCHW)},
                         {"fc": (out, H.DF_NHWC)})["fc"]
            assert np.array_equal(got.reshape(4, 1000), want[:4])


def test_runner_reports_bad_arguments_and_a_failing_shard(orc):
    import mace_b200
    from mace_b200 import hostapi as H
    image = 64
    layers = mn.build(orc, seed=0, calib_images=1, image=image)
    w = W.NetDefWriter(quantized=True, name="mobilenet_v1_u8")
    mn.build_engine(W.WriterModule(H, w), layers, 1, image=image)
    w.add_output("fc", (1, 1, 1, 1000), data_type=W.DT_UINT8)
    with pytest.raises(mace_b200.MaceB200Error) as e:
        H.MultiModel(w.netdef(), w.weights(), [0, 4096])          # no such device
    assert "shard 1" in str(e.value)
    with pytest.raises(mace_b200.MaceB200Error):
        H.MultiModel(b"\xff\xff\xff", b"", [0])                  # not a NetDef
    x = mn.random_images(4, seed=1, image=image)
    with H.MultiModel(w.netdef(), w.weights(), [0, 0]) as mm:
        small = np.zeros((2, 1, 1, 1000), np.uint8)
        with pytest.raises(mace_b200.MaceB200Error) as e:          # the buffer holds 2 rows, the batch 4
            mm.run({"input": (x, H.DF_NHWC)}, {"fc": (small, H.DF_NHWC)})
        assert "fewer rows" in str(e.value)
        with pytest.raises(mace_b200.MaceB200Error) as e:
            mm.run({"nonsense": (x, H.DF_NHWC)}, {"fc": (np.zeros((4, 1, 1, 1000), np.uint8), H.DF_NHWC)})
        assert "shard 0" in str(e.value) and "does not belong" in str(e.value)
