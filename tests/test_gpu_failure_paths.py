"""Failure paths on the GPU, without a GPU fault: a bounded device wait that runs out (a barrier
nobody arrives at, a short budget; the kernel returns normally with a status word), allocator
failures injected on the host (MACE_RUNTIME_FAILURE_RATIO, mace/core/runtime_failure_mock.cc:25)
travelling out of SerialNet::Run and MaceEngine::Run as MACE_OUT_OF_RESOURCES, and recovery
afterwards on the same context."""
import ctypes as C

import numpy as np
import pytest

from helpers import gemm_case
from mace_b200.harness import mobilenet_v1 as mn
from mace_b200.harness import netdef_wire as W

pytestmark = pytest.mark.gpu


def test_a_bounded_wait_that_runs_out_is_reported_and_the_context_survives(orc):
    import mace_b200
    L = mace_b200.lib()
    ctx = mace_b200.Context(0)
    try:
        waited = C.c_longlong(0)
        budget = 200000  # SM clocks: about 0.1 ms
        assert L.mb_wait_timeout_selftest(ctx.h, budget, C.byref(waited)) == 0
        assert budget <= waited.value < 100 * budget, waited.value
        with pytest.raises(mace_b200.MaceB200Error) as e:
            ctx.sync()
        assert e.value.code == 4                      # MACE_RUNTIME_ERROR
        assert "gave up a bounded wait" in str(e.value) and "status 1" in str(e.value)
        ctx.sync()                                    # the word was cleared: the next sync is clean
        # the context still computes: a tensor-core GEMM (whose own waits use the same helper)
        M, N, K = 256, 256, 512
        case = gemm_case(orc, 3, 1, M, N, K, bias_len=N)
        A, B, bias, out = ctx.upload(case["A"]), ctx.upload(case["B"]), ctx.upload(case["bias"]), ctx.alloc(M * N)
        before = ctx.launches_tensor_core
        ctx.gemm_u8(A, B, bias, out, 1, M, N, K, case["zp_a"], case["zp_b"], case["mult"], case["shift"], case["zp_c"])
        got = ctx.download(out, (M * N,), np.uint8)
        ctx.sync()
        assert ctx.launches_tensor_core == before + 1
        exp = orc.gemm_u8(case["A"], case["B"], case["bias"], 1, M, N, K, case["zp_a"], case["zp_b"],
                          case["mult"], case["shift"], case["zp_c"])
        assert np.array_equal(got, exp)
        # arguments outside the allowed budget are refused before anything is launched
        assert L.mb_wait_timeout_selftest(ctx.h, 0, None) == 1
        assert L.mb_wait_timeout_selftest(ctx.h, 1 << 40, None) == 1
        # without the host buffer the call does not wait; the report still comes at the sync
        assert L.mb_wait_timeout_selftest(ctx.h, 50000, None) == 0
        with pytest.raises(mace_b200.MaceB200Error):
            ctx.sync()
        ctx.sync()
    finally:
        ctx.close()


def test_allocator_failures_come_out_of_the_net_and_the_engine_recovers(orc):
    import mace_b200
    from mace_b200 import hostapi as H
    L = mace_b200.lib()
    rng = np.random.Generator(np.random.PCG64(9))
    x = rng.integers(0, 256, size=(2, 8, 8, 16), dtype=np.uint8)
    f = rng.integers(1, 256, size=(32, 1, 1, 16), dtype=np.uint8)
    mult_scale = 0.02 * 0.01 * 4 * 74 * 74 * 3 / 127
    try:
        with H.HostEngine(0) as net:
            net.add_tensor("X", x, scale=0.02, zero_point=128)
            net.add_tensor("F", f, scale=0.01, zero_point=120, is_weight=True)
            net.op("Conv2D", "pw", ["X", "F"], ["Y"], T=H.DT_UINT8, ints={"strides": [1, 1], "dilations": [1, 1]},
                   i={"padding": H.VALID}, out_quant=[(mult_scale, 100)])
            # every allocation fails: the operator's output cannot be resized, and the code comes
            # out of SerialNet::Run
            assert L.mb_set_runtime_failure_ratio(1.0) == 0
            with pytest.raises(mace_b200.MaceB200Error) as e:
                net.run()
            assert e.value.code == 2 and "mock runtime failure" in str(e.value)   # MACE_OUT_OF_RESOURCES
            with pytest.raises(mace_b200.MaceB200Error) as e:
                net.add_tensor("Z", x)
            assert e.value.code == 2
            # the caller's retry (mace_run re-creates the engine, mace/tools/mace_run.cc:552-595;
            # here the same engine simply runs again) succeeds once allocations do
            assert L.mb_set_runtime_failure_ratio(0.0) == 0
            net.run()
            m, sh = orc.output_multiplier_and_shift(np.float32(0.02), np.float32(0.01), np.float32(mult_scale))
            want = orc.conv2d_u8(x, f, None, (1, 1), (0, 0), (8, 8), 128, 120, m, sh, 100)
            assert np.array_equal(net.read("Y", np.uint8), want)
        # the model-level API: creation fails while allocations fail, works afterwards
        layers = mn.build(orc, seed=0, calib_images=1, image=64)
        w = W.NetDefWriter(quantized=True, name="mobilenet_v1_u8")
        mn.build_engine(W.WriterModule(H, w), layers, 1, image=64)
        w.add_output("fc", (1, 1, 1, 1000), data_type=W.DT_UINT8)
        L.mb_set_runtime_failure_ratio(1.0)
        with pytest.raises(mace_b200.MaceB200Error) as e:
            H.Model(w.netdef(), w.weights())
        assert e.value.code == 2
        L.mb_set_runtime_failure_ratio(0.0)
        xin = mn.random_images(2, seed=4, image=64)
        out = np.zeros((2, 1, 1, 1000), np.uint8)
        with H.Model(w.netdef(), w.weights()) as model:
            L.mb_set_runtime_failure_ratio(1.0)
            with pytest.raises(mace_b200.MaceB200Error) as e:   # MaceEngine::Run: the input is resized to batch 2
                model.run({"input": (xin, H.DF_NHWC)}, {"fc": (out, H.DF_NHWC)})
            assert e.value.code == 2
            L.mb_set_runtime_failure_ratio(0.0)
            got = model.run({"input": (xin, H.DF_NHWC)}, {"fc": (out, H.DF_NHWC)})["fc"]
            assert np.array_equal(got.reshape(2, 1000), mn.oracle_forward(orc, layers, xin))
    finally:
        L.mb_set_runtime_failure_ratio(0.0)
