"""Quantized MobileNet-v1 (224x224, uint8 NHWC, random weights) through the C++ host
engine on the GPU against the CPU oracle chain: every layer's activation and the final
uint8 logits must be bit-exact."""
import numpy as np
import pytest

from mace_b200.harness import mobilenet_v1 as mn

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def layers(orc):
    return mn.build(orc, seed=0)


def test_mobilenet_chain_every_layer(orc, layers):
    from mace_b200 import hostapi
    batch = 3
    x = mn.random_images(batch, seed=11)
    exp_logits, exp_acts = mn.oracle_forward(orc, layers, x, keep=True)
    eng = mn.build_engine(hostapi, layers, batch)
    try:
        eng.write("input", x)
        eng.run()
        for L, exp in zip(layers, exp_acts):
            got = eng.read(L["name"], np.uint8)
            assert np.array_equal(got.reshape(exp.shape), exp), "layer %s differs" % L["name"]
        assert len(np.unique(exp_logits)) > 50
        # a linear chain needs two activation buffers (plus the logits, which nobody reads):
        # planned memory is the two largest consecutive activations, and the logits stay exact
        separate, shared = eng.plan_memory()
        assert shared < separate / 2, (separate, shared)
        eng.write("input", x)
        eng.run()
        assert np.array_equal(eng.read("fc", np.uint8).reshape(exp_logits.shape), exp_logits)
        eng.capture()
        eng.run()
        assert np.array_equal(eng.read("fc", np.uint8).reshape(exp_logits.shape), exp_logits)
    finally:
        eng.close()


def test_mobilenet_layers_in_isolation_full_range(orc, layers):
    """Each layer alone on fresh uniform [0, 255] input, so that late layers see
    full-range data (chained activations are ReLU6-skewed)."""
    from mace_b200 import hostapi
    rng = np.random.Generator(np.random.PCG64(77))
    sizes = {"stem": 224}
    h, c = 112, 32
    for L in layers:
        if L["kind"] not in ("conv", "dw"):
            continue
        if L["name"] == "stem":
            hin, cin = 224, 3
        else:
            hin, cin = h, c
        x = rng.integers(0, 256, size=(2, hin, hin, cin), dtype=np.uint8)
        eng = hostapi.HostEngine(0)
        try:
            eng.add_tensor("in", x, scale=L["s_in"], zero_point=0)
            eng.add_tensor("w", L["w"], scale=L["s_f"], zero_point=L["zp_f"], is_weight=True)
            eng.add_tensor("b", L["bias"], scale=L["bias_scale"], zero_point=0, is_weight=True)
            optype = "Conv2D" if L["kind"] == "conv" else "DepthwiseConv2d"
            eng.op(optype, L["name"], ["in", "w", "b"], ["out"],
                   out_quant=[(L["s_out"], L["zp_out"])],
                   ints={"strides": [L["stride"]] * 2, "dilations": [1, 1]},
                   i={"padding": hostapi.SAME})
            eng.run()
            got = eng.read("out", np.uint8)
        finally:
            eng.close()
        one = [dict(L)]
        exp = mn.oracle_forward(orc, one, x)
        assert np.array_equal(got, exp), "layer %s differs" % L["name"]
        if L["name"] != "stem":
            h, c = exp.shape[1], exp.shape[3]


def eng_launches(eng):
    import ctypes
    import mace_b200
    return int(mace_b200.lib().mb_launch_count(ctypes.c_void_p(eng.context)))


def test_mobilenet_batch64_logits_and_host_buffers(orc, layers):
    """The benchmark configuration: batch 64, through the host-buffer entry point
    (H2D + chain + D2H), logits bit-exact against the oracle."""
    from mace_b200 import hostapi
    batch = 64
    x = mn.random_images(batch, seed=0)
    exp = mn.oracle_forward(orc, layers, x)
    eng = mn.build_engine(hostapi, layers, batch)
    try:
        out = np.empty((batch, 1, 1, mn.NUM_CLASSES), np.uint8)
        eng.run_host("input", x, "fc", out)
        assert np.array_equal(out.reshape(batch, -1), exp)
        # idempotence: a second run on the same input gives the same bytes
        out2 = np.empty_like(out)
        eng.run_host("input", x, "fc", out2)
        assert np.array_equal(out, out2)
        prof = eng.run_profiled()
        assert len(prof) == len(layers)
        # the same chain replayed from a CUDA graph, on a different input
        x2 = mn.random_images(batch, seed=5)
        exp2 = mn.oracle_forward(orc, layers, x2)
        eng.capture()
        launches_before = eng_launches(eng)
        eng.run_host("input", x2, "fc", out2)
        assert np.array_equal(out2.reshape(batch, -1), exp2)
        assert eng_launches(eng) - launches_before >= len(layers)  # replay counts its kernels
        eng.run_host("input", x, "fc", out2)
        assert np.array_equal(out2, out)
    finally:
        eng.close()


@pytest.mark.parametrize("captured", [True, False])
def test_mobilenet_pipelined_uploads_do_not_overtake_the_stem(orc, layers, captured):
    """The pipelined entry point uploads call i + 1's images straight into the input tensor as soon
    as call i's net has passed the operator that reads it.  Batch 32 from pinned buffers, twelve
    calls back to back with alternating, very different inputs (all black / random): had an
    upload started before the stem of the call in front had read its images, that call's logits
    would be those of the wrong input.  Replayed from the (split) graph and operator by operator."""
    import ctypes
    import mace_b200
    from mace_b200 import hostapi
    batch = 32
    xs = [mn.random_images(batch, seed=40), np.zeros_like(mn.random_images(batch, seed=40)),
          mn.random_images(batch, seed=41)]
    exps = [mn.oracle_forward(orc, layers, x) for x in xs]
    assert not np.array_equal(exps[0], exps[1]) and not np.array_equal(exps[0], exps[2])
    eng = mn.build_engine(hostapi, layers, batch)
    try:
        L = mace_b200.lib()
        ctx = ctypes.c_void_p(eng.context)

        def pinned(nbytes):
            p = ctypes.c_void_p()
            assert L.mb_host_alloc(ctx, int(nbytes), ctypes.byref(p)) == 0
            return np.ctypeslib.as_array((ctypes.c_uint8 * int(nbytes)).from_address(p.value))

        hin = [pinned(x.nbytes) for x in xs]
        for h, x in zip(hin, xs):
            h[:] = x.ravel()
        houts = [pinned(batch * mn.NUM_CLASSES) for _ in range(2)]
        eng.write("input", xs[0])
        eng.run()
        if captured:
            eng.capture()
        order = [0, 1, 2, 1, 0, 2, 1, 1, 0, 2, 0, 1]
        prev = None
        for i, k in enumerate(order):
            slot = eng.run_host_pipelined("input", hin[k], "fc", houts[i & 1])
            if prev is not None:
                eng.wait_slot(prev[0])
                assert np.array_equal(houts[prev[1]].reshape(batch, -1), exps[prev[2]]), "call %d" % (i - 1)
            prev = (slot, i & 1, k)
        eng.wait_slot(prev[0])
        assert np.array_equal(houts[prev[1]].reshape(batch, -1), exps[prev[2]])
        eng.sync()
        # a plain run after the pipelined ones, then pipelined again
        out = np.empty((batch, mn.NUM_CLASSES), np.uint8)
        eng.run_host("input", xs[2], "fc", out)
        assert np.array_equal(out, exps[2])
        slot = eng.run_host_pipelined("input", hin[0], "fc", houts[0])
        eng.wait_slot(slot)
        assert np.array_equal(houts[0].reshape(batch, -1), exps[0])
    finally:
        eng.close()


def test_mobilenet_pipelined_host_runs(orc, layers):
    """mbh_run_host_pipelined: every call's logits, read after wait_slot, are those of ITS input
    (pageable host arrays here; the upload goes straight into the input tensor once the previous
    call's stem has read it)."""
    from mace_b200 import hostapi
    batch = 4
    xs = [mn.random_images(batch, seed=20 + i) for i in range(6)]
    exps = [mn.oracle_forward(orc, layers, x) for x in xs]
    eng = mn.build_engine(hostapi, layers, batch)
    try:
        eng.write("input", xs[0])
        eng.run()
        eng.capture()
        outs = [np.zeros((batch, mn.NUM_CLASSES), np.uint8) for _ in range(2)]
        prev = None
        for i, x in enumerate(xs):
            slot = eng.run_host_pipelined("input", x, "fc", outs[i & 1])
            if prev is not None:
                eng.wait_slot(prev[0])
                assert np.array_equal(outs[prev[1]], exps[prev[2]]), "call %d" % prev[2]
            prev = (slot, i & 1, i)
        eng.wait_slot(prev[0])
        assert np.array_equal(outs[prev[1]], exps[prev[2]])
        eng.sync()
        # the ordinary entry point still works afterwards
        out = np.empty((batch, mn.NUM_CLASSES), np.uint8)
        eng.run_host("input", xs[2], "fc", out)
        assert np.array_equal(out, exps[2])
    finally:
        eng.close()
