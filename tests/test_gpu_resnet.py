"""The float operators between the convolutions (Pooling, Eltwise, Activation, Softmax) through
the C++ host layer, and a ResNet-50-shaped graph end to end on the device against the CPU
oracle's direct fp32 convolutions.  Tolerance for the chain: 1e-3 of each activation's range
(the bound the 3x3 Winograd path is specified with); the observed error is far smaller."""
import numpy as np
import pytest

from mace_b200.harness import resnet50 as rn

pytestmark = pytest.mark.gpu


@pytest.fixture()
def net():
    from mace_b200 import hostapi
    e = hostapi.HostEngine(0)
    yield e
    e.close()


def test_pooling_op_literals(net):
    """PoolingOpTest.MAX_VALID, AVG_VALID, MAX_SAME, MAX_VALID_DILATION
    (test/ccunit/mace/ops/pooling_test.cc:27-128, 301-336) through PoolingOp<RT_CUDA,float>."""
    from mace_b200 import hostapi as H
    x = np.arange(32, dtype=np.float32).reshape(1, 2, 4, 4)
    net.add_tensor("Input", x)
    common = {"kernels": [2, 2], "strides": [2, 2], "dilations": [1, 1]}
    net.op("Pooling", "max", ["Input"], ["OutMax"], T=H.DT_FLOAT, ints=common,
           i={"padding": H.VALID, "pooling_type": H.MAX})
    net.op("Pooling", "avg", ["Input"], ["OutAvg"], T=H.DT_FLOAT, ints=common,
           i={"padding": H.VALID, "pooling_type": H.AVG})
    net.add_tensor("In3", np.arange(9, dtype=np.float32).reshape(1, 1, 3, 3))
    net.op("Pooling", "same", ["In3"], ["OutSame"], T=H.DT_FLOAT, ints=common,
           i={"padding": H.SAME, "pooling_type": H.MAX})
    net.add_tensor("In4", np.arange(16, dtype=np.float32).reshape(1, 1, 4, 4))
    net.op("Pooling", "dil", ["In4"], ["OutDil"], T=H.DT_FLOAT,
           ints={"kernels": [2, 2], "strides": [1, 1], "dilations": [2, 2]},
           i={"padding": H.VALID, "pooling_type": H.MAX})
    net.run()
    assert net.shape("OutMax") == (1, 2, 2, 2)
    assert net.read("OutMax", np.float32).ravel().tolist() == [5, 7, 13, 15, 21, 23, 29, 31]
    assert net.read("OutAvg", np.float32).ravel().tolist() == [2.5, 4.5, 10.5, 12.5, 18.5, 20.5, 26.5, 28.5]
    assert net.shape("OutSame") == (1, 1, 2, 2)
    assert net.read("OutSame", np.float32).ravel().tolist() == [4, 5, 7, 8]
    assert net.read("OutDil", np.float32).ravel().tolist() == [10, 11, 14, 15]


def test_eltwise_activation_softmax_ops(net):
    """EltwiseOpTest.CPUSimpleTensorTensor / CPUSimpleTensorScalar literals
    (test/ccunit/mace/ops/eltwise_test.cc:253-294, 476-491), SoftmaxOpTest.CPUSimple
    (softmax_test.cc:32-97) and a ReLU, through the operators of the CUDA runtime."""
    from mace_b200 import hostapi as H
    a = np.arange(1, 7, dtype=np.float32).reshape(1, 1, 2, 3)
    net.add_tensor("A", a)
    net.add_tensor("B", a.copy())
    F = H.DT_FLOAT
    net.op("Eltwise", "sum", ["A", "B"], ["Sum"], T=F, i={"type": 0})
    net.op("Eltwise", "wsum", ["A", "B"], ["WSum"], T=F, i={"type": 0}, floats={"coeff": [0.1, 0.1]})
    net.op("Eltwise", "prod", ["A", "B"], ["Prod"], T=F, i={"type": 2})
    net.op("Eltwise", "subs", ["A"], ["SubS"], T=F, i={"type": 1}, f={"scalar_input": 1.0})
    net.op("Eltwise", "rsub", ["A"], ["RSub"], T=F, i={"type": 1, "scalar_input_index": 0},
           f={"scalar_input": 1.0})
    net.op("Eltwise", "maxs", ["A"], ["MaxS"], T=F, i={"type": 5}, f={"scalar_input": 3.0})
    net.op("Eltwise", "neg", ["A"], ["Neg"], T=F, i={"type": 6})
    net.op("Activation", "relu", ["RSub"], ["Relu"], T=F, s={"activation": "RELU"})
    net.add_tensor("Logits", np.array([1, 1, 1, 1, 1, 2, 3, 4], np.float32).reshape(2, 4))
    net.op("Softmax", "sm", ["Logits"], ["Prob"], T=F)
    net.op("Softmax", "lsm", ["Logits"], ["LogProb"], T=F, i={"use_log": 1})
    net.run()
    assert net.read("Sum", np.float32).ravel().tolist() == [2, 4, 6, 8, 10, 12]
    assert np.allclose(net.read("WSum", np.float32).ravel(), [0.2, 0.4, 0.6, 0.8, 1, 1.2], atol=1e-5)
    assert net.read("Prod", np.float32).ravel().tolist() == [1, 4, 9, 16, 25, 36]
    assert net.read("SubS", np.float32).ravel().tolist() == [0, 1, 2, 3, 4, 5]
    assert net.read("RSub", np.float32).ravel().tolist() == [0, -1, -2, -3, -4, -5]
    assert net.read("MaxS", np.float32).ravel().tolist() == [3, 3, 3, 4, 5, 6]
    assert net.read("Neg", np.float32).ravel().tolist() == [-1, -2, -3, -4, -5, -6]
    assert net.read("Relu", np.float32).ravel().tolist() == [0] * 6
    assert np.allclose(net.read("Prob", np.float32).ravel(),
                       [0.25, 0.25, 0.25, 0.25, 0.0320586, 0.08714432, 0.23688282, 0.6439142], atol=1e-5)
    assert np.allclose(net.read("LogProb", np.float32).ravel(),
                       [-1.3862944] * 4 + [-3.4401896, -2.4401896, -1.4401897, -0.44018975], atol=1e-5)


def test_eltwise_rejects_what_is_not_built(net):
    from mace_b200 import hostapi as H
    net.add_tensor("A", np.ones((1, 4, 2, 2), np.float32))
    net.add_tensor("V", np.ones((1, 4, 1, 1), np.float32))
    net.op("Eltwise", "bcast", ["A", "V"], ["Out"], T=H.DT_FLOAT, i={"type": 0})
    from mace_b200 import MaceB200Error
    with pytest.raises(MaceB200Error) as e:
        net.run()
    assert "broadcast" in str(e.value)


@pytest.mark.parametrize("cfg", [
    {"batch": 2, "image": 64, "width_div": 4},     # every layer kind, small enough for the oracle
    {"batch": 3, "image": 96, "width_div": 8},     # odd batch, 3x3 convs above and below the F(6,3) limit
])
def test_resnet50_graph_against_oracle(orc, cfg):
    from mace_b200 import hostapi
    nodes, weights = rn.build(seed=0, image=cfg["image"], width_div=cfg["width_div"])
    x = rn.random_images(cfg["batch"], 1, cfg["image"])
    ref_logits, ref = rn.oracle_forward(orc, nodes, weights, x, keep=True)
    eng = rn.build_engine(hostapi, nodes, weights, cfg["batch"], image=cfg["image"])
    try:
        eng.write("input", x)
        eng.run()
        worst = 0.0
        for n in nodes:
            got = eng.read(n["name"], np.float32)
            want = ref[n["name"]]
            assert got.shape == want.shape, n["name"]
            err = float(np.abs(got.astype(np.float64) - want).max() / max(np.abs(want).max(), 1e-30))
            worst = max(worst, err)
            assert err <= 1e-3, (n["name"], err)
        assert worst <= 1e-4, worst        # what the kernels actually deliver
        assert np.array_equal(eng.read("fc", np.float32).argmax(1).ravel(), ref_logits.argmax(1).ravel())
        # a second run through a captured CUDA graph gives the same bytes
        first = eng.read("fc", np.float32)
        eng.capture()
        eng.run()
        assert np.array_equal(eng.read("fc", np.float32), first)
        # residual sums merged with their ReLUs: one merged pair per bottleneck block, the same
        # bytes in every tensor that is still written
        kept = {n["name"]: eng.read(n["name"], np.float32) for n in nodes if n["op"] != "add"}
        assert eng.fuse_activations() == sum(1 for n in nodes if n["op"] == "add") == 16
        eng.write("input", x)
        eng.run()
        for name, want in kept.items():
            assert np.array_equal(eng.read(name, np.float32), want), name
        eng.capture()
        eng.run()
        assert np.array_equal(eng.read("fc", np.float32), first)
        # residual sums merged into the 1x1 convolutions that feed them: the sum and the ReLU
        # run in the GEMM's epilogue (for the 7x7-pixel stage: one in-place pass after it)
        before = {n["name"]: eng.read(n["name"], np.float32) for n in nodes if n["op"] in ("relu", "fc", "maxpool")}
        assert eng.fuse_residual_sums() == 16
        eng.run()
        for name, want in before.items():
            got = eng.read(name, np.float32)
            assert float(np.abs(got - want).max() / max(np.abs(want).max(), 1e-30)) <= 1e-6, name
        # activation memory shared between tensors with disjoint lifetimes: same logits from
        # less than a third of the memory, also through a re-captured graph and for new inputs
        fused_logits = eng.read("fc", np.float32)
        separate, shared = eng.plan_memory()
        assert 0 < shared < separate / 3, (separate, shared)
        eng.run()
        assert np.array_equal(eng.read("fc", np.float32), fused_logits)
        eng.capture()
        x2 = rn.random_images(cfg["batch"], 7, cfg["image"])
        eng.write("input", x2)
        eng.run()
        ref2 = rn.oracle_forward(orc, nodes, weights, x2)
        got2 = eng.read("fc", np.float32)
        assert float(np.abs(got2 - ref2).max() / np.abs(ref2).max()) <= 1e-4
    finally:
        eng.close()


def test_resnet50_full_width_224_against_oracle(orc):
    """The benchmarked network itself (width_div 1, 224 x 224), batch 2: the logits, and three
    activations from different stages (the Winograd output of the first block, the stride-2
    opening of stage 3, the last block), against the oracle's direct fp32 convolutions --
    element-wise |got - ref| <= abs_err + rel_err * |ref| with rel_err 1e-3 (the chain contains
    F(6,3) Winograd convolutions) and abs_err = rel_err * rms(ref), and range-normalised 1e-3 (the
    measured values are printed);
    then the same logits from the merged, memory-planned, graph-replayed net."""
    from helpers import near_ratio
    from mace_b200 import hostapi
    batch = 2
    nodes, weights = rn.build(seed=0)
    x = rn.random_images(batch, 11)
    ref_logits, ref = rn.oracle_forward(orc, nodes, weights, x, keep=True)
    eng = rn.build_engine(hostapi, nodes, weights, batch)
    try:
        eng.write("input", x)
        eng.run()
        report = {}
        for name in ("res2a_branch2b", "res3a_branch1", "res4f", "res5c", "pool5", "fc"):
            got, want = eng.read(name, np.float32), ref[name]
            assert got.shape == want.shape, name
            ratio = near_ratio(got, want, 1e-3)
            rng_err = float(np.abs(got.astype(np.float64) - want).max() / np.abs(want).max())
            report[name] = (ratio, rng_err)
            assert ratio <= 1.0, (name, ratio)
            assert rng_err <= 1e-3, (name, rng_err)
        print("full-width ResNet-50, element-wise ratio / range-normalised error:", report)
        assert np.array_equal(eng.read("fc", np.float32).argmax(1).ravel(), ref_logits.argmax(1).ravel())
        first = eng.read("fc", np.float32)
        eng.share_subsampled_inputs()
        eng.fuse_activations()
        eng.run()
        eng.fuse_residual_sums()
        eng.run()
        eng.plan_memory()
        eng.run()
        eng.capture()
        eng.run()
        merged = eng.read("fc", np.float32)
        assert near_ratio(merged, ref_logits, 1e-3) <= 1.0
        assert float(np.abs(merged - first).max() / np.abs(first).max()) <= 1e-5
    finally:
        eng.close()


def test_strided_pointwise_convolutions_share_one_gather(orc):
    """ShareSubsampledInputs: the two stride-2 1x1 convolutions that open a ResNet stage read the
    same pixels; with the pass every tensor of the graph still matches the oracle, before and
    after the merging passes, memory planning and graph capture."""
    from mace_b200 import hostapi
    cfg = {"batch": 3, "image": 64, "width_div": 4}
    nodes, weights = rn.build(seed=0, image=cfg["image"], width_div=cfg["width_div"])
    x = rn.random_images(cfg["batch"], 2, cfg["image"])
    ref_logits, ref = rn.oracle_forward(orc, nodes, weights, x, keep=True)
    eng = rn.build_engine(hostapi, nodes, weights, cfg["batch"], image=cfg["image"])
    try:
        assert eng.share_subsampled_inputs() == 3          # res3a, res4a, res5a
        assert eng.share_subsampled_inputs() == 0          # nothing strided is left
        eng.write("input", x)
        eng.run()
        for n in nodes:
            got, want = eng.read(n["name"], np.float32), ref[n["name"]]
            assert got.shape == want.shape, n["name"]
            assert float(np.abs(got - want).max() / max(np.abs(want).max(), 1e-30)) <= 1e-4, n["name"]
        # the gathered tensor holds exactly every second pixel of the stage's input
        sub = eng.read("res2c/subsampled_2x2", np.float32)
        assert np.array_equal(sub, eng.read("res2c", np.float32)[:, :, ::2, ::2])
        assert eng.fuse_activations() == 16 and eng.fuse_residual_sums() == 16
        eng.run()
        eng.plan_memory()
        eng.run()
        eng.capture()
        eng.run()
        got = eng.read("fc", np.float32)
        assert float(np.abs(got - ref_logits).max() / np.abs(ref_logits).max()) <= 1e-4
    finally:
        eng.close()


def test_subsample_kernel_and_its_limits():
    import mace_b200
    ctx = mace_b200.Context(0)
    try:
        rng = np.random.Generator(np.random.PCG64(3))
        for planes, H, W, sh, sw in [(6, 56, 56, 2, 2), (5, 7, 9, 2, 3), (3, 1, 1, 2, 2), (2, 13, 4, 1, 2), (4, 8, 8, 3, 1)]:
            x = rng.standard_normal((planes, H, W)).astype(np.float32)
            want = x[:, ::sh, ::sw]
            dx, do = ctx.upload(x), ctx.alloc(want.size * 4)
            ctx.subsample_f32(dx, do, planes, H, W, (sh, sw))
            assert np.array_equal(ctx.download(do, want.shape, np.float32), want)
        with pytest.raises(mace_b200.MaceB200Error):
            ctx.subsample_f32(dx, do, 1, 4, 4, (0, 1))
        with pytest.raises(mace_b200.MaceB200Error):
            ctx.subsample_f32(dx, dx, 1, 4, 4, (2, 2))
    finally:
        ctx.close()


def test_a_single_strided_convolution_or_a_padded_one_is_left_alone(net):
    from mace_b200 import hostapi as H
    rng = np.random.Generator(np.random.PCG64(4))
    F = H.DT_FLOAT
    net.add_tensor("X", rng.standard_normal((1, 8, 10, 10)).astype(np.float32))
    net.add_tensor("Y", rng.standard_normal((1, 8, 10, 10)).astype(np.float32))
    for name in ("w1", "w2", "w3", "w4"):
        net.add_tensor(name, rng.standard_normal((8, 8, 1, 1)).astype(np.float32), is_weight=True)
    net.add_tensor("w5", rng.standard_normal((8, 8, 3, 3)).astype(np.float32), is_weight=True)
    s2 = {"strides": [2, 2], "dilations": [1, 1]}
    net.op("Conv2D", "a", ["X", "w1"], ["A"], T=F, ints=s2, i={"padding": H.SAME})      # alone on X
    net.op("Conv2D", "b", ["Y", "w2"], ["B"], T=F, ints=s2, i={"padding": H.VALID})     # pair on Y ...
    net.op("Conv2D", "c", ["Y", "w3"], ["C"], T=F, ints=s2, i={"padding": H.SAME})
    net.op("Conv2D", "d", ["Y", "w4"], ["D"], T=F, ints={"strides": [2, 1], "dilations": [1, 1]},
           i={"padding": H.SAME})                                                        # ... other strides
    net.op("Conv2D", "e", ["Y", "w5"], ["E"], T=F, ints=s2, i={"padding": H.SAME})      # 3x3: not pointwise
    net.run()
    before = {k: net.read(k, np.float32) for k in "ABCDE"}
    assert net.share_subsampled_inputs() == 1
    net.run()
    for k, want in before.items():
        got = net.read(k, np.float32)
        assert got.shape == want.shape and np.abs(got - want).max() <= 1e-5 * np.abs(want).max(), k


def test_activation_is_not_merged_when_the_sum_has_another_reader(net):
    from mace_b200 import hostapi as H
    a = np.arange(-3, 3, dtype=np.float32).reshape(1, 1, 2, 3)
    net.add_tensor("A", a)
    net.add_tensor("B", np.ones_like(a))
    F = H.DT_FLOAT
    net.op("Eltwise", "sum", ["A", "B"], ["Sum"], T=F, i={"type": 0})
    net.op("Activation", "relu", ["Sum"], ["Relu"], T=F, s={"activation": "RELU"})
    net.op("Eltwise", "neg", ["Sum"], ["Neg"], T=F, i={"type": 6})          # second reader of Sum
    net.op("Eltwise", "sum2", ["A", "A"], ["Sum2"], T=F, i={"type": 0})
    net.op("Activation", "relux", ["Sum2"], ["Relux"], T=F, s={"activation": "RELUX"}, f={"max_limit": 3.0})
    assert net.fuse_activations() == 1       # only sum2 + relux
    net.run()
    assert net.read("Sum", np.float32).ravel().tolist() == [-2, -1, 0, 1, 2, 3]
    assert net.read("Relu", np.float32).ravel().tolist() == [0, 0, 0, 1, 2, 3]
    assert net.read("Neg", np.float32).ravel().tolist() == [2, 1, 0, -1, -2, -3]
    assert net.read("Relux", np.float32).ravel().tolist() == [0, 0, 0, 0, 2, 3]
