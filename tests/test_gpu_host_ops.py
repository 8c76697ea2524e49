"""The C++ host layer (operators -> delegators -> C ABI) on the GPU, driven the way the
reference's unit tests drive MACE's operators (OpsTestNet + OpDefBuilder): add named input
tensors with scale / zero point, define the operator with its args, set the output tensor's
scale / zero point, run, compare.  Expected values: the reference's known-answer literals
and the CPU oracle, bit-exact."""
import numpy as np
import pytest

from helpers import gemm_case

pytestmark = pytest.mark.gpu


@pytest.fixture()
def net():
    from mace_b200 import hostapi
    e = hostapi.HostEngine(0)
    yield e
    e.close()


def test_conv2d_quant_simple3x3(net, kats):
    """TestQuantSimple3x3, test/ccunit/mace/ops/conv_2d_test.cc:1240-1275."""
    from mace_b200 import hostapi as H
    k = kats["conv2d_u8_3x3"]
    net.add_tensor("Filter", np.array(k["filter"], np.uint8).reshape(k["filter_ohwi_shape"]),
                   scale=k["filter_scale"], zero_point=k["filter_zp"], is_weight=True)
    net.add_tensor("Input", np.array(k["input"], np.uint8).reshape(k["input_nhwc_shape"]),
                   scale=k["input_scale"], zero_point=k["input_zp"])
    net.add_tensor("Bias", np.array(k["bias"], np.int32), scale=k["bias_scale"], zero_point=0,
                   is_weight=True)
    net.op("Conv2D", "Conv2dTest", ["Input", "Filter", "Bias"], ["Output"],
           ints={"strides": [1, 1], "dilations": [1, 1]}, i={"padding": H.VALID})
    net.set_quant("Output", k["output_scale"], k["output_zp"])
    net.run()
    assert net.shape("Output") == (1, 1, 1, 1)
    assert net.read("Output", np.uint8).ravel().tolist() == k["expected"]


def test_depthwise_quant_simple_valid(net, kats):
    """QuantSimpleValidTest, test/ccunit/mace/ops/depthwise_conv2d_test.cc:333-372."""
    from mace_b200 import hostapi as H
    k = kats["dwconv_u8_3x3"]
    net.add_tensor("Input", np.array(k["input"], np.uint8).reshape(k["input_nhwc_shape"]),
                   scale=k["input_scale"], zero_point=k["input_zp"])
    net.add_tensor("Filter", np.array(k["filter"], np.uint8).reshape(k["filter_hwim_shape"]),
                   scale=k["filter_scale"], zero_point=k["filter_zp"], is_weight=True)
    net.add_tensor("Bias", np.array(k["bias"], np.int32), scale=k["bias_scale"], zero_point=0,
                   is_weight=True)
    net.op("DepthwiseConv2d", "DepthwiseConv2DTest", ["Input", "Filter", "Bias"], ["Output"],
           ints={"strides": [1, 1], "dilations": [1, 1]}, i={"padding": H.VALID})
    net.set_quant("Output", k["output_scale"], k["output_zp"])
    net.run()
    assert net.read("Output", np.uint8).ravel().tolist() == k["expected"]


@pytest.mark.parametrize("ta,tb", [(False, False), (True, False), (False, True), (True, True)])
@pytest.mark.parametrize("shape", [((1,), 64, 128, 32), ((2, 3), 31, 61, 67), ((16,), 32, 64, 96)])
def test_matmul_quant(net, orc, ta, tb, shape):
    """Quantized MatMul over the transpose / batch combinations of matmul_test.cc:400-426;
    uint8 and int32 outputs, bit-exact against the oracle."""
    from mace_b200 import hostapi as H
    batch_dims, M, K, N = shape
    batch = int(np.prod(batch_dims))
    case = gemm_case(orc, 31, batch, M, N, K, a_col_major=ta, b_col_major=tb)
    a_shape = tuple(batch_dims) + ((K, M) if ta else (M, K))
    b_shape = tuple(batch_dims) + ((N, K) if tb else (K, N))
    s_a, s_b = np.float32(0.02), np.float32(0.005)
    net.add_tensor("A", case["A"].reshape(a_shape), scale=s_a, zero_point=case["zp_a"])
    net.add_tensor("B", case["B"].reshape(b_shape), scale=s_b, zero_point=case["zp_b"])
    args = {"transpose_a": int(ta), "transpose_b": int(tb)}
    net.op("MatMul", "QuantizeMatMulTest", ["A", "B"], ["Output"], i=args,
           out_quant=[(case["s_c"], case["zp_c"])])
    net.op("MatMul", "QuantizeMatMulInt32", ["A", "B"], ["Output32"], i=args, out_dtype=H.DT_INT32)
    net.run()
    assert net.shape("Output") == tuple(batch_dims) + (M, N)
    exp = orc.gemm_u8(case["A"], case["B"], None, batch, M, N, K, case["zp_a"], case["zp_b"],
                      case["mult"], case["shift"], case["zp_c"], a_col_major=ta, b_col_major=tb)
    assert np.array_equal(net.read("Output", np.uint8).ravel(), exp)
    exp32 = orc.gemm_u8(case["A"], case["B"], None, batch, M, N, K, case["zp_a"], case["zp_b"],
                        a_col_major=ta, b_col_major=tb, out_int32=True)
    assert np.array_equal(net.read("Output32", np.int32).ravel(), exp32)
    scale, zp = net.quant("Output32")
    assert abs(scale - s_a * s_b) < 1e-12 and zp == 0  # C.scale = sA * sB, zero point 0


def test_matmul_one_side_batched_and_errors(net, orc):
    import mace_b200
    case = gemm_case(orc, 32, 3, 16, 32, 48, b_batched=False)
    net.add_tensor("A", case["A"].reshape(3, 16, 48), scale=0.02, zero_point=case["zp_a"])
    net.add_tensor("B", case["B"].reshape(48, 32), scale=0.005, zero_point=case["zp_b"])
    net.op("MatMul", "mm", ["A", "B"], ["Out"], out_quant=[(case["s_c"], case["zp_c"])])
    net.run()
    exp = orc.gemm_u8(case["A"], case["B"], None, 3, 16, 32, 48, case["zp_a"], case["zp_b"],
                      case["mult"], case["shift"], case["zp_c"], b_batched=False)
    assert np.array_equal(net.read("Out", np.uint8).ravel(), exp)
    # depth mismatch -> MACE_INVALID_ARGS from Validate()
    net.add_tensor("Bad", np.zeros((7, 5), np.uint8), scale=0.005, zero_point=0)
    net.op("MatMul", "bad", ["A", "Bad"], ["OutBad"], out_quant=[(1.0, 0)])
    with pytest.raises(mace_b200.MaceB200Error) as e:
        net.run()
    assert e.value.code == 1
    # unknown operator type / missing input
    with pytest.raises(mace_b200.MaceB200Error) as e:
        net.op("Softmax", "sm", ["A"], ["S"])
    assert e.value.code == 3
    with pytest.raises(mace_b200.MaceB200Error) as e:
        net.op("MatMul", "mm2", ["A", "Nope"], ["S"])
    assert e.value.code == 1


@pytest.mark.parametrize("shape", [(1, 4, 4, 32, 16), (5, 1, 1, 1024, 1000), (2, 7, 7, 64, 33)])
def test_fully_connected_quant(net, orc, shape):
    """Quantized FullyConnected (fully_connected_test.cc:210-314 shapes): weight OHWI,
    input NHWC, float-multiplier Gemv rule with the output zero point added."""
    n, h, w, c, o = shape
    rng = np.random.Generator(np.random.PCG64(5))
    x = rng.integers(0, 256, size=(n, h, w, c), dtype=np.uint8)
    wt = rng.integers(1, 256, size=(o, h, w, c), dtype=np.uint8)
    bias = np.rint(rng.normal(0, 500, size=o)).astype(np.int32)
    s_x, s_w = np.float32(0.03), np.float32(0.004)
    K = h * w * c
    s_o = np.float32(s_x * s_w * np.sqrt(K) * 74 * 74 * 3 / 127)
    net.add_tensor("Input", x, scale=s_x, zero_point=127)
    net.add_tensor("Weight", wt, scale=s_w, zero_point=128, is_weight=True)
    net.add_tensor("Bias", bias, scale=s_x * s_w, zero_point=0, is_weight=True)
    net.op("FullyConnected", "fc", ["Input", "Weight", "Bias"], ["Output"], out_quant=[(s_o, 119)])
    net.run()
    assert net.shape("Output") == (n, 1, 1, o)
    exp = orc.gemv_u8(wt.reshape(1, o, K), x.reshape(n, K), bias, n, o, K, 128, 127,
                      np.float32(s_w * s_x / s_o), 119, True)
    got = net.read("Output", np.uint8).ravel()
    assert np.array_equal(got, exp) and len(np.unique(got)) > 8


def test_conv_bias_rescale_and_explicit_paddings(net, orc):
    """GetBiasData rescales a bias whose scale is not input_scale * filter_scale; explicit
    `padding_values` take the CalcOutputSize path."""
    rng = np.random.Generator(np.random.PCG64(9))
    x = rng.integers(0, 256, size=(2, 9, 10, 16), dtype=np.uint8)
    f = rng.integers(1, 256, size=(24, 3, 3, 16), dtype=np.uint8)
    bias = np.rint(rng.normal(0, 50, size=24)).astype(np.int32)
    s_in, s_f, s_bias = np.float32(0.02), np.float32(0.01), np.float32(0.003)
    s_out = np.float32(s_in * s_f * 12 * 74 * 74 * 3 / 127)
    net.add_tensor("Input", x, scale=s_in, zero_point=120)
    net.add_tensor("Filter", f, scale=s_f, zero_point=131, is_weight=True)
    net.add_tensor("Bias", bias, scale=s_bias, zero_point=0, is_weight=True)
    net.op("Conv2D", "conv", ["Input", "Filter", "Bias"], ["Output"], out_quant=[(s_out, 100)],
           ints={"strides": [2, 1], "dilations": [1, 1], "padding_values": [2, 4]})
    net.run()
    bias_adj = orc.get_bias_data(bias, s_bias, s_in, s_f, 24)
    assert not np.array_equal(bias_adj, bias)
    ho, wo = (9 + 2 - 3) // 2 + 1, (10 + 4 - 3) // 1 + 1
    assert net.shape("Output") == (2, ho, wo, 24)
    m, sh = orc.output_multiplier_and_shift(s_f, s_in, s_out)
    exp = orc.conv2d_u8(x, f, bias_adj, (2, 1), (2, 4), (ho, wo), 120, 131, m, sh, 100)
    assert np.array_equal(net.read("Output", np.uint8), exp)


def test_pooling_keeps_quantization(net, orc):
    from mace_b200 import hostapi as H
    rng = np.random.Generator(np.random.PCG64(2))
    x = rng.integers(0, 256, size=(3, 7, 7, 96), dtype=np.uint8)
    net.add_tensor("Input", x, scale=0.0123, zero_point=7)
    net.op("Pooling", "pool", ["Input"], ["Output"],
           ints={"kernels": [7, 7], "strides": [1, 1], "dilations": [1, 1]},
           i={"padding": H.VALID, "pooling_type": H.AVG})
    net.run()
    scale, zp = net.quant("Output")
    assert abs(scale - np.float32(0.0123)) < 1e-9 and zp == 7
    exp = orc.avgpool_u8(x, (7, 7), (1, 1), (0, 0), (1, 1))
    assert np.array_equal(net.read("Output", np.uint8), exp)


# ---- fp32 operators -------------------------------------------------------------------

def _rel(got, ref):
    return float(np.abs(got.astype(np.float64) - ref).max() / max(np.abs(ref).max(), 1e-30))


def test_conv2d_float_simple3x3(net, kats):
    """TestNHWCSimple3x3VALID / SAME (conv_2d_test.cc:35-153) on NCHW tensors: 18.1 ..."""
    from mace_b200 import hostapi as H
    for name, pad in (("conv2d_f32_3x3_valid", H.VALID), ("conv2d_f32_3x3_same", H.SAME)):
        k = kats[name]
        net.add_tensor("Input" + name, np.ones((1, 2, 3, 3), np.float32))
        net.add_tensor("Filter" + name, np.ones((1, 2, 3, 3), np.float32), is_weight=True)
        net.add_tensor("Bias" + name, np.array(k["bias"], np.float32), is_weight=True)
        net.op("Conv2D", "Conv2dTest" + name, ["Input" + name, "Filter" + name, "Bias" + name],
               ["Output" + name], T=H.DT_FLOAT, ints={"strides": [1, 1], "dilations": [1, 1]},
               i={"padding": pad})
    net.run()
    for name in ("conv2d_f32_3x3_valid", "conv2d_f32_3x3_same"):
        k = kats[name]
        got = net.read("Output" + name, np.float32)
        np.testing.assert_allclose(got.ravel(), np.array(k["expected"], np.float32), rtol=1e-5)


@pytest.mark.parametrize("case", [(2, 16, 20, 20, 24, 3, 1, "RELU"),     # -> K3x3Winograd, F(6,3)
                                  (1, 8, 12, 12, 8, 3, 1, "NOOP"),       # -> K3x3Winograd, F(2,3)
                                  (1, 4, 12, 12, 8, 3, 1, "RELUX"),      # C < 8 -> general
                                  (2, 32, 14, 14, 64, 1, 1, "RELU"),     # -> K1x1
                                  (1, 3, 30, 30, 16, 7, 2, "LEAKYRELU")])
def test_conv2d_float_delegator_selection(net, orc, case):
    from mace_b200 import hostapi as H
    N, C, Hh, W, O, k, st, act = case
    rng = np.random.Generator(np.random.PCG64(C + O))
    x = rng.random((N, C, Hh, W), dtype=np.float32)
    f = (rng.standard_normal((O, C, k, k)) * np.sqrt(2.0 / (C * k * k))).astype(np.float32)
    bias = (rng.standard_normal(O) * 0.01).astype(np.float32)
    net.add_tensor("Input", x)
    net.add_tensor("Filter", f, is_weight=True)
    net.add_tensor("Bias", bias, is_weight=True)
    net.op("Conv2D", "conv", ["Input", "Filter", "Bias"], ["Output"], T=H.DT_FLOAT,
           ints={"strides": [st, st], "dilations": [1, 1]}, i={"padding": H.SAME},
           s={"activation": act}, f={"max_limit": 0.3, "activation_coefficient": 0.2})
    net.run()
    net.run()  # second run reuses the cached transformed filter
    Ho, Wo, ph, pw = orc.calc_padding_and_output_size(Hh, W, k, k, (1, 1), (st, st), 1)
    code = {"NOOP": 0, "RELU": 1, "RELUX": 2, "LEAKYRELU": 6}[act]
    ref = orc.conv2d_f32(x, f, bias, (st, st), (1, 1), (ph >> 1, pw >> 1), (Ho, Wo), code, 0.3, 0.2)
    got = net.read("Output", np.float32)
    assert got.shape == ref.shape
    assert _rel(got, ref) <= (1e-3 if (k == 3 and C >= 8) else 1e-4)


def test_matmul_and_fully_connected_float(net, orc):
    from mace_b200 import hostapi as H
    rng = np.random.Generator(np.random.PCG64(12))
    A = rng.standard_normal((2, 3, 40, 24)).astype(np.float32)
    B = rng.standard_normal((2, 3, 56, 24)).astype(np.float32)
    net.add_tensor("A", A)
    net.add_tensor("B", B)
    net.op("MatMul", "mm", ["A", "B"], ["C"], T=H.DT_FLOAT, i={"transpose_b": 1})
    x = rng.standard_normal((5, 32, 2, 2)).astype(np.float32)
    w = rng.standard_normal((10, 32, 2, 2)).astype(np.float32)
    b = rng.standard_normal(10).astype(np.float32)
    net.add_tensor("X", x)
    net.add_tensor("W", w, is_weight=True)
    net.add_tensor("Bfc", b, is_weight=True)
    net.op("FullyConnected", "fc", ["X", "W", "Bfc"], ["Y"], T=H.DT_FLOAT)
    net.run()
    ref = orc.gemm_f32(A, B, 6, 40, 56, 24, b_col_major=True)
    assert net.shape("C") == (2, 3, 40, 56)
    assert _rel(net.read("C", np.float32).ravel(), ref) <= 1e-4
    ref = orc.gemv_f32(w.reshape(10, 128), x.reshape(5, 128), b, 5, 10, 128)
    assert net.shape("Y") == (5, 10, 1, 1)
    assert _rel(net.read("Y", np.float32).ravel(), ref) <= 1e-4


@pytest.mark.parametrize("values", [[-2, -1, 0, 1, 2, 3, 4], [0, 1, 2, 3, 4], [2, 3, 4, 5, 6], [2, 4, 6, 8],
                                    [-2, -4, -6, -8]])
@pytest.mark.parametrize("non_zero", [0, 1])
def test_quantize_dequantize_ops(net, orc, values, non_zero):
    """QuantizeTest.TestQuantize (test/ccunit/mace/ops/quantize_test.cc:22-77) through
    QuantizeOp / DequantizeOp of the CUDA runtime: the range comes from the data."""
    from mace_b200 import hostapi as H
    x = np.array(values, np.float32)
    net.add_tensor("Input", x)
    net.op("Quantize", "QuantizeTest", ["Input"], ["QuantizeOutput"], T=H.DT_UINT8, out_dtype=H.DT_UINT8,
           i={"non_zero": non_zero})
    net.op("Dequantize", "DeQuantizeTest", ["QuantizeOutput"], ["Output"], T=H.DT_UINT8, out_dtype=H.DT_FLOAT)
    net.run()
    q = net.read("QuantizeOutput", np.uint8)
    scale, zp = net.quant("QuantizeOutput")
    assert (scale, zp) == orc.adjust_range(*orc.find_min_max(x), bool(non_zero))
    assert np.array_equal(q, orc.quantize(x, scale, zp))
    if non_zero:
        assert (q > 0).all()
    out = net.read("Output", np.float32)
    assert np.array_equal(out, orc.dequantize(q, scale, zp))
    assert np.abs(out - x).max() <= 0.1


def test_quantize_with_given_range_then_conv(net, orc):
    """A float input quantized with the output tensor's preset scale (the converter's
    quantize_info), fed to a quantized 1x1 convolution and dequantized again."""
    from mace_b200 import hostapi as H
    rng = np.random.Generator(np.random.PCG64(5))
    x = rng.random((2, 9, 9, 16), dtype=np.float32) * 4 - 1
    w = rng.integers(0, 256, (8, 1, 1, 16), dtype=np.uint8)
    net.add_tensor("Input", x)
    net.add_tensor("W", w, scale=0.01, zero_point=120, is_weight=True)
    net.op("Quantize", "q", ["Input"], ["Xq"], T=H.DT_UINT8, out_dtype=H.DT_UINT8, out_quant=[(4 / 255.0, 64)])
    net.op("Conv2D", "conv", ["Xq", "W"], ["Yq"], out_quant=[(0.05, 100)],
           ints={"strides": [1, 1], "dilations": [1, 1]}, i={"padding": H.VALID})
    net.op("Dequantize", "dq", ["Yq"], ["Y"], T=H.DT_UINT8, out_dtype=H.DT_FLOAT)
    net.run()
    xq = orc.quantize(x, np.float32(4 / 255.0), 64)
    assert np.array_equal(net.read("Xq", np.uint8), xq)
    m, sh = orc.output_multiplier_and_shift(np.float32(4 / 255.0), np.float32(0.01), np.float32(0.05))
    yq = orc.conv2d_u8(xq, w, None, (1, 1), (0, 0), (9, 9), 64, 120, m, sh, 100)
    assert np.array_equal(net.read("Yq", np.uint8), yq)
    assert np.array_equal(net.read("Y", np.float32), orc.dequantize(yq, np.float32(0.05), 100))
