"""The CPU oracle against the reference's own known-answer tests.

These literals come from the reference's unit tests (tests/golden/reference_kats.json
cites file:line for each); they are what pins the oracle.
"""
import numpy as np
import pytest

PAD = {"VALID": 0, "SAME": 1, "FULL": 2}


def test_conv2d_u8_kat(orc, kats):
    k = kats["conv2d_u8_3x3"]
    x = np.array(k["input"], np.uint8).reshape(k["input_nhwc_shape"])
    f = np.array(k["filter"], np.uint8).reshape(k["filter_ohwi_shape"])
    bias = orc.get_bias_data(np.array(k["bias"], np.int32), k["bias_scale"],
                             k["input_scale"], k["filter_scale"], f.shape[0])
    oh, ow, ph, pw = orc.calc_padding_and_output_size(3, 3, 3, 3, (1, 1), k["strides"],
                                                      PAD[k["padding"]])
    assert (oh, ow, ph, pw) == (1, 1, 0, 0)
    # Pipeline::Make(bias, channels, filter scale, input scale, output scale, zp)
    mult, shift = orc.output_multiplier_and_shift(k["filter_scale"], k["input_scale"],
                                                  k["output_scale"])
    out = orc.conv2d_u8(x, f, bias, k["strides"], (ph, pw), (oh, ow), k["input_zp"],
                        k["filter_zp"], mult, shift, k["output_zp"])
    assert out.ravel().tolist() == k["expected"]


def test_dwconv_u8_kat(orc, kats):
    k = kats["dwconv_u8_3x3"]
    x = np.array(k["input"], np.uint8).reshape(k["input_nhwc_shape"])
    f = np.array(k["filter"], np.uint8).reshape(k["filter_hwim_shape"])
    bias = orc.get_bias_data(np.array(k["bias"], np.int32), k["bias_scale"],
                             k["input_scale"], k["filter_scale"], 2)
    mult, shift = orc.output_multiplier_and_shift(k["input_scale"], k["filter_scale"],
                                                  k["output_scale"])
    out = orc.dwconv_u8(x, f, bias, k["strides"], (1, 1), (0, 0), (1, 1), k["input_zp"],
                        k["filter_zp"], mult, shift, k["output_zp"])
    assert out.ravel().tolist() == k["expected"]


def _nhwc_to_nchw(a):
    return np.ascontiguousarray(np.transpose(a, (0, 3, 1, 2)))


def _nchw_to_nhwc(a):
    return np.ascontiguousarray(np.transpose(a, (0, 2, 3, 1)))


def _run_f32_conv(orc, k, fn):
    shape = k["input_nhwc_shape"]
    x = np.full(shape, k["input_fill"], np.float32)
    f = np.full(k["filter_oihw_shape"], k["filter_fill"], np.float32)
    oh, ow, ph, pw = orc.calc_padding_and_output_size(shape[1], shape[2], 3, 3, (1, 1),
                                                      k["strides"], PAD[k["padding"]])
    out = fn(_nhwc_to_nchw(x), f, np.array(k["bias"], np.float32), (ph >> 1, pw >> 1),
             (oh, ow))
    exp = np.array(k["expected"], np.float32).reshape(k["expected_nhwc_shape"])
    np.testing.assert_allclose(_nchw_to_nhwc(out), exp, rtol=k["rel_tol"], atol=1e-8)


def test_conv2d_f32_literals(orc, kats):
    for name in ("conv2d_f32_3x3_valid", "conv2d_f32_3x3_same"):
        _run_f32_conv(orc, kats[name],
                      lambda x, f, b, pad, ohw: orc.conv2d_f32(x, f, b, (1, 1), (1, 1), pad, ohw))


def test_winograd_f32_literals(orc, kats):
    # The reference reaches its Winograd delegator through the same Conv2D
    # literals when channels >= 8 on ARM; the oracle's Winograd path must agree
    # with them too (both tile sizes).
    for name in ("conv2d_f32_3x3_valid", "conv2d_f32_3x3_same"):
        for tile in (2, 6):
            _run_f32_conv(orc, kats[name],
                          lambda x, f, b, pad, ohw: orc.winograd_f32(x, f, b, pad, ohw, tile=tile))


def test_dwconv_f32_literal(orc, kats):
    k = kats["dwconv_f32_2x2_valid"]
    x = np.array(k["input"], np.float32).reshape(k["input_nhwc_shape"])
    f = np.array(k["filter"], np.float32).reshape(k["filter_mihw_shape"])
    out = orc.dwconv_f32(_nhwc_to_nchw(x), f, np.array(k["bias"], np.float32), (1, 1), (1, 1),
                         (0, 0), (2, 2))
    exp = np.array(k["expected"], np.float32).reshape(k["expected_nhwc_shape"])
    np.testing.assert_allclose(_nchw_to_nhwc(out), exp, rtol=k["rel_tol"])


def test_matmul_f32_literals(orc):
    # test/ccunit/mace/ops/matmul_test.cc:55-72
    a = np.arange(1, 7, dtype=np.float32)
    out = orc.gemm_f32(a, a, 1, 2, 2, 3)
    assert out.tolist() == [22, 28, 49, 64]
    a = np.arange(1, 26, dtype=np.float32)
    out = orc.gemm_f32(a, a, 1, 5, 5, 5)
    assert out.tolist() == [215, 230, 245, 260, 275, 490, 530, 570, 610, 650, 765, 830, 895,
                            960, 1025, 1040, 1130, 1220, 1310, 1400, 1315, 1430, 1545, 1660,
                            1775]


def test_requant_primitives(orc):
    # the arithmetic of the Conv2D pin, step by step: 353 * 1392511872 >> 31, +1 -> 230
    mult, shift = orc.output_multiplier_and_shift(0.0226, 0.0204, 0.000711)
    assert 0 < mult < 2 ** 31 and shift >= 0
    # the doubling high-mul rounds exact ties towards +infinity ...
    assert orc.requant_fixed(1, 1 << 30, 0, 0) == 1      # 0.5 -> 1
    assert orc.requant_fixed(3, 1 << 30, 1, 10) == 11    # 1.5 -> 2, then 2/2 = 1
    assert orc.requant_fixed(-1, 1 << 30, 0, 10) == 10   # -0.5 -> 0
    assert orc.requant_fixed(-3, 1 << 30, 0, 10) == 9    # -1.5 -> -1
    # ... and the rounding right shift rounds ties away from zero
    assert orc.requant_fixed(-2, 2 ** 31 - 1, 2, 10) == 9    # -2 * ~1 = -2; -2/4 = -0.5 -> -1
    assert orc.requant_fixed(2, 2 ** 31 - 1, 2, 10) == 11    # 0.5 -> 1
    assert orc.requant_fixed(-(1 << 20), 2 ** 31 - 1, 0, 0) == 0  # clamp low
    assert orc.requant_fixed(1 << 20, 2 ** 31 - 1, 0, 0) == 255   # clamp high


def test_adjust_range(orc):
    s, z = orc.adjust_range(-1.0, 1.0, False)
    assert abs(s - 2.0 / 255) < 1e-7 and z in (127, 128)
    s, z = orc.adjust_range(0.0, 6.0, False)
    assert z == 0 and abs(s - 6.0 / 255) < 1e-7
    # non_zero nudges the range so that the minimum quantizes to >= 1
    s, z = orc.adjust_range(-1.0, 1.0, True)
    q = orc.quantize(np.array([-1.0, 1.0], np.float32), s, z)
    assert q[0] >= 1 and q[1] == 255


def test_padding_rules(orc):
    # stride-2 3x3 SAME on an even size: total pad 1 -> 0 before, 1 after
    assert orc.calc_padding_and_output_size(224, 224, 3, 3, (1, 1), (2, 2), 1) == (112, 112, 1, 1)
    assert orc.calc_padding_and_output_size(112, 112, 3, 3, (1, 1), (1, 1), 1) == (112, 112, 2, 2)
    assert orc.calc_padding_and_output_size(5, 5, 3, 3, (1, 1), (1, 1), 2) == (7, 7, 4, 4)
    assert orc.calc_padding_and_output_size(7, 7, 3, 3, (2, 2), (1, 1), 0) == (3, 3, 0, 0)


def _flat_nhwc_to_nchw(values, shape):
    return np.ascontiguousarray(np.asarray(values, np.float32).reshape(shape).transpose(0, 3, 1, 2))


def _nchw_to_flat_nhwc(t):
    return t.transpose(0, 2, 3, 1).ravel().tolist()


def test_pooling_f32_known_answers(orc):
    # PoolingOpTest.MAX_VALID / AVG_VALID (test/ccunit/mace/ops/pooling_test.cc:27-61, 301-336):
    # NHWC [1,4,4,2] whose two channels count 0..15 and 16..31, 2x2 window, stride 2, VALID
    x = _flat_nhwc_to_nchw([v for i in range(16) for v in (i, 16 + i)], (1, 4, 4, 2))
    out = orc.pooling_f32(x, (2, 2), (2, 2), (1, 1), (0, 0), (2, 2), 2)
    assert _nchw_to_flat_nhwc(out) == [5, 21, 7, 23, 13, 29, 15, 31]
    out = orc.pooling_f32(x, (2, 2), (2, 2), (1, 1), (0, 0), (2, 2), 1)
    assert _nchw_to_flat_nhwc(out) == [2.5, 18.5, 4.5, 20.5, 10.5, 26.5, 12.5, 28.5]
    # MAX_SAME (:63-94): 3x3 counting from 0, 2x2 stride 2 SAME -> pad 0 before, 1 after
    x = _flat_nhwc_to_nchw(range(9), (1, 3, 3, 1))
    ho, wo, ph, pw = orc.calc_padding_and_output_size(3, 3, 2, 2, (1, 1), (2, 2), 1)
    out = orc.pooling_f32(x, (2, 2), (2, 2), (1, 1), (ph // 2, pw // 2), (ho, wo), 2)
    assert _nchw_to_flat_nhwc(out) == [4, 5, 7, 8]
    # MAX_VALID_DILATION (:96-128): 4x4 counting from 0, 2x2 window, dilation 2
    x = _flat_nhwc_to_nchw(range(16), (1, 4, 4, 1))
    out = orc.pooling_f32(x, (2, 2), (1, 1), (2, 2), (0, 0), (2, 2), 2)
    assert _nchw_to_flat_nhwc(out) == [10, 11, 14, 15]
    # MAX_k2x2s2x2 (:130-162): [1,2,9,1] counting from 0, SAME -> the last window is cut
    x = _flat_nhwc_to_nchw(range(18), (1, 2, 9, 1))
    ho, wo, ph, pw = orc.calc_padding_and_output_size(2, 9, 2, 2, (1, 1), (2, 2), 1)
    out = orc.pooling_f32(x, (2, 2), (2, 2), (1, 1), (ph // 2, pw // 2), (ho, wo), 2)
    assert (ho, wo) == (1, 5) and _nchw_to_flat_nhwc(out) == [10, 12, 14, 16, 17]
    # SimpleAvgPoolingTest (:338-366): [1,2,8,1] counting from 0, 2x2 stride 2 SAME
    x = _flat_nhwc_to_nchw(range(16), (1, 2, 8, 1))
    out = orc.pooling_f32(x, (2, 2), (2, 2), (1, 1), (0, 0), (1, 4), 1)
    assert _nchw_to_flat_nhwc(out) == [4.5, 6.5, 8.5, 10.5]


def test_eltwise_f32_known_answers(orc):
    # EltwiseOpTest.CPUSimpleTensorScalar (test/ccunit/mace/ops/eltwise_test.cc:253-294)
    one_to_six = np.arange(1, 7, dtype=np.float32)
    SUM, SUB, PROD, DIV, MIN, MAX, NEG, ABS, SQR_DIFF = range(9)
    assert orc.eltwise_f32(np.ones(1, np.float32), None, SUM, scalar=1.0).tolist() == [2]
    assert orc.eltwise_f32(one_to_six, None, SUB, scalar=1.0).tolist() == [0, 1, 2, 3, 4, 5]
    assert orc.eltwise_f32(one_to_six, None, PROD, scalar=2.0).tolist() == [2, 4, 6, 8, 10, 12]
    assert orc.eltwise_f32(2 * one_to_six, None, DIV, scalar=2.0).tolist() == [1, 2, 3, 4, 5, 6]
    assert orc.eltwise_f32(one_to_six, None, MIN, scalar=1.0).tolist() == [1] * 6
    assert orc.eltwise_f32(one_to_six, None, MAX, scalar=3.0).tolist() == [3, 3, 3, 4, 5, 6]
    assert orc.eltwise_f32(one_to_six, None, NEG, scalar=3.0).tolist() == [-1, -2, -3, -4, -5, -6]
    assert orc.eltwise_f32(-one_to_six, None, ABS, scalar=3.0).tolist() == [1, 2, 3, 4, 5, 6]
    assert orc.eltwise_f32(one_to_six, None, SQR_DIFF, scalar=1.0).tolist() == [0, 1, 4, 9, 16, 25]
    # CPUSimpleTensorTensor (:476-491): same-shape operands, with and without coeff
    a = np.arange(1, 7, dtype=np.float32)
    assert orc.eltwise_f32(a, a, SUM).tolist() == [2, 4, 6, 8, 10, 12]
    assert np.allclose(orc.eltwise_f32(a, a, SUM, coeff=(0.1, 0.1)), [0.2, 0.4, 0.6, 0.8, 1, 1.2], atol=1e-5)
    assert orc.eltwise_f32(a, a, SUB).tolist() == [0] * 6
    assert orc.eltwise_f32(a, a, PROD).tolist() == [1, 4, 9, 16, 25, 36]
    assert orc.eltwise_f32(a, a, DIV).tolist() == [1] * 6
    # swapped operands: SUB and DIV are computed the other way round, SUM swaps its coefficients
    b = np.array([6, 5, 4, 3, 2, 1], np.float32)
    assert orc.eltwise_f32(a, b, SUB, swapped=True).tolist() == [5, 3, 1, -1, -3, -5]
    assert orc.eltwise_f32(a, b, SUM, coeff=(1.0, 2.0), swapped=True).tolist() == [8, 9, 10, 11, 12, 13]


def test_softmax_f32_known_answers(orc):
    # SoftmaxOpTest.CPUSimple / LogSoftmaxOpTest.CPUSimple (test/ccunit/mace/ops/softmax_test.cc:
    # 32-97): rows (1,1,1,1) and (1,2,3,4), as NHWC [1,1,2,4] and as a 2-D tensor [2,4]
    x = np.array([1, 1, 1, 1, 1, 2, 3, 4], np.float32)
    want = [0.25, 0.25, 0.25, 0.25, 0.0320586, 0.08714432, 0.23688282, 0.6439142]
    got = orc.softmax_f32(x, 2, 4, 1)
    assert np.allclose(got, want, atol=1e-5)
    want_log = [-1.3862944, -1.3862944, -1.3862944, -1.3862944, -3.4401896, -2.4401896,
                -1.4401897, -0.44018975]
    assert np.allclose(orc.softmax_f32(x, 2, 4, 1, use_log=True), want_log, atol=1e-5)
    # the same rows as the channels of an NCHW tensor [1,4,2,1]: softmax over C at each pixel
    nchw = np.ascontiguousarray(x.reshape(2, 4).T).reshape(1, 4, 2, 1)
    got = orc.softmax_f32(nchw, 1, 4, 2).reshape(4, 2).T.ravel()
    assert np.allclose(got, want, atol=1e-5)


QUANT_CASES = [[-2, -1, 0, 1, 2, 3, 4], [0, 1, 2, 3, 4], [2, 3, 4, 5, 6], [2, 4, 6, 8], [-2, -4, -6, -8]]


@pytest.mark.parametrize("values", QUANT_CASES)
@pytest.mark.parametrize("non_zero", [False, True])
def test_quantize_dequantize_known_answers(orc, values, non_zero):
    """QuantizeTest.TestQuantize (test/ccunit/mace/ops/quantize_test.cc:22-77): the range is
    found from the data, a round trip stays within 0.1, non_zero leaves no 0 in the output."""
    x = np.array(values, np.float32)
    mn, mx = orc.find_min_max(x)
    scale, zp = orc.adjust_range(mn, mx, non_zero)
    q = orc.quantize(x, scale, zp)
    if non_zero:
        assert (q > 0).all()
    assert np.abs(orc.dequantize(q, scale, zp) - x).max() <= 0.1
    assert 0 <= zp <= 255
    # zero is exactly representable
    assert orc.dequantize(np.array([zp], np.uint8), scale, zp)[0] == 0.0
