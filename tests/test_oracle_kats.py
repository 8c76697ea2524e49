"""The CPU oracle against the reference's own known-answer tests.

These literals come from the reference's unit tests (tests/golden/reference_kats.json
cites file:line for each); they are what pins the oracle.
"""
import numpy as np

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
