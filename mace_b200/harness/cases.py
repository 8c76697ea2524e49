"""Seeded problem generators shared by the tests, the smoke check and the benchmark."""
import numpy as np


def gemm_case(orc, seed, batch, M, N, K, bias_len=None, a_batched=True, b_batched=True,
              a_col_major=False, b_col_major=False, zp_a=128, zp_b=120):
    """Operands, bias and output quantization in the style of the 1024^3 config:
    uint8 uniform operands, scales 0.02 / 0.005, int32 bias ~ round(N(0, 1000)), output
    scale / zero point from the fp32 product's min / max, fixed-point multiplier."""
    rng = np.random.Generator(np.random.PCG64(seed))
    A = rng.integers(0, 256, size=((batch if a_batched else 1), M, K), dtype=np.uint8)
    B = rng.integers(0, 256, size=((batch if b_batched else 1), K, N), dtype=np.uint8)
    bias = None
    if bias_len:
        bias = np.rint(rng.normal(0, 1000, size=bias_len)).astype(np.int32)
    # stored layouts
    A_st = np.ascontiguousarray(np.swapaxes(A, 1, 2)) if a_col_major else A
    B_st = np.ascontiguousarray(np.swapaxes(B, 1, 2)) if b_col_major else B
    s_a, s_b = np.float32(0.02), np.float32(0.005)
    acc = orc.gemm_u8(A_st, B_st, None, batch, M, N, K, zp_a, zp_b, a_col_major=a_col_major,
                      b_col_major=b_col_major, a_batched=a_batched, b_batched=b_batched,
                      out_int32=True).astype(np.float32)
    real = acc * (s_a * s_b)
    s_c, zp_c = orc.adjust_range(real.min(), real.max(), False)
    mult, shift = orc.output_multiplier_and_shift(s_a, s_b, s_c)
    return dict(A=A_st, B=B_st, bias=bias, zp_a=zp_a, zp_b=zp_b, mult=mult, shift=shift,
                zp_c=zp_c, s_c=s_c)


def conv_quant(orc, rng, x_shape_nhwc, f_shape, depth):
    """Random uint8 tensors + plausible quantization parameters for a conv."""
    x = rng.integers(0, 256, size=x_shape_nhwc, dtype=np.uint8)
    f = rng.integers(1, 256, size=f_shape, dtype=np.uint8)
    # zero points near mid-range keep the accumulator centred, so the requantized
    # output spreads over the uint8 range instead of saturating
    zp_in = int(rng.integers(118, 139))
    zp_f = int(rng.integers(118, 139))
    # typical magnitude of the accumulator: sqrt(depth) * 74 * 74
    mult, shift = orc.output_multiplier_and_shift(
        np.float32(0.02), np.float32(0.01),
        np.float32(0.02 * 0.01 * np.sqrt(depth) * 74 * 74 * 3 / 127))
    return x, f, zp_in, zp_f, mult, shift


def near_ratio(got, ref, rel_err, abs_err=None):
    """The reference's element-wise tensor comparison (ExpectTensorNear,
    test/ccutils/mace/ops/testing/test_utils.h:208-233): every element must satisfy
    |got - ref| <= abs_err + rel_err * |ref|.  Returns max |got - ref| / (abs_err + rel_err * |ref|),
    so a value <= 1 passes.  abs_err defaults to rel_err * rms(ref): an element much smaller than
    the tensor's typical magnitude is a sum that cancelled, and no summation order keeps a
    relative bound there."""
    got = np.asarray(got, dtype=np.float64).ravel()
    ref = np.asarray(ref, dtype=np.float64).ravel()
    assert got.shape == ref.shape
    if abs_err is None:
        abs_err = rel_err * float(np.sqrt(np.mean(ref * ref)))
    bound = abs_err + rel_err * np.abs(ref)
    return float((np.abs(got - ref) / np.maximum(bound, 1e-300)).max())
