"""ctypes binding of the CPU oracle (``oracle/_build/liboracle.so``).

Test infrastructure only: imported by ``tests/``, by the smoke check and by the
CPU-baseline leg of ``bench.py``.  The product package never imports it.
All wrappers take and return numpy arrays on the host.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_build", "liboracle.so")


def build(force=False):
    """Compile the oracle with make when the library is missing or stale."""
    src = [os.path.join(_HERE, f) for f in ("oracle.cc", "oracle.h", "Makefile")]
    stale = (not os.path.exists(_LIB_PATH)) or any(
        os.path.getmtime(s) > os.path.getmtime(_LIB_PATH) for s in src)
    if force or stale:
        subprocess.check_call(["make", "-C", _HERE], stdout=subprocess.DEVNULL)
    return _LIB_PATH


_lib = None

_u8p = C.POINTER(C.c_uint8)
_i32p = C.POINTER(C.c_int32)
_f32p = C.POINTER(C.c_float)
_i64 = C.c_int64
_i32 = C.c_int32
_int = C.c_int
_f32 = C.c_float
_vp = C.c_void_p


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(_LIB_PATH)
        _lib.orc_requant_fixed.restype = C.c_uint8
        _lib.orc_requant_fixed.argtypes = [_i32, _i32, _i32, _i32]
        _lib.orc_rounding_stages.restype = _i32
        _lib.orc_rounding_stages.argtypes = [_i32, _i32, _i32]
        _lib.orc_adjust_range_u8.restype = None
        _lib.orc_adjust_range_u8.argtypes = [_f32, _f32, _int, _f32p, _i32p]
        _lib.orc_quantize_u8.restype = None
        _lib.orc_quantize_u8.argtypes = [_vp, _i64, _f32, _i32, _vp]
        _lib.orc_output_multiplier_and_shift.argtypes = [_f32, _f32, _f32, _i32p, _i32p]
        _lib.orc_get_bias_data.restype = None
        _lib.orc_get_bias_data.argtypes = [_vp, _f32, _f32, _f32, _i64, _vp]
        _lib.orc_calc_padding_and_output_size.argtypes = (
            [_i64] * 4 + [_int] * 5 + [C.POINTER(_i64)] * 2 + [C.POINTER(_int)] * 2)
        _lib.orc_gemm_u8.argtypes = ([_vp] * 4 + [_int] + [_i64] * 4 + [_int] * 5 +
                                     [_i32] * 5 + [_int])
        _lib.orc_gemv_u8.argtypes = ([_vp] * 4 + [_int] + [_i64] * 3 + [_int] * 2 +
                                     [_i32] * 2 + [_f32, _i32, _int])
        _lib.orc_conv2d_u8_nhwc.argtypes = ([_vp] * 4 + [_i64] * 7 + [_int] * 4 +
                                            [_i64] * 2 + [_i32] * 5)
        _lib.orc_dwconv_u8_nhwc.argtypes = ([_vp] * 4 + [_i64] * 7 + [_int] * 6 +
                                            [_i64] * 2 + [_i32] * 5)
        _lib.orc_dwconv_u8_nhwc_general.argtypes = ([_vp] * 4 + [_i64] * 7 + [_int] * 6 +
                                                    [_i64] * 2 + [_i32] * 2 + [_f32, _i32])
        _lib.orc_avgpool_u8_nhwc.argtypes = ([_vp] * 2 + [_i64] * 6 + [_int] * 4 + [_i64] * 2)
        _lib.orc_conv2d_f32_nchw.argtypes = ([_vp] * 4 + [_i64] * 7 + [_int] * 6 +
                                             [_i64] * 2 + [_int, _f32, _f32])
        _lib.orc_dwconv_f32_nchw.argtypes = ([_vp] * 4 + [_i64] * 7 + [_int] * 6 +
                                             [_i64] * 2 + [_int, _f32, _f32])
        _lib.orc_gemm_f32.argtypes = [_vp] * 3 + [_i64] * 4 + [_int] * 5
        _lib.orc_gemv_f32.argtypes = [_vp] * 4 + [_i64] * 3 + [_int] * 2
        _lib.orc_conv3x3_winograd_f32_nchw.argtypes = (
            [_vp] * 4 + [_i64] * 5 + [_int] * 2 + [_i64] * 2 + [_int, _f32, _f32, _int])
        _lib.orc_pooling_f32_nchw.argtypes = [_vp] * 2 + [_i64] * 6 + [_int] * 6 + [_i64] * 2 + [_int]
        _lib.orc_eltwise_f32.argtypes = [_vp] * 3 + [_i64, _int, _f32, _int, _f32, _f32, _int]
        _lib.orc_activation_f32.argtypes = [_vp] * 2 + [_i64, _int, _f32, _f32]
        _lib.orc_softmax_f32.argtypes = [_vp] * 2 + [_i64] * 3 + [_int]
        _lib.orc_dequantize_u8.restype = None
        _lib.orc_dequantize_u8.argtypes = [_vp, _i64, _f32, _i32, _vp]
        _lib.orc_dequantize_i32.restype = None
        _lib.orc_dequantize_i32.argtypes = [_vp, _i64, _f32, _i32, _vp]
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(_vp)


def _c(a, dt):
    return None if a is None else np.ascontiguousarray(a, dtype=dt)


def set_threads(n):
    return lib().orc_set_threads(int(n))


def get_threads():
    return lib().orc_get_threads()


def adjust_range(mn, mx, non_zero):
    s, z = _f32(), _i32()
    lib().orc_adjust_range_u8(float(mn), float(mx), int(bool(non_zero)), C.byref(s), C.byref(z))
    return np.float32(s.value), int(z.value)


def quantize(x, scale, zp):
    x = _c(x, np.float32)
    out = np.empty(x.shape, np.uint8)
    lib().orc_quantize_u8(_p(x), x.size, float(scale), int(zp), _p(out))
    return out


def output_multiplier_and_shift(ls, rs, os_):
    m, s = _i32(), _i32()
    st = lib().orc_output_multiplier_and_shift(float(ls), float(rs), float(os_),
                                               C.byref(m), C.byref(s))
    if st != 0:
        raise ValueError("real multiplier outside (0,1)")
    return int(m.value), int(s.value)


def requant_fixed(acc, mult, shift, zp):
    return int(lib().orc_requant_fixed(int(acc), int(mult), int(shift), int(zp)))


def rounding_stages(acc, mult, shift):
    return int(lib().orc_rounding_stages(int(acc), int(mult), int(shift)))


def get_bias_data(bias, bias_scale, in_scale, f_scale, channels):
    bias = _c(bias, np.int32)
    out = np.empty(channels, np.int32)
    lib().orc_get_bias_data(_p(bias), float(bias_scale), float(in_scale), float(f_scale),
                            channels, _p(out))
    return out


def calc_padding_and_output_size(in_h, in_w, k_h, k_w, dil, strides, padding_type):
    oh, ow, ph, pw = _i64(), _i64(), _int(), _int()
    st = lib().orc_calc_padding_and_output_size(
        in_h, in_w, k_h, k_w, dil[0], dil[1], strides[0], strides[1], padding_type,
        C.byref(oh), C.byref(ow), C.byref(ph), C.byref(pw))
    if st != 0:
        raise ValueError("invalid conv arguments")
    return int(oh.value), int(ow.value), int(ph.value), int(pw.value)


def gemm_u8(A, B, bias, batch, M, N, K, zp_a, zp_b, mult=0, shift=0, zp_c=0,
            a_col_major=False, b_col_major=False, c_col_major=False,
            a_batched=True, b_batched=True, out_int32=False, bias_per_row=False):
    A, B, bias = _c(A, np.uint8), _c(B, np.uint8), _c(bias, np.int32)
    out = np.empty(batch * M * N, np.int32 if out_int32 else np.uint8)
    st = lib().orc_gemm_u8(_p(A), _p(B), _p(bias), _p(out), int(out_int32), batch, M, N, K,
                           int(a_col_major), int(b_col_major), int(c_col_major),
                           int(a_batched), int(b_batched), zp_a, zp_b, mult, shift, zp_c,
                           int(bias_per_row))
    assert st == 0
    return out


def gemv_u8(lhs, rhs, bias, batch, rows, K, zp_l, zp_r, multiplier=0.0, zp_out=0,
            add_zp_out=True, lhs_batched=False, rhs_batched=True, out_int32=False):
    lhs, rhs, bias = _c(lhs, np.uint8), _c(rhs, np.uint8), _c(bias, np.int32)
    out = np.empty(batch * rows, np.int32 if out_int32 else np.uint8)
    st = lib().orc_gemv_u8(_p(lhs), _p(rhs), _p(bias), _p(out), int(out_int32), batch, rows,
                           K, int(lhs_batched), int(rhs_batched), zp_l, zp_r,
                           float(multiplier), zp_out, int(add_zp_out))
    assert st == 0
    return out


def conv2d_u8(x, f, bias, strides, pads_total, out_hw, zp_in, zp_f, mult, shift, zp_out):
    """x NHWC, f OHWI."""
    x, f, bias = _c(x, np.uint8), _c(f, np.uint8), _c(bias, np.int32)
    N, H, W, Cc = x.shape
    O, KH, KW, _ = f.shape
    Ho, Wo = out_hw
    out = np.empty((N, Ho, Wo, O), np.uint8)
    st = lib().orc_conv2d_u8_nhwc(_p(x), _p(f), _p(bias), _p(out), N, H, W, Cc, O, KH, KW,
                                  strides[0], strides[1], pads_total[0], pads_total[1],
                                  Ho, Wo, zp_in, zp_f, mult, shift, zp_out)
    assert st == 0
    return out


def dwconv_u8(x, f, bias, strides, dil, pad_tl, out_hw, zp_in, zp_f, mult, shift, zp_out):
    """x NHWC, f HWIM."""
    x, f, bias = _c(x, np.uint8), _c(f, np.uint8), _c(bias, np.int32)
    N, H, W, Cc = x.shape
    KH, KW, _, Mc = f.shape
    Ho, Wo = out_hw
    out = np.empty((N, Ho, Wo, Cc * Mc), np.uint8)
    st = lib().orc_dwconv_u8_nhwc(_p(x), _p(f), _p(bias), _p(out), N, H, W, Cc, Mc, KH, KW,
                                  strides[0], strides[1], dil[0], dil[1], pad_tl[0],
                                  pad_tl[1], Ho, Wo, zp_in, zp_f, mult, shift, zp_out)
    assert st == 0
    return out


def dwconv_u8_general(x, f, bias, strides, dil, pad_tl, out_hw, zp_in, zp_f, multiplier,
                      zp_out):
    x, f, bias = _c(x, np.uint8), _c(f, np.uint8), _c(bias, np.int32)
    N, H, W, Cc = x.shape
    KH, KW, _, Mc = f.shape
    Ho, Wo = out_hw
    out = np.empty((N, Ho, Wo, Cc * Mc), np.uint8)
    st = lib().orc_dwconv_u8_nhwc_general(
        _p(x), _p(f), _p(bias), _p(out), N, H, W, Cc, Mc, KH, KW, strides[0], strides[1],
        dil[0], dil[1], pad_tl[0], pad_tl[1], Ho, Wo, zp_in, zp_f, float(multiplier), zp_out)
    assert st == 0
    return out


def avgpool_u8(x, kernel, strides, pad_tl, out_hw):
    x = _c(x, np.uint8)
    N, H, W, Cc = x.shape
    Ho, Wo = out_hw
    out = np.empty((N, Ho, Wo, Cc), np.uint8)
    st = lib().orc_avgpool_u8_nhwc(_p(x), _p(out), N, H, W, Cc, kernel[0], kernel[1],
                                   strides[0], strides[1], pad_tl[0], pad_tl[1], Ho, Wo)
    assert st == 0
    return out


def conv2d_f32(x, f, bias, strides, dil, pad_tl, out_hw, act=0, max_limit=0.0, coef=0.0):
    """x NCHW, f OIHW."""
    x, f, bias = _c(x, np.float32), _c(f, np.float32), _c(bias, np.float32)
    N, Cc, H, W = x.shape
    O, _, KH, KW = f.shape
    Ho, Wo = out_hw
    out = np.empty((N, O, Ho, Wo), np.float32)
    st = lib().orc_conv2d_f32_nchw(_p(x), _p(f), _p(bias), _p(out), N, Cc, H, W, O, KH, KW,
                                   strides[0], strides[1], dil[0], dil[1], pad_tl[0],
                                   pad_tl[1], Ho, Wo, act, max_limit, coef)
    assert st == 0
    return out


def dwconv_f32(x, f, bias, strides, dil, pad_tl, out_hw, act=0, max_limit=0.0, coef=0.0):
    """x NCHW, f [multiplier, Cin, kh, kw]."""
    x, f, bias = _c(x, np.float32), _c(f, np.float32), _c(bias, np.float32)
    N, Cc, H, W = x.shape
    Mc, _, KH, KW = f.shape
    Ho, Wo = out_hw
    out = np.empty((N, Cc * Mc, Ho, Wo), np.float32)
    st = lib().orc_dwconv_f32_nchw(_p(x), _p(f), _p(bias), _p(out), N, Cc, H, W, Mc, KH, KW,
                                   strides[0], strides[1], dil[0], dil[1], pad_tl[0],
                                   pad_tl[1], Ho, Wo, act, max_limit, coef)
    assert st == 0
    return out


def gemm_f32(A, B, batch, M, N, K, a_col_major=False, b_col_major=False, c_col_major=False,
             a_batched=True, b_batched=True):
    A, B = _c(A, np.float32), _c(B, np.float32)
    out = np.empty(batch * M * N, np.float32)
    st = lib().orc_gemm_f32(_p(A), _p(B), _p(out), batch, M, N, K, int(a_col_major),
                            int(b_col_major), int(c_col_major), int(a_batched), int(b_batched))
    assert st == 0
    return out


def gemv_f32(lhs, rhs, bias, batch, rows, K, lhs_batched=False, rhs_batched=True):
    lhs, rhs, bias = _c(lhs, np.float32), _c(rhs, np.float32), _c(bias, np.float32)
    out = np.empty(batch * rows, np.float32)
    st = lib().orc_gemv_f32(_p(lhs), _p(rhs), _p(bias), _p(out), batch, rows, K,
                            int(lhs_batched), int(rhs_batched))
    assert st == 0
    return out


def winograd_f32(x, f, bias, pad_tl, out_hw, act=0, max_limit=0.0, coef=0.0, tile=0):
    x, f, bias = _c(x, np.float32), _c(f, np.float32), _c(bias, np.float32)
    N, Cc, H, W = x.shape
    O = f.shape[0]
    Ho, Wo = out_hw
    out = np.empty((N, O, Ho, Wo), np.float32)
    st = lib().orc_conv3x3_winograd_f32_nchw(_p(x), _p(f), _p(bias), _p(out), N, Cc, H, W, O,
                                             pad_tl[0], pad_tl[1], Ho, Wo, act, max_limit,
                                             coef, tile)
    assert st == 0
    return out


def pooling_f32(x, kernel, strides, dil, pad_tl, out_hw, pooling_type):
    """x NCHW; pooling_type 1 AVG, 2 MAX."""
    x = _c(x, np.float32)
    N, Cc, H, W = x.shape
    Ho, Wo = out_hw
    out = np.empty((N, Cc, Ho, Wo), np.float32)
    st = lib().orc_pooling_f32_nchw(_p(x), _p(out), N, Cc, H, W, kernel[0], kernel[1], strides[0],
                                    strides[1], dil[0], dil[1], pad_tl[0], pad_tl[1], Ho, Wo,
                                    pooling_type)
    assert st == 0
    return out


def eltwise_f32(a, b, type_, coeff=None, swapped=False, scalar=1.0):
    """b None: the tensor-scalar form with `scalar` as second operand."""
    a = _c(a, np.float32)
    b = _c(b, np.float32) if b is not None else None
    out = np.empty_like(a)
    c = coeff if coeff else (0.0, 0.0)
    st = lib().orc_eltwise_f32(_p(a), _p(b) if b is not None else None, _p(out), a.size, type_,
                               scalar, 1 if coeff else 0, c[0], c[1], 1 if swapped else 0)
    assert st == 0
    return out


def activation_f32(x, act, max_limit=0.0, coef=0.0):
    x = _c(x, np.float32)
    out = np.empty_like(x)
    st = lib().orc_activation_f32(_p(x), _p(out), x.size, act, max_limit, coef)
    assert st == 0
    return out


def softmax_f32(x, outer, classes, inner, use_log=False):
    x = _c(x, np.float32)
    out = np.empty_like(x)
    st = lib().orc_softmax_f32(_p(x), _p(out), outer, classes, inner, 1 if use_log else 0)
    assert st == 0
    return out


def dequantize(q, scale, zp):
    """uint8 or int32 -> float32: scale * (q - zp)."""
    q = np.ascontiguousarray(q)
    out = np.empty(q.shape, np.float32)
    if q.dtype == np.uint8:
        lib().orc_dequantize_u8(_p(q), q.size, scale, zp, _p(out))
    else:
        q = _c(q, np.int32)
        lib().orc_dequantize_i32(_p(q), q.size, scale, zp, _p(out))
    return out


def find_min_max(x):
    """FindMinMax (mace/core/quantize.h:90-102)."""
    x = np.asarray(x, np.float32)
    return float(x.min()), float(x.max())
