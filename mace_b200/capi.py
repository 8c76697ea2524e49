"""ctypes binding of ``libmace_b200.so`` (the C ABI of include/mace_b200.h)."""
import ctypes as C
import os
import subprocess

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = os.path.join(_HERE, "libmace_b200.so")

STATUS = {0: "MACE_SUCCESS", 1: "MACE_INVALID_ARGS", 2: "MACE_OUT_OF_RESOURCES",
          3: "MACE_UNSUPPORTED", 4: "MACE_RUNTIME_ERROR"}


class MaceB200Error(RuntimeError):
    def __init__(self, code, msg):
        super().__init__("%s: %s" % (STATUS.get(code, code), msg))
        self.code = code


def lib_path():
    return _LIB


def build(verbose=False):
    """Compile the device library for sm_100a with nvcc (in-tree)."""
    out = None if verbose else subprocess.DEVNULL
    subprocess.check_call(["make", "-C", os.path.join(_HERE, "csrc"), "-j8"], stdout=out)
    return _LIB


_vp = C.c_void_p
_i64 = C.c_int64
_i32 = C.c_int32
_int = C.c_int
_f32 = C.c_float
_sz = C.c_size_t

# name -> (restype, argtypes); every symbol that include/mace_b200.h declares
PROTOTYPES = {
    "mb_init": (_int, [_int, C.POINTER(_vp)]),
    "mb_destroy": (_int, [_vp]),
    "mb_last_error": (C.c_char_p, [_vp]),
    "mb_malloc": (_int, [_vp, _sz, C.POINTER(_vp)]),
    "mb_free": (_int, [_vp, _vp]),
    "mb_host_alloc": (_int, [_vp, _sz, C.POINTER(_vp)]),
    "mb_host_free": (_int, [_vp, _vp]),
    "mb_memcpy_h2d": (_int, [_vp, _vp, _vp, _sz]),
    "mb_memcpy_d2h": (_int, [_vp, _vp, _vp, _sz]),
    "mb_memset": (_int, [_vp, _vp, _int, _sz]),
    "mb_memcpy_d2d": (_int, [_vp, _vp, _vp, _sz]),
    "mb_upload_h2d": (_int, [_vp, _vp, _vp, _sz]),
    "mb_upload_wait_event": (_int, [_vp, _vp]),
    "mb_upload_signal": (_int, [_vp]),
    "mb_download_d2h": (C.c_int, [_vp, _vp, _vp, C.c_size_t, _vp]),
    "mb_stream_wait_event": (C.c_int, [_vp, _vp]),
    "mb_event_sync": (_int, [_vp, _vp]),
    "mb_stream_sync": (_int, [_vp]),
    "mb_stream": (_vp, [_vp]),
    "mb_event_create": (_int, [_vp, C.POINTER(_vp)]),
    "mb_event_record": (_int, [_vp, _vp]),
    "mb_event_elapsed_ms": (_int, [_vp, _vp, _vp, C.POINTER(_f32)]),
    "mb_event_destroy": (_int, [_vp, _vp]),
    "mb_graph_begin": (_int, [_vp]),
    "mb_graph_end": (_int, [_vp, C.POINTER(_vp)]),
    "mb_graph_launch": (_int, [_vp, _vp]),
    "mb_graph_destroy": (_int, [_vp, _vp]),
    "mb_launch_count": (C.c_uint64, [_vp]),
    "mb_launch_count_tensor_core": (C.c_uint64, [_vp]),
    "mb_launch_count_pair": (C.c_uint64, [_vp]),
    "mb_pair_clusters": (C.c_int, [_vp]),
    "mb_set_option": (_int, [_vp, C.c_char_p, _int]),
    "mb_gemm_u8": (_int, [_vp] * 5 + [_int] + [_i64] * 4 + [_int] * 5 + [_i32] * 5 + [_int]),
    "mb_gemv_u8": (_int, [_vp] * 5 + [_int] + [_i64] * 3 + [_int] * 2 + [_i32] * 2 +
                   [_f32, _i32, _int]),
    "mb_conv2d_u8_nhwc": (_int, [_vp] * 5 + [_i64] * 7 + [_int] * 4 + [_i64] * 2 + [_i32] * 5),
    "mb_dwconv_u8_nhwc": (_int, [_vp] * 5 + [_i64] * 7 + [_int] * 6 + [_i64] * 2 + [_i32] * 5 +
                          [_int, _f32]),
    "mb_dwconv_u8_nhwc_prepacked": (_int, [_vp] * 6 + [_i64] * 7 + [_int] * 6 + [_i64] * 2 +
                                    [_i32] * 5 + [_int, _f32]),
    "mb_dwconv3x3_u8_prepacked_bytes": (C.c_size_t, [_i64]),
    "mb_dwconv3x3_u8_prepack": (_int, [_vp] * 3 + [_i64, _i32, _i32, _vp]),
    "mb_avgpool_u8_nhwc": (_int, [_vp] * 3 + [_i64] * 6 + [_int] * 4 + [_i64] * 2),
    "mb_gemm_f32": (_int, [_vp] * 4 + [_i64] * 4 + [_int] * 5),
    "mb_gemv_f32": (_int, [_vp] * 5 + [_i64] * 3 + [_int] * 2),
    "mb_conv2d_f32_nchw": (_int, [_vp] * 5 + [_i64] * 7 + [_int] * 6 + [_i64] * 2 + [_int, _f32, _f32]),
    "mb_conv2d_f32_nchw_residual": (_int, [_vp] * 6 + [_i64] * 7 + [_int] * 6 + [_i64] * 2 + [_int, _f32, _f32]),
    "mb_dwconv_f32_nchw": (_int, [_vp] * 5 + [_i64] * 7 + [_int] * 6 + [_i64] * 2 + [_int, _f32, _f32]),
    "mb_winograd_transform_filter_f32": (_int, [_vp] * 3 + [_i64] * 2 + [_int]),
    "mb_conv3x3_winograd_f32_nchw": (_int, [_vp] * 6 + [_i64] * 5 + [_int] * 2 + [_i64] * 2 +
                                     [_int, _f32, _f32, _int]),
    "mb_pooling_f32_nchw": (_int, [_vp] * 3 + [_i64] * 6 + [_int] * 6 + [_i64] * 2 + [_int]),
    "mb_eltwise_f32": (_int, [_vp] * 4 + [_i64, _int, _f32, _int, _f32, _f32, _int]),
    "mb_eltwise_act_f32": (_int, [_vp] * 4 + [_i64, _int, _f32, _int, _f32, _f32, _int, _int, _f32, _f32]),
    "mb_activation_f32": (_int, [_vp] * 3 + [_i64, _int, _f32, _f32]),
    "mb_softmax_f32": (_int, [_vp] * 3 + [_i64] * 3 + [_int]),
    "mb_quantize_f32_u8": (_int, [_vp] * 3 + [_i64, _f32, _i32]),
    "mb_dequantize_f32": (_int, [_vp, _vp, _int, _vp, _i64, _f32, _i32]),
    "mb_minmax_f32": (_int, [_vp, _vp, _i64, C.POINTER(_f32), C.POINTER(_f32)]),
    "mb_transpose2d_batched": (_int, [_vp, _vp, _vp, _i64, _i64, _i64, _int]),
    "mb_subsample_f32_nchw": (_int, [_vp, _vp, _vp, _i64, _i64, _i64, _int, _int]),
    "mb_gemm_u8_static_scratch": (_int, [_vp] * 5 + [_int] + [_i64] * 3 + [_int] * 2 +
                                  [_i32] * 5 + [_int, C.c_char_p, _sz]),
    "mb_gemm_u8_static_scratch_status": (_int, [_vp, C.POINTER(_int)]),
    "mb_histogram_f32": (_int, [_vp, _vp, _i64, _f32, _f32, _int, C.POINTER(_i32)]),
    "mb_set_runtime_failure_ratio": (_int, [_f32]),
    "mb_should_mock_runtime_failure": (_int, []),
    "mb_wait_timeout_selftest": (_int, [_vp, C.c_longlong, C.POINTER(C.c_longlong)]),
}

_lib = None


def lib():
    """Load the library; raises if it has not been built (no fallback)."""
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB):
            raise ImportError(
                "libmace_b200.so is missing: run `python -c 'import __graft_entry__ as g; "
                "g.build()'` (or make -C mace_b200/csrc). There is no CPU fallback.")
        _lib = C.CDLL(_LIB)
        for name, (res, args) in PROTOTYPES.items():
            fn = getattr(_lib, name)
            fn.restype = res
            fn.argtypes = args
    return _lib


class DeviceBuffer:
    """A device allocation owned by a Context."""

    def __init__(self, ctx, nbytes):
        self.ctx = ctx
        self.nbytes = int(nbytes)
        p = _vp()
        ctx._check(lib().mb_malloc(ctx.h, max(self.nbytes, 1), C.byref(p)))
        self.ptr = p.value

    def free(self):
        if self.ptr:
            lib().mb_free(self.ctx.h, self.ptr)
            self.ptr = None


class Context:
    """One device context (stream + scratch arena) on a GPU."""

    def __init__(self, device=0):
        self.h = _vp()
        st = lib().mb_init(int(device), C.byref(self.h))
        if st != 0:
            raise MaceB200Error(st, "mb_init failed (no sm_100a CUDA device?)")
        self._bufs = []

    def _check(self, st):
        if st != 0:
            raise MaceB200Error(st, lib().mb_last_error(self.h).decode())

    def close(self):
        if self.h:
            for b in self._bufs:
                b.free()
            for p in getattr(self, "_pinned", []):
                lib().mb_host_free(self.h, p)
            lib().mb_destroy(self.h)
            self.h = None

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    # -- memory ---------------------------------------------------------------
    def alloc(self, nbytes):
        b = DeviceBuffer(self, nbytes)
        self._bufs.append(b)
        return b

    def upload(self, arr):
        """numpy array -> new device buffer (synchronous)."""
        import numpy as np
        arr = np.ascontiguousarray(arr)
        b = self.alloc(arr.nbytes)
        if arr.nbytes:
            self._check(lib().mb_memcpy_h2d(self.h, b.ptr, arr.ctypes.data, arr.nbytes))
            self.sync()
        return b

    def download(self, buf, shape, dtype):
        import numpy as np
        out = np.empty(shape, dtype)
        if out.nbytes:
            self._check(lib().mb_memcpy_d2h(self.h, out.ctypes.data, buf.ptr, out.nbytes))
        self.sync()
        return out

    def sync(self):
        self._check(lib().mb_stream_sync(self.h))

    def event(self):
        e = _vp()
        self._check(lib().mb_event_create(self.h, C.byref(e)))
        return e

    def record(self, event):
        self._check(lib().mb_event_record(self.h, event))

    def elapsed_ms(self, start, stop):
        ms = _f32()
        self._check(lib().mb_event_elapsed_ms(self.h, start, stop, C.byref(ms)))
        return float(ms.value)

    def host_alloc(self, nbytes):
        """Pinned host memory as a numpy uint8 array (freed with the context)."""
        import numpy as np
        p = _vp()
        self._check(lib().mb_host_alloc(self.h, max(int(nbytes), 1), C.byref(p)))
        self._pinned = getattr(self, "_pinned", [])
        self._pinned.append(p.value)
        return np.ctypeslib.as_array((C.c_uint8 * int(nbytes)).from_address(p.value))

    def h2d(self, buf, arr):
        """Asynchronous copy of a (pinned) numpy array into a device buffer."""
        self._check(lib().mb_memcpy_h2d(self.h, buf.ptr, arr.ctypes.data, arr.nbytes))

    def d2h(self, arr, buf):
        self._check(lib().mb_memcpy_d2h(self.h, arr.ctypes.data, buf.ptr, arr.nbytes))

    def set_option(self, name, value):
        self._check(lib().mb_set_option(self.h, name.encode(), int(value)))

    @property
    def launches(self):
        return int(lib().mb_launch_count(self.h))

    @property
    def launches_tensor_core(self):
        return int(lib().mb_launch_count_tensor_core(self.h))

    @property
    def launches_pair(self):
        return int(lib().mb_launch_count_pair(self.h))

    @property
    def stream(self):
        return lib().mb_stream(self.h)

    # -- ops (device pointers in, status checked) --------------------------------
    def gemm_u8(self, A, B, bias, Cout, batch, M, N, K, zp_a, zp_b, mult=1 << 30, shift=0,
                zp_c=0, a_col_major=False, b_col_major=False, c_col_major=False,
                a_batched=True, b_batched=True, out_int32=False, bias_per_row=False):
        self._check(lib().mb_gemm_u8(
            self.h, A.ptr, B.ptr, bias.ptr if bias is not None else None, Cout.ptr,
            int(out_int32), batch, M, N, K, int(a_col_major), int(b_col_major),
            int(c_col_major), int(a_batched), int(b_batched), zp_a, zp_b, mult, shift, zp_c,
            int(bias_per_row)))

    def gemv_u8(self, lhs, rhs, bias, out, batch, rows, K, zp_l, zp_r, multiplier=0.0,
                zp_out=0, add_zp_out=True, lhs_batched=False, rhs_batched=True,
                out_int32=False):
        self._check(lib().mb_gemv_u8(
            self.h, lhs.ptr, rhs.ptr, bias.ptr if bias is not None else None, out.ptr,
            int(out_int32), batch, rows, K, int(lhs_batched), int(rhs_batched), zp_l, zp_r,
            float(multiplier), zp_out, int(add_zp_out)))

    def conv2d_u8(self, x, f, bias, out, N, H, W, Cc, O, KH, KW, strides, pad_tl, out_hw,
                  zp_in, zp_f, mult, shift, zp_out):
        self._check(lib().mb_conv2d_u8_nhwc(
            self.h, x.ptr, f.ptr, bias.ptr if bias is not None else None, out.ptr, N, H, W, Cc,
            O, KH, KW, strides[0], strides[1], pad_tl[0], pad_tl[1], out_hw[0], out_hw[1],
            zp_in, zp_f, mult, shift, zp_out))

    def dwconv3x3_u8_prepack(self, f, bias, Cc, zp_in, zp_f):
        """Returns a device buffer with the fast path's tap words for a constant filter."""
        nbytes = lib().mb_dwconv3x3_u8_prepacked_bytes(Cc)
        if nbytes == 0:
            raise ValueError("channel count not eligible for the 3x3 fast path")
        packed = self.alloc(nbytes)
        self._check(lib().mb_dwconv3x3_u8_prepack(
            self.h, f.ptr, bias.ptr if bias is not None else None, Cc, zp_in, zp_f, packed.ptr))
        return packed

    def dwconv_u8(self, x, f, bias, out, N, H, W, Cc, Mc, KH, KW, strides, dil, pad_tl, out_hw,
                  zp_in, zp_f, mult=1 << 30, shift=0, zp_out=0, float_multiplier=None,
                  prepacked=None):
        if prepacked is not None:
            self._check(lib().mb_dwconv_u8_nhwc_prepacked(
                self.h, x.ptr, f.ptr, bias.ptr if bias is not None else None, prepacked.ptr,
                out.ptr, N, H, W, Cc, Mc, KH, KW, strides[0], strides[1], dil[0], dil[1],
                pad_tl[0], pad_tl[1], out_hw[0], out_hw[1], zp_in, zp_f, mult, shift, zp_out,
                int(float_multiplier is not None), float(float_multiplier or 0.0)))
            return
        self._check(lib().mb_dwconv_u8_nhwc(
            self.h, x.ptr, f.ptr, bias.ptr if bias is not None else None, out.ptr, N, H, W, Cc,
            Mc, KH, KW, strides[0], strides[1], dil[0], dil[1], pad_tl[0], pad_tl[1],
            out_hw[0], out_hw[1], zp_in, zp_f, mult, shift, zp_out,
            int(float_multiplier is not None), float(float_multiplier or 0.0)))

    def gemm_f32(self, A, B, Cout, batch, M, N, K, a_col_major=False, b_col_major=False,
                 c_col_major=False, a_batched=True, b_batched=True):
        self._check(lib().mb_gemm_f32(self.h, A.ptr, B.ptr, Cout.ptr, batch, M, N, K,
                                      int(a_col_major), int(b_col_major), int(c_col_major),
                                      int(a_batched), int(b_batched)))

    def gemv_f32(self, lhs, rhs, bias, out, batch, rows, K, lhs_batched=False, rhs_batched=True):
        self._check(lib().mb_gemv_f32(self.h, lhs.ptr, rhs.ptr,
                                      bias.ptr if bias is not None else None, out.ptr, batch,
                                      rows, K, int(lhs_batched), int(rhs_batched)))

    def conv2d_f32(self, x, f, bias, out, N, Cc, H, W, O, KH, KW, strides, dil, pad_tl, out_hw,
                   act=0, max_limit=0.0, coef=0.0):
        self._check(lib().mb_conv2d_f32_nchw(
            self.h, x.ptr, f.ptr, bias.ptr if bias is not None else None, out.ptr, N, Cc, H, W,
            O, KH, KW, strides[0], strides[1], dil[0], dil[1], pad_tl[0], pad_tl[1], out_hw[0],
            out_hw[1], act, max_limit, coef))

    def conv2d_f32_residual(self, x, f, bias, residual, out, N, Cc, H, W, O, KH, KW, strides, dil, pad_tl,
                            out_hw, act=0, max_limit=0.0, coef=0.0):
        self._check(lib().mb_conv2d_f32_nchw_residual(
            self.h, x.ptr, f.ptr, bias.ptr if bias is not None else None, residual.ptr, out.ptr, N, Cc, H,
            W, O, KH, KW, strides[0], strides[1], dil[0], dil[1], pad_tl[0], pad_tl[1], out_hw[0],
            out_hw[1], act, max_limit, coef))

    def dwconv_f32(self, x, f, bias, out, N, Cc, H, W, Mc, KH, KW, strides, dil, pad_tl, out_hw,
                   act=0, max_limit=0.0, coef=0.0):
        self._check(lib().mb_dwconv_f32_nchw(
            self.h, x.ptr, f.ptr, bias.ptr if bias is not None else None, out.ptr, N, Cc, H, W,
            Mc, KH, KW, strides[0], strides[1], dil[0], dil[1], pad_tl[0], pad_tl[1], out_hw[0],
            out_hw[1], act, max_limit, coef))

    def winograd_f32(self, x, f, bias, out, N, Cc, H, W, O, pad_tl, out_hw, act=0, max_limit=0.0,
                     coef=0.0, tile=0, transformed=None):
        self._check(lib().mb_conv3x3_winograd_f32_nchw(
            self.h, x.ptr, f.ptr if f is not None else None,
            transformed.ptr if transformed is not None else None,
            bias.ptr if bias is not None else None, out.ptr, N, Cc, H, W, O, pad_tl[0],
            pad_tl[1], out_hw[0], out_hw[1], act, max_limit, coef, tile))

    def winograd_transform_filter(self, f, out, Cc, O, tile):
        self._check(lib().mb_winograd_transform_filter_f32(self.h, f.ptr, out.ptr, Cc, O, tile))

    def pooling_f32(self, x, out, N, Cc, H, W, kernel, strides, dil, pad_tl, out_hw, pooling_type):
        self._check(lib().mb_pooling_f32_nchw(
            self.h, x.ptr, out.ptr, N, Cc, H, W, kernel[0], kernel[1], strides[0], strides[1],
            dil[0], dil[1], pad_tl[0], pad_tl[1], out_hw[0], out_hw[1], pooling_type))

    def eltwise_f32(self, a, b, out, size, type_, coeff=None, swapped=False, scalar=1.0, act=0,
                    max_limit=0.0, coef=0.0):
        c = coeff if coeff else (0.0, 0.0)
        self._check(lib().mb_eltwise_act_f32(
            self.h, a.ptr, b.ptr if b is not None else None, out.ptr, size, type_, scalar,
            1 if coeff else 0, c[0], c[1], 1 if swapped else 0, act, max_limit, coef))

    def activation_f32(self, x, out, size, act, max_limit=0.0, coef=0.0):
        self._check(lib().mb_activation_f32(self.h, x.ptr, out.ptr, size, act, max_limit, coef))

    def softmax_f32(self, x, out, outer, classes, inner, use_log=False):
        self._check(lib().mb_softmax_f32(self.h, x.ptr, out.ptr, outer, classes, inner,
                                         1 if use_log else 0))

    def quantize_f32_u8(self, x, out, size, scale, zero_point):
        self._check(lib().mb_quantize_f32_u8(self.h, x.ptr, out.ptr, size, scale, zero_point))

    def dequantize_f32(self, q, out, size, scale, zero_point, int32=False):
        self._check(lib().mb_dequantize_f32(self.h, q.ptr, 1 if int32 else 0, out.ptr, size, scale,
                                            zero_point))

    def minmax_f32(self, x, size):
        mn, mx = _f32(), _f32()
        self._check(lib().mb_minmax_f32(self.h, x.ptr, size, C.byref(mn), C.byref(mx)))
        return mn.value, mx.value

    def subsample_f32(self, x, out, planes, H, W, strides):
        """out[p][ho][wo] = x[p][ho * sh][wo * sw]."""
        self._check(lib().mb_subsample_f32_nchw(self.h, x.ptr, out.ptr, planes, H, W, strides[0], strides[1]))

    def transpose2d_batched(self, x, out, batch, rows, cols, elem_bytes):
        """out[b][c][r] = x[b][r][c]; NHWC -> NCHW is rows = H * W, cols = C."""
        self._check(lib().mb_transpose2d_batched(self.h, x.ptr, out.ptr, batch, rows, cols, elem_bytes))

    def avgpool_u8(self, x, out, N, H, W, Cc, kernel, strides, pad_tl, out_hw):
        self._check(lib().mb_avgpool_u8_nhwc(
            self.h, x.ptr, out.ptr, N, H, W, Cc, kernel[0], kernel[1], strides[0], strides[1],
            pad_tl[0], pad_tl[1], out_hw[0], out_hw[1]))
