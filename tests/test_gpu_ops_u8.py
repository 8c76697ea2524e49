"""uint8 GEMV, Conv2D, DepthwiseConv2d and pooling on the GPU against the CPU oracle
(bit-exact), including the reference's two quantized known-answer tests."""
import numpy as np
import pytest

from helpers import conv_quant

pytestmark = pytest.mark.gpu

PAD = {"VALID": 0, "SAME": 1, "FULL": 2}


@pytest.fixture(scope="module")
def ctx():
    import mace_b200
    c = mace_b200.Context(0)
    yield c
    c.close()


# ---- known-answer tests through the C ABI ---------------------------------------

def test_conv2d_kat_230(ctx, orc, kats):
    k = kats["conv2d_u8_3x3"]
    x = np.array(k["input"], np.uint8).reshape(k["input_nhwc_shape"])
    f = np.array(k["filter"], np.uint8).reshape(k["filter_ohwi_shape"])
    bias = orc.get_bias_data(np.array(k["bias"], np.int32), k["bias_scale"], k["input_scale"],
                             k["filter_scale"], 1)
    mult, shift = orc.output_multiplier_and_shift(k["filter_scale"], k["input_scale"],
                                                  k["output_scale"])
    dx, df, db, do = ctx.upload(x), ctx.upload(f), ctx.upload(bias), ctx.alloc(16)
    ctx.conv2d_u8(dx, df, db, do, 1, 3, 3, 2, 1, 3, 3, (1, 1), (0, 0), (1, 1), k["input_zp"],
                  k["filter_zp"], mult, shift, k["output_zp"])
    assert ctx.download(do, (1,), np.uint8).tolist() == k["expected"]


def test_dwconv_kat_255_21(ctx, orc, kats):
    k = kats["dwconv_u8_3x3"]
    x = np.array(k["input"], np.uint8).reshape(k["input_nhwc_shape"])
    f = np.array(k["filter"], np.uint8).reshape(k["filter_hwim_shape"])
    bias = orc.get_bias_data(np.array(k["bias"], np.int32), k["bias_scale"], k["input_scale"],
                             k["filter_scale"], 2)
    mult, shift = orc.output_multiplier_and_shift(k["input_scale"], k["filter_scale"],
                                                  k["output_scale"])
    dx, df, db, do = ctx.upload(x), ctx.upload(f), ctx.upload(bias), ctx.alloc(16)
    ctx.dwconv_u8(dx, df, db, do, 1, 3, 3, 2, 1, 3, 3, (1, 1), (1, 1), (0, 0), (1, 1),
                  k["input_zp"], k["filter_zp"], mult, shift, k["output_zp"])
    assert ctx.download(do, (2,), np.uint8).tolist() == k["expected"]


# ---- GEMV --------------------------------------------------------------------------

@pytest.mark.parametrize("shape", [(1, 16, 4), (1, 16, 256), (2, 16, 256), (3, 63, 257),
                                   (1, 4096, 4096), (64, 1000, 1024), (1, 256, 30000)])
@pytest.mark.parametrize("lhs_batched", [False, True])
def test_gemv_u8(ctx, orc, shape, lhs_batched):
    """Shapes of test/ccunit/mace/ops/arm/q8/gemv_test.cc plus the FullyConnected and the
    M=1 sweep shapes; uint8 (both zero-point formulas) and int32 outputs."""
    batch, rows, K = shape
    if lhs_batched and batch * rows * K > (1 << 26):
        pytest.skip("batched copy of the matrix not needed at this size")
    rng = np.random.Generator(np.random.PCG64(rows * 7 + K))
    lhs = rng.integers(0, 256, size=((batch if lhs_batched else 1), rows, K), dtype=np.uint8)
    rhs = rng.integers(0, 256, size=(batch, K), dtype=np.uint8)
    bias = np.rint(rng.normal(0, 1000, size=rows)).astype(np.int32)
    zl, zr = 127, 128
    mult = np.float32(1.0 / (np.sqrt(K) * 74 * 74 * 3 / 127))
    dl, dr, db = ctx.upload(lhs), ctx.upload(rhs), ctx.upload(bias)
    do = ctx.alloc(batch * rows * 4)
    for add_zp in (True, False):
        ctx.gemv_u8(dl, dr, db, do, batch, rows, K, zl, zr, mult, 31, add_zp,
                    lhs_batched=lhs_batched)
        got = ctx.download(do, (batch * rows,), np.uint8)
        exp = orc.gemv_u8(lhs, rhs, bias, batch, rows, K, zl, zr, mult, 31, add_zp,
                          lhs_batched=lhs_batched)
        assert np.array_equal(got, exp)
        assert len(np.unique(got)) > 2
    ctx.gemv_u8(dl, dr, None, do, batch, rows, K, zl, zr, lhs_batched=lhs_batched,
                out_int32=True)
    got = ctx.download(do, (batch * rows,), np.int32)
    exp = orc.gemv_u8(lhs, rhs, None, batch, rows, K, zl, zr, lhs_batched=lhs_batched,
                      out_int32=True)
    assert np.array_equal(got, exp)
    for b in (dl, dr, db, do):
        b.free()


@pytest.mark.parametrize("shape", [(4096, 4096), (1000, 1024), (300, 4112), (777, 20000), (5000, 256),
                                   (296, 65536), (1201, 8192)])
def test_gemv_u8_streaming_kernel(ctx, orc, shape):
    """One vector against a large matrix runs through the bulk-copy streaming kernel (a ring of
    row chunks per warp): rows that are not a multiple of the warp count, K below, equal to and
    above the chunk size, with a ragged last chunk; the same bytes as the warp-per-row kernel,
    and as the oracle."""
    rows, K = shape
    rng = np.random.Generator(np.random.PCG64(rows + K))
    lhs = rng.integers(0, 256, size=(1, rows, K), dtype=np.uint8)
    rhs = rng.integers(0, 256, size=(1, K), dtype=np.uint8)
    bias = np.rint(rng.normal(0, 1000, size=rows)).astype(np.int32)
    mult = np.float32(1.0 / (np.sqrt(K) * 74 * 74 * 3 / 127))
    dl, dr, db, do = ctx.upload(lhs), ctx.upload(rhs), ctx.upload(bias), ctx.alloc(rows * 4 + 64)
    L = __import__("mace_b200").lib()
    for zl, zr, add_zp, out_int32 in ((127, 128, True, False), (0, 255, False, False), (120, 0, True, True)):
        exp = orc.gemv_u8(lhs, rhs, bias, 1, rows, K, zl, zr, mult, 31, add_zp, out_int32=out_int32)
        got = {}
        for stream in (1, 0):
            ctx.set_option("gemv_stream", stream)
            try:
                ctx._check(L.mb_memset(ctx.h, do.ptr, 0xA5, do.nbytes))
                before = ctx.launches
                ctx.gemv_u8(dl, dr, db, do, 1, rows, K, zl, zr, mult, 31, add_zp, out_int32=out_int32)
                assert ctx.launches == before + 1
                raw = ctx.download(do, (do.nbytes,), np.uint8)
            finally:
                ctx.set_option("gemv_stream", 1)
            n = rows * (4 if out_int32 else 1)
            assert (raw[n:] == 0xA5).all(), "wrote past the output"
            got[stream] = raw[:n].view(np.int32 if out_int32 else np.uint8)
            assert np.array_equal(got[stream], exp), (stream, zl, zr)
    ctx.sync()
    for b in (dl, dr, db, do):
        b.free()


def test_gemv_u8_chain_with_constant_matrices(ctx, orc):
    """A stack of one-vector products, each consuming the previous one's output, with the
    matrices declared constant (what the Gemv delegator does for weight tensors): the kernels
    fetch their first matrix bytes ahead of the dependency wait, the vector only after it.
    Every stage must equal the oracle chain, also when replayed from a graph."""
    import ctypes
    rows = K = 1024
    depth = 6
    rng = np.random.Generator(np.random.PCG64(77))
    mats = [rng.integers(0, 256, size=(1, rows, K), dtype=np.uint8) for _ in range(depth)]
    x0 = rng.integers(0, 256, size=(1, K), dtype=np.uint8)
    mult = np.float32(1.0 / (np.sqrt(K) * 74))  # keeps the spread of the values from stage to stage
    exp, v = [], x0
    for m in mats:
        v = orc.gemv_u8(m, v, None, 1, rows, K, 127, 128, mult, 128, True).reshape(1, K)
        exp.append(v.copy())
    assert len({e.tobytes() for e in exp}) == depth and all(e.std() > 30 for e in exp), "degenerate chain"
    dm = [ctx.upload(m) for m in mats]
    acts = [ctx.upload(x0)] + [ctx.alloc(rows) for _ in range(depth)]
    L = __import__("mace_b200").lib()

    def enqueue():
        for i in range(depth):
            ctx.gemv_u8(dm[i], acts[i], None, acts[i + 1], 1, rows, K, 127, 128, mult, 128, True)

    ctx.set_option("gemv_lhs_const", 1)
    try:
        enqueue()
        for i in range(depth):
            assert np.array_equal(ctx.download(acts[i + 1], (1, K), np.uint8), exp[i]), i
        ctx._check(L.mb_graph_begin(ctx.h))
        enqueue()
        graph = ctypes.c_void_p()
        ctx._check(L.mb_graph_end(ctx.h, ctypes.byref(graph)))
        for _ in range(3):
            for a in acts[1:]:
                ctx._check(L.mb_memset(ctx.h, a.ptr, 0, a.nbytes))
            ctx._check(L.mb_graph_launch(ctx.h, graph))
            for i in range(depth):
                assert np.array_equal(ctx.download(acts[i + 1], (1, K), np.uint8), exp[i]), i
        ctx._check(L.mb_graph_destroy(ctx.h, graph))
    finally:
        ctx.set_option("gemv_lhs_const", 0)
    ctx.sync()
    for b in dm + acts:
        b.free()


# ---- Conv2D ------------------------------------------------------------------------
# shapes in the style of conv_2d_test.cc:1348-1397: N, H, W, C, O, KH, KW, stride, padding

def _conv_case(ctx, orc, N, H, W, C, O, KH, KW, stride, padding, seed=0):
    rng = np.random.Generator(np.random.PCG64(seed + H * 131 + C))
    x, f, zp_in, zp_f, mult, shift = conv_quant(orc, rng, (N, H, W, C), (O, KH, KW, C),
                                                C * KH * KW)
    bias = np.rint(rng.normal(0, 2000, size=O)).astype(np.int32)
    Ho, Wo, ph, pw = orc.calc_padding_and_output_size(H, W, KH, KW, (1, 1), (stride, stride),
                                                      PAD[padding])
    zp_out = int(rng.integers(96, 161))
    exp = orc.conv2d_u8(x, f, bias, (stride, stride), (ph, pw), (Ho, Wo), zp_in, zp_f, mult,
                        shift, zp_out)
    dx, df, db = ctx.upload(x), ctx.upload(f), ctx.upload(bias)
    do = ctx.alloc(exp.size)
    ctx.conv2d_u8(dx, df, db, do, N, H, W, C, O, KH, KW, (stride, stride), (ph >> 1, pw >> 1),
                  (Ho, Wo), zp_in, zp_f, mult, shift, zp_out)
    got = ctx.download(do, exp.shape, np.uint8)
    for b in (dx, df, db, do):
        b.free()
    assert np.array_equal(got, exp)
    assert len(np.unique(got)) > min(4, got.size // 2)
    return got


@pytest.mark.parametrize("case", [
    (1, 2, 3, 3, 1, 1, 1, 1, "VALID"),
    (1, 16, 16, 64, 64, 1, 1, 1, "VALID"),
    (9, 7, 9, 32, 128, 1, 1, 1, "SAME"),
    (1, 32, 32, 3, 32, 3, 3, 2, "SAME"),      # MobileNet stem shape (reduced size)
    (2, 17, 19, 3, 10, 3, 3, 1, "VALID"),     # 3-channel input, O not a multiple of 4
    (1, 9, 9, 3, 7, 3, 3, 3, "SAME"),
    (2, 17, 19, 32, 64, 3, 3, 1, "SAME"),     # patch gather + tensor-core GEMM
    (1, 31, 33, 16, 24, 3, 3, 2, "VALID"),
    (1, 15, 17, 8, 16, 5, 5, 1, "FULL"),
    (1, 12, 12, 64, 96, 3, 3, 3, "SAME"),
    (1, 9, 11, 5, 7, 1, 5, 1, "SAME"),
    (1, 9, 11, 5, 7, 5, 1, 2, "VALID"),
    (1, 20, 20, 16, 17, 7, 7, 2, "SAME"),
])
def test_conv2d_u8(ctx, orc, case):
    _conv_case(ctx, orc, *case)


def test_conv2d_u8_pointwise_uses_tensor_core(ctx, orc):
    before = ctx.launches_tensor_core
    _conv_case(ctx, orc, 2, 28, 28, 256, 256, 1, 1, 1, "VALID")
    assert ctx.launches_tensor_core == before + 1


@pytest.mark.parametrize("case", [
    # N, H, W, O, stride, padding, zp_in, zp_out  (None: drawn by the case)
    (1, 32, 32, 32, 4, "SAME", None, None),      # 64 output pixels: below one group, integer kernel both times
    (1, 16, 16, 32, 1, "SAME", None, None),      # exactly two groups of 128 pixels
    (2, 32, 32, 32, 1, "SAME", None, None),
    (1, 224, 224, 32, 2, "SAME", None, None),    # MobileNet stem at full size
    (3, 17, 23, 16, 2, "VALID", None, None),     # ragged last group, narrowest channel count
    (2, 9, 9, 64, 1, "SAME", None, None),
    (1, 30, 30, 256, 2, "SAME", None, None),     # widest channel count (whole accumulator block)
    (1, 40, 36, 48, 1, "VALID", None, None),     # accumulator columns rounded up to 64
    (2, 64, 64, 32, 2, "SAME", 0, 0),
    (2, 64, 64, 32, 2, "SAME", 255, 255),        # padding bytes and outputs at the top of the range
    (200, 3, 3, 32, 1, "VALID", None, None),     # one output pixel per image: row and column divisors of 1
    (2, 13, 131, 32, 1, "SAME", None, None),     # prime row length, borders on every side
])
def test_conv2d_u8_three_channel_stem_on_tensor_cores(ctx, orc, case):
    """A 3x3 filter over 3 channels runs as one 128 x O x 32 tensor-core product per 128 pixels; the
    integer kernel it replaces stays selectable.  Both must equal the reference arithmetic
    (conv_2d.cc:206-318 of the reference's quantized Conv2d) and leave the bytes behind the output
    alone."""
    N, H, W, O, stride, padding, zi_forced, zo_forced = case
    rng = np.random.Generator(np.random.PCG64(H * 131 + O))
    x, f, zp_in, zp_f, mult, shift = conv_quant(orc, rng, (N, H, W, 3), (O, 3, 3, 3), 27)
    if zi_forced is not None:
        zp_in = zi_forced
    bias = np.rint(rng.normal(0, 2000, size=O)).astype(np.int32)
    Ho, Wo, ph, pw = orc.calc_padding_and_output_size(H, W, 3, 3, (1, 1), (stride, stride),
                                                      PAD[padding])
    zp_out = int(rng.integers(96, 161)) if zo_forced is None else zo_forced
    exp = orc.conv2d_u8(x, f, bias, (stride, stride), (ph, pw), (Ho, Wo), zp_in, zp_f, mult,
                        shift, zp_out)
    dx, df, db = ctx.upload(x), ctx.upload(f), ctx.upload(bias)
    do = ctx.alloc(exp.size + 64)
    import mace_b200
    L = mace_b200.lib()
    try:
        for tc in (1, 0):
            ctx.set_option("stem_tc", tc)
            ctx._check(L.mb_memset(ctx.h, do.ptr, 0xA5, do.nbytes))
            before = ctx.launches
            ctx.conv2d_u8(dx, df, db, do, N, H, W, 3, O, 3, 3, (stride, stride),
                          (ph >> 1, pw >> 1), (Ho, Wo), zp_in, zp_f, mult, shift, zp_out)
            assert ctx.launches == before + 1
            raw = ctx.download(do, (do.nbytes,), np.uint8)
            assert np.array_equal(raw[:exp.size].reshape(exp.shape), exp), "stem_tc=%d" % tc
            assert (raw[exp.size:] == 0xA5).all()
        ctx.sync()   # raises if a block gave up its bounded wait
    finally:
        ctx.set_option("stem_tc", 1)
        for b in (dx, df, db, do):
            b.free()
    assert len(np.unique(exp)) > 4


@pytest.mark.parametrize("case", [
    # N, H, W, C, O, zp_in, zp_out, bias
    (2, 112, 112, 32, 64, None, None, True),     # MobileNet's first pointwise layer (reduced batch)
    (6, 56, 57, 64, 128, None, None, True),      # depth 64: two products per group of pixels
    (3, 80, 80, 128, 128, None, None, True),     # depth 128
    (1, 150, 127, 32, 16, None, None, True),     # ragged last group, narrowest channel count
    (2, 100, 100, 64, 48, None, None, True),     # accumulator columns rounded up
    (1, 139, 137, 128, 80, None, None, True),
    (2, 112, 112, 32, 64, 0, 0, False),          # no bias, zero points 0 (the packed requantization)
    (2, 112, 112, 64, 128, 255, 255, True),
    (2, 112, 112, 32, 32, None, None, True),
])
def test_conv2d_u8_pointwise_with_short_depth(ctx, orc, case):
    """Pointwise layers of depth 32 (by default), 64 and 128 (by option) can run on the
    thread-per-pixel tensor-core kernel instead of the persistent GEMM: both must equal the
    reference arithmetic (conv_2d.cc:206-318) and leave the bytes behind the output alone."""
    import mace_b200
    N, H, W, C, O, zi_forced, zo_forced, with_bias = case
    rng = np.random.Generator(np.random.PCG64(H * 131 + O + C))
    x, f, zp_in, zp_f, mult, shift = conv_quant(orc, rng, (N, H, W, C), (O, 1, 1, C), C)
    if zi_forced is not None:
        zp_in = zi_forced
    bias = np.rint(rng.normal(0, 2000, size=O)).astype(np.int32) if with_bias else None
    zp_out = int(rng.integers(96, 161)) if zo_forced is None else zo_forced
    exp = orc.conv2d_u8(x, f, bias, (1, 1), (0, 0), (H, W), zp_in, zp_f, mult, shift, zp_out)
    dx, df = ctx.upload(x), ctx.upload(f)
    db = ctx.upload(bias) if with_bias else None
    do = ctx.alloc(exp.size + 64)
    L = mace_b200.lib()
    try:
        for level in (3, 0):
            ctx.set_option("thin_pw", level)
            ctx._check(L.mb_memset(ctx.h, do.ptr, 0xA5, do.nbytes))
            tc_before = ctx.launches_tensor_core
            ctx.conv2d_u8(dx, df, db, do, N, H, W, C, O, 1, 1, (1, 1), (0, 0), (H, W), zp_in, zp_f,
                          mult, shift, zp_out)
            # (the persistent GEMM counts as a tensor-core GEMM launch, the per-pixel kernel does not)
            assert (ctx.launches_tensor_core == tc_before) == (level == 3)
            raw = ctx.download(do, (do.nbytes,), np.uint8)
            assert np.array_equal(raw[:exp.size].reshape(exp.shape), exp), "thin_pw=%d" % level
            assert (raw[exp.size:] == 0xA5).all()
        ctx.sync()   # raises if a block gave up its bounded wait
    finally:
        ctx.set_option("thin_pw", 1)
        for b in (dx, df, db, do):
            if b is not None:
                b.free()
    assert len(np.unique(exp)) > 4


def test_conv2d_u8_thread_per_pixel_grid_multiples(ctx, orc):
    """More blocks than are resident at once (option stem_grid) change no byte."""
    try:
        for g in (2, 3):
            ctx.set_option("stem_grid", g)
            _conv_case(ctx, orc, 2, 224, 224, 3, 32, 3, 3, 2, "SAME")
            _conv_case(ctx, orc, 2, 112, 112, 32, 64, 1, 1, 1, "VALID")
    finally:
        ctx.set_option("stem_grid", 1)


def test_conv2d_u8_weights_read_before_the_wait(ctx, orc):
    """With the filter declared constant the thread-per-pixel kernels fetch it before they wait for
    the kernel in front; a chain of such convolutions (each reads the previous one's output) must
    still equal the oracle."""
    rng = np.random.Generator(np.random.PCG64(5))
    N, H, W = 2, 112, 112
    x, f1, zp_in, zp_f1, mult1, shift1 = conv_quant(orc, rng, (N, H, W, 32), (32, 1, 1, 32), 32)
    f2 = rng.integers(0, 256, size=(64, 1, 1, 32), dtype=np.uint8)
    y1 = orc.conv2d_u8(x, f1, None, (1, 1), (0, 0), (H, W), zp_in, zp_f1, mult1, shift1, 0)
    y2 = orc.conv2d_u8(y1, f2, None, (1, 1), (0, 0), (H, W), 0, 119, mult1, shift1, 3)
    dx, d1, d2 = ctx.upload(x), ctx.upload(f1), ctx.upload(f2)
    o1, o2 = ctx.alloc(y1.size), ctx.alloc(y2.size)
    try:
        ctx.set_option("conv_filter_const", 1)
        for _ in range(3):
            ctx.conv2d_u8(dx, d1, None, o1, N, H, W, 32, 32, 1, 1, (1, 1), (0, 0), (H, W), zp_in, zp_f1,
                          mult1, shift1, 0)
            ctx.conv2d_u8(o1, d2, None, o2, N, H, W, 32, 64, 1, 1, (1, 1), (0, 0), (H, W), 0, 119,
                          mult1, shift1, 3)
        assert np.array_equal(ctx.download(o1, y1.shape, np.uint8), y1)
        assert np.array_equal(ctx.download(o2, y2.shape, np.uint8), y2)
    finally:
        ctx.set_option("conv_filter_const", 0)
        for b in (dx, d1, d2, o1, o2):
            b.free()


def test_conv2d_u8_three_channel_input_off_the_word_grid(ctx, orc):
    """The word-wise window loads of the 3x3x3 kernels need a 4-byte aligned input; any other input
    address takes the byte-wise gather and must give the same bytes."""
    import types
    rng = np.random.Generator(np.random.PCG64(77))
    N, H, W, O = 2, 20, 24, 32
    x, f, zp_in, zp_f, mult, shift = conv_quant(orc, rng, (N, H, W, 3), (O, 3, 3, 3), 27)
    Ho, Wo, ph, pw = orc.calc_padding_and_output_size(H, W, 3, 3, (1, 1), (1, 1), PAD["SAME"])
    exp = orc.conv2d_u8(x, f, None, (1, 1), (ph, pw), (Ho, Wo), zp_in, zp_f, mult, shift, 90)
    raw = np.zeros(x.size + 8, np.uint8)
    df, do = ctx.upload(f), ctx.alloc(exp.size)
    try:
        for shift_bytes in (1, 2, 3):
            raw[:] = 0
            raw[shift_bytes:shift_bytes + x.size] = x.reshape(-1)
            dx = ctx.upload(raw)
            view = types.SimpleNamespace(ptr=dx.ptr + shift_bytes)
            for tc in (1, 0):
                ctx.set_option("stem_tc", tc)
                ctx.conv2d_u8(view, df, None, do, N, H, W, 3, O, 3, 3, (1, 1), (ph >> 1, pw >> 1),
                              (Ho, Wo), zp_in, zp_f, mult, shift, 90)
                assert np.array_equal(ctx.download(do, exp.shape, np.uint8), exp), (shift_bytes, tc)
            dx.free()
    finally:
        ctx.set_option("stem_tc", 1)
        df.free()
        do.free()


# ---- DepthwiseConv2d ---------------------------------------------------------------

@pytest.mark.parametrize("case", [
    # N, H, W, C, mult, KH, KW, stride, dilation, padding   (depthwise_conv2d_test.cc:464-492)
    (1, 56, 56, 128, 1, 3, 3, 1, 1, "SAME"),
    (3, 28, 28, 128, 1, 3, 3, 2, 1, "SAME"),
    (1, 14, 14, 512, 1, 3, 3, 1, 1, "VALID"),
    (2, 7, 7, 1024, 1, 3, 3, 1, 1, "SAME"),
    (1, 33, 31, 32, 1, 3, 3, 2, 1, "SAME"),
    (1, 9, 5, 36, 1, 3, 3, 1, 1, "FULL"),
    (1, 13, 14, 12, 2, 3, 3, 1, 1, "SAME"),     # channel multiplier 2 -> general kernel
    (1, 13, 14, 7, 1, 5, 5, 2, 1, "SAME"),
    (1, 15, 15, 16, 1, 3, 3, 1, 2, "SAME"),     # dilated -> float-multiplier rule
])
def test_dwconv_u8(ctx, orc, case):
    N, H, W, C, mc, KH, KW, stride, dil, padding = case
    rng = np.random.Generator(np.random.PCG64(H * 17 + C))
    x, f, zp_in, zp_f, mult, shift = conv_quant(orc, rng, (N, H, W, C), (KH, KW, C, mc), KH * KW)
    bias = np.rint(rng.normal(0, 500, size=C * mc)).astype(np.int32)
    Ho, Wo, ph, pw = orc.calc_padding_and_output_size(H, W, KH, KW, (dil, dil), (stride, stride),
                                                      PAD[padding])
    zp_out = int(rng.integers(96, 161))
    args = (x, f, bias, (stride, stride), (dil, dil), (ph >> 1, pw >> 1), (Ho, Wo), zp_in, zp_f)
    dx, df, db = ctx.upload(x), ctx.upload(f), ctx.upload(bias)
    do = ctx.alloc(N * Ho * Wo * C * mc)
    if dil == 1:
        exp = orc.dwconv_u8(*args, mult, shift, zp_out)
        ctx.dwconv_u8(dx, df, db, do, N, H, W, C, mc, KH, KW, (stride, stride), (dil, dil),
                      (ph >> 1, pw >> 1), (Ho, Wo), zp_in, zp_f, mult, shift, zp_out)
    else:
        mf = np.float32(1.0 / (3 * 74 * 74 * 3 / 127))
        exp = orc.dwconv_u8_general(*args, mf, zp_out)
        ctx.dwconv_u8(dx, df, db, do, N, H, W, C, mc, KH, KW, (stride, stride), (dil, dil),
                      (ph >> 1, pw >> 1), (Ho, Wo), zp_in, zp_f, zp_out=zp_out,
                      float_multiplier=mf)
    got = ctx.download(do, exp.shape, np.uint8)
    for b in (dx, df, db, do):
        b.free()
    assert np.array_equal(got, exp)
    assert len(np.unique(got)) > 4


@pytest.mark.parametrize("stride", [1, 2])
@pytest.mark.parametrize("variant", ["zp_out_0", "shift_0", "shift_0_zp_out_0", "filter_zp_far", "huge_bias",
                                     "input_zp_0"])
def test_dwconv_u8_3x3_variants(ctx, orc, stride, variant):
    """The 3x3 fast path over its requantization variants (output zero point 0, shift 0), a
    filter zero point far from 128 (weights beyond the signed 8-bit range in most channels),
    accumulators near the int32 limits, and ragged sizes (W not a multiple of 4, odd H)."""
    N, H, W, C = 3, 23, 21, 40
    rng = np.random.Generator(np.random.PCG64(stride * 7 + len(variant)))
    x = rng.integers(0, 256, size=(N, H, W, C), dtype=np.uint8)
    f = rng.integers(0, 256, size=(3, 3, C, 1), dtype=np.uint8)
    zp_in, zp_f, zp_out = 131, 127, 77
    bias = np.rint(rng.normal(0, 500, size=C)).astype(np.int32)
    scale = 0.02 * 0.01 * 3 * 74 * 74 * 3 / 127
    if variant in ("zp_out_0", "shift_0_zp_out_0"):
        zp_out = 0
    if variant == "filter_zp_far":
        zp_f = 40
    if variant == "input_zp_0":
        zp_in = 0
    if variant == "huge_bias":
        bias = rng.integers(-2 ** 31 + 600000, 2 ** 31 - 600000, size=C, dtype=np.int64).astype(np.int32)
        bias[::3] = np.rint(rng.normal(0, 500, size=bias[::3].size)).astype(np.int32)
    mult, shift = orc.output_multiplier_and_shift(np.float32(0.02), np.float32(0.01), np.float32(scale))
    if variant.startswith("shift_0"):
        shift = 0
        x = rng.integers(126, 137, size=(N, H, W, C), dtype=np.uint8)  # small accumulators
    Ho, Wo, ph, pw = orc.calc_padding_and_output_size(H, W, 3, 3, (1, 1), (stride, stride), PAD["SAME"])
    exp = orc.dwconv_u8(x, f, bias, (stride, stride), (1, 1), (ph >> 1, pw >> 1), (Ho, Wo), zp_in,
                        zp_f, mult, shift, zp_out)
    dx, df, db = ctx.upload(x), ctx.upload(f), ctx.upload(bias)
    do = ctx.alloc(exp.size)
    ctx.dwconv_u8(dx, df, db, do, N, H, W, C, 1, 3, 3, (stride, stride), (1, 1), (ph >> 1, pw >> 1),
                  (Ho, Wo), zp_in, zp_f, mult, shift, zp_out)
    got = ctx.download(do, exp.shape, np.uint8)
    # the same through a prepacked filter (what the delegator caches for weights), twice
    packed = ctx.dwconv3x3_u8_prepack(df, db, C, zp_in, zp_f)
    for _ in range(2):
        ctx._check(__import__("mace_b200").lib().mb_memset(ctx.h, do.ptr, 0, do.nbytes))
        ctx.dwconv_u8(dx, df, db, do, N, H, W, C, 1, 3, 3, (stride, stride), (1, 1),
                      (ph >> 1, pw >> 1), (Ho, Wo), zp_in, zp_f, mult, shift, zp_out, prepacked=packed)
        assert np.array_equal(ctx.download(do, exp.shape, np.uint8), exp)
    for b in (dx, df, db, do, packed):
        b.free()
    assert np.array_equal(got, exp)
    assert len(np.unique(got)) > 4


@pytest.mark.parametrize("stride", [1, 2])
@pytest.mark.parametrize("zp_in", [0, 129])      # 0: rows through shared memory by TMA; else the register kernel
@pytest.mark.parametrize("rows", [(0,), (1,), (2,), (0, 2), (0, 1, 2), ()])
def test_dwconv_u8_nine_bit_taps_in_chosen_filter_rows(ctx, orc, stride, zp_in, rows):
    """Weights beyond the signed 8-bit range take a second multiply pass, which runs per filter row
    and only for the rows that hold such a tap: place them in chosen rows of a few channels."""
    N, H, W, C = 2, 19, 22, 64
    rng = np.random.Generator(np.random.PCG64(stride * 11 + zp_in + sum(rows) * 3 + len(rows)))
    x = rng.integers(0, 256, size=(N, H, W, C), dtype=np.uint8)
    zp_f, zp_out = 100, 0
    f = rng.integers(0, 228, size=(3, 3, C, 1), dtype=np.uint8)   # f - 100 <= 127 everywhere
    for i, kh in enumerate(rows):
        for c in (3 + 8 * i, 17 + 4 * i, 40):                         # f - 100 = 140 .. 155 there
            f[kh, int(rng.integers(0, 3)), c, 0] = int(rng.integers(240, 256))
    bias = np.rint(rng.normal(0, 500, size=C)).astype(np.int32)
    mult, shift = orc.output_multiplier_and_shift(np.float32(0.02), np.float32(0.01),
                                                  np.float32(0.02 * 0.01 * 3 * 74 * 74 * 3 / 127))
    Ho, Wo, ph, pw = orc.calc_padding_and_output_size(H, W, 3, 3, (1, 1), (stride, stride), PAD["SAME"])
    exp = orc.dwconv_u8(x, f, bias, (stride, stride), (1, 1), (ph >> 1, pw >> 1), (Ho, Wo), zp_in,
                        zp_f, mult, shift, zp_out)
    dx, df, db = ctx.upload(x), ctx.upload(f), ctx.upload(bias)
    do = ctx.alloc(exp.size)
    ctx.dwconv_u8(dx, df, db, do, N, H, W, C, 1, 3, 3, (stride, stride), (1, 1), (ph >> 1, pw >> 1),
                  (Ho, Wo), zp_in, zp_f, mult, shift, zp_out)
    got = ctx.download(do, exp.shape, np.uint8)
    for b in (dx, df, db, do):
        b.free()
    assert np.array_equal(got, exp)
    assert len(np.unique(got)) > 4


@pytest.mark.parametrize("option,value", [("dw_fixed_groups", 0), ("dw_tma_fill", 8), ("dw_tma_fill", 1),
                                          ("dw_lane_setup", 0), ("dw_tma", 0)])
@pytest.mark.parametrize("shape", [(3, 14, 14, 512, 1), (2, 28, 28, 256, 2), (2, 56, 56, 64, 1)])
def test_dwconv_u8_launch_variants(ctx, orc, option, value, shape):
    """The switches that pick the depthwise kernel variant and its launch geometry (generic instead of
    fixed channel-group count, other grid fill rules, one thread instead of a lane per row for the
    copy requests, the register kernel) change no byte of the result."""
    N, H, W, C, stride = shape
    defaults = {"dw_fixed_groups": 1, "dw_tma_fill": 4, "dw_lane_setup": 1, "dw_tma": 1}
    rng = np.random.Generator(np.random.PCG64(H * 7 + C + stride))
    x = rng.integers(0, 256, size=(N, H, W, C), dtype=np.uint8)
    f = rng.integers(0, 256, size=(3, 3, C, 1), dtype=np.uint8)
    bias = np.rint(rng.normal(0, 500, size=C)).astype(np.int32)
    zp_in, zp_f, zp_out = 0, 121, 0
    mult, shift = orc.output_multiplier_and_shift(np.float32(0.02), np.float32(0.01),
                                                  np.float32(0.02 * 0.01 * 3 * 74 * 74 * 3 / 127))
    Ho, Wo, ph, pw = orc.calc_padding_and_output_size(H, W, 3, 3, (1, 1), (stride, stride), PAD["SAME"])
    exp = orc.dwconv_u8(x, f, bias, (stride, stride), (1, 1), (ph >> 1, pw >> 1), (Ho, Wo), zp_in,
                        zp_f, mult, shift, zp_out)
    dx, df, db = ctx.upload(x), ctx.upload(f), ctx.upload(bias)
    do = ctx.alloc(exp.size)
    try:
        ctx.set_option(option, value)
        ctx.dwconv_u8(dx, df, db, do, N, H, W, C, 1, 3, 3, (stride, stride), (1, 1), (ph >> 1, pw >> 1),
                      (Ho, Wo), zp_in, zp_f, mult, shift, zp_out)
        got = ctx.download(do, exp.shape, np.uint8)
    finally:
        ctx.set_option(option, defaults[option])
        for b in (dx, df, db, do):
            b.free()
    assert np.array_equal(got, exp)
    assert len(np.unique(got)) > 4


@pytest.mark.parametrize("case", [
    # N, H, W, C, stride: the MobileNet layer shapes at a small batch ...
    (2, 112, 112, 32, 1), (2, 112, 112, 64, 2), (3, 56, 56, 128, 1), (2, 56, 56, 128, 2), (4, 28, 28, 256, 1),
    (2, 28, 28, 256, 2), (3, 14, 14, 512, 1), (5, 14, 14, 512, 2), (6, 7, 7, 1024, 1),
    # ... and shapes that exercise the tiling: channels that only 16-byte chunks divide, a single
    # row / column, widths beyond one column tile and beyond the 256-column box limit, odd sizes
    (1, 9, 13, 48, 1), (2, 5, 6, 16, 2), (1, 3, 3, 16, 1), (1, 1, 1, 32, 1), (1, 40, 300, 16, 1), (1, 33, 515, 16, 2),
    (2, 31, 29, 80, 1), (1, 64, 7, 2048, 2),
])
def test_dwconv_u8_tma_tiled_kernel(ctx, orc, case):
    """Input zero point 0 (out-of-image taps read as zero): the depthwise kernel whose input rows
    arrive in shared memory by TMA.  Same bytes as the register kernel and as the oracle, with
    filters that need the second weight pass, an int32 bias and SAME padding (stride 2 pads only
    bottom / right)."""
    N, H, W, C, stride = case
    rng = np.random.Generator(np.random.PCG64(H * 1000 + W + C))
    x = rng.integers(0, 256, size=(N, H, W, C), dtype=np.uint8)
    f = rng.integers(1, 256, size=(3, 3, C, 1), dtype=np.uint8)
    bias = np.rint(rng.normal(0, 2000, size=C)).astype(np.int32)
    zp_in, zp_f, zp_out = 0, int(rng.integers(110, 140)), int(rng.integers(0, 2)) * 7
    mult, shift = orc.output_multiplier_and_shift(np.float32(0.02), np.float32(0.01), np.float32(0.02 * 0.01 * 3 * 128 * 74 * 3 / 127))
    Ho, Wo, ph, pw = orc.calc_padding_and_output_size(H, W, 3, 3, (1, 1), (stride, stride), PAD["SAME"])
    exp = orc.dwconv_u8(x, f, bias, (stride, stride), (1, 1), (ph >> 1, pw >> 1), (Ho, Wo), zp_in, zp_f, mult, shift,
                        zp_out)
    dx, df, db = ctx.upload(x), ctx.upload(f), ctx.upload(bias)
    do = ctx.alloc(exp.size + 64)
    packed = ctx.dwconv3x3_u8_prepack(df, db, C, zp_in, zp_f)
    L = __import__("mace_b200").lib()
    got = {}
    for tma in (1, 0):
        ctx.set_option("dw_tma", tma)
        try:
            for pre in (None, packed):
                ctx._check(L.mb_memset(ctx.h, do.ptr, 0xA5, do.nbytes))
                ctx.dwconv_u8(dx, df, db, do, N, H, W, C, 1, 3, 3, (stride, stride), (1, 1), (ph >> 1, pw >> 1),
                              (Ho, Wo), zp_in, zp_f, mult, shift, zp_out, prepacked=pre)
                raw = ctx.download(do, (do.nbytes,), np.uint8)
                assert (raw[exp.size:] == 0xA5).all(), "wrote past the output"
                got[tma] = raw[:exp.size].reshape(exp.shape)
                assert np.array_equal(got[tma], exp), (tma, pre is not None)
        finally:
            ctx.set_option("dw_tma", 1)
    ctx.sync()
    assert len(np.unique(exp)) > 4
    for b in (dx, df, db, do, packed):
        b.free()


def test_dwconv_u8_repack_into_the_same_buffer_then_run_at_once(ctx, orc):
    """The depthwise kernel fetches cached tap words before it waits for the kernel in front of
    it.  When that kernel is the one that (re)wrote the tap words -- a delegator's first run, or
    a weight update -- the fetch has to wait: alternate two filters through ONE prepacked
    buffer, launching the convolution right behind each repack with nothing in between."""
    rng = np.random.Generator(np.random.PCG64(77))
    N, H, W, C = 8, 56, 56, 256
    x = rng.integers(0, 256, size=(N, H, W, C), dtype=np.uint8)
    zp_in, zp_f, zp_out = 0, 128, 0
    mult, shift = orc.output_multiplier_and_shift(np.float32(0.02), np.float32(0.01), np.float32(3.0))
    filters = [rng.integers(1, 256, size=(3, 3, C, 1), dtype=np.uint8) for _ in range(2)]
    biases = [np.rint(rng.normal(0, 500, size=C)).astype(np.int32) for _ in range(2)]
    exps = [orc.dwconv_u8(x, f, b, (1, 1), (1, 1), (1, 1), (H, W), zp_in, zp_f, mult, shift, zp_out)
            for f, b in zip(filters, biases)]
    assert not np.array_equal(exps[0], exps[1])
    dx, do = ctx.upload(x), ctx.alloc(x.size)
    dfs, dbs = [ctx.upload(f) for f in filters], [ctx.upload(b) for b in biases]
    packed = ctx.dwconv3x3_u8_prepack(dfs[0], dbs[0], C, zp_in, zp_f)
    L = __import__("mace_b200").lib()
    for it in range(6):
        k = it & 1
        ctx._check(L.mb_dwconv3x3_u8_prepack(ctx.h, dfs[k].ptr, dbs[k].ptr, C, zp_in, zp_f, packed.ptr))
        ctx.dwconv_u8(dx, dfs[k], dbs[k], do, N, H, W, C, 1, 3, 3, (1, 1), (1, 1), (1, 1), (H, W),
                      zp_in, zp_f, mult, shift, zp_out, prepacked=packed)
        assert np.array_equal(ctx.download(do, x.shape, np.uint8), exps[k]), it
        # a second launch may fetch early again: the tap words are settled
        ctx.dwconv_u8(dx, dfs[k], dbs[k], do, N, H, W, C, 1, 3, 3, (1, 1), (1, 1), (1, 1), (H, W),
                      zp_in, zp_f, mult, shift, zp_out, prepacked=packed)
        assert np.array_equal(ctx.download(do, x.shape, np.uint8), exps[k]), it
    for b in [dx, do, packed] + dfs + dbs:
        b.free()


# ---- pooling -----------------------------------------------------------------------

@pytest.mark.parametrize("case", [(64, 7, 7, 1024, 7, 7, 1, "VALID"), (2, 9, 11, 24, 3, 3, 2, "SAME"),
                                  (1, 8, 8, 5, 2, 2, 2, "VALID")])
def test_avgpool_u8(ctx, orc, case):
    N, H, W, C, KH, KW, stride, padding = case
    rng = np.random.Generator(np.random.PCG64(3))
    x = rng.integers(0, 256, size=(N, H, W, C), dtype=np.uint8)
    Ho, Wo, ph, pw = orc.calc_padding_and_output_size(H, W, KH, KW, (1, 1), (stride, stride),
                                                      PAD[padding])
    exp = orc.avgpool_u8(x, (KH, KW), (stride, stride), (ph >> 1, pw >> 1), (Ho, Wo))
    dx, do = ctx.upload(x), ctx.alloc(exp.size)
    ctx.avgpool_u8(dx, do, N, H, W, C, (KH, KW), (stride, stride), (ph >> 1, pw >> 1), (Ho, Wo))
    got = ctx.download(do, exp.shape, np.uint8)
    assert np.array_equal(got, exp)


@pytest.mark.parametrize("size", [1, 7, 4096, 1000003])
def test_quantize_dequantize_minmax(ctx, orc, size):
    """Quantize / Dequantize / FindMinMax on the device, bit-exact against the oracle, with
    values that hit both saturation ends and exact rounding ties."""
    rng = np.random.Generator(np.random.PCG64(size))
    x = (rng.standard_normal(size) * 3).astype(np.float32)
    x[:: max(1, size // 50)] = 0.5 * 0.0625 * np.arange(len(x[:: max(1, size // 50)]))  # ties at scale 1/16
    dx, dq, dy = ctx.upload(x), ctx.alloc(size), ctx.alloc(size * 4)
    assert ctx.minmax_f32(dx, size) == orc.find_min_max(x)
    for scale, zp in ((0.0625, 128), (0.02, 3), (0.11, 250)):
        ctx.quantize_f32_u8(dx, dq, size, scale, zp)
        q = ctx.download(dq, (size,), np.uint8)
        assert np.array_equal(q, orc.quantize(x, scale, zp))
        ctx.dequantize_f32(dq, dy, size, scale, zp)
        assert np.array_equal(ctx.download(dy, (size,), np.float32), orc.dequantize(q, scale, zp))
    acc = rng.integers(-2 ** 20, 2 ** 20, size=size, dtype=np.int32)
    da = ctx.upload(acc)
    ctx.dequantize_f32(da, dy, size, 3.7e-4, 0, int32=True)
    assert np.array_equal(ctx.download(dy, (size,), np.float32), orc.dequantize(acc, 3.7e-4, 0))
    for b in (dx, dq, dy, da):
        b.free()
